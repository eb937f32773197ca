"""b200moe_route_noalloc: routing for hosts that cannot hand the library a scratch buffer.

Some processes that embed this library have no device memory left to give and no way
to ask for more: an inference server that reserved all free HBM for its cache pool at
start-up, or a plugin living under an allocator it does not control.  For them the
library keeps the routing scratch in a fixed 1 MiB array of its own.  This test drives
the entry point through the C ABI, twice in a row on different inputs (the array keeps
what the previous call left there, which must not matter), and requires the four output
arrays to be bit-identical to those of b200moe_route with a caller-provided workspace.

Collected last on purpose (file name), and it must pass both alone in a fresh process
and after every other test has run in the same process.
"""
import ctypes

import pytest
import torch

from applied_ai_b200 import _lib
from oracle import grouped as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _outputs(R, E):
    return [torch.full((n,), -7, dtype=torch.int32, device=DEV) for n in (E, E + 1, max(R, 1), max(R, 1))]


def _route_with_workspace(lib, ids, E):
    R = ids.numel()
    need = ctypes.c_size_t(0)
    assert lib.b200moe_route_workspace_bytes(R, E, ctypes.byref(need)) == 0
    ws = torch.empty(max(need.value, 4), dtype=torch.uint8, device=DEV)
    out = _outputs(R, E)
    rc = lib.b200moe_route(ids.data_ptr(), R, E, *[t.data_ptr() for t in out], ws.data_ptr(), ws.numel(), None,
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def _route_noalloc(lib, ids, E):
    R = ids.numel()
    out = _outputs(R, E)
    rc = lib.b200moe_route_noalloc(ids.data_ptr(), R, E, *[t.data_ptr() for t in out], None,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return out


def test_route_noalloc_matches_route_on_two_calls_in_a_row():
    lib = _lib.load()
    g = torch.Generator().manual_seed(2024)
    # first call: large, fills most of the array; second: small and different, reuses it dirty
    cases = [(32768 * 8, 256), (4096 * 2, 8), (1000 * 3, 100), (7, 2048), (32768, 2048)]
    for R, E in cases:
        ids = torch.randint(0, E, (R,), generator=g, dtype=torch.int32).to(DEV)
        got = _route_noalloc(lib, ids, E)
        ref = _route_with_workspace(lib, ids, E)
        torch.cuda.synchronize()
        for a, b, name in zip(got, ref, ("m_sizes", "offsets", "perm", "inv_perm")):
            assert torch.equal(a, b), f"{name} differs for R={R} E={E}"
        assert int(got[0].sum()) == R
        # and against the CPU restatement of the ordering itself, not only against the sibling entry point
        for a, b, name in zip(got, O.route_ref(ids.cpu(), E), ("m_sizes", "offsets", "perm", "inv_perm")):
            assert torch.equal(a.cpu(), b), f"{name} differs from the oracle for R={R} E={E}"


def test_route_noalloc_rejects_sizes_beyond_its_array():
    lib = _lib.load()
    R, E = 300000, 2048          # 1024 chunks x 2048 experts of counts would need 8 MiB
    ids = torch.zeros(R, dtype=torch.int32, device=DEV)
    out = _outputs(R, E)
    rc = lib.b200moe_route_noalloc(ids.data_ptr(), R, E, *[t.data_ptr() for t in out], None,
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == -7
    torch.cuda.synchronize()
    assert all(bool((t == -7).all()) for t in out)   # nothing was enqueued
    assert "beyond" in _lib.ERROR_NAMES[-7]
