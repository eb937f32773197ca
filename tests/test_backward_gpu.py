"""grouped_gemm_backward on the GPU against the oracle and the fixture produced by the reference's
`_pytorch_reference_backward`; tolerance rtol = atol = 1e-2 as in the reference's own check
(kernels/MoE/group_GEMM/triton/testing/fast_verification.py:111-122), plus the normalised bound."""
import pytest
import torch

from applied_ai_b200.tgroup_gemm_backwards import grouped_gemm_backward
from oracle import grouped as O
from tests.helpers import BF16_REL_TOL, bf16_from_bits, load_npz, random_m_sizes

pytestmark = pytest.mark.gpu
DEV = "cuda"


def check(dy, x, w, m, cta):
    gx, gw = grouped_gemm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), m.to(DEV), cta_group=cta)
    rx, rw = O.grouped_gemm_backward_ref(dy, x, w, m)
    assert gx.shape == x.shape and gw.shape == w.shape and gx.dtype == gw.dtype == torch.bfloat16
    assert O.rel_err(gx.cpu().float(), rx) <= BF16_REL_TOL
    assert O.rel_err(gw.cpu().float(), rw) <= BF16_REL_TOL
    assert torch.allclose(gx.cpu().float(), rx, rtol=1e-2, atol=1e-2 * max(1.0, float(rx.abs().max())))
    assert torch.allclose(gw.cpu().float(), rw, rtol=1e-2, atol=1e-2 * max(1.0, float(rw.abs().max())))
    return gx, gw


@pytest.mark.parametrize("cta", [1, 2])
def test_golden_from_reference_function(cta):
    z = load_npz("backward.npz")
    for i in range(int(z["n_cases"])):
        x, w, dy = (bf16_from_bits(z[f"{n}{i}"]) for n in ("x", "w", "dy"))
        m = torch.from_numpy(z[f"m_sizes{i}"])
        gx, gw = grouped_gemm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), m.to(DEV), cta_group=cta)
        assert O.rel_err(gx.cpu().float(), torch.from_numpy(z[f"grad_x{i}"])) <= BF16_REL_TOL
        assert O.rel_err(gw.cpu().float(), torch.from_numpy(z[f"grad_w{i}"])) <= BF16_REL_TOL


@pytest.mark.parametrize("cta", [1, 2])
def test_fast_verification_shape_and_ragged_cases(cta):
    g = torch.Generator().manual_seed(61)
    # the reference's own check: G=20, M=1024, N=512, K=256, even split, block-layout grad_output
    G, M, N, K = 20, 1024, 512, 256
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(G * N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    dy = torch.randn(M, N * G, generator=g).to(torch.bfloat16)
    m = torch.full((G,), M // G, dtype=torch.int32)
    m[-1] += M - int(m.sum())
    check(dy, x, w, m, cta)
    # ragged: empty groups, sizes straddling 64 / 128 / 256, sum < M, [M, N] layout, odd N and K tiles
    for (G, M, N, K, sizes) in [(6, 700, 192, 320, [0, 1, 63, 65, 0, 300]), (3, 520, 264, 136, [129, 256, 130]),
                                (1, 100, 64, 64, [100])]:
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        m = torch.tensor(sizes, dtype=torch.int32)
        check(torch.randn(M, N * G, generator=g).to(torch.bfloat16), x, w, m, cta)
        gx, gw = check(torch.randn(M, N, generator=g).to(torch.bfloat16), x, w, m, cta)
        rows = int(m.sum())
        assert bool((gx[rows:] == 0).all())
        for e, s in enumerate(sizes):
            if s == 0:
                assert bool((gw[e] == 0).all())


def test_random_groups_and_errors():
    g = torch.Generator().manual_seed(62)
    G, M, N, K = 16, 2048, 256, 512
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(G * N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    dy = torch.randn(M, N * G, generator=g).to(torch.bfloat16)
    check(dy, x, w, random_m_sizes(G, M, g), 0)
    with pytest.raises(ValueError):
        grouped_gemm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), torch.full((G,), 200, dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError):
        grouped_gemm_backward(dy.to(DEV)[:, :100].contiguous(), x.to(DEV), w.to(DEV),
                              torch.full((G,), 128, dtype=torch.int32, device=DEV))
