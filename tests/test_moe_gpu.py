"""Routing, gather, SwiGLU, combine, quantiser and the whole MoE layer on the GPU against
the CPU oracle and the fixtures produced by the reference's code."""
import numpy as np
import pytest
import torch

import applied_ai_b200 as B
from applied_ai_b200 import configs as C
from oracle import grouped as O
from tests.helpers import BF16_REL_TOL, bf16_from_bits, load_npz

pytestmark = pytest.mark.gpu
DEV = "cuda"


def check_route(ids, E):
    m_sizes, offsets, perm, inv = B.route(ids.to(DEV), E)
    rm, ro, rp, ri = O.route_ref(ids, E)
    assert torch.equal(m_sizes.cpu(), rm) and torch.equal(offsets.cpu(), ro)
    assert torch.equal(perm.cpu(), rp) and torch.equal(inv.cpu(), ri)
    for t in (m_sizes, offsets, perm, inv):
        assert t.dtype == torch.int32


def test_route_bit_exact():
    g = torch.Generator().manual_seed(1)
    check_route(torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=torch.int32), 5)  # docstring example
    for (T, k, E) in [(1, 1, 1), (7, 2, 8), (4096, 2, 8), (1000, 8, 256), (333, 3, 1000), (50, 2, 2048), (32768, 8, 256)]:
        check_route(torch.randint(0, E, (T, k), generator=g, dtype=torch.int32), E)
    # heavy skew: everything on one expert, and experts that receive nothing
    check_route(torch.full((5000, 2), 3, dtype=torch.int32), 8)
    _, ids = C.routing(4096, 8, 2, 1002)
    check_route(ids, 8)


def test_route_rejects_bad_ids():
    ids = torch.tensor([[0, 9]], dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):
        B.route(ids, 4)
    check_route(torch.tensor([[0, 3]], dtype=torch.int32), 4)
    with pytest.raises(RuntimeError):  # more experts than the routing kernels support
        B.route(torch.zeros(4, 2, dtype=torch.int32, device=DEV), 4096)


def test_moe_align_block_size_matches_reference_format():
    """Docstring example of the reference (v0_moe_fused.py:157-165) and random cases vs the oracle."""
    import json
    import os
    from tests.helpers import GOLDEN
    ex = json.load(open(os.path.join(GOLDEN, "align_example.json")))
    ids = torch.tensor(ex["topk_ids"], dtype=torch.int32)
    s, e, p = B.moe_align_block_size(ids.to(DEV), ex["block_size"], 5)
    assert s.numel() == ids.numel() + 5 * (ex["block_size"] - 1) and e.numel() == ids.numel() + 5
    assert s[: int(p)].tolist() == ex["sorted_token_ids"] and int(p) == 16
    assert e[: int(p) // ex["block_size"]].tolist() == [1, 2, 3, 4]
    g = torch.Generator().manual_seed(8)
    for (T, k, E, blk) in [(64, 2, 8, 16), (1000, 8, 256, 64), (4096, 2, 8, 64), (5, 1, 3, 128)]:
        ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
        s, e, p = B.moe_align_block_size(ids.to(DEV), blk, E)
        rs, re_, rp = O.moe_align_block_size_ref(ids, blk, E)
        assert torch.equal(p.cpu(), rp) and torch.equal(s.cpu(), rs)
        nb = int(rp) // blk
        assert torch.equal(e.cpu()[:nb], re_[:nb])


def test_gather_rows():
    g = torch.Generator().manual_seed(2)
    for (T, H, k, dtype) in [(64, 4096, 2, torch.bfloat16), (33, 7168, 8, torch.bfloat16), (50, 56, 2, torch.float32),
                             (9, 7, 3, torch.uint8)]:
        src = torch.randint(0, 255, (T, H), generator=g).to(dtype)
        idx = torch.randperm(T * k, generator=g).to(torch.int32)
        out = B.gather_rows(src.to(DEV), idx.to(DEV), div=k)
        assert torch.equal(out.cpu(), src[(idx // k).long()])


def test_silu_and_mul():
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(77, 2 * 264, generator=g) * 3).to(torch.bfloat16)
    out = B.silu_and_mul(x.to(DEV)).cpu().float()
    ref = O.silu_and_mul_ref(x.float())
    torch.testing.assert_close(out, ref, rtol=1e-2, atol=1e-2)


def test_combine_topk():
    g = torch.Generator().manual_seed(4)
    T, k, H = 100, 3, 264
    y = torch.randn(T * k, H, generator=g).to(torch.bfloat16)
    w = torch.rand(T, k, generator=g)
    inv = torch.randperm(T * k, generator=g).to(torch.int32)
    out = B.combine_topk(y.to(DEV), inv.to(DEV), w.to(DEV), T, k).cpu().float()
    ref = (y.float()[inv.long()].view(T, k, H) * w.view(T, k, 1)).sum(1)
    torch.testing.assert_close(out, ref, rtol=1e-2, atol=1e-2)


def test_quant_1x128_bit_exact():
    z = load_npz("quant_1x128.npz")
    x = torch.from_numpy(z["x"])
    for inp in (x, x.to(torch.bfloat16)):
        q, s = B.float8_groupwise_quantize(inp.to(DEV))
        rq, rs = O.quant_1x128_ref(inp)
        assert torch.equal(s.cpu(), rs)
        assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    np.testing.assert_array_equal(B.float8_groupwise_quantize(x.to(DEV))[1].cpu().numpy(), z["scales"])
    g = torch.Generator().manual_seed(5)
    big = torch.randn(3, 500, 1024, generator=g).to(torch.bfloat16)
    q, s = B.float8_groupwise_quantize(big.to(DEV))
    rq, rs = O.quant_1x128_ref(big)
    assert s.shape == (3, 500, 8) and torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))


@pytest.mark.parametrize("cta", [1, 2])
def test_fused_moe_golden(cta):
    """Inputs and outputs of the reference's `torch_moe` (test_moe_gemm.py:16-30)."""
    z = load_npz("torch_moe.npz")
    for i in range(int(z["n_cases"])):
        a, w1, w2 = (bf16_from_bits(z[f"{n}{i}"]).to(DEV) for n in ("a", "w1", "w2"))
        tw = torch.from_numpy(z[f"topk_weight{i}"]).to(DEV)
        ids = torch.from_numpy(z[f"topk_ids{i}"]).to(DEV)
        ref = torch.from_numpy(z[f"out{i}"])
        out = B.fused_moe(a, w1, w2, tw, ids, cta_group=cta).cpu().float()
        assert O.rel_err(out, ref) <= BF16_REL_TOL
        # the reference's own acceptance bound (test_moe_gemm.py:78)
        assert torch.allclose(out, ref, atol=1e-2, rtol=0)


def test_fused_moe_layer_and_inplace():
    hidden, w1, w2, tw, ids = C.c3_mixtral_layer(T=256, H=512, I=768, E=8, k=2)
    ref = O.torch_moe_ref(hidden, w1, w2, tw, ids)
    h = hidden.to(DEV)
    out = B.fused_moe(h, w1.to(DEV), w2.to(DEV), tw.to(DEV), ids.to(DEV))
    assert O.rel_err(out.cpu().float(), ref) <= BF16_REL_TOL
    ret = B.fused_moe(h, w1.to(DEV), w2.to(DEV), tw.to(DEV), ids.to(DEV), inplace=True)
    assert ret.data_ptr() == h.data_ptr() and torch.equal(h, out)


def test_full_size_mixtral_layer():
    """The Mixtral-8x7B FFN layer shapes at full size (T=4096, H=4096, I=14336, E=8, top-2): routing bit-exact
    on all 8192 routed rows, the layer output on 64 sampled tokens against the reference's `torch_moe`
    procedure (kernels/triton/inference/col_major_moe_gemm/test_moe_gemm.py:16-30, routing fed as at :54-57)."""
    T, H, I, E, k = 4096, 4096, 14336, 8, 2
    tw, ids = C.routing(T, E, k, 1002)
    gd = torch.Generator(device=DEV).manual_seed(1002)
    hidden = torch.randn(T, H, generator=gd, device=DEV).to(torch.bfloat16)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=DEV)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=DEV)
    for e in range(E):
        w1[e] = (torch.randn(2 * I, H, generator=gd, device=DEV) * H ** -0.5).to(torch.bfloat16)
        w2[e] = (torch.randn(H, I, generator=gd, device=DEV) * I ** -0.5).to(torch.bfloat16)
    got = B.route(ids.to(DEV), E)
    for a, b, name in zip(got, O.route_ref(ids, E), ("m_sizes", "offsets", "perm", "inv_perm")):
        assert torch.equal(a.cpu(), b), name
    out = B.fused_moe(hidden, w1, w2, tw.to(DEV), ids.to(DEV))
    assert tuple(out.shape) == (T, H) and bool(torch.isfinite(out.float()).all())
    pick = torch.randperm(T, generator=torch.Generator().manual_seed(5))[:64]
    ref = O.torch_moe_ref(hidden[pick.to(DEV)].cpu(), w1.cpu(), w2.cpu(), tw[pick], ids[pick])
    got_rows = out[pick.to(DEV)].cpu().float()
    assert O.rel_err(got_rows, ref) <= BF16_REL_TOL
    assert torch.allclose(got_rows, ref, atol=1e-2 * float(ref.abs().max()), rtol=1.6e-2)


def test_fused_moe_replays_from_a_cuda_graph():
    """With check=False the layer is a fixed sequence of launches on the current stream (no host read, no
    allocation outside torch's caching allocator), so it can be captured once and replayed on new inputs and
    new routing written into the same tensors."""
    T, H, I, E, k = 256, 512, 768, 8, 2
    hidden, w1, w2, tw, ids = (t.to(DEV) for t in C.c3_mixtral_layer(T=T, H=H, I=I, E=E, k=k, seed=1002))
    hidden2, _, _, tw2, ids2 = (t.to(DEV) for t in C.c3_mixtral_layer(T=T, H=H, I=I, E=E, k=k, seed=2002))
    want1 = B.fused_moe(hidden, w1, w2, tw, ids)
    want2 = B.fused_moe(hidden2, w1, w2, tw2, ids2)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # first calls on this stream create its status word and workspace
            B.fused_moe(hidden, w1, w2, tw, ids, check=False)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        out = B.fused_moe(hidden, w1, w2, tw, ids, check=False)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want1)
    hidden.copy_(hidden2)
    tw.copy_(tw2)
    ids.copy_(ids2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want2)
    assert B.pending_status() is None
