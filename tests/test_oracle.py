"""The CPU oracle against fixtures produced by the reference's own test code
(tests/golden/make_golden.py).  Runs without a GPU."""
import json
import os

import numpy as np
import torch

from oracle import grouped as O
from tests.helpers import GOLDEN, bf16_from_bits, load_npz


def test_grouped_loop_matches_reference_expected():
    z = load_npz("grouped_bf16.npz")
    for i in range(int(z["n_cases"])):
        G, M, N, K = [int(v) for v in z[f"shape{i}"]]
        a, b = bf16_from_bits(z[f"a{i}"]), bf16_from_bits(z[f"b{i}"])
        m_sizes = torch.from_numpy(z[f"m_sizes{i}"])
        expected = bf16_from_bits(z[f"expected{i}"]).float()
        assert a.shape == (M, K) and b.shape == (G * N, K) and int(m_sizes.sum()) == M
        y = O.grouped_gemm_ref(a, b, m_sizes)
        # The reference's expected values went through a bf16 matmul and a bf16 store;
        # the oracle keeps fp32.  One bf16 rounding separates them.
        assert O.rel_err(y, expected) < 4e-3
        torch.testing.assert_close(y.to(torch.bfloat16).float(), expected, rtol=1.6e-2, atol=2e-2)
        # block layout holds the same numbers on the diagonal blocks and zeros elsewhere
        y_ng = O.grouped_gemm_ref(a, b, m_sizes, layout="NG")
        start = 0
        for g in range(G):
            m = int(m_sizes[g])
            assert torch.equal(y_ng[start:start + m, g * N:(g + 1) * N], y[start:start + m])
            start += m
        assert float(y_ng.abs().sum()) == float(y.abs().sum()) or abs(
            float(y_ng.abs().sum()) - float(y.abs().sum())) < 1e-3 * float(y.abs().sum())


def test_fp8_rowwise_loop_matches_reference_expected():
    """Fixture = the expected values of the reference's own (switched-off) FP8 row-wise test,
    computed by its loop at dev/triton_groupGEMM/testing/base_testing.py:75-88."""
    z = load_npz("grouped_fp8_rowwise.npz")
    for i in range(int(z["n_cases"])):
        G, M, N, K = [int(v) for v in z[f"shape{i}"]]
        a = torch.from_numpy(z[f"a{i}"]).view(torch.float8_e4m3fn)
        b = torch.from_numpy(z[f"b{i}"]).view(torch.float8_e4m3fn)
        a_s, b_s = torch.from_numpy(z[f"a_scale{i}"]), torch.from_numpy(z[f"b_scale{i}"])
        m_sizes = torch.from_numpy(z[f"m_sizes{i}"])
        expected = bf16_from_bits(z[f"expected{i}"]).float()
        assert a.shape == (M, K) and b.shape == (G * N, K) and int(m_sizes.sum()) == M
        y = O.grouped_gemm_fp8_rowwise_ref(a, b, m_sizes, a_s, b_s)
        # the reference stores its fp32 loop result as bf16: one rounding apart, then its own tolerance (:90)
        assert torch.equal(y.to(torch.bfloat16).float(), expected) or O.rel_err(y, expected) < 4e-3
        torch.testing.assert_close(y.to(torch.bfloat16).float(), expected, rtol=float(z["rtol"]), atol=float(z["atol"]))


def test_torch_moe_matches_reference_output():
    z = load_npz("torch_moe.npz")
    for i in range(int(z["n_cases"])):
        a, w1, w2 = (bf16_from_bits(z[f"{n}{i}"]) for n in ("a", "w1", "w2"))
        tw = torch.from_numpy(z[f"topk_weight{i}"])
        ids = torch.from_numpy(z[f"topk_ids{i}"])
        ref = torch.from_numpy(z[f"out{i}"])
        out = O.torch_moe_ref(a, w1, w2, tw, ids)
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-6)


def test_route_matches_docstring_example():
    ex = json.load(open(os.path.join(GOLDEN, "align_example.json")))
    ids = torch.tensor(ex["topk_ids"], dtype=torch.int32)
    E = int(ids.max()) + 1  # the example's ids run 1..4
    sorted_ids, expert_ids, post = O.moe_align_block_size_ref(ids, ex["block_size"], E)
    numel = ids.numel()
    # slot 0 is empty in the example; the documented list starts at expert 1
    got = sorted_ids[: int(post)].tolist()
    assert got == ex["sorted_token_ids"]
    assert int(post) == len(ex["sorted_token_ids"])
    assert expert_ids[: int(post) // ex["block_size"]].tolist() == [1, 2, 3, 4]
    assert sorted_ids.numel() == numel + E * (ex["block_size"] - 1)
    m_sizes, offsets, perm, inv = O.route_ref(ids, E)
    assert perm.tolist() == [v for v in ex["sorted_token_ids"] if v != numel]
    assert inv[perm.long()].tolist() == list(range(numel))
    assert m_sizes.tolist() == [0, 3, 3, 3, 3] and offsets.tolist() == [0, 0, 3, 6, 9, 12]


def test_route_order_is_the_mask_order_of_torch_moe():
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 7, (50, 3), generator=g, dtype=torch.int32)
    _, _, perm, _ = O.route_ref(ids, 7)
    flat = ids.reshape(-1)
    by_mask = torch.cat([torch.nonzero(flat == e).reshape(-1) for e in range(7)])
    assert perm.tolist() == by_mask.tolist()


def test_quant_matches_reference_kernel():
    """Scales are bit-identical to the reference kernel's.  The fixture's e4m3 bytes come
    from Triton's CPU interpreter, whose fp32->e4m3 conversion drops the carry when
    rounding overflows the mantissa (1.96 becomes 1.0 instead of 2.0); hardware conversion
    carries.  Every byte must agree except exactly those carries, where the oracle's value
    is the power of two just above and twice the interpreter's."""
    z = load_npz("quant_1x128.npz")
    x = torch.from_numpy(z["x"])
    q, s = O.quant_1x128_ref(x)
    np.testing.assert_array_equal(s.numpy(), z["scales"])
    mine = q.view(torch.uint8).numpy()
    theirs = z["q"]
    diff = mine != theirs
    assert diff.mean() < 0.03
    v_mine = torch.from_numpy(mine[diff]).view(torch.float8_e4m3fn).float()
    v_theirs = torch.from_numpy(theirs[diff]).view(torch.float8_e4m3fn).float()
    assert torch.equal(v_mine, 2 * v_theirs)
    assert torch.equal(torch.log2(v_mine.abs()), torch.log2(v_mine.abs()).round())  # powers of two
    exact = (x.reshape(24, 4, 128) / s[..., None]).reshape(24, 512)[torch.from_numpy(diff)]
    assert bool(((exact.abs() >= 0.75 * v_mine.abs()) & (exact.abs() <= v_mine.abs())).all())  # rounded up to it


def test_fp8_forms_agree_where_they_overlap():
    g = torch.Generator().manual_seed(9)
    M, N, K, G = 96, 256, 256, 3
    m_sizes = torch.tensor([40, 0, 56], dtype=torch.int32)
    x = torch.randn(M, K, generator=g)
    w = torch.randn(G, N, K, generator=g) * K ** -0.5
    xq, xs = O.quant_1x128_ref(x)
    # a block-wise problem whose scales are constant along K is a row-wise problem
    xs_const = xs[:, :1].expand(-1, K // 128).contiguous()
    ws_blk = torch.rand(G, N // 128, 1, generator=g).expand(-1, -1, K // 128).contiguous() + 0.5
    wq = (w / 4).to(torch.float8_e4m3fn)
    y_blk = O.grouped_gemm_fp8_blockwise_ref(xq, wq, m_sizes, xs_const, ws_blk)
    w_row_scale = ws_blk[:, :, 0].repeat_interleave(128, dim=1).reshape(-1)
    y_row = O.grouped_gemm_fp8_rowwise_ref(xq, wq.reshape(G * N, K), m_sizes, xs_const[:, 0].contiguous(), w_row_scale)
    torch.testing.assert_close(y_blk, y_row, rtol=1e-4, atol=1e-4)


def test_backward_matches_reference_function():
    z = load_npz("backward.npz")
    for i in range(int(z["n_cases"])):
        x, w, dy = (bf16_from_bits(z[f"{n}{i}"]) for n in ("x", "w", "dy"))
        m = torch.from_numpy(z[f"m_sizes{i}"])
        gx, gw = O.grouped_gemm_backward_ref(dy, x, w, m)
        torch.testing.assert_close(gx, torch.from_numpy(z[f"grad_x{i}"]), rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(gw, torch.from_numpy(z[f"grad_w{i}"]), rtol=1e-5, atol=1e-5)
        # the [M, N] layout carries the same numbers
        G = m.numel()
        N = w.shape[0] // G
        dy_mn = torch.cat([dy[int(m[:g].sum()):int(m[:g + 1].sum()), g * N:(g + 1) * N] for g in range(G)])
        dy_mn = torch.cat([dy_mn, torch.zeros(x.shape[0] - dy_mn.shape[0], N, dtype=dy.dtype)])
        gx2, gw2 = O.grouped_gemm_backward_ref(dy_mn, x, w, m)
        assert torch.equal(gx, gx2) and torch.equal(gw, gw2)
