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


def test_full_size_deepseek_gate_up_shape_sampled():
    """The bench's backward shape (G=8, K=7168, N=4096, M=16384, ragged groups with partial 64-row blocks) against
    the oracle on what it can do in seconds: grad_x on sampled rows of every group (rows are independent, so the
    oracle runs on the sampled rows with the per-group counts), grad_w on sampled rows n of w in every group
    (grad_w[g][n] depends on column n of grad_output only)."""
    g = torch.Generator().manual_seed(63)
    G, M, N, K = 8, 16384, 4096, 7168
    m = random_m_sizes(G, M - 300, g)          # ragged, sum < M
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    dy = torch.randn(M, N, generator=g).to(torch.bfloat16)
    gx, gw = grouped_gemm_backward(dy.to(DEV), x.to(DEV), w.to(DEV), m.to(DEV))
    gx, gw = gx.cpu().float(), gw.cpu().float()
    # grad_x: first, last and two random rows of every non-empty group
    starts = torch.cumsum(m, 0) - m
    rows, counts = [], []
    for e in range(G):
        n_e = int(m[e])
        pick = sorted({0, n_e - 1, *torch.randint(0, max(n_e, 1), (2,), generator=g).tolist()}) if n_e else []
        rows += [int(starts[e]) + r for r in pick]
        counts.append(len(pick))
    rows = torch.tensor(rows)
    rx, _ = O.grouped_gemm_backward_ref(dy[rows], x[rows], w, torch.tensor(counts, dtype=torch.int32))
    assert O.rel_err(gx[rows], rx) <= BF16_REL_TOL
    assert bool((gx[int(m.sum()):] == 0).all())
    # grad_w: 6 sampled rows n, all groups, all K
    ns = torch.randint(0, N, (6,), generator=g)
    _, rw = O.grouped_gemm_backward_ref(dy[:, ns].contiguous(), x, w[:, ns].contiguous(), m)
    assert O.rel_err(gw[:, ns], rw) <= BF16_REL_TOL
    assert torch.allclose(gw[:, ns], rw, rtol=1e-2, atol=1e-2 * max(1.0, float(rw.abs().max())))
