"""CPU restatement of the reference's ground-truth procedures for the MoE grouped-GEMM
path.  TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs as the checker / baseline.  Nothing in the product
package imports this module and nothing here is a fallback for the CUDA path.

The reference's own ground truth is a handful of torch expressions inside its test
files; each function below restates one of them and cites it (paths are relative to
the reference repository).  Parity pins: tests/golden/*.npz hold outputs of the
reference's own test code executed on the CPU (tests/golden/make_golden.py runs the
loop of base_testing.py and `torch_moe` of test_moe_gemm.py straight from the
reference's files), and tests/test_oracle.py checks this module against them.  The
FP8 block-wise form and the permutation indices have no counterpart that can run in
the reference (FBGEMM / vLLM ops are absent): for those, parity is pinned only by the
definitions stated here.

All functions take CPU tensors and compute in fp32.
"""
import torch


def _offsets(m_sizes):
    sizes = [int(v) for v in m_sizes.tolist()]
    starts, acc = [], 0
    for s in sizes:
        starts.append(acc)
        acc += s
    return sizes, starts


def grouped_gemm_ref(x, w, m_sizes, layout="MN"):
    """Per-expert matmul loop, fp32 accumulate on the given (already rounded) inputs.

    layout "MN": y [M, N], y[rows_g] = x[rows_g] @ w[g].T
        (dev/triton_groupGEMM/testing/base_testing.py:125-131, unit_tests.py:49-55).
    layout "NG": y [M, N*G], y[rows_g, g*N:(g+1)*N] = x[rows_g] @ w[g].T, zeros elsewhere
        (kernels/MoE/group_GEMM/triton/testing/fast_verification.py:83-96).
    w is [G*N, K] or [G, N, K].  Returns fp32; rows past sum(m_sizes) stay zero."""
    G = m_sizes.numel()
    M, K = x.shape
    w3 = w.reshape(G, -1, K).float()
    N = w3.shape[1]
    xf = x.float()
    y = torch.zeros(M, N if layout == "MN" else N * G, dtype=torch.float32)
    sizes, starts = _offsets(m_sizes)
    for g in range(G):
        a, b = starts[g], starts[g] + sizes[g]
        if sizes[g] == 0:
            continue
        blk = xf[a:b] @ w3[g].T
        if layout == "MN":
            y[a:b] = blk
        else:
            y[a:b, g * N:(g + 1) * N] = blk
    return y


def grouped_gemm_fp8_rowwise_ref(xq, wq, m_sizes, x_scale, w_scale, layout="MN"):
    """Loop on the already quantised operands, scales applied after the product
    (dev/triton_groupGEMM/testing/base_testing.py:75-88)."""
    G = m_sizes.numel()
    M, K = xq.shape
    w3 = wq.reshape(G, -1, K).float()
    N = w3.shape[1]
    y = grouped_gemm_ref(xq.float(), w3, m_sizes, layout)
    ws = w_scale.reshape(G, N).float()
    sizes, starts = _offsets(m_sizes)
    for g in range(G):
        a, b = starts[g], starts[g] + sizes[g]
        cols = slice(None) if layout == "MN" else slice(g * N, (g + 1) * N)
        y[a:b, cols] = y[a:b, cols] * x_scale[a:b, None].float() * ws[g][None, :]
    return y


def grouped_gemm_fp8_blockwise_ref(xq, wq, m_sizes, x_scale, w_scale, block=128):
    """y = sum over K blocks kb of (xq[:, kb] @ wq[g][:, kb].T) * xs[:, kb, None] * ws[g, n // 128, kb].
    xq [M, K] e4m3, x_scale [M, K/128]; wq [G, N, K] e4m3, w_scale [G, N/128, K/128].
    Not present in the reference (its block-wise quantiser lives in FBGEMM,
    kernels/needs_perf_help/fp8_gemm_bench.py:16-21); defined by dequantising both
    operands with their block scales and running the per-expert loop."""
    G = m_sizes.numel()
    M, K = xq.shape
    w3 = wq.reshape(G, -1, K).float()
    N = w3.shape[1]
    xd = xq.float() * x_scale.float().repeat_interleave(block, dim=1)[:, :K]
    ws = w_scale.reshape(G, -1, w_scale.shape[-1]).float()
    wd = w3 * ws.repeat_interleave(block, dim=1)[:, :N].repeat_interleave(block, dim=2)[:, :, :K]
    return grouped_gemm_ref(xd, wd, m_sizes, "MN")


def silu_and_mul_ref(x):
    """silu(x[..., :d]) * x[..., d:] — the activation applied at
    kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:284 (vLLM silu_and_mul)."""
    d = x.shape[-1] // 2
    return torch.nn.functional.silu(x[..., :d]) * x[..., d:]


def torch_moe_ref(a, w1, w2, topk_weight, topk_ids):
    """MoE layer ground truth, same procedure as `torch_moe`
    (kernels/triton/inference/col_major_moe_gemm/test_moe_gemm.py:16-30), in fp32:
    repeat each token top-k times, run each expert's FFN on its rows, weight and sum."""
    B, D = a.shape
    k = topk_ids.shape[1]
    rep = a.float().view(B, 1, D).repeat(1, k, 1).reshape(-1, D)
    out = torch.zeros(B * k, w2.shape[1], dtype=torch.float32)
    ids = topk_ids.reshape(-1)
    for e in range(w1.shape[0]):
        mask = ids == e
        if mask.any():
            out[mask] = silu_and_mul_ref(rep[mask] @ w1[e].float().T) @ w2[e].float().T
    return (out.view(B, k, -1) * topk_weight.float().view(B, k, 1)).sum(dim=1)


def route_ref(topk_ids, num_experts):
    """Stable sort of the flattened ids by expert: (m_sizes, offsets, perm, inv_perm) int32.
    The order `out[mask]` visits rows in torch_moe (test_moe_gemm.py:26-29) and the
    sorted list of the moe_align_block_size docstring with its pad entries removed
    (kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:157-165)."""
    ids = topk_ids.reshape(-1).to(torch.int64)
    m_sizes = torch.bincount(ids, minlength=num_experts).to(torch.int32)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(m_sizes, 0)
    _, perm = torch.sort(ids, stable=True)
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel())
    return m_sizes, offsets, perm.to(torch.int32), inv.to(torch.int32)


def moe_align_block_size_ref(topk_ids, block_size, num_experts):
    """(sorted_token_ids, expert_ids, num_tokens_post_padded) as documented at
    v0_moe_fused.py:138-180: each expert's rows padded to a multiple of block_size with the
    pad id numel; buffer sizes numel + E*(block_size-1) and numel + E."""
    ids = topk_ids.reshape(-1)
    numel = ids.numel()
    m_sizes, _, perm, _ = route_ref(ids, num_experts)
    sorted_ids = torch.full((numel + num_experts * (block_size - 1),), numel, dtype=torch.int32)
    expert_ids = torch.zeros(numel + num_experts, dtype=torch.int32)
    pos, src, blk = 0, 0, 0
    for e in range(num_experts):
        m = int(m_sizes[e])
        sorted_ids[pos:pos + m] = perm[src:src + m]
        padded = (m + block_size - 1) // block_size * block_size
        nb = padded // block_size
        expert_ids[blk:blk + nb] = e
        blk += nb
        pos += padded
        src += m
    return sorted_ids, expert_ids, torch.tensor([pos], dtype=torch.int32)


def quant_1x128_ref(x, block=128):
    """scale = max(amax, 1e-12) / 448; q = clamp(x / scale, +-448) -> e4m3
    (kernels/triton/inference/fp8/float8_groupwise_quant.py:36-46), IEEE fp32 arithmetic."""
    xf = x.float().reshape(*x.shape[:-1], x.shape[-1] // block, block)
    scale = xf.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
    q = (xf / scale[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q.reshape(x.shape), scale


def grouped_gemm_backward_ref(grad_output, x, w, m_sizes):
    """(grad_x, grad_w) of the grouped GEMM, group by group in fp32
    (kernels/MoE/group_GEMM/triton/testing/pytorch_reference_backwards.py:165-197):
    grad_x[rows_g] = dY[rows_g, block g] @ w[g];  grad_w[g] = dY[rows_g, block g].T @ x[rows_g].
    grad_output is [M, N*G] (block layout) or [M, N]; zeros where nothing is defined."""
    G = m_sizes.numel()
    M, K = x.shape
    w3 = w.reshape(G, -1, K).float()
    N = w3.shape[1]
    dy, xf = grad_output.float(), x.float()
    blocked = dy.shape[1] == N * G and G > 1
    grad_x = torch.zeros(M, K)
    grad_w = torch.zeros(G, N, K)
    sizes, starts = _offsets(m_sizes)
    for g in range(G):
        a, b = starts[g], starts[g] + sizes[g]
        if sizes[g] == 0:
            continue
        blk = dy[a:b, g * N:(g + 1) * N] if blocked else dy[a:b]
        grad_x[a:b] = blk @ w3[g]
        grad_w[g] = blk.T @ xf[a:b]
    return grad_x, grad_w.reshape(w.shape)


def dense_gemm_ref(A, B, C, alpha=1.0, beta=0.0):
    """alpha * A @ B.T + beta * C in fp32 — what the reference's Blackwell driver compares
    against with torch.addmm (kernels/blackwell/cute_gemm_02_tma/driver.py:240-258)."""
    return alpha * (A.float() @ B.float().T) + beta * C.float()


def rel_err(y, ref):
    """max|y - ref| / max|ref|, the normalisation printed by
    kernels/blackwell/cute_gemm_02_tma/driver.py:257-258."""
    ref = ref.float()
    denom = ref.abs().max().clamp_min(1e-30)
    return float((y.float() - ref).abs().max() / denom)
