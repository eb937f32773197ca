"""Seeded synthetic inputs for the benchmark configurations.

Shapes only: "DeepSeek-V3" and "Mixtral-8x7B" name shape tuples, no model weights or
datasets are involved.  Every generator draws on the CPU from torch.Generator(seed) so
that a CPU checker and the GPU path can be fed identical bits.
"""
import torch


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1_small(seed=1000):
    """G=4, K=256, N=512, M=512, fp32; m_sizes from a uniform multinomial draw."""
    g = _gen(seed)
    idx = torch.multinomial(torch.full((4,), 0.25), 512, replacement=True, generator=g)
    m_sizes = torch.bincount(idx, minlength=4).to(torch.int32)
    x = torch.randn(512, 256, generator=g)
    w = torch.randn(4, 512, 256, generator=g) * 256 ** -0.5
    return x, w, m_sizes


def m_sizes_blocks(G, total_rows, block=128, seed=1001):
    """Row counts that are multiples of `block`, summing to total_rows, multinomial over G."""
    g = _gen(seed)
    nblk = total_rows // block
    idx = torch.multinomial(torch.full((G,), 1.0 / G), nblk, replacement=True, generator=g)
    return (torch.bincount(idx, minlength=G) * block).to(torch.int32)


def c2_deepseek_gate_up(seed=1001, M=16384, K=7168, N=4096, G=8, device="cpu"):
    """bf16 grouped GEMM at the DeepSeek-V3 routed-expert gate+up shape."""
    g = _gen(seed)
    m_sizes = m_sizes_blocks(G, M, 128, seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(device)
    w = torch.empty(G, N, K, dtype=torch.bfloat16, device=device)
    for e in range(G):  # one expert at a time bounds host memory
        w[e] = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(device)
    return x, w, m_sizes.to(device)


def m_sizes_zipf(G=128, total_rows=8192, s=1.2, n_empty=8, seed=1004):
    """Zipf(s) expert loads through a seeded permutation; the n_empty least likely experts
    are forced to zero rows (their rows go to the most likely expert)."""
    g = _gen(seed)
    p = torch.arange(1, G + 1, dtype=torch.float64) ** (-s)
    order = torch.randperm(G, generator=g)
    probs = torch.empty(G, dtype=torch.float64)
    probs[order] = p / p.sum()
    idx = torch.multinomial(probs.float(), total_rows, replacement=True, generator=g)
    counts = torch.bincount(idx, minlength=G)
    if n_empty:
        low = torch.argsort(probs)[:n_empty]
        top = torch.argmax(probs)
        moved = counts[low].sum()
        counts[low] = 0
        counts[top] += moved
    return counts.to(torch.int32)


def c5_skew(seed=1004, M=8192, K=2048, N=1408, G=128, device="cpu"):
    g = _gen(seed)
    m_sizes = m_sizes_zipf(G, M, 1.2, 8, seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(device)
    w = (torch.randn(G, N, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(device)
    return x, w, m_sizes.to(device)


def routing(T, E, k, seed):
    """softmax(randn) -> top-k, weights not renormalised (as the reference's test feeds them,
    kernels/triton/inference/col_major_moe_gemm/test_moe_gemm.py:54-57)."""
    g = _gen(seed)
    logits = torch.randn(T, E, generator=g)
    p = torch.softmax(logits.float(), dim=-1)
    w, ids = torch.topk(p, k)
    return w, ids.to(torch.int32)


def c3_mixtral_layer(seed=1002, T=4096, H=4096, I=14336, E=8, k=2, device="cpu"):
    g = _gen(seed)
    topk_w, topk_ids = routing(T, E, k, seed)
    hidden = torch.randn(T, H, generator=g).to(torch.bfloat16).to(device)
    w1 = torch.empty(E, 2 * I, H, dtype=torch.bfloat16, device=device)
    w2 = torch.empty(E, H, I, dtype=torch.bfloat16, device=device)
    for e in range(E):
        w1[e] = (torch.randn(2 * I, H, generator=g) * H ** -0.5).to(torch.bfloat16).to(device)
        w2[e] = (torch.randn(H, I, generator=g) * I ** -0.5).to(torch.bfloat16).to(device)
    return hidden, w1, w2, topk_w.to(device), topk_ids.to(device)
