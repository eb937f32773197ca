"""The MoE layer around the grouped GEMM, with the call surface of
kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py:222 (`fused_moe`).

    route -> gather rows -> grouped GEMM (gate+up) with SwiGLU epilogue
          -> grouped GEMM (down) -> weighted top-k combine

Where the reference pads every expert to the GEMM's row block
(`moe_align_block_size`, v0_moe_fused.py:138-180) this engine sorts the routed rows by
expert without padding: the grouped GEMM walks ragged groups directly.
"""
import torch

from . import _lib
from . import groupgemm as _gg

_workspaces = {}


def _stream(t):
    return torch.cuda.current_stream(t.device).cuda_stream


def _workspace(device, nbytes):
    """Scratch buffer of (device, its current stream): kernels of one stream run in order and may
    share it; two streams (or two host threads on their own streams) never get the same one."""
    idx = _gg._device_index(device)
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    with _gg._state_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", idx))
            _workspaces[key] = ws
    return ws


def route(topk_ids, num_experts, *, check=None):
    """Stable sort of the flattened expert ids.

    Returns (m_sizes [E], offsets [E+1], perm [R], inv_perm [R]), all int32:
    perm[p] = flat index t*top_k + j of the routed row at sorted position p (ordered by
    expert, then by flat index); inv_perm is its inverse.  Equals
    torch.sort(topk_ids.view(-1), stable=True) / torch.bincount bit for bit."""
    _gg._require(topk_ids.is_cuda, "topk_ids must be a CUDA tensor (no CPU path)")
    ids = topk_ids.reshape(-1)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    R, E = ids.numel(), int(num_experts)
    dev = ids.device
    m_sizes = torch.empty(E, dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    perm = torch.empty(R, dtype=torch.int32, device=dev)
    inv_perm = torch.empty(R, dtype=torch.int32, device=dev)
    lib = _lib.load()
    import ctypes
    need = ctypes.c_size_t(0)
    _lib.check(lib.b200moe_route_workspace_bytes(R, E, ctypes.byref(need)), "route")
    ws = _workspace(dev, need.value)
    word = _gg._status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.b200moe_route(ids.data_ptr(), R, E, m_sizes.data_ptr(), offsets.data_ptr(), perm.data_ptr(),
                               inv_perm.data_ptr(), ws.data_ptr(), ws.numel(), word.data_ptr(), _stream(ids))
    _lib.check(rc, "route")
    if _gg._default_check if check is None else check:
        _gg.raise_on_status(word, "route")
    return m_sizes, offsets, perm, inv_perm


def moe_align_block_size(topk_ids, block_size, num_experts):
    """(sorted_token_ids, expert_ids, num_tokens_post_padded) with the buffer sizes, pad id and
    ordering of the reference wrapper (v0_moe_fused.py:138-180): each expert's routed rows padded
    to a multiple of block_size with the id `topk_ids.numel()`.  For code written against the
    vLLM format; this engine's own GEMM does not need the padding."""
    _gg._require(topk_ids.is_cuda, "topk_ids must be a CUDA tensor (no CPU path)")
    ids = topk_ids.reshape(-1)
    if ids.dtype != torch.int32:
        ids = ids.to(torch.int32)
    ids = ids.contiguous()
    R, E, dev = ids.numel(), int(num_experts), ids.device
    sorted_ids = torch.empty(R + E * (block_size - 1), dtype=torch.int32, device=dev)
    expert_ids = torch.empty(R + E, dtype=torch.int32, device=dev)
    post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    lib = _lib.load()
    import ctypes
    need = ctypes.c_size_t(0)
    _lib.check(lib.b200moe_moe_align_workspace_bytes(R, E, ctypes.byref(need)), "moe_align_block_size")
    ws = _workspace(dev, need.value)
    word = _gg._status_word(dev)
    with torch.cuda.device(dev):
        rc = lib.b200moe_moe_align_block_size(ids.data_ptr(), R, E, int(block_size), sorted_ids.data_ptr(),
                                              expert_ids.data_ptr(), post_pad.data_ptr(), ws.data_ptr(), ws.numel(),
                                              word.data_ptr(), _stream(ids))
    _lib.check(rc, "moe_align_block_size")
    return sorted_ids, expert_ids, post_pad


def gather_rows(src, idx, div=1, out=None):
    """out[p, :] = src[idx[p] // div, :] (idx int32 on the device)."""
    _gg._require(src.is_cuda and idx.is_cuda and src.is_contiguous() and idx.is_contiguous(),
                 "src and idx must be contiguous CUDA tensors")
    _gg._require(idx.dtype == torch.int32 and src.dim() == 2, "idx must be int32, src 2-D")
    rows = idx.numel()
    if out is None:
        out = torch.empty((rows, src.shape[1]), dtype=src.dtype, device=src.device)
    lib = _lib.load()
    with torch.cuda.device(src.device):
        rc = lib.b200moe_gather_rows(src.data_ptr(), idx.data_ptr(), int(div), out.data_ptr(), rows,
                                     src.shape[1] * src.element_size(), src.shape[0], _stream(src))
    _lib.check(rc, "gather_rows")
    return out


def silu_and_mul(x, out=None):
    """out = silu(x[:, :d]) * x[:, d:]  (bf16), the activation of v0_moe_fused.py:284."""
    _gg._require(x.is_cuda and x.is_contiguous() and x.dim() == 2 and x.dtype == torch.bfloat16,
                 "x must be a contiguous 2-D bf16 CUDA tensor")
    d = x.shape[1] // 2
    if out is None:
        out = torch.empty((x.shape[0], d), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with torch.cuda.device(x.device):
        rc = lib.b200moe_swiglu(x.data_ptr(), out.data_ptr(), x.shape[0], d, _stream(x))
    _lib.check(rc, "silu_and_mul")
    return out


def combine_topk(y, inv_perm, topk_weights, num_tokens, top_k, out=None):
    """out[t] = sum_j topk_weights[t, j] * y[inv_perm[t*top_k + j]]  (fp32 sum, bf16 out)."""
    _gg._require(y.is_cuda and y.is_contiguous() and y.dtype == torch.bfloat16 and y.dim() == 2,
                 "y must be a contiguous 2-D bf16 CUDA tensor")
    H = y.shape[1]
    w = None
    if topk_weights is not None:
        w = topk_weights.reshape(-1).to(torch.float32).contiguous()
        _gg._require(w.numel() == num_tokens * top_k, "topk_weights must have tokens*top_k entries")
    _gg._require(inv_perm.dtype == torch.int32 and inv_perm.numel() == num_tokens * top_k,
                 "inv_perm must be int32 with tokens*top_k entries")
    if out is None:
        out = torch.empty((num_tokens, H), dtype=torch.bfloat16, device=y.device)
    lib = _lib.load()
    with torch.cuda.device(y.device):
        rc = lib.b200moe_combine_topk(y.data_ptr(), inv_perm.data_ptr(), 0 if w is None else w.data_ptr(),
                                      out.data_ptr(), num_tokens, top_k, H, y.shape[0], _stream(y))
    _lib.check(rc, "combine_topk")
    return out


def fused_moe(hidden_states, w1, w2, topk_weights, topk_ids, inplace=False, *, check=None, cta_group=0):
    """Mixture-of-experts FFN: for every token, sum over its top-k experts e of
    topk_weight * (silu(h @ w1[e, :I].T) * (h @ w1[e, I:].T)) @ w2[e].T.

    hidden_states [T, H] bf16; w1 [E, 2*I, H]; w2 [E, H, I]; topk_weights, topk_ids [T, k].
    Same arguments as fused_moe of v0_moe_fused.py:222-227; with inplace=True the result
    is written into hidden_states (:291-294)."""
    _gg._require(hidden_states.dim() == 2 and w1.dim() == 3 and w2.dim() == 3, "expected [T,H], [E,2I,H], [E,H,I]")
    _gg._require(hidden_states.shape[1] == w1.shape[2], "Incompatible dimensions")
    _gg._require(hidden_states.is_contiguous(), "Hidden_states must be contiguous")
    _gg._require(w1.is_contiguous(), "Expert weights1 must be contiguous")
    _gg._require(w2.is_contiguous(), "Expert weights2 must be contiguous")
    _gg._require(hidden_states.dtype == torch.bfloat16, "hidden_states must be bfloat16")
    T, H = hidden_states.shape
    E, N2, _ = w1.shape
    _gg._require(w2.shape[0] == E and w2.shape[1] == H and w2.shape[2] * 2 == N2, "w2 must be [E, H, I]")
    _gg._require(topk_ids.shape == topk_weights.shape and topk_ids.shape[0] == T, "topk tensors must be [T, k]")
    k = topk_ids.shape[1]

    m_sizes, _, perm, inv_perm = route(topk_ids, E, check=check)
    xs = gather_rows(hidden_states, perm, div=k)                          # [R, H] rows sorted by expert
    h = _gg.grouped_gemm(xs, w1, m_sizes, epilogue="swiglu", check=check, cta_group=cta_group)   # [R, I]
    y2 = _gg.grouped_gemm(h, w2, m_sizes, check=check, cta_group=cta_group)                      # [R, H]
    out = hidden_states if inplace else None
    return combine_topk(y2, inv_perm, topk_weights, T, k, out=out)
