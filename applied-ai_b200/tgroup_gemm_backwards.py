"""`grouped_gemm_backward(grad_output, x, w, m_sizes) -> (grad_x, grad_w)` with the call surface of
kernels/MoE/group_GEMM/triton/tgroup_gemm_backwards.py:382-420.

    grad_x[rows of g] = grad_output[rows of g, g*N:(g+1)*N] @ w[g*N:(g+1)*N]
    grad_w[g*N:(g+1)*N] = grad_output[rows of g, g*N:(g+1)*N].T @ x[rows of g]

grad_output is [M, N*G] (the block layout of grouped_gemm_forward) or [M, N] (the layout of
grouped_gemm); x [M, K]; w [N*G, K] or [G, N, K]; all bf16.  Rows of grad_x past sum(m_sizes) and
grad_w of empty groups are zero, as in the reference (torch.zeros_like, :413-414).
"""
import ctypes

import torch

from . import _lib
from . import groupgemm as _gg
from . import moe as _moe


def grouped_gemm_backward(grad_output, x, w, m_sizes, *, cta_group=0, check=None):
    m_sizes, G, M, N, K = _gg._prepare(x, w, m_sizes, torch.bfloat16)
    _gg._require(isinstance(grad_output, torch.Tensor) and grad_output.is_cuda and grad_output.device == x.device,
                 "grad_output must be a CUDA tensor on the same device")
    _gg._require(grad_output.dtype == torch.bfloat16 and grad_output.dim() == 2 and grad_output.shape[0] == M,
                 "grad_output must be bf16 [M, N*G] or [M, N]")
    if not grad_output.is_contiguous():
        grad_output = grad_output.contiguous()
    if grad_output.shape[1] == N * G and G > 1:
        ld, stride = N * G, N
    else:
        _gg._require(grad_output.shape[1] == N, f"grad_output must have N*G={N * G} or N={N} columns")
        ld, stride = N, 0
    _gg._require(N % 8 == 0, "N must be a multiple of 8 (16-byte rows for TMA)")
    grad_x = torch.zeros_like(x)
    grad_w = torch.empty_like(w)
    if M == 0:
        return grad_x, grad_w.zero_()
    lib = _lib.load()
    need = ctypes.c_size_t(0)
    _lib.check(lib.b200moe_backward_workspace_bytes(M, N, K, G, ctypes.byref(need)), "grouped_gemm_backward")
    ws = _moe._workspace(x.device, need.value)
    word = _gg._status_word(x.device)
    with torch.cuda.device(x.device):
        rc = lib.b200moe_grouped_gemm_backward(grad_output.data_ptr(), x.data_ptr(), w.data_ptr(), m_sizes.data_ptr(),
                                               grad_x.data_ptr(), grad_w.data_ptr(), M, N, K, G, ld, stride,
                                               ws.data_ptr(), ws.numel(), cta_group, word.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "grouped_gemm_backward")
    if _gg._default_check if check is None else check:
        _gg.raise_on_status(word, "grouped_gemm_backward")
    return grad_x, grad_w
