"""`grouped_gemm_forward(x, w, m_sizes)` in the block ("N*G") output layout of
kernels/MoE/group_GEMM/triton/tgroup_gemm_forward.py:626 (wrapper :485-623):

    y [M, N*G],  y[rows of group g, g*N:(g+1)*N] = x[rows of group g] @ w[g*N:(g+1)*N].T

Entries of y outside the G diagonal blocks are not written, as in the reference, which
allocates with torch.empty (:513); pass zero_fill=True to get zeros there.
"""
import torch

from . import groupgemm as _gg
from . import _lib


def grouped_gemm_forward(x, w, m_sizes, *, zero_fill=False, cta_group=0, check=None):
    m_sizes, G, M, N, K = _gg._prepare(x, w, m_sizes, torch.bfloat16)
    alloc = torch.zeros if zero_fill else torch.empty
    y = alloc((M, N * G), device=x.device, dtype=torch.bfloat16)
    if M > 0:
        _gg._launch_bf16(x, w, m_sizes, y, M, N, K, G, N * G, N, 0, cta_group, check, "grouped_gemm_forward")
    return y


def grouped_gemm_fp8_rowwise(x, w, m_sizes, x_scale, w_scale, *, zero_fill=False, cta_group=0, check=None):
    """FP8 row-wise variant in the same [M, N*G] layout (tgroup_gemm_forward.py:632)."""
    m_sizes, G, M, N, K = _gg._prepare(x, w, m_sizes, torch.float8_e4m3fn)
    _gg._prepare_scales(x_scale, w_scale, M, G, N, x.device)
    alloc = torch.zeros if zero_fill else torch.empty
    y = alloc((M, N * G), device=x.device, dtype=torch.bfloat16)
    if M == 0:
        return y
    lib = _lib.load()
    word = _gg._status_word(x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200moe_grouped_gemm_fp8_rowwise(x.data_ptr(), w.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(),
                                                  m_sizes.data_ptr(), y.data_ptr(), M, N, K, G, N * G, N, cta_group,
                                                  0, 0, word.data_ptr(), stream)
    _lib.check(rc, "grouped_gemm_fp8_rowwise")
    if _gg._default_check if check is None else check:
        _gg.raise_on_status(word, "grouped_gemm_fp8_rowwise")
    return y
