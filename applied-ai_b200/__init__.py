"""B200-native (sm_100a) MoE grouped-GEMM engine with the call surface of the grouped
GEMM kernels of meta-pytorch/applied-ai.  All arithmetic runs in libb200moe.so
(hand-written CUDA behind a C ABI, include/b200moe.h); torch is the host.
"""
from . import _lib  # noqa: F401
from .groupgemm import (grouped_gemm, grouped_gemm_fp8_blockwise, grouped_gemm_fp8_rowwise,  # noqa: F401
                        pending_status, set_default_check)  # noqa: F401
from .tgroup_gemm_forward import grouped_gemm_forward  # noqa: F401
from .moe import combine_topk, fused_moe, gather_rows, moe_align_block_size, route, silu_and_mul  # noqa: F401
from .quant import float8_groupwise_quantize, quantize_fp8_block, quantize_fp8_row  # noqa: F401

__all__ = [
    "grouped_gemm", "grouped_gemm_forward", "grouped_gemm_fp8_rowwise", "grouped_gemm_fp8_blockwise", "fused_moe", "moe_align_block_size", "route", "gather_rows",
    "silu_and_mul", "combine_topk", "float8_groupwise_quantize", "quantize_fp8_row", "quantize_fp8_block",
    "set_default_check", "pending_status",
]
