"""Alias of tgroup_gemm_forward under the spelling the reference's own test imports
(kernels/MoE/group_GEMM/triton/testing/fast_verification.py:20)."""
from .tgroup_gemm_forward import grouped_gemm_forward, grouped_gemm_fp8_rowwise  # noqa: F401
