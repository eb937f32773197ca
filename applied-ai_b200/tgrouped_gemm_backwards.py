"""Alias of tgroup_gemm_backwards under the spelling the reference's own test imports
(kernels/MoE/group_GEMM/triton/testing/fast_verification.py:19)."""
from .tgroup_gemm_backwards import grouped_gemm_backward  # noqa: F401
