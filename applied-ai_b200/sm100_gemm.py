"""Dense `D = alpha * A @ B.T + beta * C` with the module surface of the reference's Blackwell
extension (kernels/blackwell/cute_gemm_02_tma/sm100_gemm_pytorch.cpp:34-187): same function
names, argument order, dtypes (A, B float16; C, D float32) and helper constants.  Served by
the grouped kernel's single-group mode, so unlike the reference no dimension has to be a
multiple of the tile (only K % 8 == 0), and the launch goes to the current stream."""
import torch

from . import _lib

MMA_TILE_M = 128
MMA_TILE_N = 256
MMA_TILE_K = 64


def is_sm100_supported():
    """True when the sm_100a library is present and loadable."""
    try:
        _lib.load()
        return True
    except Exception:
        return False


def check_sm100_device():
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


def get_device_info():
    major, minor = torch.cuda.get_device_capability() if torch.cuda.is_available() else (0, 0)
    return torch.tensor([major, minor, int(is_sm100_supported()), int(check_sm100_device())], dtype=torch.int32)


def get_aligned_shape(M, N, K):
    return [(M + 127) // 128 * 128, (N + 255) // 256 * 256, (K + 63) // 64 * 64]


def create_aligned_tensor(shape, dtype, device):
    if len(shape) != 2:
        raise RuntimeError("Shape must be 2D")
    m, n, _ = get_aligned_shape(shape[0], shape[1], 64)
    return torch.zeros((m, n), dtype=dtype, device=device)


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def sm100_gemm_f16(A, B, C, alpha=1.0, beta=0.0):
    _require(A.is_cuda and B.is_cuda and C.is_cuda, "A, B and C must be CUDA tensors")
    _require(A.dtype == torch.float16 and B.dtype == torch.float16, "A and B must be float16")
    _require(C.dtype == torch.float32, "C must be float32")
    _require(A.is_contiguous() and B.is_contiguous() and C.is_contiguous(), "A, B and C must be contiguous")
    _require(A.dim() == 2 and B.dim() == 2 and C.dim() == 2, "A, B and C must be 2D")
    M, K = A.shape
    N, K_B = B.shape
    _require(K == K_B, f"Inner dimensions must match: A.shape[1]={K}, B.shape[1]={K_B}")
    _require(tuple(C.shape) == (M, N), f"C dimensions {tuple(C.shape)} must match output shape ({M}, {N})")
    _require(K % 8 == 0, "K must be a multiple of 8 (16-byte rows for TMA)")
    D = torch.empty_like(C)
    if M == 0 or N == 0:
        return D
    lib = _lib.load()
    with torch.cuda.device(A.device):
        rc = lib.b200moe_sm100_gemm_f16(A.data_ptr(), B.data_ptr(), C.data_ptr(), D.data_ptr(), M, N, K,
                                        float(alpha), float(beta), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "sm100_gemm_f16")
    return D


def sm100_gemm_f16_tma(A, B, C=None, alpha=1.0, beta=0.0, check_alignment=True):
    """The convenience wrapper of the reference's driver (driver.py:38-107): C defaults to zeros."""
    if C is None:
        C = torch.zeros(A.shape[0], B.shape[0], dtype=torch.float32, device=A.device)
    return sm100_gemm_f16(A, B, C, alpha, beta)
