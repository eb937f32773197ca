"""FP8 e4m3 quantisers.

`float8_groupwise_quantize(x, 128)` mirrors
kernels/triton/inference/fp8/float8_groupwise_quant.py:53-91: one fp32 scale per run of
128 elements of the last dimension, scale = max(amax, 1e-12) / 448, values divided by
the scale, clamped to +-448 and rounded to float8_e4m3fn.
"""
import torch

from . import _lib


def float8_groupwise_quantize(x, block_size=128):
    if x.size(-1) % block_size != 0:
        raise ValueError(f"Input tensor must have a last dimension that is a multiple of {block_size}")
    if block_size != 128:
        raise ValueError("only block_size=128 is implemented")
    if not x.is_cuda:
        raise RuntimeError("float8_groupwise_quantize needs a CUDA tensor (no CPU path)")
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("input must be bfloat16 or float32")
    if not x.is_contiguous():
        x = x.contiguous()
    K = x.size(-1)
    rows = x.numel() // K
    q = torch.empty_like(x, dtype=torch.float8_e4m3fn)
    scales = torch.empty(*x.shape[:-1], K // block_size, device=x.device, dtype=torch.float32)
    if rows:
        lib = _lib.load()
        with torch.cuda.device(x.device):
            rc = lib.b200moe_quant_1x128(x.data_ptr(), 1 if x.dtype == torch.float32 else 0, q.data_ptr(),
                                         scales.data_ptr(), rows, K, torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "float8_groupwise_quantize")
    return q, scales


def quantize_fp8_row(w):
    """Row-wise e4m3 quantisation (one fp32 scale per row): scale = max(amax_row, 1e-12) / 448.
    Set-up code for weights and test inputs, plain torch on whatever device `w` is on."""
    f = w.float()
    scale = f.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
    q = (f / scale[..., None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, scale


def quantize_fp8_block(w, block_n=128, block_k=128):
    """128x128-block e4m3 quantisation of a weight [..., N, K] (K a multiple of the block; a
    ragged last block along N is allowed): returns (q [..., N, K], scales
    [..., ceil(N/128), K/128] fp32) with the same scale formula as the 1x128 quantiser.
    Set-up code (run once per weight), plain torch."""
    *lead, N, K = w.shape
    if K % block_k:
        raise ValueError("K must be a multiple of the block size")
    nb = (N + block_n - 1) // block_n
    f = w.float()
    if nb * block_n != N:
        f = torch.nn.functional.pad(f, (0, 0, 0, nb * block_n - N))
    f = f.reshape(*lead, nb, block_n, K // block_k, block_k)
    scale = f.abs().amax(dim=(-3, -1)).clamp_min(1e-12) / 448.0
    q = (f / scale[..., :, None, :, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    q = q.reshape(*lead, nb * block_n, K)[..., :N, :].contiguous()
    return q, scale
