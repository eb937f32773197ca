"""Grouped GEMM entry points with the reference's call surface.

    grouped_gemm(x, w, m_sizes)                                  -> y [M, N]
    grouped_gemm_fp8_rowwise(x, w, m_sizes, x_scale, w_scale)    -> y [M, N]

mirror dev/triton_groupGEMM/groupgemm.py:518-531 (wrapper `_grouped_gemm` :407-515):
x [M, K] and w [G*N, K] (or [G, N, K]) contiguous, m_sizes [G] int32 on the device,
output freshly allocated bf16.  `grouped_gemm_forward` (the [M, N*G] block layout of
kernels/MoE/group_GEMM/triton/tgroup_gemm_forward.py:626) is in tgroup_gemm_forward.py.

Torch is only the host here (memory, streams); the arithmetic runs in libb200moe.so.
Errors follow what the reference's tests expect (dev/triton_groupGEMM/testing/
unit_tests.py:168-212): RuntimeError for shape/dtype/contiguity problems, ValueError
for a group count that does not fit `w`, ValueError for group sizes the device
rejects (negative, or adding up to more rows than x has).
"""
import threading

import torch

from . import _lib

_default_check = True
_status_words = {}          # (device index, stream handle) -> 4-byte status word on that device
_state_lock = threading.Lock()


def set_default_check(flag):
    """With checking on (the default) every call reads back a 4-byte status word after
    the launch (one synchronisation) and raises on bad group sizes.  Turn it off for
    benchmarking or when m_sizes is known to be valid."""
    global _default_check
    _default_check = bool(flag)


def _device_index(device):
    return device.index if device.index is not None else torch.cuda.current_device()


def _status_word(device):
    """The status word kernels launched on (device, its current stream) report into.  One word
    per stream, so that calls issued on different streams or from different host threads never
    share one (a word is sticky: the first code written stays until it is read and cleared)."""
    idx = _device_index(device)
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    with _state_lock:
        word = _status_words.get(key)
        if word is None:
            with torch.cuda.stream(torch.cuda.current_stream(idx)):
                word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
            _status_words[key] = word
    return word


def pending_status(device=None):
    """Deferred check for callers that run with check=False: synchronises, reads every status
    word of `device` (default: the current device), clears the ones that are set and raises for
    the first code found — ValueError for invalid group sizes / expert ids, B200MoeError for the
    rest (a device-side wait that ran out, an expert-parallel receive buffer that overflowed).
    Returns None when nothing is pending."""
    idx = torch.cuda.current_device() if device is None else _device_index(torch.device(device))
    with _state_lock:
        words = [w for (d, _), w in _status_words.items() if d == idx]
    torch.cuda.synchronize(idx)
    first = 0
    for w in words:
        code = int(w.item())
        if code:
            w.zero_()
            first = first or code
    if first:
        msg = f"pending device status: {_lib.describe_status(first)} (status {first})"
        if first == 1:
            raise ValueError(msg)
        raise _lib.B200MoeError(msg)


def raise_on_status(word, what):
    """Read the device status word; if set, clear it and raise."""
    code = int(word.item())
    if code == 0:
        return
    word.zero_()
    msg = f"{what}: {_lib.describe_status(code)} (status {code})"
    if code == 1:
        raise ValueError(msg)
    raise _lib.B200MoeError(msg)


def _require(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def _prepare(x, w, m_sizes, elem_dtype):
    _require(isinstance(x, torch.Tensor) and isinstance(w, torch.Tensor) and isinstance(m_sizes, torch.Tensor),
             "x, w and m_sizes must be tensors")
    _require(x.is_cuda and w.is_cuda and m_sizes.is_cuda, "x, w and m_sizes must be CUDA tensors (no CPU path)")
    _require(x.device == w.device == m_sizes.device, "x, w and m_sizes must be on the same device")
    _require(x.dim() == 2, "x must be [M, K]")
    _require(w.dim() in (2, 3), "w must be [G*N, K] or [G, N, K]")
    _require(m_sizes.dim() == 1 and m_sizes.numel() > 0, "m_sizes must be a non-empty 1-D tensor")
    _require(x.is_contiguous() and w.is_contiguous() and m_sizes.is_contiguous(),
             "x, w and m_sizes must be contiguous")
    _require(x.dtype == elem_dtype and w.dtype == elem_dtype, f"x and w must be {elem_dtype}")
    _require(m_sizes.dtype in (torch.int32, torch.int64), "m_sizes must be int32")
    if m_sizes.dtype != torch.int32:
        m_sizes = m_sizes.to(torch.int32)
    G = m_sizes.shape[0]
    M, K = x.shape
    _require(K == w.shape[-1], f"K mismatch: x has {K} columns, w has {w.shape[-1]}")
    if w.dim() == 3:
        if w.shape[0] != G:
            raise ValueError(f"m_sizes has {G} groups but w has {w.shape[0]}")
        N = w.shape[1]
    else:
        if w.shape[0] % G != 0:
            raise ValueError(f"w has {w.shape[0]} rows, not a multiple of the {G} groups in m_sizes")
        N = w.shape[0] // G
    _require(N > 0 and K > 0, "N and K must be positive")
    _require((K * x.element_size()) % 16 == 0, "K * element size must be a multiple of 16 bytes (TMA row pitch)")
    return m_sizes, G, M, N, K


def _row_map_args(out_row_map, y, device):
    """(pointer, rows of y) for the optional output row map."""
    if out_row_map is None:
        return 0, 0
    _require(isinstance(out_row_map, torch.Tensor) and out_row_map.device == device and
             out_row_map.dtype == torch.int32 and out_row_map.is_contiguous(),
             "out_row_map must be a contiguous int32 tensor on the same device")
    return out_row_map.data_ptr(), y.shape[0]


def _launch_bf16(x, w, m_sizes, y, M, N, K, G, ldy, col_stride, epilogue, cta_group, check, what, out_row_map=None):
    lib = _lib.load()
    word = _status_word(x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        map_ptr, y_rows = _row_map_args(out_row_map, y, x.device)
        rc = lib.b200moe_grouped_gemm_bf16(x.data_ptr(), w.data_ptr(), m_sizes.data_ptr(), y.data_ptr(), M, N, K, G,
                                           ldy, col_stride, epilogue, cta_group, map_ptr, y_rows, word.data_ptr(),
                                           stream)
    _lib.check(rc, what)
    if _default_check if check is None else check:
        raise_on_status(word, what)


def grouped_gemm(x, w, m_sizes, *, epilogue="none", cta_group=0, check=None, out_row_map=None, out_rows=None):
    """y[rows of group g] = x[rows of group g] @ w[g].T, bf16 in, fp32 accumulate, bf16 out.

    epilogue="swiglu": w[g] is [gate; up] (N = 2*I rows) and y gets I columns,
    silu(gate) * up computed on the fp32 accumulators.
    out_row_map (int32 [M], optional): row r of the result is stored at row out_row_map[r]
    of the output, which then has out_rows rows (default M); rows no entry points to stay
    unwritten.
    """
    m_sizes, G, M, N, K = _prepare(x, w, m_sizes, torch.bfloat16)
    epi = {"none": 0, "swiglu": 1}.get(epilogue)
    _require(epi is not None, "epilogue must be 'none' or 'swiglu'")
    if epi == 1:
        _require(N % 2 == 0, "SwiGLU needs an even number of weight rows per group")
    n_out = N // 2 if epi == 1 else N
    y = torch.empty((M if out_rows is None else out_rows, n_out), device=x.device, dtype=torch.bfloat16)
    if M > 0:
        _launch_bf16(x, w, m_sizes, y, M, N, K, G, n_out, 0, epi, cta_group, check, "grouped_gemm", out_row_map)
    return y


def _prepare_scales(x_scale, w_scale, M, G, N, device):
    _require(isinstance(x_scale, torch.Tensor) and isinstance(w_scale, torch.Tensor), "scales must be tensors")
    _require(x_scale.device == device and w_scale.device == device, "scales must be on the same device as x")
    _require(x_scale.dtype == torch.float32 and w_scale.dtype == torch.float32, "scales must be float32")
    _require(x_scale.is_contiguous() and w_scale.is_contiguous(), "scales must be contiguous")
    _require(x_scale.numel() == M, f"x_scale must have M={M} entries")
    _require(w_scale.numel() == G * N, f"w_scale must have G*N={G * N} entries")


def grouped_gemm_fp8_rowwise(x, w, m_sizes, x_scale, w_scale, *, cta_group=0, check=None):
    """(xq @ wq[g].T) * x_scale[:, None] * w_scale[None, g*N:(g+1)*N] -> bf16 [M, N].

    x, w are float8_e4m3fn; x_scale [M] and w_scale [G*N] are fp32."""
    m_sizes, G, M, N, K = _prepare(x, w, m_sizes, torch.float8_e4m3fn)
    _prepare_scales(x_scale, w_scale, M, G, N, x.device)
    y = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    if M == 0:
        return y
    lib = _lib.load()
    word = _status_word(x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.b200moe_grouped_gemm_fp8_rowwise(x.data_ptr(), w.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(),
                                                  m_sizes.data_ptr(), y.data_ptr(), M, N, K, G, N, 0, cta_group,
                                                  0, 0, word.data_ptr(), stream)
    _lib.check(rc, "grouped_gemm_fp8_rowwise")
    if _default_check if check is None else check:
        raise_on_status(word, "grouped_gemm_fp8_rowwise")
    return y


def grouped_gemm_fp8_blockwise(x, w, m_sizes, x_scale, w_scale, *, epilogue="none", cta_group=0, check=None,
                               out_row_map=None, out_rows=None):
    """FP8 grouped GEMM with 1x128 activation scales and 128x128 weight-block scales -> bf16.

    x [M, K], w [G*N, K] or [G, N, K] float8_e4m3fn; x_scale [M, K/128] fp32 (as produced by
    float8_groupwise_quantize); w_scale [G, ceil(N/128), K/128] fp32 (quantize_fp8_block).
    epilogue="swiglu": w[g] = [gate; up], output has N/2 columns.  out_row_map / out_rows as in
    grouped_gemm."""
    m_sizes, G, M, N, K = _prepare(x, w, m_sizes, torch.float8_e4m3fn)
    _require(K % 128 == 0, "K must be a multiple of 128 for block-wise scales")
    epi = {"none": 0, "swiglu": 1}.get(epilogue)
    _require(epi is not None, "epilogue must be 'none' or 'swiglu'")
    if epi == 1:
        _require(N % 256 == 0, "SwiGLU with block-wise scales needs N (gate+up rows) to be a multiple of 256")
    nblk = (N + 127) // 128
    _require(isinstance(x_scale, torch.Tensor) and isinstance(w_scale, torch.Tensor), "scales must be tensors")
    _require(x_scale.device == x.device and w_scale.device == x.device, "scales must be on the same device as x")
    _require(x_scale.dtype == torch.float32 and w_scale.dtype == torch.float32, "scales must be float32")
    _require(x_scale.is_contiguous() and w_scale.is_contiguous(), "scales must be contiguous")
    _require(tuple(x_scale.shape) == (M, K // 128), f"x_scale must be [M, K/128] = [{M}, {K // 128}]")
    _require(w_scale.numel() == G * nblk * (K // 128), f"w_scale must be [G, ceil(N/128), K/128] = [{G}, {nblk}, {K // 128}]")
    n_out = N // 2 if epi == 1 else N
    y = torch.empty((M if out_rows is None else out_rows, n_out), device=x.device, dtype=torch.bfloat16)
    if M == 0:
        return y
    lib = _lib.load()
    word = _status_word(x.device)
    with torch.cuda.device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        map_ptr, y_rows = _row_map_args(out_row_map, y, x.device)
        rc = lib.b200moe_grouped_gemm_fp8_blockwise(x.data_ptr(), w.data_ptr(), x_scale.data_ptr(), w_scale.data_ptr(),
                                                    m_sizes.data_ptr(), y.data_ptr(), M, N, K, G, n_out, 0, epi,
                                                    cta_group, map_ptr, y_rows, word.data_ptr(), stream)
    _lib.check(rc, "grouped_gemm_fp8_blockwise")
    if _default_check if check is None else check:
        raise_on_status(word, "grouped_gemm_fp8_blockwise")
    return y


KIND_BF16, KIND_FP8_ROWWISE, KIND_FP8_BLOCKWISE = 0, 1, 2


def grouped_gemm_ex(kind, x, w, m_sizes, *, x_scale=None, w_scale=None, epilogue="none", cta_group=0, y=None,
                    out_row_map=None, out_row_tags=None, peer_bases=None, n_peers=0, out_rows=None, check=False,
                    return_fp32=False):
    """Struct-described grouped GEMM (b200moe_grouped_gemm_ex).  Besides everything the plain
    entry points do, result rows can be sent to (rank, row) destinations: out_row_tags int64 [M]
    = (rank << 32) | row and peer_bases = int64 device tensor of n_peers base addresses of bf16
    buffers with out_rows rows each (this rank's own buffer included).  Returns y, or None when
    rows go to peer buffers.  epilogue="swiglu_fp8" (block-wise kind): returns (e4m3 [M, N/2],
    fp32 scales [M, N/256]) — silu(gate)*up quantised 1x128 inside the GEMM with the formula of
    float8_groupwise_quantize (IEEE division); return_fp32=True appends the fp32 values [M, N/2]
    that were quantised, so a caller can check the bytes against the stand-alone quantiser."""
    import ctypes
    m_sizes, G, M, N, K = _prepare(x, w, m_sizes, torch.bfloat16 if kind == KIND_BF16 else torch.float8_e4m3fn)
    epi = {"none": 0, "swiglu": 1, "swiglu_fp8": 3}[epilogue]
    n_out = N // 2 if epi != 0 else N
    d = _lib.GemmDesc()
    y_scale = None
    if epi == 3:
        _require(kind == KIND_FP8_BLOCKWISE and N % 256 == 0 and out_row_map is None and out_row_tags is None,
                 "the quantising SwiGLU epilogue needs the block-wise kind, N % 256 == 0 and plain row placement")
        y = torch.empty((M, n_out), device=x.device, dtype=torch.float8_e4m3fn)
        y_scale = torch.empty((M, n_out // 128), device=x.device, dtype=torch.float32)
        d.y_scale_out = y_scale.data_ptr()
        y_f32 = torch.empty((M, n_out), device=x.device, dtype=torch.float32) if return_fp32 else None
        d.y_fp32_out = 0 if y_f32 is None else y_f32.data_ptr()
    d.x, d.w, d.m_sizes = x.data_ptr(), w.data_ptr(), m_sizes.data_ptr()
    d.x_scale = 0 if x_scale is None else x_scale.data_ptr()
    d.w_scale = 0 if w_scale is None else w_scale.data_ptr()
    d.M, d.N, d.K, d.G = M, N, K, G
    d.ldy, d.y_col_group_stride = n_out, 0
    d.kind, d.epilogue, d.cta_group = kind, epi, cta_group
    word = _status_word(x.device)
    d.status = word.data_ptr()
    if out_row_tags is not None:
        _require(out_row_tags.dtype == torch.int64 and out_row_tags.is_contiguous() and out_row_tags.numel() >= M,
                 "out_row_tags must be a contiguous int64 tensor with one entry per row of x")
        _require(peer_bases is not None and peer_bases.dtype == torch.int64 and n_peers > 0 and out_rows,
                 "peer_bases (int64 device tensor), n_peers and out_rows are needed with out_row_tags")
        d.y_row_tags, d.y_peer_bases, d.n_peers, d.y_rows = out_row_tags.data_ptr(), peer_bases.data_ptr(), n_peers, out_rows
        d.y = 0  # every row goes to a peer buffer
    else:
        if y is None:
            y = torch.empty((M if out_rows is None else out_rows, n_out), device=x.device, dtype=torch.bfloat16)
        d.y = y.data_ptr()
        if out_row_map is not None:
            d.y_row_map, d.y_rows = _row_map_args(out_row_map, y, x.device)
    if M > 0:
        lib = _lib.load()
        with torch.cuda.device(x.device):
            rc = lib.b200moe_grouped_gemm_ex(ctypes.addressof(d), torch.cuda.current_stream().cuda_stream)
        _lib.check(rc, "grouped_gemm_ex")
        if check:
            raise_on_status(word, "grouped_gemm_ex")
    if epi == 3:
        return (y, y_scale, y_f32) if return_fp32 else (y, y_scale)
    return None if out_row_tags is not None else y
