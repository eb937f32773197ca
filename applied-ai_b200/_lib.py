"""ctypes binding of libb200moe.so.

The library is the only compute path of this package: if it cannot be loaded the
import of any operator fails with an error that says so.  There is no fallback to
torch or to the CPU.
"""
import ctypes
import os
import threading

from . import build as _build

_c_int = ctypes.c_int
_c_i64 = ctypes.c_int64
_c_vp = ctypes.c_void_p
_c_sz = ctypes.c_size_t

ERROR_NAMES = {
    -1: "bad argument",
    -2: "misaligned pointer or K * element size not a multiple of 16 bytes",
    -3: "more than 1024 groups",
    -4: "cuTensorMapEncodeTiled not available from the driver",
    -5: "the driver rejected a tensor map",
    -6: "current device is not a compute-capability 10.x GPU",
    -7: "workspace too small or size beyond the supported maximum",
}
STATUS_NAMES = {
    1: "invalid group sizes / expert ids (negative entry, sum(m_sizes) > rows of x, or id outside [0, E))",
    16: "device-side wait ran out (TMA producer)",
    17: "device-side wait ran out (MMA issuer, operand stage)",
    18: "device-side wait ran out (MMA issuer, accumulator)",
    19: "device-side wait ran out (epilogue)",
    20: "self-test wait ran out (expected)",
    24: "expert-parallel dispatch: a rank would receive more rows than its receive buffer holds",
    25: "expert-parallel barrier: a peer rank's flag did not arrive within the limit",
    32: "kernel image not built for sm_100a",
}

# name -> argtypes; every function returns int.  Must list every symbol that
# include/b200moe.h declares (a CPU test checks this).
SIGNATURES = {
    "b200moe_version": [],
    "b200moe_build_id": [],
    "b200moe_kernel_launches": [],     # returns long long (restype set in load)
    "b200moe_grouped_gemm_bf16": [_c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_i64, _c_i64,
                                  _c_int, _c_int, _c_vp, _c_int, _c_vp, _c_vp],
    "b200moe_grouped_gemm_fp8_rowwise": [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                                         _c_i64, _c_i64, _c_int, _c_vp, _c_int, _c_vp, _c_vp],
    "b200moe_grouped_gemm_fp8_blockwise": [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                                           _c_i64, _c_i64, _c_int, _c_int, _c_vp, _c_int, _c_vp, _c_vp],
    "b200moe_grouped_gemm_ex": [_c_vp, _c_vp],
    "b200moe_ep_plan": [_c_vp, _c_int, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp],
    "b200moe_ep_push": [_c_vp, _c_i64, _c_vp, _c_i64, _c_vp, _c_int, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int,
                        _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_i64, _c_vp],
    "b200moe_ep_barrier": [_c_vp, _c_int, _c_int, _c_int, _c_int, ctypes.c_uint64, _c_vp, _c_vp],
    "b200moe_enable_peer_access": [_c_int],
    "b200moe_ipc_export": [_c_vp, _c_vp, ctypes.POINTER(ctypes.c_uint64)],
    "b200moe_ipc_open": [_c_vp, ctypes.POINTER(_c_vp)],
    "b200moe_ipc_close": [_c_vp],
    "b200moe_peer_probe": [_c_vp, _c_vp],
    "b200moe_sm100_gemm_f16": [_c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, ctypes.c_float, ctypes.c_float,
                               _c_vp],
    "b200moe_backward_workspace_bytes": [_c_int, _c_int, _c_int, _c_int, ctypes.POINTER(_c_sz)],
    "b200moe_grouped_gemm_backward": [_c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_i64,
                                      _c_i64, _c_vp, _c_sz, _c_int, _c_vp, _c_vp],
    "b200moe_selftest_wait_timeout": [ctypes.c_uint64, _c_vp, _c_vp],
    "b200moe_selftest_tmem_read": [_c_int, _c_int, _c_int, _c_int, _c_vp, _c_vp],
    "b200moe_route_workspace_bytes": [_c_int, _c_int, ctypes.POINTER(_c_sz)],
    "b200moe_route": [_c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_sz, _c_vp, _c_vp],
    "b200moe_route_noalloc": [_c_vp, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp, _c_vp],
    "b200moe_moe_align_workspace_bytes": [_c_int, _c_int, ctypes.POINTER(_c_sz)],
    "b200moe_moe_align_block_size": [_c_vp, _c_int, _c_int, _c_int, _c_vp, _c_vp, _c_vp, _c_vp, _c_sz, _c_vp, _c_vp],
    "b200moe_gather_rows": [_c_vp, _c_vp, _c_int, _c_vp, _c_int, _c_i64, _c_int, _c_vp],
    "b200moe_swiglu": [_c_vp, _c_vp, _c_i64, _c_int, _c_vp],
    "b200moe_combine_topk": [_c_vp, _c_vp, _c_vp, _c_vp, _c_int, _c_int, _c_int, _c_int, _c_vp],
    "b200moe_quant_1x128": [_c_vp, _c_int, _c_vp, _c_vp, _c_i64, _c_int, _c_vp],
}

def launch_count():
    """Kernels this library has enqueued in this process so far (counted inside the library at every
    launch site: b200moe_kernel_launches)."""
    lib = load()
    return int(lib.b200moe_kernel_launches())


_lock = threading.Lock()
_lib = None


class GemmDesc(ctypes.Structure):
    """Mirror of b200moe_gemm_desc (include/b200moe.h)."""
    _fields_ = [("x", _c_vp), ("w", _c_vp), ("m_sizes", _c_vp), ("y", _c_vp), ("x_scale", _c_vp), ("w_scale", _c_vp),
                ("M", _c_int), ("N", _c_int), ("K", _c_int), ("G", _c_int), ("ldy", _c_i64),
                ("y_col_group_stride", _c_i64), ("kind", _c_int), ("epilogue", _c_int), ("cta_group", _c_int),
                ("y_rows", _c_int), ("y_row_map", _c_vp), ("y_row_tags", _c_vp), ("y_peer_bases", _c_vp),
                ("n_peers", _c_int), ("status", _c_vp), ("y_scale_out", _c_vp), ("y_fp32_out", _c_vp)]


class B200MoeError(RuntimeError):
    """A C entry point returned a non-zero code."""


def lib_path():
    return _build.LIB_PATH


def load(build_if_missing=True):
    """Load and return the ctypes library.  A library that is missing, or that was built from
    other sources than the ones on disk, is rebuilt first when that is allowed and nvcc is here;
    otherwise loading fails loudly (never a silent run on an old binary)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB_PATH
        custom = bool(os.environ.get("B200MOE_LIBRARY"))  # a build the caller made with other flags: taken as is
        if not custom and _build.is_stale():
            if build_if_missing and _build.have_nvcc():
                _build.build_library()
            elif not os.path.exists(path):
                raise ImportError(f"{path} is missing; run `python applied-ai_b200/build.py`")
            else:
                raise ImportError(f"{path} was built from other sources than those in {_build.CSRC}; "
                                  "run `python applied-ai_b200/build.py`")
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise ImportError(f"cannot load {path}: {exc}. This package has no fallback path.") from exc
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = stale library
            fn.argtypes = argtypes
            fn.restype = _c_int
        lib.b200moe_kernel_launches.argtypes = []
        lib.b200moe_kernel_launches.restype = ctypes.c_longlong
        if not custom and lib.b200moe_build_id() != _build.source_id():
            raise ImportError(f"{path} does not carry the id of the sources in {_build.CSRC}; rebuild it")
        _lib = lib
        return lib


def check(rc, what):
    """Raise for a non-zero return code of entry point `what`."""
    if rc == 0:
        return
    if rc < 0:
        msg = ERROR_NAMES.get(rc, "unknown error")
        exc = ValueError if rc == -3 else B200MoeError
        raise exc(f"{what}: {msg} (code {rc})")
    raise B200MoeError(f"{what}: CUDA error {rc}")


def describe_status(code):
    return STATUS_NAMES.get(int(code), f"unknown status {int(code)}")
