"""Builds libb200moe.so (hand-written sm_100a CUDA behind a C ABI) in-tree with nvcc.

Run as a script (`python applied-ai_b200/build.py`) or call `build_library()`.  nvcc
cross-compiles without a GPU, so this works on a CPU-only machine.
"""
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
# B200MOE_LIBRARY: load another build of the library (e.g. one made with other nvcc flags) instead of the in-tree one
LIB_PATH = os.environ.get("B200MOE_LIBRARY") or os.path.join(PKG_DIR, "libb200moe.so")
SOURCES = ["capi.cu", "grouped_gemm.cu", "grouped_gemm_fp8_block.cu", "grouped_gemm_dw.cu", "moe_kernels.cu", "ep_kernels.cu", "selftest.cu"]
HEADERS = ["b200moe_internal.h", "moe_kernels.h", "ptx.cuh", "gg_common.cuh", os.path.join("..", "..", "include", "b200moe.h")]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "static",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libb200moe.so cannot be built")


def source_id():
    """31-bit id of the sources the library is built from (sha256 over their contents and the
    nvcc flags).  It is compiled into the library (b200moe_build_id) and written next to it, so a
    library older than the sources is recognised whatever the files' time stamps say."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for name in SOURCES + HEADERS:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode() + b"\0" + f.read())
    return int.from_bytes(h.digest()[:4], "big") & 0x7FFFFFFF


def _id_path():
    return LIB_PATH + ".id"


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    try:
        with open(_id_path()) as f:
            return int(f.read().strip()) != source_id()
    except (OSError, ValueError):
        return True


def have_nvcc():
    try:
        _nvcc()
        return True
    except RuntimeError:
        return False


def build_library(force=False, verbose=False):
    """Compile the library if it is missing or was built from other sources. Returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    sid = source_id()
    cmd = [_nvcc()] + NVCC_FLAGS + [f"-DB200MOE_BUILD_ID={sid}"] + (["-Xptxas", "-v"] if verbose else [])
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB_PATH]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose:
        sys.stderr.write(res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    with open(_id_path(), "w") as f:
        f.write(str(sid))
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
