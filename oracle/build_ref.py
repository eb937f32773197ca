"""Builds the reference's own Blackwell GEMM (kernels/blackwell/cute_gemm_02_tma/sm100_gemm.cu,
C entry point launch_sm100_gemm_f16_tma, sm100_gemm.h:33-36) straight from the reference
checkout into oracle/_ref/libsm100_gemm_ref.so, with the nvcc flags of the reference's
setup.py:45-58 and the CUTLASS/CuTe headers that ship inside the Python environment
(nothing of either is copied into this repository).  TEST/BENCH INFRASTRUCTURE: it is the
baseline `bench.py --workload dense` times next to this package's dense mode and a second
opinion for tests; the product never loads it.

Needs the reference checkout (its path in $APPLIED_AI_REFERENCE, else a directory named
`reference` beside this repository); without it the function returns None and an already
built library, if any, is used as is.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libsm100_gemm_ref.so")


def _cutlass_include():
    import importlib.util
    for pkg, sub in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        spec = importlib.util.find_spec(pkg)
        if spec and spec.submodule_search_locations:
            p = os.path.join(list(spec.submodule_search_locations)[0], sub)
            if os.path.isdir(os.path.join(p, "cute")):
                return p
    return None


def build_reference_gemm(force=False):
    # the checkout named by the environment, else one that sits beside this repository
    ref = os.environ.get("APPLIED_AI_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    src = os.path.join(ref, "kernels/blackwell/cute_gemm_02_tma/sm100_gemm.cu")
    if not os.path.exists(src):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force:
        return LIB
    inc = _cutlass_include()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if inc is None or not os.path.exists(nvcc):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = [nvcc, "-O3", "-std=c++17", "--expt-relaxed-constexpr", "--expt-extended-lambda",
           "-gencode=arch=compute_100a,code=sm_100a", "-DCUTLASS_ARCH_MMA_SM100_SUPPORTED", "-DCUTE_SM100_ENABLED",
           "--use_fast_math", "-Xcompiler=-fPIC", "-DCUTE_ARCH_TCGEN05_TMEM_ENABLED=1", "-shared", "-cudart", "static",
           "-I", inc, "-I", os.path.join(os.path.dirname(inc), "tools", "util", "include"),
           "-I", os.path.dirname(src), src, "-o", LIB]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stderr[-2000:])
        return None
    return LIB


if __name__ == "__main__":
    print(build_reference_gemm(force="--force" in sys.argv))
