"""The C-ABI library builds, loads and exports everything include/b200moe.h declares.
No compute call is made: this runs without a GPU."""
import ctypes
import os
import re

import pytest
import torch

import applied_ai_b200 as B
from applied_ai_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|long long)\s+(b200moe_\w+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build_library()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = declared_symbols()
    assert len(names) >= 9
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/b200moe.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signatures and header disagree"
    assert _lib.load().b200moe_version() >= 1


def test_error_codes_are_described():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    for code in re.findall(r"#define B200MOE_E\w+ \((-\d+)\)", text):
        assert int(code) in _lib.ERROR_NAMES


def test_argument_errors_need_no_device():
    lib = _lib.load()
    n = ctypes.c_size_t(0)
    assert lib.b200moe_route_workspace_bytes(1000, 8, ctypes.byref(n)) == 0 and n.value == 4 * 8 * 4
    assert lib.b200moe_route_workspace_bytes(262144, 256, ctypes.byref(n)) == 0 and n.value == 1024 * 256 * 4
    assert lib.b200moe_route_workspace_bytes(10, 0, ctypes.byref(n)) == -1
    assert lib.b200moe_route_workspace_bytes(10, 2048, ctypes.byref(n)) == 0
    assert lib.b200moe_route_workspace_bytes(10, 2049, ctypes.byref(n)) == -1
    # null pointers / bad sizes are rejected before any CUDA call
    assert lib.b200moe_grouped_gemm_bf16(None, None, None, None, 8, 8, 8, 1, 8, 0, 0, 0, None, 0, None, None) == -1
    assert lib.b200moe_swiglu(None, None, 4, 8, None) == -1
    assert lib.b200moe_quant_1x128(None, 0, None, None, 4, 100, None) == -1


def test_wrappers_reject_cpu_tensors_loudly():
    x = torch.randn(8, 8).to(torch.bfloat16)
    w = torch.randn(16, 8).to(torch.bfloat16)
    m = torch.tensor([4, 4], dtype=torch.int32)
    with pytest.raises(RuntimeError, match="CUDA"):
        B.grouped_gemm(x, w, m)
    with pytest.raises(RuntimeError, match="CUDA"):
        B.grouped_gemm_forward(x, w, m)
    with pytest.raises(RuntimeError, match="CUDA"):
        B.route(torch.zeros(4, 2, dtype=torch.int32), 4)
    with pytest.raises(RuntimeError, match="CUDA"):
        B.float8_groupwise_quantize(torch.randn(4, 128))
    with pytest.raises(ValueError):
        B.float8_groupwise_quantize(torch.randn(4, 100))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "applied-ai_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, f"{f} mentions the oracle"
