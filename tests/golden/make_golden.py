"""Generates the golden fixtures of this directory by running the REFERENCE's own test
code on the CPU.  Needs the reference checkout (its path in $APPLIED_AI_REFERENCE); the fixtures it writes are committed so the tests need only them.

Nothing of the reference is copied: functions are pulled out of its files with `ast`
at run time and executed in a namespace where

  * `grouped_gemm` (the Triton entry point that cannot run here) is a recorder that
    keeps the inputs the reference's test generated and returns zeros, and
  * `torch.testing.assert_close` is a recorder that keeps the `expected_result` the
    reference's per-expert loop computed (dev/triton_groupGEMM/testing/base_testing.py:125-131).

  grouped_bf16.npz : inputs + expected outputs of `_test_grouped_gemm_bf16` for a few
                     shapes the reference tests (base_testing.py:135-138, unit_tests.py:99-103)
  torch_moe.npz    : inputs + output of `torch_moe` (kernels/triton/inference/
                     col_major_moe_gemm/test_moe_gemm.py:16-30) on a small bf16 case
  align_example.json : the worked example in the moe_align_block_size docstring
                     (v0_moe_fused.py:157-165), read from the docstring text
  grouped_fp8_rowwise.npz : the same for `_test_grouped_gemm_fp8_rowwise`, whose body the reference
                     keeps as a string (base_testing.py:43-96, the test is switched off there because
                     FBGEMM's quantize_fp8_row is absent): the string is parsed and its expected-value
                     loop (:75-88) executed with a stand-in row quantiser (scale = amax/448 per row)
  backward.npz     : `_pytorch_reference_backward` (kernels/MoE/group_GEMM/triton/testing/
                     pytorch_reference_backwards.py:165-197) on three small cases
  quant_1x128.npz  : `_float8_groupwise_quant_kernel` (float8_groupwise_quant.py:20-50)
                     executed by Triton's CPU interpreter, if that is available

bf16 tensors are stored as their uint16 bit patterns, e4m3 as uint8.
"""
import ast
import json
import os
import re
import sys
import types

import numpy as np
import torch

REF = os.environ.get("APPLIED_AI_REFERENCE")
if not REF or not os.path.isdir(REF):
    sys.exit("set APPLIED_AI_REFERENCE to a checkout of the reference repository")
HERE = os.path.dirname(os.path.abspath(__file__))


def bits16(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def find_function(path, name):
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == name:
            return node
    raise KeyError(name)


def compile_function(node, namespace, filename):
    mod = ast.Module(body=[node], type_ignores=[])
    ast.fix_missing_locations(mod)
    exec(compile(mod, filename, "exec"), namespace)
    return namespace[node.name]


class TorchProxy:
    """The torch module with torch.testing.assert_close replaced by a recorder."""

    def __init__(self, record):
        self.testing = types.SimpleNamespace(assert_close=record)

    def __getattr__(self, name):
        return getattr(torch, name)


def golden_grouped():
    path = os.path.join(REF, "dev/triton_groupGEMM/testing/base_testing.py")
    node = find_function(path, "_test_grouped_gemm_bf16")
    captured = {}

    def fake_grouped_gemm(a, b, m_sizes):
        captured["a"], captured["b"], captured["m_sizes"] = a.clone(), b.clone(), m_sizes.clone()
        G = m_sizes.numel()
        return torch.zeros(a.shape[0], b.shape[0] // G, dtype=torch.bfloat16)

    def record(result, expected, **kw):
        captured["expected"] = expected.clone()
        captured["tol"] = kw

    self_stub = types.SimpleNamespace(assertTrue=lambda c: None)
    from typing import Tuple
    ns = {"torch": TorchProxy(record), "grouped_gemm": fake_grouped_gemm, "self": self_stub, "Tuple": Tuple}
    fn = compile_function(node, ns, path)
    out = {}
    shapes = [(1, 64, 256, 256), (4, 64, 256, 256), (4, 128, 128, 256), (8, 256, 256, 128), (8, 128, 64, 64),
              (16, 512, 64, 128)]
    torch.manual_seed(0)  # base_testing.py:41
    for i, shape in enumerate(shapes):
        fn(shape, torch.device("cpu"))
        out[f"shape{i}"] = np.array(shape, dtype=np.int32)
        out[f"a{i}"] = bits16(captured["a"])
        out[f"b{i}"] = bits16(captured["b"])
        out[f"m_sizes{i}"] = captured["m_sizes"].numpy().astype(np.int32)
        out[f"expected{i}"] = bits16(captured["expected"])
    out["n_cases"] = np.array(len(shapes))
    out["rtol"] = np.array(captured["tol"]["rtol"])
    out["atol"] = np.array(captured["tol"]["atol"])
    np.savez_compressed(os.path.join(HERE, "grouped_bf16.npz"), **out)
    print("grouped_bf16.npz:", len(shapes), "cases, tol", captured["tol"])


def golden_fp8_rowwise():
    """The reference keeps its FP8 row-wise test as a string expression inside the test class
    (dev/triton_groupGEMM/testing/base_testing.py:43-96).  Parse that string, take
    `_test_grouped_gemm_fp8_rowwise` out of it and run it on the CPU: the Triton entry point is a
    recorder, `quantize_fp8_row` (FBGEMM, absent) is a stand-in with the published row-wise
    recipe (one fp32 scale per row, amax / 448, e4m3 values), and torch.testing.assert_close
    records the `expected_result` the reference's own loop computed (:75-88) and its tolerances (:90)."""
    import textwrap
    path = os.path.join(REF, "dev/triton_groupGEMM/testing/base_testing.py")
    tree = ast.parse(open(path).read())
    body = None
    for node in ast.walk(tree):
        if (isinstance(node, ast.Expr) and isinstance(node.value, ast.Constant) and isinstance(node.value.value, str)
                and "_test_grouped_gemm_fp8_rowwise" in node.value.value):
            body = node.value.value
    if body is None:
        raise KeyError("the FP8 row-wise test body was not found in " + path)
    inner = ast.parse(textwrap.dedent(body))
    fn_node = next(n for n in ast.walk(inner)
                   if isinstance(n, ast.FunctionDef) and n.name == "_test_grouped_gemm_fp8_rowwise")
    captured = {}

    def quantize_fp8_row(t):
        f = t.float()
        scale = f.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
        q = (f / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
        return q, scale

    def fake_fp8(a_fp8, b_fp8, m_sizes, a_scale, b_scale):
        captured.update(a=a_fp8.clone(), b=b_fp8.clone(), m_sizes=m_sizes.clone(), a_scale=a_scale.clone(),
                        b_scale=b_scale.clone())
        return torch.zeros(a_fp8.shape[0], b_fp8.shape[0] // m_sizes.numel(), dtype=torch.bfloat16)

    def record(result, expected, **kw):
        captured["expected"] = expected.clone()
        captured["tol"] = kw

    from typing import Tuple
    ns = {"torch": TorchProxy(record), "grouped_gemm_fp8_rowwise": fake_fp8, "quantize_fp8_row": quantize_fp8_row,
          "self": types.SimpleNamespace(assertTrue=lambda c: None), "Tuple": Tuple}
    fn = compile_function(fn_node, ns, path)
    out = {}
    shapes = [(1, 64, 256, 256), (4, 64, 256, 256), (4, 512, 256, 256), (16, 512, 256, 256)]  # :92-96 uses these
    torch.manual_seed(0)  # base_testing.py:41
    for i, shape in enumerate(shapes):
        fn(shape, torch.device("cpu"))
        out[f"shape{i}"] = np.array(shape, dtype=np.int32)
        out[f"a{i}"] = captured["a"].view(torch.uint8).numpy()
        out[f"b{i}"] = captured["b"].view(torch.uint8).numpy()
        out[f"a_scale{i}"] = captured["a_scale"].numpy().astype(np.float32)
        out[f"b_scale{i}"] = captured["b_scale"].numpy().astype(np.float32)
        out[f"m_sizes{i}"] = captured["m_sizes"].numpy().astype(np.int32)
        out[f"expected{i}"] = bits16(captured["expected"])
    out["n_cases"] = np.array(len(shapes))
    out["rtol"] = np.array(captured["tol"]["rtol"])
    out["atol"] = np.array(captured["tol"]["atol"])
    np.savez_compressed(os.path.join(HERE, "grouped_fp8_rowwise.npz"), **out)
    print("grouped_fp8_rowwise.npz:", len(shapes), "cases, tol", captured["tol"])


def golden_torch_moe():
    path = os.path.join(REF, "kernels/triton/inference/col_major_moe_gemm/test_moe_gemm.py")
    node = find_function(path, "torch_moe")

    class SiluAndMul:  # stand-in for vllm.model_executor.layers.activation.SiluAndMul (forward_native)
        def __call__(self, x):
            d = x.shape[-1] // 2
            return torch.nn.functional.silu(x[..., :d]) * x[..., d:]

    fn = compile_function(node, {"torch": torch, "SiluAndMul": SiluAndMul}, path)
    out = {}
    cases = [(16, 64, 128, 8, 2, 3227), (33, 96, 64, 4, 2, 3228), (8, 32, 64, 16, 4, 3229)]  # m, I, H, E, topk, seed
    for i, (m, n, k, e, topk, seed) in enumerate(cases):
        g = torch.Generator().manual_seed(seed)
        a = (torch.randn(m, k, generator=g) / 10).to(torch.bfloat16)
        w1 = (torch.randn(e, 2 * n, k, generator=g) / 10).to(torch.bfloat16)
        w2 = (torch.randn(e, k, n, generator=g) / 10).to(torch.bfloat16)
        score = torch.softmax(torch.randn(m, e, generator=g), dim=-1)
        topk_weight, topk_ids = torch.topk(score, topk)
        # run the reference procedure in fp32 on the bf16-rounded inputs
        res = fn(a.float(), w1.float(), w2.float(), topk_weight.float(), topk_ids)
        out[f"a{i}"], out[f"w1{i}"], out[f"w2{i}"] = bits16(a), bits16(w1), bits16(w2)
        out[f"topk_weight{i}"] = topk_weight.numpy().astype(np.float32)
        out[f"topk_ids{i}"] = topk_ids.numpy().astype(np.int32)
        out[f"out{i}"] = res.numpy().astype(np.float32)
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "torch_moe.npz"), **out)
    print("torch_moe.npz:", len(cases), "cases")


def golden_align_example():
    path = os.path.join(REF, "kernels/triton/inference/col_major_moe_gemm/v0_moe_fused.py")
    doc = ast.get_docstring(find_function(path, "moe_align_block_size"))
    lists = re.findall(r"\[[\d,\s\[\]]+\]", doc)
    topk_ids = json.loads(next(s for s in lists if s.startswith("[[")))
    sorted_ids = json.loads(next(s for s in lists if s.startswith("[3")))
    nums = dict(re.findall(r"(block_size|num_experts) = (\d+)", doc))
    ex = {"topk_ids": topk_ids, "sorted_token_ids": sorted_ids, "block_size": int(nums["block_size"]),
          "num_experts_in_text": int(nums["num_experts"]),
          "note": "ids in the example run 1..4, so the arrays cover 5 expert slots with slot 0 empty"}
    json.dump(ex, open(os.path.join(HERE, "align_example.json"), "w"), indent=1)
    print("align_example.json:", ex["sorted_token_ids"])


def golden_quant():
    os.environ["TRITON_INTERPRET"] = "1"
    try:
        sys.path.insert(0, os.path.join(REF, "kernels/triton/inference/fp8"))
        import float8_groupwise_quant as ref_q
        g = torch.Generator().manual_seed(77)
        x = torch.randn(24, 512, generator=g) * torch.logspace(-3, 2, 24)[:, None]
        x[3, :128] = 0.0  # an all-zero run exercises the 1e-12 floor
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):
            q, s = ref_q.float8_groupwise_quantize(x, 128)
        np.savez_compressed(os.path.join(HERE, "quant_1x128.npz"), x=x.numpy(),
                            q=q.view(torch.uint8).numpy(), scales=s.numpy())
        print("quant_1x128.npz: reference kernel ran under the Triton interpreter")
    except Exception as exc:  # interpreter missing or incompatible: leave the fixture out
        print("quant_1x128.npz NOT written:", repr(exc))


def golden_backward():
    """`_pytorch_reference_backward` (kernels/MoE/group_GEMM/triton/testing/
    pytorch_reference_backwards.py:165-197) pulled out of the reference file and run on the CPU in
    fp32 on bf16-rounded inputs."""
    path = os.path.join(REF, "kernels/MoE/group_GEMM/triton/testing/pytorch_reference_backwards.py")
    fn = compile_function(find_function(path, "_pytorch_reference_backward"), {"torch": torch}, path)
    out = {}
    cases = [(4, 96, 64, 48, [30, 0, 41, 25], 51), (3, 200, 32, 72, [64, 100, 36], 52), (2, 128, 128, 64, [128, 0], 53)]
    for i, (G, M, N, K, ms, seed) in enumerate(cases):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(G * N, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        dy = torch.randn(M, N * G, generator=g).to(torch.bfloat16)
        m_sizes = torch.tensor(ms, dtype=torch.int32)
        gx, gw = fn(dy.float(), x.float(), w.float(), m_sizes)
        out[f"x{i}"], out[f"w{i}"], out[f"dy{i}"] = bits16(x), bits16(w), bits16(dy)
        out[f"m_sizes{i}"] = m_sizes.numpy()
        out[f"grad_x{i}"], out[f"grad_w{i}"] = gx.numpy().astype(np.float32), gw.numpy().astype(np.float32)
    out["n_cases"] = np.array(len(cases))
    np.savez_compressed(os.path.join(HERE, "backward.npz"), **out)
    print("backward.npz:", len(cases), "cases")


if __name__ == "__main__":
    if "--only-backward" in sys.argv:
        golden_backward()
        sys.exit(0)
    if "--only-fp8-rowwise" in sys.argv:
        golden_fp8_rowwise()
        sys.exit(0)
    golden_grouped()
    golden_fp8_rowwise()
    golden_torch_moe()
    golden_align_example()
    golden_quant()
    golden_backward()
