"""Generate the golden fixtures of the 8-bit (FP8 / SmoothQuant INT8) linears by running the REFERENCE's own
Python functions and the torch comparators its unit tests use (not the oracle, not the product).

Run once, in a container that has the reference checkout (CPU is enough):

    python tests/golden/make_q8_golden.py /path/to/reference

Imported unmodified from the reference:
  * per_tensor_quantize, static_per_tensor_quantize, per_token_quantize, fp8_gemm, FP8DynamicLinear
    (LLMQRT/runtime_refact/nn_models/modules/linear/linear_fp8.py:11-268),
  * quantize_activation_per_tensor_absmax (LLMQRT/runtime_refact/nn_models/modules/linear/linear_sq.py:19-28).
The compiled GEMMs themselves need sm_89 hardware and are not run; their comparators are what the reference's
unit tests compare them with: torch._scaled_mm (unittest/test_fp8_tensorwise_linear.py:33-44) and an fp16
nn.Linear on dequantised operands (unittest/test_sq_linear.py:18-27), plus an exact integer matmul.

Fixtures (seeded; shapes follow the reference's unit tests, reduced where noted):
  q8_quant.npz        activations in bf16 and fp16 -> bytes and scales of the four quantisers (CPU torch: a division
                      by a python number is a true division there).
  q8_fp8_gemm.npz     128 x 256 e4m3 activations, 512 x 256 e4m3 weights (the unit tests' shapes), bf16 bias:
                      torch._scaled_mm per-tensor output + bias; per-row scaled float64 product for the rowwise form;
                      FP8DynamicLinear(impl_mode="fp8_gemm") forward of the reference, per tensor and per token.
  q8_int8_gemm.npz    64 x 512 int8 activations, 256 x 512 int8 weights (unit test: 128 x 512, 1024 x 512), fp16 bias:
                      exact int32 product, fp16 nn.Linear comparator of the unit test.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch


def _install_stubs():
    acc = types.ModuleType("accelerate")
    big = types.ModuleType("accelerate.big_modeling")
    acc.big_modeling = big
    for name in ("init_empty_weights", "load_checkpoint_and_dispatch", "infer_auto_device_map", "dispatch_model"):
        setattr(acc, name, lambda *a, **k: None)
        setattr(big, name, lambda *a, **k: None)
    sys.modules.setdefault("accelerate", acc)
    sys.modules.setdefault("accelerate.big_modeling", big)
    rt = types.ModuleType("runtime")
    ext = types.ModuleType("runtime.sq_fp8_kernels")

    def _absent(*a, **k):
        raise NotImplementedError("compiled extension is not part of golden generation")

    for name in ("cutlass_f8f8bf16_tensorwise_sm89", "cutlass_f8f8bf16_rowwise_sm89",
                 "w8a8_int8_linear_bbf16_obf16_per_tensor", "awq_gemm", "awq_gemv", "awq_gemv_coalesced", "awq_gemm_db",
                 "awq_gemm_cutlass"):
        setattr(ext, name, _absent)
    rt.sq_fp8_kernels = ext
    sys.modules["runtime"] = rt
    sys.modules["runtime.sq_fp8_kernels"] = ext


def _bits(t: torch.Tensor) -> np.ndarray:
    """16-bit float tensor -> uint16 bit patterns; fp8 / int8 -> uint8 bytes."""
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().view(torch.uint8).numpy()


def main(ref_root: str) -> None:
    import transformers  # noqa: F401  (before the stand-in modules exist)
    _install_stubs()
    sys.path.insert(0, os.path.join(ref_root, "LLMQRT"))
    from runtime_refact.nn_models.modules.linear import linear_fp8 as ref_fp8
    from runtime_refact.nn_models.modules.linear import linear_sq as ref_sq
    here = os.path.dirname(os.path.abspath(__file__))

    # ---- quantisers ---------------------------------------------------------------------------------------------
    out = {}
    g = torch.Generator().manual_seed(1234)
    for tag, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        x = torch.randn(6, 64, generator=g) * torch.tensor([0.01, 0.3, 1.0, 7.0, 30.0, 1.0]).view(6, 1)
        x[5, :8] = torch.tensor([0.0, -0.0, 1e-4, -1e-4, 448.0, -448.0, 0.5, -0.5])
        x = x.to(dt)
        out[f"x_{tag}"] = _bits(x)
        q, s = ref_fp8.per_tensor_quantize(x.clone())
        out[f"pt_q_{tag}"], out[f"pt_s_{tag}"] = _bits(q), s.reshape(1).numpy()
        q, s = ref_fp8.per_token_quantize(x.clone())
        out[f"tok_q_{tag}"], out[f"tok_s_{tag}"] = _bits(q), s.reshape(-1).numpy()
        q = ref_fp8.static_per_tensor_quantize(x.clone(), torch.tensor([0.037], dtype=torch.float32))
        out[f"st_q_{tag}"] = _bits(q)
        q, s = ref_sq.quantize_activation_per_tensor_absmax(x.clone())
        out[f"sq_q_{tag}"], out[f"sq_s_{tag}"] = _bits(q), s.float().reshape(1).numpy()
        # alpha of the module forward: 16-bit scale times a python float (linear_sq.py:97)
        out[f"sq_alpha_{tag}"] = (s * 0.0123).float().reshape(1).numpy()
    out["static_scale"] = np.array([0.037], dtype=np.float32)
    out["sq_weight_scale"] = np.array([0.0123], dtype=np.float32)
    np.savez_compressed(os.path.join(here, "q8_quant.npz"), **out)

    # ---- fp8 GEMM -----------------------------------------------------------------------------------------------
    torch.manual_seed(42)
    a = torch.randn(128, 256, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
    b = torch.randn(512, 256, dtype=torch.bfloat16).to(torch.float8_e4m3fn)
    bias = torch.randn(512, dtype=torch.bfloat16)
    scale_a, scale_b = torch.tensor(0.5), torch.tensor(1.2)
    y = torch._scaled_mm(a, b.t(), scale_a=scale_a, scale_b=scale_b, out_dtype=torch.bfloat16)
    y_bias = y + bias.reshape(1, -1)
    sa = torch.rand(128, 1, dtype=torch.float32)
    sb = torch.rand(1, 512, dtype=torch.float32)
    prod = a.double() @ b.double().t()
    y_row = (prod * sa.double() * sb.double())
    # the reference's own dequantise-and-matmul forward (impl_mode="fp8_gemm"), per tensor and per token
    xin = (torch.randn(2, 8, 256) * 3).to(torch.bfloat16)
    mods = {}
    for per_tensor in (True, False):
        m = ref_fp8.FP8DynamicLinear(256, 512, True, dev="cpu", dtype=torch.bfloat16, per_tensor=per_tensor,
                                     impl_mode="fp8_gemm")
        m.weight.data = b.to(torch.bfloat16)
        m.weight_scale.data = torch.tensor([0.02]) if per_tensor else (torch.rand(512, 1) * 0.05 + 0.01)
        m.bias.data = bias.clone()
        mods["tensor" if per_tensor else "token"] = (m.weight_scale.data.clone(), m(xin.clone()))
    np.savez_compressed(
        os.path.join(here, "q8_fp8_gemm.npz"), a=_bits(a), b=_bits(b), bias=_bits(bias),
        alpha=np.array([0.5 * 1.2], dtype=np.float32), scaled_mm=_bits(y), scaled_mm_bias=_bits(y_bias),
        row_sa=sa.numpy(), row_sb=sb.numpy(), row_f64=y_row.numpy().astype(np.float32),
        mod_x=_bits(xin), mod_ws_tensor=mods["tensor"][0].numpy(), mod_y_tensor=_bits(mods["tensor"][1]),
        mod_ws_token=mods["token"][0].numpy(), mod_y_token=_bits(mods["token"][1]))

    # ---- int8 GEMM ----------------------------------------------------------------------------------------------
    torch.manual_seed(7)
    B, K, N = 64, 512, 256
    weight = torch.randint(-128, 127, (N, K), dtype=torch.int8)
    x = torch.randint(-128, 127, (B, K), dtype=torch.int8)
    bias = torch.randn(N, dtype=torch.float16)
    alpha, input_scale = 0.00334, 0.002
    linear = torch.nn.Linear(K, N, bias=True)
    linear.weight.data = weight.to(torch.float16) * alpha
    linear.bias.data = bias.to(torch.float16)
    with torch.no_grad():
        y_gt = linear(x.to(torch.float16) * input_scale)
    acc = x.int() @ weight.int().t()
    np.savez_compressed(os.path.join(here, "q8_int8_gemm.npz"), x=x.numpy(), w=weight.numpy(), bias=bias.numpy(),
                        alpha=np.array([alpha * input_scale], dtype=np.float32), acc=acc.numpy().astype(np.int32),
                        y_fp16_linear=y_gt.numpy())
    print("wrote q8_quant.npz, q8_fp8_gemm.npz, q8_int8_gemm.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_q8_golden.py /path/to/reference")
    main(sys.argv[1])
