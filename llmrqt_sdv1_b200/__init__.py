"""B200 (sm_100a) implementation of the AWQ W4A16 quantized-linear hot path.

Public surface:
  AWQLinear_GEMM, AWQLinearMMFunction   module API of the reference runtime
  AWQGatedMLP                           gate/up/down of a decoder layer in two launches (fused epilogues)
  GraphedStep                           a fixed sequence of module calls captured in a CUDA graph (decode step)
  FP8DynamicLinear, FP8StaticLinear, FP8Native*Linear, SqW8A8BBF16OBF16PerTensor
                                        the reference's FP8 / SmoothQuant module classes on the 8-bit GEMM
  get_concrete_linear_module            quant_method -> module class, as the reference's linear package maps it
  sq_fp8_kernels                        function API of the reference extension
  kernels                               torch wrappers over the C ABI (include/awq_b200.h)
"""
from .linear_awq import AWQLinear_GEMM, AWQLinearMMFunction, WQLinear_GEMM, WQLinearMMFunction, pack_awq_int4
from .graph import GraphedStep
from .mlp_awq import AWQGatedMLP
from .linear_fp8 import FP8DynamicLinear, FP8NativeDynamicLinear, FP8NativeStaticLinear, FP8StaticLinear
from .linear_sq import SqW8A8BBF16OBF16PerTensor

# quant_method of a checkpoint's config -> module class, as the reference's linear package maps it
# (LLMQRT/runtime_refact/nn_models/modules/linear/__init__.py:10-20)
method_to_linear = {
    "awq": AWQLinear_GEMM,
    "sq": SqW8A8BBF16OBF16PerTensor,
    "fp8_static_quant": FP8StaticLinear,
    "fp8_dynamic_quant": FP8DynamicLinear,
    "fp8_native_static_quant": FP8NativeStaticLinear,
    "fp8_native_dynamic_quant": FP8NativeDynamicLinear,
}


def get_concrete_linear_module(quant_method):
    return method_to_linear[quant_method]


__all__ = ["AWQGatedMLP", "AWQLinear_GEMM", "GraphedStep", "AWQLinearMMFunction", "WQLinear_GEMM", "WQLinearMMFunction",
           "pack_awq_int4", "FP8DynamicLinear", "FP8StaticLinear", "FP8NativeDynamicLinear", "FP8NativeStaticLinear",
           "SqW8A8BBF16OBF16PerTensor", "method_to_linear", "get_concrete_linear_module"]
