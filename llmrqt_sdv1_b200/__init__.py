"""B200 (sm_100a) implementation of the AWQ W4A16 quantized-linear hot path.

Public surface:
  AWQLinear_GEMM, AWQLinearMMFunction   module API of the reference runtime
  AWQGatedMLP                           gate/up/down of a decoder layer in two launches (fused epilogues)
  GraphedStep                           a fixed sequence of module calls captured in a CUDA graph (decode step)
  sq_fp8_kernels                        function API of the reference extension
  kernels                               torch wrappers over the C ABI (include/awq_b200.h)
"""
from .linear_awq import AWQLinear_GEMM, AWQLinearMMFunction, WQLinear_GEMM, WQLinearMMFunction, pack_awq_int4
from .graph import GraphedStep
from .mlp_awq import AWQGatedMLP

__all__ = ["AWQGatedMLP", "AWQLinear_GEMM", "GraphedStep", "AWQLinearMMFunction", "WQLinear_GEMM", "WQLinearMMFunction", "pack_awq_int4"]
