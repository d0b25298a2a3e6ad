"""`runtime.sq_fp8_kernels`, the module name the reference extension is built under."""
from llmrqt_sdv1_b200.sq_fp8_kernels import (  # noqa: F401
    awq_gemm,
    awq_gemm_cutlass,
    awq_gemm_db,
    awq_gemv,
    awq_gemv_coalesced,
    cutlass_f8f8bf16_rowwise_sm89,
    cutlass_f8f8bf16_tensorwise_sm89,
    w8a8_int8_linear_bbf16_obf16_per_tensor,
)
