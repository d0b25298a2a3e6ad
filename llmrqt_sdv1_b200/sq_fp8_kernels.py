"""Drop-in for the reference's compiled extension module `runtime.sq_fp8_kernels`
(LLMQRT/runtime_refact/csrc/bindings.cpp:9-47): same function names, argument
order and return shapes for the five AWQ entry points, backed by the sm_100a
kernels.  The arguments are the ON-DISK tensors; the kernel-layout repack is
done once per weight tensor and cached on the tensor's identity.

The three non-AWQ entry points (FP8 tensorwise / rowwise, SmoothQuant INT8) keep the
reference's names, `_sm89` included, and run 8-bit tensor-memory GEMMs.
"""
from __future__ import annotations

import weakref

import torch

from . import kernels, q8

_cache: dict[int, tuple] = {}


def _drop(key: int) -> None:
    _cache.pop(key, None)


def packed_for(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int):
    """Kernel-layout weight for these on-disk tensors, repacked on first use.

    Keyed on the qweight tensor object and its in-place version counter, so a
    buffer replaced after loading (as `fuse_qkv` does,
    LLMQRT/runtime_refact/utils/fused_utils.py:88-105) or overwritten by
    `load_state_dict` is repacked again.
    """
    key = id(qweight)
    hit = _cache.get(key)
    if hit is not None:
        ref, version, ptr, zptr, sptr, pw = hit
        if (ref() is qweight and version == qweight._version and ptr == qweight.data_ptr()
                and zptr == qzeros.data_ptr() and sptr == scales.data_ptr() and pw.group_size == group_size):
            return pw
    pw = kernels.make_packed(qweight, qzeros, scales, group_size)
    _cache[key] = (weakref.ref(qweight, lambda _r, k=key: _drop(k)), qweight._version, qweight.data_ptr(),
                   qzeros.data_ptr(), scales.data_ptr(), pw)
    return pw


def _linear(in_feats, pw):
    overlap, pw.fresh = not pw.fresh, False   # the call right after a repack must not prefetch weights
    return kernels.linear(in_feats, pw, overlap=overlap)


def _infer_group(kernel: torch.Tensor, scaling_factors: torch.Tensor) -> int:
    return kernel.shape[0] // scaling_factors.shape[0]


def awq_gemv(in_feats, kernel, scaling_factors, zeros, group_size):
    """[M, K] fp16 -> [M, N] fp16 (csrc/awq/gemv.cu:171-208).  The reference launches nothing
    unless group_size == 128 and returns uninitialised memory; here any multiple of 128 works
    and anything else raises ValueError."""
    pw = packed_for(kernel, zeros, scaling_factors, group_size)
    return _linear(in_feats, pw)


def awq_gemv_coalesced(in_feats, kernel, scaling_factors, zeros, group_size, version=2):
    """Same contract as awq_gemv (csrc/awq/gemv_coalesced.cu:263-303); `version` selected
    between two reference kernels and has no effect here."""
    return awq_gemv(in_feats, kernel, scaling_factors, zeros, group_size)


def awq_gemm(in_feats, kernel, scaling_factors, zeros, split_k_iters=8):
    """[M, K] fp16 -> [M, N] fp16 (csrc/awq/gemm.cu:407-467).  `split_k_iters` is accepted and
    ignored: accumulation stays in fp32 tensor memory, there are no fp16 partial sums to add.
    Rows <= 16 are routed to the decode kernel inside the library, because the reference's own
    dispatch sends 8 <= M <= 16 here (linear_awq.py:167-185)."""
    pw = packed_for(kernel, zeros, scaling_factors, _infer_group(kernel, scaling_factors))
    return _linear(in_feats, pw)


def awq_gemm_db(in_feats, kernel, scaling_factors, zeros, split_k_iters=8):
    """csrc/awq/gemm_db.cu:670-732; same contract as awq_gemm."""
    return awq_gemm(in_feats, kernel, scaling_factors, zeros, split_k_iters)


def awq_gemm_cutlass(in_feats, kernel, scaling_factors, zeros, split_k_iters=8):
    """csrc/awq/gemm_cutlass.cu:314-374; same contract as awq_gemm."""
    return awq_gemm(in_feats, kernel, scaling_factors, zeros, split_k_iters)


_DTYPE_STR = {"bfloat16": torch.bfloat16, "float16": torch.float16}


def cutlass_f8f8bf16_tensorwise_sm89(XQ, WQ, bias, alpha, beta, dtype_str):
    """[M, K] e4m3 x [K, N] e4m3 (stride [1, K]) -> [M, N] `dtype_str`: alpha * (XQ @ WQ) + beta * bias
    (csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:316-328; checks :272-311, dtype dispatch :228-262).  The name is
    the reference's; the kernel is an sm_100a one.  `alpha` may also be a one-element CUDA tensor, which is then
    read on the device instead of being converted to a python float (the reference's binding forces that read)."""
    if dtype_str not in _DTYPE_STR:
        raise RuntimeError(f"currently only support bf16 or fp16 output dtype, the passed dtype is {dtype_str}")
    out_dtype = _DTYPE_STR[dtype_str]
    if bias is not None and bias.dtype != out_dtype:
        raise RuntimeError("if bias has value, dtype passed in should same as bias dtype")
    return q8.gemm_tensorwise(XQ, WQ, bias, alpha, beta, out_dtype)


def cutlass_f8f8bf16_rowwise_sm89(XQ, WQ, bias, x_scale, w_scale, use_fast_accum=True):
    """[M, K] e4m3 / e5m2 x [K, N] e4m3 -> [M, N] bf16: (XQ @ WQ) * x_scale[M, 1] * w_scale[1, N] + bias
    (csrc/fp8/sm89_fp8_rowwise_fbgemm.cu:2222-2248; checks :2170-2218).  `use_fast_accum` selected between two
    accumulation schemes of the sm_89 kernel; here the accumulator is always fp32 in tensor memory."""
    return q8.gemm_rowwise(XQ, WQ, bias, x_scale, w_scale)


def w8a8_int8_linear_bbf16_obf16_per_tensor(input, weight, bias, alpha, beta):
    """[M, K] int8 x [K, N] int8 (stride [1, K]) -> [M, N]: alpha * int32(input @ weight) + beta * bias
    (csrc/smoothquant/sq_gemm.cu:30-190).  The reference requires a bias tensor (zeros when the layer has none),
    writes fp16 whatever the bias dtype and reads a bf16 bias as if it were fp16; here the output takes the
    bias's dtype (fp16 or bf16) and a bf16 bias is read as bf16."""
    if bias is None:
        raise RuntimeError("w8a8_int8_linear_bbf16_obf16_per_tensor: bias is required (pass zeros)")
    return q8.gemm_tensorwise(input, weight, bias, alpha, beta, bias.dtype, int8=True)
