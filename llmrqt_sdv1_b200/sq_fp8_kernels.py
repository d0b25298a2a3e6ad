"""Drop-in for the reference's compiled extension module `runtime.sq_fp8_kernels`
(LLMQRT/runtime_refact/csrc/bindings.cpp:9-47): same function names, argument
order and return shapes for the five AWQ entry points, backed by the sm_100a
kernels.  The arguments are the ON-DISK tensors; the kernel-layout repack is
done once per weight tensor and cached on the tensor's identity.

The three non-AWQ names exist only so that the reference's `linear` package
imports (linear_fp8.py:7-8, linear_sq.py:14); calling them raises.
"""
from __future__ import annotations

import weakref

import torch

from . import kernels

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


def _not_awq(name):
    def fn(*_a, **_k):
        raise NotImplementedError(f"{name}: only the AWQ W4A16 path is implemented for sm_100a")
    fn.__name__ = name
    return fn


cutlass_f8f8bf16_tensorwise_sm89 = _not_awq("cutlass_f8f8bf16_tensorwise_sm89")
cutlass_f8f8bf16_rowwise_sm89 = _not_awq("cutlass_f8f8bf16_rowwise_sm89")
w8a8_int8_linear_bbf16_obf16_per_tensor = _not_awq("w8a8_int8_linear_bbf16_obf16_per_tensor")
