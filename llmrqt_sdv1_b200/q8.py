"""8-bit quantized linears (FP8 e4m3 / SmoothQuant INT8) on the sm_100a library: thin, checked wrappers over the
C ABI (`awq_b200_fp8_gemm_*`, `awq_b200_int8_gemm_tensorwise`, `awq_b200_q8_quantize`).

Operand convention is the reference's: activations `XQ` [M, K] with unit inner stride, weights `WQ` as the
[K, N] view with stride [1, ld] of a row-major [N, K] tensor (`qweight.t()`), see
LLMQRT/runtime_refact/csrc/fp8/sm89_fp8_tensorwise_cutlassgemm.cu:272-311 (check_inputs).
There is no CPU or torch fallback.
"""
from __future__ import annotations

import torch

from ._lib import check, lib
from .kernels import _prep

_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)
_BIAS_KIND = {torch.bfloat16: 1, torch.float16: 2, torch.float32: 3}
_scratch: dict[tuple[int, int], torch.Tensor] = {}

QUANT_FP8_PER_TENSOR, QUANT_FP8_PER_TOKEN, QUANT_FP8_STATIC, QUANT_INT8_PER_TENSOR = range(4)


def _scratch_words(dev: torch.device, stream: int) -> torch.Tensor:
    """Per (device, stream): word 0 = status of the GEMM kernels, word 64 = |x| maximum scratch of the quantiser."""
    key = (dev.index, stream)
    t = _scratch.get(key)
    if t is None:
        t = torch.zeros(128, dtype=torch.int32, device=dev)
        _scratch[key] = t
    return t


def status(dev: torch.device | None = None) -> int:
    """OR of the status words the 8-bit GEMM kernels left on this device (0 = no bounded wait ran out).  Synchronises."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    out = 0
    for (index, _stream), t in _scratch.items():
        if index == dev.index:
            out |= int(t[0].item())
    return out


def _operands(XQ: torch.Tensor, WQ: torch.Tensor, dtypes, what: str):
    if XQ.dim() != 2 or WQ.dim() != 2:
        raise RuntimeError(f"{what}: XQ and WQ must be 2-D")
    if XQ.dtype not in dtypes or WQ.dtype not in dtypes:
        raise RuntimeError(f"{what}: operand dtypes {XQ.dtype}, {WQ.dtype} not supported")
    if XQ.size(1) != WQ.size(0):
        raise RuntimeError(f"{what}: XQ is [M, K] = {tuple(XQ.shape)} but WQ is [K, N] = {tuple(WQ.shape)}")
    M, K = XQ.shape
    N = WQ.size(1)
    if M > 1 and (XQ.stride(1) != 1 or XQ.stride(0) < K):
        raise RuntimeError(f"{what}: XQ must be row-major (stride {XQ.stride()})")
    if K > 1 and XQ.stride(1) != 1:
        raise RuntimeError(f"{what}: XQ must have unit inner stride")
    if K > 1 and WQ.stride(0) != 1:
        raise RuntimeError(f"{what}: WQ must be the [K, N] view with stride [1, ld] of a row-major [N, K] weight")
    ldx = XQ.stride(0) if M > 1 else max(K, 16)
    ldw = WQ.stride(1) if N > 1 else max(K, 16)
    if N > 1 and ldw < K:
        raise RuntimeError(f"{what}: WQ column pitch {ldw} < K = {K}")
    return M, N, K, ldx, ldw


def _bias(bias, N: int, dev, allowed, what: str):
    if bias is None:
        return None, 0
    if bias.dtype not in allowed:
        raise RuntimeError(f"{what}: bias dtype {bias.dtype} not supported")
    if bias.dim() != 1 or bias.numel() != N or bias.stride(0) != 1:
        raise RuntimeError(f"{what}: bias must be a contiguous [N] vector")
    if bias.device != dev:
        raise RuntimeError(f"{what}: bias is on {bias.device}, the operands on {dev}")
    return bias, _BIAS_KIND[bias.dtype]


def _alpha(alpha, dev):
    """(host float, device pointer or 0, keep-alive).  A tensor alpha stays on the device: no host read-back."""
    if isinstance(alpha, torch.Tensor):
        if alpha.numel() != 1:
            raise RuntimeError("alpha must have one element")
        if alpha.device.type == "cuda":
            a = alpha.detach().reshape(1)
            if a.dtype != torch.float32:
                a = a.float()
            if a.device != dev:
                a = a.to(dev)
            return 1.0, a.data_ptr(), a
        return float(alpha), 0, None
    return float(alpha), 0, None


def gemm_tensorwise(XQ, WQ, bias, alpha, beta, out_dtype: torch.dtype, alpha2=None, int8: bool = False,
                    out: torch.Tensor | None = None, split: bool = True) -> torch.Tensor:
    """`alpha * alpha2 * (XQ @ WQ) + beta * bias` in `out_dtype` (bf16 / fp16).  `alpha` / `alpha2` may be python
    numbers or one-element CUDA tensors (read on the device).  `split=False` forbids the K split of small problems."""
    what = "int8_gemm_tensorwise" if int8 else "fp8_gemm_tensorwise"
    dtypes = (torch.int8,) if int8 else (torch.float8_e4m3fn,)
    M, N, K, ldx, ldw = _operands(XQ, WQ, dtypes, what)
    if out_dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"{what}: output dtype must be bfloat16 or float16, got {out_dtype}")
    dev = _prep(XQ, WQ)
    bias, kind = _bias(bias, N, dev, (torch.bfloat16, torch.float16), what)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    elif out.dtype != out_dtype or not out.is_contiguous() or out.numel() != M * N or out.device != dev:
        raise ValueError(f"{what}: out must be a contiguous {out_dtype} tensor of {M} x {N} elements on {dev}")
    if M == 0 or N == 0:
        return out
    if K == 0:
        raise RuntimeError(f"{what}: K = 0")
    a_host, a_ptr, keep1 = _alpha(alpha, dev)
    a2_host, a2_ptr, keep2 = _alpha(1.0 if alpha2 is None else alpha2, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    st = _scratch_words(dev, stream)
    fn = lib.awq_b200_int8_gemm_tensorwise if int8 else lib.awq_b200_fp8_gemm_tensorwise
    check(fn(XQ.data_ptr(), ldx, WQ.data_ptr(), ldw, bias.data_ptr() if bias is not None else None, kind,
             out.data_ptr(), M, N, K, a_host * a2_host, a_ptr or None, a2_ptr or None, float(beta),
             1 if out_dtype == torch.bfloat16 else 0, 0 if split else 1, st.data_ptr(), stream), "awq_b200_" + what)
    del keep1, keep2
    return out


def gemm_rowwise(XQ, WQ, bias, x_scale, w_scale, out: torch.Tensor | None = None, split: bool = True) -> torch.Tensor:
    """bf16 `((XQ @ WQ) * x_scale[m]) * w_scale[n] + bias[n]`; x_scale [M, 1], w_scale [1, N] fp32."""
    what = "fp8_gemm_rowwise"
    if XQ.dtype not in _FP8 or WQ.dtype != torch.float8_e4m3fn:
        raise RuntimeError(f"{what}: XQ must be e4m3 or e5m2 and WQ e4m3, got {XQ.dtype}, {WQ.dtype}")
    M, N, K, ldx, ldw = _operands(XQ, WQ, _FP8, what)
    dev = _prep(XQ, WQ, x_scale, w_scale)
    if x_scale.dtype != torch.float32 or w_scale.dtype != torch.float32:
        raise RuntimeError(f"{what}: scales must be fp32")
    if x_scale.dim() != 2 or w_scale.dim() != 2 or tuple(x_scale.shape) != (M, 1) or tuple(w_scale.shape) != (1, N):
        raise RuntimeError(f"{what}: x_scale must be [M, 1] and w_scale [1, N], got {tuple(x_scale.shape)}, "
                           f"{tuple(w_scale.shape)}")
    if (M > 1 and x_scale.stride(0) != 1) or (N > 1 and w_scale.stride(1) != 1):
        raise RuntimeError(f"{what}: scales must be contiguous")
    bias, kind = _bias(bias, N, dev, (torch.bfloat16, torch.float32), what)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    elif out.dtype != torch.bfloat16 or not out.is_contiguous() or out.numel() != M * N or out.device != dev:
        raise ValueError(f"{what}: out must be a contiguous bfloat16 tensor of {M} x {N} elements on {dev}")
    if M == 0 or N == 0:
        return out
    if K == 0:
        raise RuntimeError(f"{what}: K = 0")
    stream = torch.cuda.current_stream(dev).cuda_stream
    st = _scratch_words(dev, stream)
    check(lib.awq_b200_fp8_gemm_rowwise(XQ.data_ptr(), ldx, 1 if XQ.dtype == torch.float8_e5m2 else 0, WQ.data_ptr(), ldw,
                                        bias.data_ptr() if bias is not None else None, kind, x_scale.data_ptr(),
                                        w_scale.data_ptr(), out.data_ptr(), M, N, K, 0 if split else 1, st.data_ptr(),
                                        stream),
          "awq_b200_fp8_gemm_rowwise")
    return out


def quantize(x: torch.Tensor, mode: int, static_scale: torch.Tensor | None = None, weight_scale: float = 1.0):
    """Quantise activations `x` [..., K] (fp16 / bf16) -> (xq [..., K], scales fp32).

    mode QUANT_FP8_PER_TENSOR: scales [1];  QUANT_FP8_PER_TOKEN: scales [..., 1];  QUANT_FP8_STATIC: scales is
    `static_scale` itself;  QUANT_INT8_PER_TENSOR: scales [2] = (scale, scale * weight_scale rounded to x's dtype).
    """
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"quantize: x must be fp16 or bf16, got {x.dtype}")
    if not x.is_contiguous():
        x = x.contiguous()
    K = x.shape[-1]
    M = x.numel() // K if K else 0
    qdtype = torch.int8 if mode == QUANT_INT8_PER_TENSOR else torch.float8_e4m3fn
    dev = _prep(x)
    xq = torch.empty(x.shape, dtype=qdtype, device=dev)
    if mode == QUANT_FP8_STATIC:
        if static_scale is None or static_scale.dtype != torch.float32 or static_scale.numel() != 1:
            raise RuntimeError("quantize: static mode needs a one-element fp32 scale")
        if static_scale.device != dev:
            raise RuntimeError("quantize: scale and x must be on one device")
        scales = static_scale
    elif mode == QUANT_FP8_PER_TOKEN:
        scales = torch.empty((*x.shape[:-1], 1), dtype=torch.float32, device=dev)
    else:
        scales = torch.empty(2 if mode == QUANT_INT8_PER_TENSOR else 1, dtype=torch.float32, device=dev)
    if M == 0:
        return xq, scales
    stream = torch.cuda.current_stream(dev).cuda_stream
    words = _scratch_words(dev, stream)
    check(lib.awq_b200_q8_quantize(x.data_ptr(), 1 if x.dtype == torch.bfloat16 else 0, M, K, mode,
                                   static_scale.data_ptr() if mode == QUANT_FP8_STATIC else None, float(weight_scale),
                                   xq.data_ptr(), None if mode == QUANT_FP8_STATIC else scales.data_ptr(),
                                   words.data_ptr() + 64 * 4, stream), "awq_b200_q8_quantize")
    return xq, scales
