"""FP8 (e4m3) quantized linears of the reference runtime on sm_100a kernels: same classes, constructor arguments,
parameter names and shapes as LLMQRT/runtime_refact/nn_models/modules/linear/linear_fp8.py:134-454, so the
reference's checkpoints load by name.

What differs is how a forward runs.  The reference quantises the activations with half a dozen torch launches,
reads the product of the two scales back to the host to pass it as a float, and (for 16-bit "legacy" checkpoints)
casts the whole weight to e4m3 on every call.  Here a forward is: one quantisation pass (two launches for the
tensor-wide dynamic scale), one tensor-memory GEMM whose epilogue reads both scales on the device, and the e4m3
weight is cast once and kept.  No host synchronisation, so a decode step can be captured in a CUDA graph.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import q8
from .sq_fp8_kernels import cutlass_f8f8bf16_rowwise_sm89, cutlass_f8f8bf16_tensorwise_sm89

dtype_to_str = {torch.bfloat16: "bfloat16", torch.float16: "float16"}


def per_tensor_quantize(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 tensor, fp32 scale [1]): scale = max|x| / 448 in x's dtype, q = clamp(x / scale) (linear_fp8.py:11-33;
    the reference returns a 0-dim scale, here it has one element)."""
    if tensor.numel() == 0:
        return torch.empty_like(tensor, dtype=torch.float8_e4m3fn), torch.full((1,), 16.0 / 448.0, device=tensor.device)
    return q8.quantize(tensor, q8.QUANT_FP8_PER_TENSOR)


def static_per_tensor_quantize(tensor: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """e4m3 clamp(x / scale) with a given fp32 scale (linear_fp8.py:35-38)."""
    if tensor.numel() == 0:
        return torch.empty_like(tensor, dtype=torch.float8_e4m3fn)
    return q8.quantize(tensor, q8.QUANT_FP8_STATIC, static_scale=scale.detach().reshape(1))[0]


def per_token_quantize(tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(e4m3 tensor, fp32 scales [..., 1]), one scale per row (linear_fp8.py:41-64)."""
    if tensor.numel() == 0:
        return (torch.empty_like(tensor, dtype=torch.float8_e4m3fn),
                torch.ones((*tensor.shape[:-1], 1), dtype=torch.float32, device=tensor.device))
    return q8.quantize(tensor, q8.QUANT_FP8_PER_TOKEN)


def fp8_gemm(A, A_scale, B, B_scale, bias, out_dtype):
    """Dequantise-and-matmul path of the reference (linear_fp8.py:66-104), kept as the module's
    impl_mode="fp8_gemm": torch operations on the device, no custom kernel."""
    if A.numel() == 0:
        return torch.empty(size=(0, B.shape[0]), dtype=out_dtype, device=A.device)
    return torch.nn.functional.linear(A.to(out_dtype) * A_scale.to(out_dtype), B.to(out_dtype) * B_scale.to(out_dtype),
                                      bias=bias)


class _FP8Base(torch.nn.Module):
    """Shared storage: `weight` [out, in] (16-bit legacy or e4m3 native), `weight_scale`, optional `bias`."""

    def _init_common(self, in_features, out_features, bias, dev, dtype, qdtype, per_tensor_weight_scale):
        self.dtype = dtype
        self.qdtype = qdtype
        self.in_features = in_features
        self.out_features = out_features
        self.weight = torch.nn.Parameter(torch.randn((out_features, in_features), dtype=dtype, device=dev),
                                         requires_grad=False)
        shape = (1,) if per_tensor_weight_scale else (out_features, 1)
        self.weight_scale = torch.nn.Parameter(torch.randn(shape, dtype=torch.float32, device=dev), requires_grad=False)
        if bias:
            self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=dev), requires_grad=False)
        else:
            self.bias = None
        self._qcache = None

    def _get_quantized_weight(self) -> torch.Tensor:
        """e4m3 [out, in].  The reference casts on every call (linear_fp8.py:267-268); the cast is kept here and
        redone only when the parameter is replaced or written in place."""
        w = self.weight
        if w.dtype == self.qdtype:
            return w.data
        key = (w.data_ptr(), w._version, w.device)
        if self._qcache is None or self._qcache[0] != key:
            self._qcache = (key, w.data.to(self.qdtype))
        return self._qcache[1]

    def _check_devices(self, x):
        assert x.device == self.weight.device, "when fp8 linear fwd, input and qweight must be same device!"
        assert self.weight_scale.device == self.weight.device, "when fp8 linear fwd, scale and qweight must be same device!"


class FP8DynamicLinear(_FP8Base):
    """Dynamic activation scale, per tensor or per token (linear_fp8.py:134-268)."""

    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True, impl_mode="cutlass"):
        super().__init__()
        assert impl_mode in ["cutlass", "fp8_gemm"], f"impl_mode must be 'cutlass' or 'fp8_gemm', got {impl_mode}"
        self.impl_mode = impl_mode
        self.per_tensor = per_tensor
        self._init_common(in_features, out_features, bias, dev, dtype, qdtype, per_tensor)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit=8, group_size=0, init_only=True, dtype=torch.bfloat16,
                    per_tensor=True, impl_mode="cutlass"):
        assert group_size == 0, "not support group wise fp8 quant yet! pls set group_size = 0"
        layer = cls(in_features=module.in_features, out_features=module.out_features, bias=module.bias is not None,
                    dev=module.weight.device, dtype=dtype, per_tensor=per_tensor, impl_mode=impl_mode)
        if init_only:
            return layer
        # The reference returns None here (linear_fp8.py:189-190): quantising is the offline tool's job.
        return None

    def forward(self, x):
        self._check_devices(x)
        x_shape = x.shape
        out_shape = x.shape[:-1] + (self.out_features,)
        if x.shape[0] == 0:
            return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        qweight = self._get_quantized_weight()
        if self.per_tensor:
            qinput, x_scale = per_tensor_quantize(x)
        else:
            qinput, x_scale = per_token_quantize(x)
        if self.impl_mode == "cutlass":
            qinput = qinput.view(-1, x_shape[-1])
            if self.per_tensor:
                # alpha = weight_scale * x_scale, multiplied on the device by the GEMM's epilogue
                output = q8.gemm_tensorwise(qinput, qweight.t(), self._bias_for(self.dtype), x_scale, 1.0, self.dtype,
                                            alpha2=self.weight_scale.data)
            else:
                output = cutlass_f8f8bf16_rowwise_sm89(qinput, qweight.t(), self.bias, x_scale.view(-1, 1),
                                                       self.weight_scale.data.to(torch.float32).t(), True)
        elif self.impl_mode == "fp8_gemm":
            output = fp8_gemm(A=qinput, A_scale=x_scale if not self.per_tensor else x_scale.reshape(()),
                              B=qweight, B_scale=self.weight_scale.data, bias=self.bias, out_dtype=self.dtype)
        else:
            raise ValueError(f"Unknown impl_mode: {self.impl_mode}")
        return output.view(*x_shape[:-1], -1)

    def _bias_for(self, dtype):
        if self.bias is not None and self.bias.dtype != dtype:
            raise RuntimeError("if bias has value, dtype passed in should same as bias dtype")
        return self.bias


class FP8StaticLinear(_FP8Base):
    """Static (calibrated) per-tensor activation scale, optional fake-quantised output (linear_fp8.py:270-362)."""

    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True, quantize_output=False):
        super().__init__()
        self.per_tensor = per_tensor
        self._init_common(in_features, out_features, bias, dev, dtype, qdtype, True)
        self.input_scale = torch.nn.Parameter(torch.randn(1, dtype=torch.float32, device=dev), requires_grad=False)
        self.quantize_output = quantize_output
        self.output_scale = torch.nn.Parameter(torch.randn(1, dtype=torch.float32, device=dev), requires_grad=False)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit=8, group_size=0, init_only=True, dtype=torch.bfloat16,
                    per_tensor=True, quantize_output=False):
        assert group_size == 0, "not support group wise fp8 quant yet! pls set group_size = 0"
        layer = cls(in_features=module.in_features, out_features=module.out_features, bias=module.bias is not None,
                    dev=module.weight.device, dtype=dtype, per_tensor=True, quantize_output=quantize_output)
        if init_only:
            return layer
        return None

    def forward(self, x):
        self._check_devices(x)
        x_shape = x.shape
        out_shape = x.shape[:-1] + (self.out_features,)
        if x.shape[0] == 0:
            return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        assert self.per_tensor, "[error!!] static activation quant only support per tensor!"
        if self.bias is not None and self.bias.dtype != self.dtype:
            raise RuntimeError("if bias has value, dtype passed in should same as bias dtype")
        qweight = self._get_quantized_weight()
        qinput = static_per_tensor_quantize(x, self.input_scale.data).view(-1, x_shape[-1])
        output = q8.gemm_tensorwise(qinput, qweight.t(), self.bias, self.weight_scale.data, 1.0, self.dtype,
                                    alpha2=self.input_scale.data)
        output = output.view(*x_shape[:-1], -1)
        if self.quantize_output:
            qoutput = static_per_tensor_quantize(output, self.output_scale.data)
            output = qoutput.to(output.dtype) * self.output_scale
        return output


class _NativeWeight:
    """Checkpoint weight already e4m3: no cast, and a weight converted by a global dtype change is refused
    (linear_fp8.py:395-403, :445-453)."""

    def _native_init(self, dev):
        self.weight = torch.nn.Parameter(torch.empty((self.out_features, self.in_features), dtype=self.qdtype, device=dev),
                                         requires_grad=False)

    def _get_quantized_weight(self):
        if self.weight.dtype != self.qdtype:
            raise RuntimeError("Native FP8 checkpoint weight was converted to "
                               f"{self.weight.dtype}; expected {self.qdtype}. "
                               "Load it without a global dtype conversion.")
        return self.weight.data


class FP8NativeDynamicLinear(_NativeWeight, FP8DynamicLinear):
    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True, impl_mode="cutlass"):
        FP8DynamicLinear.__init__(self, in_features, out_features, bias, dev=dev, dtype=dtype, qdtype=qdtype,
                                  per_tensor=per_tensor, impl_mode=impl_mode)
        self._native_init(dev)


class FP8NativeStaticLinear(_NativeWeight, FP8StaticLinear):
    def __init__(self, in_features, out_features, bias, dev="cuda:0", dtype=torch.bfloat16,
                 qdtype=torch.float8_e4m3fn, per_tensor=True, quantize_output=False):
        FP8StaticLinear.__init__(self, in_features, out_features, bias, dev=dev, dtype=dtype, qdtype=qdtype,
                                 per_tensor=per_tensor, quantize_output=quantize_output)
        self._native_init(dev)
