"""SmoothQuant W8A8 linear (int8 weights, dynamic per-tensor int8 activations) on sm_100a kernels: same class name,
constructor arguments and buffers as LLMQRT/runtime_refact/nn_models/modules/linear/linear_sq.py:44-147.

A forward is two small launches that quantise the activations (|x| maximum, then scale / round / clamp) and leave
`alpha = input_scale * weight_scale` on the device, and one int8 tensor-memory GEMM whose epilogue reads it.  The
reference reads `weight_scale` back to the host on every call (`.item()`, linear_sq.py:97) and the extension's
float argument forces a second read of alpha; here the weight scale is read once and nothing else synchronises.

The per-channel class of the reference calls an extension function that its bindings do not export
(csrc/bindings.cpp:10-11, commented out) and its package does not list it (linear/__init__.py:9); it has no
counterpart here.
"""
from __future__ import annotations

import torch

from . import q8


@torch.no_grad()
def quantize_activation_per_tensor_absmax(t: torch.Tensor, n_bits: int = 8):
    """(int8 tensor, scale in t's dtype [1]): scale = clamp(max|t|, 1e-5) / 127, q = clamp(round(t / scale))
    (linear_sq.py:19-28; the reference's scale is 0-dim)."""
    assert n_bits == 8, "only 8-bit activations"
    qt, scales = q8.quantize(t, q8.QUANT_INT8_PER_TENSOR)
    return qt, scales[:1].to(t.dtype)


class SqW8A8BBF16OBF16PerTensor(torch.nn.Module):
    def __init__(self, w_bit, group_size, in_features, out_features, bias, dev="cuda:0", dtype=torch.float16,
                 weight_scale=1.0, input_scale=1.0, alpha=1.0, beta=1.0, impl_mode="cutlass"):
        super().__init__()
        self.w_bit = w_bit
        self.group_size = group_size
        self.in_features = in_features
        self.out_features = out_features
        self.dtype = dtype
        assert impl_mode in ["cutlass", "naive"], f"impl_mode must be 'cutlass' or 'naive', got {impl_mode}"
        self.impl_mode = impl_mode
        self.register_buffer("qweight", torch.randint(-127, 127, (out_features, in_features), dtype=torch.int8, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=dtype, device=dev))
        else:
            self.bias = None
        self.register_buffer("weight_scale", torch.tensor(weight_scale, device=dev))
        self.register_buffer("input_scale", torch.tensor(input_scale, device=dev))
        self._ws_host = None
        self._zero_bias = None

    def _weight_scale_host(self) -> float:
        """weight_scale as a host number: read back once per value of the buffer, not once per forward."""
        ws = self.weight_scale
        key = (ws.data_ptr(), ws._version)
        if self._ws_host is None or self._ws_host[0] != key:
            self._ws_host = (key, float(ws.item()))
        return self._ws_host[1]

    @torch.no_grad()
    def forward(self, x):
        assert x.device == self.qweight.device, "when sq linear fwd, input and qweight must be same device!"
        assert self.weight_scale.device == self.qweight.device, "when sq linear fwd, scale and qweight must be same device!"
        assert self.input_scale.device == self.qweight.device, "when sq linear fwd, scale and qweight must be same device!"
        x_shape = x.shape
        x = x.reshape(-1, x_shape[-1])
        if x.shape[0] == 0:
            return torch.zeros((*x_shape[:-1], self.out_features), dtype=x.dtype, device=x.device)
        ws = self._weight_scale_host()
        qx, scales = q8.quantize(x, q8.QUANT_INT8_PER_TENSOR, weight_scale=ws)   # scales = (input scale, alpha)
        if self.impl_mode == "cutlass":
            bias = self.bias
            if bias is None:
                # the reference passes a zero vector in x's dtype (linear_sq.py:107-109): the output takes that dtype
                if self._zero_bias is None or self._zero_bias.dtype != x.dtype or self._zero_bias.device != x.device:
                    self._zero_bias = torch.zeros(self.out_features, dtype=x.dtype, device=x.device)
                bias = self._zero_bias
            y = q8.gemm_tensorwise(qx, self.qweight.t(), bias, scales[1:2], 1.0, bias.dtype, int8=True)
        elif self.impl_mode == "naive":
            # dequantise + matmul (linear_sq.py:111-127); the reference's forward overwrites impl_mode with
            # "cutlass" first (linear_sq.py:99), so this branch is unreachable there
            x_dequant = qx.to(x.dtype).mul(scales[0].to(x.dtype))
            weight_dequant = (self.qweight.to(x.dtype) * ws).t()
            y = torch.matmul(x_dequant, weight_dequant)
            if self.bias is not None:
                y += self.bias.unsqueeze(0)
        else:
            raise ValueError(f"Unknown impl_mode: {self.impl_mode}")
        return y.view(*x_shape[:-1], -1)

    @classmethod
    def from_linear(cls, module: torch.nn.Linear, w_bit, group_size, init_only=True, dtype=torch.float16, per_tensor=True,
                    impl_mode="cutlass"):
        layer = cls(w_bit=w_bit, group_size=group_size, in_features=module.in_features, out_features=module.out_features,
                    bias=module.bias is not None, dev=module.weight.device, dtype=dtype, impl_mode=impl_mode)
        if init_only:
            return layer
        return None
