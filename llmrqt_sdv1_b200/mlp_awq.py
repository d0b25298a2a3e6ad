"""`AWQGatedMLP`: the gated MLP of a Llama / Qwen decoder layer over AWQ linears, in two launches.

The reference keeps `gate_proj`, `up_proj` and `down_proj` as three `AWQLinear_GEMM` modules inside
Hugging Face's MLP (`down_proj(act_fn(gate_proj(x)) * up_proj(x))`, called from
LLMQRT/runtime_refact/nn_models/modules/nonlinear/transformer_layer.py:139-151 as `h + self.mlp.forward(...)`):
three linear launches and three elementwise ones per layer.  Here gate and up become one weight whose columns
alternate (gate j, up j), so that the first kernel's epilogue applies SiLU(gate) * up, and the second kernel's
epilogue can add the layer's residual.  Every intermediate is rounded to fp16 exactly where the separate fp16
tensor operations round, so the result matches the three-module form up to the last place of exp().

The buffers are regular on-disk-format AWQ tensors (`gate_up_qweight` [K, 2I/8] etc.), built once from the
three source modules; the kernel-layout repack is cached as for `AWQLinear_GEMM`.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .linear_awq import AWQLinear_GEMM, _kernels


class AWQGatedMLP(nn.Module):
    def __init__(self, gate_proj: AWQLinear_GEMM, up_proj: AWQLinear_GEMM, down_proj: AWQLinear_GEMM):
        super().__init__()
        if (gate_proj.in_features, gate_proj.out_features, gate_proj.group_size) != \
                (up_proj.in_features, up_proj.out_features, up_proj.group_size):
            raise ValueError("gate_proj and up_proj must have the same shape and group size")
        if down_proj.in_features != gate_proj.out_features:
            raise ValueError("down_proj must take the intermediate size as input")
        if gate_proj.out_features % 8 != 0:
            raise ValueError("the intermediate size must be a multiple of 8")
        kernels, _ = _kernels()
        self.in_features = gate_proj.in_features
        self.intermediate_size = gate_proj.out_features
        self.group_size = gate_proj.group_size
        self.impl_mode = "auto"       # or "dequant_matmul", as on AWQLinear_GEMM
        self.register_buffer("gate_up_qweight", kernels.interleave_columns(gate_proj.qweight, up_proj.qweight))
        self.register_buffer("gate_up_qzeros", kernels.interleave_columns(gate_proj.qzeros, up_proj.qzeros))
        self.register_buffer("gate_up_scales", torch.stack((gate_proj.scales, up_proj.scales), dim=-1)
                             .reshape(gate_proj.scales.shape[0], -1).contiguous())
        if (gate_proj.bias is None) != (up_proj.bias is None):
            raise ValueError("gate_proj and up_proj must both have a bias or neither")
        if gate_proj.bias is not None:
            self.register_buffer("gate_up_bias", kernels.interleave_bias(gate_proj.bias, up_proj.bias))
        else:
            self.gate_up_bias = None
        self.down_proj = down_proj

    def prepare(self):
        """Repack now instead of on the first forward."""
        _, ext = _kernels()
        ext.packed_for(self.gate_up_qweight, self.gate_up_qzeros, self.gate_up_scales, self.group_size)
        self.down_proj.prepare()
        return self

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """`down_proj(silu(gate_proj(x)) * up_proj(x))`, plus `residual` when given (same shape as the
        result).  Unlike `AWQLinear_GEMM.forward`, the result keeps the rank of `x`."""
        kernels, ext = _kernels()
        down = self.down_proj
        input_dtype = x.dtype
        if input_dtype != torch.float16:
            x = x.to(torch.float16)
            residual = residual.to(torch.float16) if residual is not None else None
        lead = x.shape[:-1]
        if x.numel() == 0:
            out = torch.zeros(lead + (down.out_features,), dtype=torch.float16, device=x.device)
        elif self.impl_mode == "dequant_matmul" or down.impl_mode == "dequant_matmul":
            # explicit reference path: materialised fp16 weights, library matmuls, separate elementwise kernels
            y = torch.matmul(x, kernels.dequantize(self.gate_up_qweight, self.gate_up_qzeros, self.gate_up_scales,
                                                   self.group_size))
            if self.gate_up_bias is not None:
                y = y + self.gate_up_bias
            h = F.silu(y[..., 0::2]) * y[..., 1::2]
            down.restore_qweight()
            out = torch.matmul(h, kernels.dequantize(down.qweight, down.qzeros, down.scales, down.group_size))
            if down.bias is not None:
                out = out + down.bias
            if residual is not None:
                out = residual + out
        else:
            x2 = x.reshape(-1, self.in_features)
            pw_gu = ext.packed_for(self.gate_up_qweight, self.gate_up_qzeros, self.gate_up_scales, self.group_size)
            overlap, pw_gu.fresh = not pw_gu.fresh, False
            h = kernels.linear_fused(x2, pw_gu, bias=self.gate_up_bias, gated=True, overlap=overlap)
            pw_d = down.packed()
            overlap, pw_d.fresh = not pw_d.fresh, False
            out = kernels.linear_fused(h, pw_d, bias=down.bias, residual=residual, overlap=overlap,
                                       out_shape=lead + (down.out_features,))
        return out if input_dtype == torch.float16 else out.to(input_dtype)

    def extra_repr(self) -> str:
        return "in_features={}, intermediate_size={}, group_size={}".format(
            self.in_features, self.intermediate_size, self.group_size)
