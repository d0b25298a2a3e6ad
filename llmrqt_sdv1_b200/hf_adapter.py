"""Swap the decoder `nn.Linear`s of a Hugging Face causal LM for `AWQLinear_GEMM` modules.

The reference does this in its loader (`_load_quantized_modules`,
LLMQRT/runtime_refact/core/base.py:229-261: every nn.Linear of each decoder layer becomes an
`AWQLinear_GEMM`, `lm_head` stays fp16, core/config.py:16) and then fills the buffers from a
checkpoint.  Real AWQ checkpoints are not available here, so `quantize_model_` derives the tensors
from the model's own (random-init) weights with the reference's round-to-nearest quantiser instead.
Attention, norms and the KV cache stay Hugging Face's (the un-fused path the reference's RAG
client uses, RAG/generation_backends.py:206-213).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .linear_awq import AWQLinear_GEMM
from .mlp_awq import AWQGatedMLP
from .quantize import quantize_weight


def decoder_layers(model) -> nn.ModuleList:
    return model.model.layers


@torch.no_grad()
def quantize_model_(model, group_size: int = 128, skip=("lm_head",)) -> int:
    """Replace, in place, every nn.Linear inside the decoder layers.  Returns how many were replaced."""
    replaced = 0
    for layer in decoder_layers(model):
        for parent in layer.modules():
            for name, child in list(parent.named_children()):
                if not isinstance(child, nn.Linear) or name in skip:
                    continue
                w = child.weight.data.half()
                qweight, qzeros, scales = quantize_weight(w, group_size)
                q = AWQLinear_GEMM(4, group_size, child.in_features, child.out_features, child.bias is not None,
                                   w.device)
                q.qweight, q.qzeros, q.scales = qweight, qzeros, scales
                if child.bias is not None:
                    q.bias = child.bias.data.half().clone()
                setattr(parent, name, q)
                replaced += 1
    return replaced


@torch.no_grad()
def fuse_mlp_(model) -> int:
    """Replace, in place, every decoder layer's gated MLP whose three projections are `AWQLinear_GEMM`
    modules and whose activation is SiLU by an `AWQGatedMLP` (gate and up in one launch with the
    SiLU(gate) * up epilogue).  Call it after the checkpoint tensors are in place.  Returns how many
    were replaced.  The reference's fusers stop at q/k/v (utils/fused_utils.py:43-105) and leave the MLP
    as Hugging Face built it."""
    replaced = 0
    for layer in decoder_layers(model):
        mlp = getattr(layer, "mlp", None)
        projs = [getattr(mlp, n, None) for n in ("gate_proj", "up_proj", "down_proj")]
        act = getattr(mlp, "act_fn", None)
        is_silu = isinstance(act, nn.SiLU) or getattr(act, "__name__", "") == "silu" or \
            type(act).__name__ in ("SiLUActivation", "SiLU")
        if mlp is None or not all(isinstance(p, AWQLinear_GEMM) for p in projs) or not is_silu:
            continue
        layer.mlp = AWQGatedMLP(*projs)
        replaced += 1
    return replaced


def set_impl_mode(model, mode: str) -> None:
    """"auto" = the sm_100a kernels, "dequant_matmul" = materialise the fp16 weight + library matmul."""
    for m in model.modules():
        if isinstance(m, (AWQLinear_GEMM, AWQGatedMLP)):
            m.impl_mode = mode
