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


def fuse_qkv(q_proj: AWQLinear_GEMM, k_proj: AWQLinear_GEMM, v_proj: AWQLinear_GEMM) -> AWQLinear_GEMM:
    """One `AWQLinear_GEMM` whose output columns are q, k and v side by side: the buffers of the three modules
    concatenated along N, as the reference's `fuse_qkv` does
    (LLMQRT/runtime_refact/utils/fused_utils.py:43-105)."""
    for m in (k_proj, v_proj):
        if (m.in_features, m.group_size, m.bias is None) != (q_proj.in_features, q_proj.group_size, q_proj.bias is None):
            raise ValueError("q/k/v projections must share in_features, group size and the presence of a bias")
    n = q_proj.out_features + k_proj.out_features + v_proj.out_features
    qkv = AWQLinear_GEMM(q_proj.w_bit, q_proj.group_size, q_proj.in_features, n, q_proj.bias is not None,
                         q_proj.qweight.device)
    qkv.qweight = torch.cat([q_proj.qweight, k_proj.qweight, v_proj.qweight], dim=1).contiguous()
    qkv.qzeros = torch.cat([q_proj.qzeros, k_proj.qzeros, v_proj.qzeros], dim=1).contiguous()
    qkv.scales = torch.cat([q_proj.scales, k_proj.scales, v_proj.scales], dim=1).contiguous()
    if q_proj.bias is not None:
        qkv.bias = torch.cat([q_proj.bias, k_proj.bias, v_proj.bias], dim=0)
    qkv.impl_mode = q_proj.impl_mode
    return qkv


class FusedQKVAttention(nn.Module):
    """A Hugging Face Qwen3 / Llama-style attention module with q, k and v computed by ONE quantized linear
    (`qkv_proj`), then sliced - the layout of the reference's fused attention
    (LLMQRT/runtime_refact/nn_models/modules/nonlinear/attention.py:299-309; fuser
    nn_models/models/qwen3.py:97-164).  Per-head q/k RMSNorm, rotary embedding, cache update and the
    attention kernel itself stay Hugging Face's (`q_norm` / `k_norm` may be absent, as in Llama)."""

    def __init__(self, attn: nn.Module):
        super().__init__()
        self.config, self.layer_idx = attn.config, attn.layer_idx
        self.head_dim, self.scaling = attn.head_dim, attn.scaling
        self.num_key_value_groups = attn.num_key_value_groups
        self.attention_dropout, self.is_causal = attn.attention_dropout, True
        self.sliding_window = getattr(attn, "sliding_window", None)
        self.q_size = attn.q_proj.out_features
        self.kv_size = attn.k_proj.out_features
        self.qkv_proj = fuse_qkv(attn.q_proj, attn.k_proj, attn.v_proj)
        self.o_proj = attn.o_proj
        self.q_norm, self.k_norm = getattr(attn, "q_norm", None), getattr(attn, "k_norm", None)

    def forward(self, hidden_states, position_embeddings, attention_mask=None, past_key_values=None, **kwargs):
        from transformers.models.qwen3.modeling_qwen3 import (ALL_ATTENTION_FUNCTIONS, apply_rotary_pos_emb,
                                                               eager_attention_forward)
        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, self.head_dim)
        qkv = self.qkv_proj(hidden_states).view(*input_shape, -1)
        q, k, v = qkv.split((self.q_size, self.kv_size, self.kv_size), dim=-1)
        q, k, v = q.reshape(hidden_shape), k.reshape(hidden_shape), v.reshape(hidden_shape)
        if self.q_norm is not None:
            q = self.q_norm(q)
        if self.k_norm is not None:
            k = self.k_norm(k)
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        cos, sin = position_embeddings
        q, k = apply_rotary_pos_emb(q, k, cos, sin)
        if past_key_values is not None:
            k, v = past_key_values.update(k, v, self.layer_idx)
        interface = ALL_ATTENTION_FUNCTIONS.get_interface(self.config._attn_implementation, eager_attention_forward)
        out, weights = interface(self, q, k, v, attention_mask, dropout=0.0, scaling=self.scaling,
                                 sliding_window=self.sliding_window, **kwargs)
        out = out.reshape(*input_shape, -1).contiguous()
        out = self.o_proj(out)
        return out.view(*input_shape, -1), weights


@torch.no_grad()
def fuse_qkv_(model) -> int:
    """Replace, in place, every decoder layer's attention whose q/k/v projections are `AWQLinear_GEMM`
    modules by a `FusedQKVAttention`.  Returns how many were replaced."""
    replaced = 0
    for layer in decoder_layers(model):
        attn = getattr(layer, "self_attn", None)
        if attn is None or isinstance(attn, FusedQKVAttention):
            continue
        if all(isinstance(getattr(attn, n, None), AWQLinear_GEMM) for n in ("q_proj", "k_proj", "v_proj")):
            layer.self_attn = FusedQKVAttention(attn)
            replaced += 1
    return replaced


def set_impl_mode(model, mode: str) -> None:
    """"auto" = the sm_100a kernels, "dequant_matmul" = materialise the fp16 weight + library matmul."""
    for m in model.modules():
        if isinstance(m, (AWQLinear_GEMM, AWQGatedMLP)):
            m.impl_mode = mode
