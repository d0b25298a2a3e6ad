"""`GraphedDecoder`: greedy decoding of a Llama / Qwen3-style causal LM whose decoder linears are this
package's quantized linears, with the WHOLE per-token step - embedding, 28 x {norm, qkv, per-head q/k norm,
rotary embedding, KV-cache write, attention, o (+ residual), norm, MLP (+ residual)}, final norm, lm_head,
argmax - captured once in a CUDA graph and replayed per token.

The step the reference runs per token is `LlamaLikeModel.forward`
(LLMQRT/runtime_refact/nn_models/modules/nonlinear/model.py:33-64) over its fused attention block
(nn_models/modules/nonlinear/attention.py:281-330: qkv_proj -> slices -> q_norm / k_norm -> rope -> cache
update -> attention -> o_proj), driven by Hugging Face's `generate`; at batch 1 that path spends most of a
token's time in Python and in launch gaps between a few hundred small kernels.  Here everything a step
needs lives in static device buffers - the KV cache [layers][1, kv_heads, max_len, head_dim], the position
and the current token as device scalars, rotary tables indexed by the position - so the graph is the same
for every token and the host only replays it.  Attention runs over the whole fixed-length cache under a
mask derived from the position (scaled_dot_product_attention; the reference's attention kernel itself is
outside the quantized-linear path and is not rebuilt).

Works on any module tree with `model.model.{embed_tokens, layers, norm}`, `model.lm_head` and layers with
`input_layernorm`, `self_attn` (either `hf_adapter.FusedQKVAttention` or separate q/k/v projections),
`post_attention_layernorm`, `mlp`.  On CPU tensors (no graph) `forward_tokens` / `step_eager` still run,
which is how the host-side tests check the arithmetic against Hugging Face's own forward.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def _rms(x: torch.Tensor, norm: nn.Module) -> torch.Tensor:
    eps = getattr(norm, "variance_epsilon", None)
    if eps is None:
        eps = getattr(norm, "eps", 1e-6)
    if x.is_cuda and x.dtype == torch.float16 and norm.weight.dtype == torch.float16 and x.is_contiguous():
        from . import kernels
        return kernels.rmsnorm(x, norm.weight, eps)       # one launch (F.rms_norm's arithmetic and rounding)
    return F.rms_norm(x, (x.shape[-1],), norm.weight, eps)


def _call_linear(mod: nn.Module, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """`mod(x) (+ residual)`; the package's quantized modules add the residual in the kernel's epilogue."""
    from .linear_awq import AWQLinear_GEMM
    from .mlp_awq import AWQGatedMLP
    if isinstance(mod, (AWQLinear_GEMM, AWQGatedMLP)):
        return mod(x, residual=residual).view(*x.shape[:-1], -1)
    y = mod(x)
    return y if residual is None else residual + y


class GraphedDecoder:
    def __init__(self, model: nn.Module, max_len: int, capture: bool | None = None, attn_split: bool | None = None):
        """`attn_split`: let the attention launch cut long contexts into chunks of positions, one CTA each (None:
        when `max_len` exceeds 512; a launch with chunk CTAs costs 0.1-0.2 us more at short contexts)."""
        core = model.model
        self.model, self.core = model, core
        self.layers = list(core.layers)
        cfg = model.config
        self.n_heads, self.n_kv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.max_len = int(max_len)
        self._attn_split = (self.max_len > 512) if attn_split is None else bool(attn_split)
        emb = core.embed_tokens.weight
        self.device, self.dtype = emb.device, emb.dtype
        dev = self.device
        L = len(self.layers)
        self.k_cache = torch.zeros((L, 1, self.n_kv, self.max_len, self.head_dim), dtype=self.dtype, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        # rotary tables for every position, from the model's own rotary module
        pos_ids = torch.arange(self.max_len, device=dev).unsqueeze(0)
        with torch.no_grad():
            cos, sin = core.rotary_emb(torch.zeros((1, 1, 1), dtype=self.dtype, device=dev), pos_ids)
        half = self.head_dim // 2
        self.cos_tab = cos[0].to(self.dtype).contiguous()                              # [max_len, head_dim]
        # rotate_half(x) * sin == roll(x, head_dim / 2) * sin_signed with the first half of sin negated
        self.sin_signed_tab = torch.cat((-sin[0, :, :half], sin[0, :, half:]), dim=-1).to(self.dtype).contiguous()
        self.sin_tab = sin[0].to(self.dtype).contiguous()
        # per-head q / k norm weights as one [heads + kv_heads, head_dim] tensor (ones where a model has none)
        self.qk_weights = []
        for layer in self.layers:
            attn = layer.self_attn
            qn, kn = getattr(attn, "q_norm", None), getattr(attn, "k_norm", None)
            if qn is None and kn is None:
                self.qk_weights.append(None)
            else:
                w = torch.cat((qn.weight.expand(self.n_heads, -1), kn.weight.expand(self.n_kv, -1)), dim=0)
                self.qk_weights.append((w.to(self.dtype).contiguous(), getattr(qn, "variance_epsilon", 1e-6)))
        # device-side state of a generation
        self.token = torch.zeros((1, 1), dtype=torch.long, device=dev)
        self.pos = torch.zeros((1,), dtype=torch.long, device=dev)
        self.out_tokens = torch.zeros((1, self.max_len), dtype=torch.long, device=dev)
        self.positions = torch.arange(self.max_len, device=dev)
        self.last_logits = None
        self.graph = None
        self._capture = (dev.type == "cuda") if capture is None else capture
        # On the GPU the step's attention-side plumbing (per-head q/k norm, rotary embedding, cache write, the
        # single-query attention) runs as two small library kernels instead of a dozen tensor operations.
        self._glue = dev.type == "cuda" and self.dtype == torch.float16 and self.head_dim in (64, 128)
        if self._glue:
            self._q_buf = torch.empty((self.n_heads, self.head_dim), dtype=self.dtype, device=dev)
            self._attn_buf = torch.empty((1, 1, self.n_heads * self.head_dim), dtype=self.dtype, device=dev)
            self._qk_norm = []
            for layer in self.layers:
                qn, kn = getattr(layer.self_attn, "q_norm", None), getattr(layer.self_attn, "k_norm", None)
                if qn is None or kn is None:
                    self._qk_norm.append((None, None, 0.0))
                else:
                    self._qk_norm.append((qn.weight.detach().to(self.dtype).contiguous(),
                                          kn.weight.detach().to(self.dtype).contiguous(),
                                          float(getattr(qn, "variance_epsilon", 1e-6))))

    # ------------------------------------------------------------------ pieces of a step
    def _qkv(self, attn, x):
        if hasattr(attn, "qkv_proj"):
            return attn.qkv_proj(x).view(*x.shape[:-1], -1)
        return torch.cat((attn.q_proj(x).view(*x.shape[:-1], -1), attn.k_proj(x).view(*x.shape[:-1], -1),
                          attn.v_proj(x).view(*x.shape[:-1], -1)), dim=-1)

    def _qk_norm_rope(self, li, qkv, cos, sin_signed):
        """qkv [1, S, (H + 2 KV) * D] -> q [1, H, S, D], k [1, KV, S, D], v [1, KV, S, D]; q and k normalised per
        head (where the model has q/k norms) and rotated.  cos / sin_signed: [S, D]."""
        S = qkv.shape[1]
        H, KV, D = self.n_heads, self.n_kv, self.head_dim
        qk = qkv[..., :(H + KV) * D].reshape(1, S, H + KV, D)
        v = qkv[..., (H + KV) * D:].reshape(1, S, KV, D)
        w = self.qk_weights[li]
        if w is not None:
            qk = F.rms_norm(qk, (D,), None, w[1]) * w[0]       # rounds after the normalisation and after the weight
        c, s = cos.unsqueeze(1), sin_signed.unsqueeze(1)        # [S, 1, D]
        qk = torch.addcmul(qk * c, torch.roll(qk, D // 2, dims=-1), s)
        return qk[:, :, :H].transpose(1, 2), qk[:, :, H:].transpose(1, 2), v.transpose(1, 2)

    def _layer_tail(self, layer, h, attn_out):
        attn = layer.self_attn
        h = _call_linear(attn.o_proj, attn_out, residual=h)
        x = _rms(h, layer.post_attention_layernorm)
        from .mlp_awq import AWQGatedMLP
        if isinstance(layer.mlp, AWQGatedMLP):
            return _call_linear(layer.mlp, x, residual=h)
        return h + layer.mlp(x)

    # ------------------------------------------------------------------ whole sequences (prefill, teacher forcing)
    @torch.no_grad()
    def forward_tokens(self, tokens: torch.Tensor, fill_cache: bool = True) -> torch.Tensor:
        """Logits [1, S, vocab] of `tokens` [1, S] processed from position 0 (causal), writing the KV cache."""
        S = tokens.shape[1]
        if S > self.max_len:
            raise ValueError(f"{S} tokens exceed the decoder's max_len {self.max_len}")
        h = self.core.embed_tokens(tokens)
        cos, sin_signed = self.cos_tab[:S], self.sin_signed_tab[:S]
        for li, layer in enumerate(self.layers):
            x = _rms(h, layer.input_layernorm)
            q, k, v = self._qk_norm_rope(li, self._qkv(layer.self_attn, x), cos, sin_signed)
            if fill_cache:
                self.k_cache[li, :, :, :S].copy_(k)
                self.v_cache[li, :, :, :S].copy_(v)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=(self.n_kv != self.n_heads))
            h = self._layer_tail(layer, h, a.transpose(1, 2).reshape(1, S, -1))
        h = _rms(h, self.core.norm)
        return self.model.lm_head(h)

    # ------------------------------------------------------------------ one token
    def _step(self):
        """One decode step on the device-side state: consumes `token` at `pos`, appends the arg-max token."""
        pos = self.pos
        h = self.core.embed_tokens(self.token)                                  # [1, 1, hidden]
        if not self._glue:
            cos, sin_signed = self.cos_tab.index_select(0, pos), self.sin_signed_tab.index_select(0, pos)
            mask = (self.positions <= pos).view(1, 1, 1, self.max_len)          # attend to cache slots 0..pos
        for li, layer in enumerate(self.layers):
            x = _rms(h, layer.input_layernorm)
            qkv = self._qkv(layer.self_attn, x)
            if self._glue:
                from . import kernels
                qw, kw, eps = self._qk_norm[li]
                # q/k norm + rope + cache append + attention of the one new token: one launch
                kernels.attn_step(qkv, qw, kw, eps, self.cos_tab, self.sin_tab, pos, self.k_cache[li], self.v_cache[li],
                                  self._attn_buf,
                                  layer.self_attn.scaling if hasattr(layer.self_attn, "scaling") else self.head_dim ** -0.5,
                                  split=self._attn_split)
                h = self._layer_tail(layer, h, self._attn_buf)
                continue
            q, k, v = self._qk_norm_rope(li, qkv, cos, sin_signed)
            self.k_cache[li].index_copy_(2, pos, k)
            self.v_cache[li].index_copy_(2, pos, v)
            a = F.scaled_dot_product_attention(q, self.k_cache[li], self.v_cache[li], attn_mask=mask,
                                               enable_gqa=(self.n_kv != self.n_heads))
            h = self._layer_tail(layer, h, a.transpose(1, 2).reshape(1, 1, -1))
        h = _rms(h, self.core.norm)
        logits = self.model.lm_head(h)
        nxt = logits.argmax(dim=-1)                                             # [1, 1]
        self.pos.add_(1)
        self.out_tokens.index_copy_(1, self.pos, nxt)
        self.token.copy_(nxt)
        return logits

    @torch.no_grad()
    def step_eager(self) -> torch.Tensor:
        return self._step()

    @torch.no_grad()
    def _ensure_graph(self):
        if self.graph is not None or not self._capture:
            return
        # Warm-up on a side stream (workspaces are per stream; the first call after a repack must not be captured),
        # on a copy of the state so that the generation in progress is not disturbed.
        saved = (self.token.clone(), self.pos.clone(), self.out_tokens.clone())
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(3):
                self.pos.fill_(min(8, self.max_len - 2))
                self._step()
            side.synchronize()
            self.pos.fill_(min(8, self.max_len - 2))
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self._graph_logits = self._step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._side = side
        self.token.copy_(saved[0]); self.pos.copy_(saved[1]); self.out_tokens.copy_(saved[2])

    # ------------------------------------------------------------------ generation
    @torch.no_grad()
    def prefill(self, prompt: torch.Tensor) -> torch.Tensor:
        """Process the prompt [1, S]; leaves the first generated token in the device-side state."""
        S = prompt.shape[1]
        logits = self.forward_tokens(prompt)
        nxt = logits[:, -1:].argmax(dim=-1)
        self.out_tokens[:, :S].copy_(prompt)
        self.out_tokens[:, S:S + 1].copy_(nxt)
        self.token.copy_(nxt)
        self.pos.fill_(S)
        return logits

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy decoding: returns [1, S + new_tokens] (prompt followed by the generated tokens)."""
        S = prompt.shape[1]
        if S + new_tokens + 1 > self.max_len:
            raise ValueError("prompt + new tokens exceed the decoder's max_len")
        self._ensure_graph()
        self.prefill(prompt)
        for _ in range(new_tokens - 1):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._step()
        return self.out_tokens[:, :S + new_tokens].clone()

    # ------------------------------------------------------------------ measurements used by the benchmark
    @torch.no_grad()
    def time_step_at(self, position: int, iters: int = 20) -> float:
        """ms per token of the decode step with `position` tokens in the cache (whatever the cache holds): device
        time of the captured step alone, the position put back before every replay.  The generation state (token,
        position, output tokens) is restored afterwards; cache row `position` is overwritten."""
        if not 0 <= position < self.max_len - 1:
            raise ValueError(f"position {position} outside the decoder's cache of {self.max_len}")
        self._ensure_graph()
        saved = (self.token.clone(), self.pos.clone(), self.out_tokens.clone())
        run = self.graph.replay if self.graph is not None else self._step
        total = 0.0
        for it in range(iters + 3):
            self.pos.fill_(position)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            run()
            b.record()
            b.synchronize()
            if it >= 3:
                total += a.elapsed_time(b)
        self.token.copy_(saved[0]); self.pos.copy_(saved[1]); self.out_tokens.copy_(saved[2])
        return total / iters

    @torch.no_grad()
    def teacher_forced_error(self, seq: torch.Tensor, logits_ref: torch.Tensor) -> float:
        """max |logits - logits_ref| / max |logits_ref| with `seq` fed as it is (no cache effects)."""
        mine = self.forward_tokens(seq, fill_cache=False).float()
        return float((mine - logits_ref.float()).abs().max() / logits_ref.float().abs().max())

    @torch.no_grad()
    def time_linears_only(self, iters: int = 20) -> float:
        """ms per token spent in the layers' linears alone: the same calls as a step makes (qkv, o + residual,
        MLP per layer) on fixed inputs, captured in a CUDA graph and replayed."""
        from .graph import GraphedStep
        from .mlp_awq import AWQGatedMLP
        hidden = self.core.embed_tokens.weight.shape[1]
        x = torch.randn((1, 1, hidden), device=self.device).to(self.dtype)
        a = torch.randn((1, 1, self.n_heads * self.head_dim), device=self.device).to(self.dtype)

        def chain(x_, a_):
            y = None
            for layer in self.layers:
                self._qkv(layer.self_attn, x_)
                _call_linear(layer.self_attn.o_proj, a_, residual=x_)
                mlp = layer.mlp
                if isinstance(mlp, AWQGatedMLP):
                    y = _call_linear(mlp, x_, residual=x_)
                else:
                    y = mlp(x_)
            return y
        gs = GraphedStep(chain, (x, a))
        gs.replay()
        torch.cuda.synchronize(self.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            gs.replay()
        e1.record()
        torch.cuda.synchronize(self.device)
        return e0.elapsed_time(e1) / iters
