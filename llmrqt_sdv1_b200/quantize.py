"""Round-to-nearest int4 quantisation and packing of an fp16 weight into the
on-disk AWQ tensors, on whole tensors (CPU or CUDA).  Restates the quantizer's
zero-point branch (LLMQT/quant/quantization/awq/quantizer.py:115-125) and the
`from_linear` packer (LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:313-361);
used to build checkpoints-in-memory for tests and benchmarks, where real AWQ
checkpoints are not available."""
from __future__ import annotations

import torch

from .linear_awq import pack_awq_int4


def rtn_quantize(w: torch.Tensor, group_size: int):
    """w fp16 [N, K] -> (w_fake fp16 [N, K], scales fp16 [N, K/G], zeros fp16 [N, K/G]).
    Every op runs on fp16 tensors, as in the reference."""
    assert w.dtype == torch.float16 and w.dim() == 2 and w.shape[1] % group_size == 0
    N, K = w.shape
    g = w.reshape(-1, group_size)
    max_val = g.amax(dim=1, keepdim=True)
    min_val = g.amin(dim=1, keepdim=True)
    scales = (max_val - min_val).clamp(min=1e-5) / 15
    zeros = (-torch.round(min_val / scales)).clamp_(0, 15)
    fake = (torch.clamp(torch.round(g / scales) + zeros, 0, 15) - zeros) * scales
    return fake.reshape(N, K), scales.view(N, -1), zeros.view(N, -1)


def quantize_weight(w: torch.Tensor, group_size: int = 128):
    """w fp16 [N, K] -> (qweight int32 [K, N/8], qzeros int32 [K/G, N/8], scales fp16 [K/G, N])."""
    fake, scales, zeros = rtn_quantize(w, group_size)
    scales = scales.t().contiguous()
    zeros = zeros.t().contiguous()
    scale_zeros = zeros * scales
    codes = torch.round((fake.t() + scale_zeros.repeat_interleave(group_size, dim=0))
                        / scales.repeat_interleave(group_size, dim=0)).to(torch.int32)
    # The reference ORs unmasked codes into the word; a code outside 0..15 would spill into the
    # neighbouring nibble there.  fp16 rounding cannot produce one (|w + z*s| <= 15*s up to half
    # an ulp), and the clamp makes that explicit.
    codes = codes.clamp_(0, 15)
    return pack_awq_int4(codes.contiguous()), pack_awq_int4(zeros.to(torch.int32)), scales.half()


def random_awq_tensors(K: int, N: int, group_size: int = 128, seed: int = 0, std: float = 0.02,
                       device: str | torch.device = "cpu"):
    """Seeded stand-in for a checkpoint tensor triple: W ~ N(0, std) fp16, RTN-quantised."""
    gen = torch.Generator(device=device).manual_seed(seed)
    w = (torch.randn((N, K), generator=gen, device=device, dtype=torch.float32) * std).half()
    return quantize_weight(w, group_size)
