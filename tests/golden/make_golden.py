"""Generate the golden fixtures in this directory by running the REFERENCE's own
Python functions (not the oracle, not the product).

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports, unmodified,
  * `dequantize_gemm` (LLMQRT/runtime_refact/utils/packing_utils.py:65-80),
  * `AWQLinear_GEMM` with `from_linear` and `forward(impl_mode="dequant_matmul")`
    (LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:216-398),
  * `AwqQuantizer.pseudo_quantize_tensor`
    (LLMQT/quant/quantization/awq/quantizer.py:99-141),
and stores their inputs and outputs as small .npz files.  The reference needs
`accelerate` and its compiled extension merely to be importable; neither is on
the path exercised here, so empty stand-in modules are registered for them.

Fixtures (all seeded, a few hundred KB in total):
  awq_small.npz      K=256 N=128 G=128, M=3: the full quantise -> pack ->
                     dequantise -> forward chain of the reference.
  awq_bias_3d.npz    K=128 N=64 with bias, x of shape [2, 3, K] and a bf16 case.
  awq_all_pairs.npz  every (q, z) pair with adversarial fp16 scales (subnormal,
                     largest finite, negative, 1e-5 clamp value): pins the
                     single-rounding dequant arithmetic.
  awq_config1_slice.npz  config-1 shaped (K=2048, N=6144, M=1, seed 0) output of
                     the reference forward, plus a checksum of its dequantised
                     weight and a 64-column slice of it.
"""
from __future__ import annotations

import hashlib
import os
import sys
import types

import numpy as np
import torch


def _install_stubs():
    acc = types.ModuleType("accelerate")
    big = types.ModuleType("accelerate.big_modeling")
    acc.big_modeling = big
    for name in ("init_empty_weights", "load_checkpoint_and_dispatch", "infer_auto_device_map",
                 "dispatch_model"):
        setattr(acc, name, lambda *a, **k: None)
        setattr(big, name, lambda *a, **k: None)
    sys.modules.setdefault("accelerate", acc)
    sys.modules.setdefault("accelerate.big_modeling", big)
    rt = types.ModuleType("runtime")
    ext = types.ModuleType("runtime.sq_fp8_kernels")

    def _absent(*a, **k):
        raise NotImplementedError("compiled extension is not part of golden generation")

    for name in ("cutlass_f8f8bf16_tensorwise_sm89", "cutlass_f8f8bf16_rowwise_sm89",
                 "w8a8_int8_linear_bbf16_obf16_per_tensor"):
        setattr(ext, name, _absent)
    rt.sq_fp8_kernels = ext
    sys.modules["runtime"] = rt
    sys.modules["runtime.sq_fp8_kernels"] = ext


def _quantise_with_reference(AwqQuantizer, AWQLinear_GEMM, w: torch.Tensor, G: int, bias=None):
    """Follow AwqQuantizer._apply_quant (quantizer.py:249-297) for one nn.Linear."""
    fake_self = types.SimpleNamespace(group_size=G, zero_point=True, w_bit=4)
    N, K = w.shape
    lin = torch.nn.Linear(K, N, bias=bias is not None).half()
    lin.weight.data = w.clone()
    if bias is not None:
        lin.bias.data = bias.clone()
    w_fake, scales, zeros = AwqQuantizer.pseudo_quantize_tensor(fake_self, lin.weight.data)
    lin.weight.data = w_fake
    scales = scales.t().contiguous()
    zeros = zeros.t().contiguous()
    q = AWQLinear_GEMM.from_linear(linear=lin, w_bit=4, group_size=G, init_only=False,
                                   scales=scales, zeros=zeros)
    return q, w_fake, scales, zeros


def main(ref_root: str):
    import transformers  # noqa: F401  (must be imported before the stand-in modules exist)
    _install_stubs()
    sys.path.insert(0, os.path.join(ref_root, "LLMQRT"))
    sys.path.insert(0, os.path.join(ref_root, "LLMQT"))
    from runtime_refact.utils.packing_utils import dequantize_gemm
    from runtime_refact.nn_models.modules.linear.linear_awq import AWQLinear_GEMM
    import quant.nn_models  # noqa: F401  (the only entry order that avoids the quantizer's import cycle)
    from quant.quantization.awq.quantizer import AwqQuantizer

    out_dir = os.path.dirname(os.path.abspath(__file__))
    torch.set_num_threads(8)

    # ---- awq_small: full chain --------------------------------------------------
    torch.manual_seed(0)
    K, N, G, M = 256, 128, 128, 3
    w = (torch.randn(N, K) * 0.02).half()
    x = torch.randn(M, K).half()
    q, w_fake, scales, zeros = _quantise_with_reference(AwqQuantizer, AWQLinear_GEMM, w, G)
    W = dequantize_gemm(q.qweight, q.qzeros, q.scales, 4, G)
    q.impl_mode = "dequant_matmul"
    y = q(x)
    np.savez_compressed(
        os.path.join(out_dir, "awq_small.npz"),
        w=w.numpy(), x=x.numpy(), w_fake=w_fake.numpy(), scales_kn=scales.numpy(),
        zeros_kn=zeros.numpy().astype(np.float16), qweight=q.qweight.numpy(),
        qzeros=q.qzeros.numpy(), scales=q.scales.numpy(), W=W.numpy(), y=y.numpy(),
        group_size=np.int32(G))

    # ---- awq_bias_3d: module I/O conventions ------------------------------------
    torch.manual_seed(1)
    K, N, G = 128, 64, 128
    w = (torch.randn(N, K) * 0.02).half()
    b = torch.randn(N).half()
    q, *_ = _quantise_with_reference(AwqQuantizer, AWQLinear_GEMM, w, G, bias=b)
    q.impl_mode = "dequant_matmul"
    x3 = torch.randn(2, 3, K).half()
    y3 = q(x3)
    xbf = torch.randn(5, K).bfloat16()
    ybf = q(xbf)                       # 2-D input comes back as [1, 5, N], bf16
    y_empty = q(torch.zeros(0, K).half())
    np.savez_compressed(
        os.path.join(out_dir, "awq_bias_3d.npz"),
        qweight=q.qweight.numpy(), qzeros=q.qzeros.numpy(), scales=q.scales.numpy(),
        bias=q.bias.detach().numpy(), x3=x3.numpy(), y3=y3.numpy(),
        xbf_as_f32=xbf.float().numpy(), ybf_as_f32=ybf.float().numpy(),
        ybf_shape=np.array(ybf.shape), y_empty_shape=np.array(y_empty.shape),
        group_size=np.int32(G))

    # ---- awq_all_pairs: dequant arithmetic --------------------------------------
    # K = 256 (two groups of 128), N = 128.  Row k of group g carries q = k % 16 in
    # every column; column n carries z = n % 16; scales sweep adversarial values.
    K, N, G = 256, 128, 128
    specials = torch.tensor(
        [5.9604645e-08, 6.0975552e-05, 1e-5, 65504.0, -0.0123, 0.33325, -65504.0, 2.0 ** -14,
         1.0, 0.0, -0.0, 3.0517578e-05, 0.1, 1e-3, 7.0, 4366.0], dtype=torch.float32).half()
    torch.manual_seed(2)
    scales = (torch.randn(K // G, N) * 0.01).half()
    scales[0, :16] = specials
    scales[1, 16:32] = specials
    qv = (torch.arange(K)[:, None] % 16).expand(K, N).contiguous()
    qv[128:] = (qv[128:] + torch.arange(N)[None, :] // 16) % 16   # second group: vary with n too
    zv = (torch.arange(N)[None, :] % 16).expand(K // G, N).contiguous()
    order = [0, 2, 4, 6, 1, 3, 5, 7]

    def pack(v):
        o = torch.zeros(v.shape[0], v.shape[1] // 8, dtype=torch.int32)
        for c in range(v.shape[1] // 8):
            for i in range(8):
                o[:, c] |= v[:, c * 8 + order[i]].to(torch.int32) << (4 * i)
        return o

    qweight, qzeros = pack(qv), pack(zv)
    W = dequantize_gemm(qweight, qzeros, scales, 4, G)
    np.savez_compressed(
        os.path.join(out_dir, "awq_all_pairs.npz"),
        qweight=qweight.numpy(), qzeros=qzeros.numpy(), scales=scales.numpy(),
        W_bits=W.numpy().view(np.uint16), q=qv.numpy().astype(np.uint8),
        z=zv.numpy().astype(np.uint8), group_size=np.int32(G))

    # ---- awq_config1_slice: config-1 shape through the reference forward --------
    sys.path.insert(0, os.path.join(os.path.dirname(out_dir), ".."))
    from oracle import awq_oracle as orc   # only as the seeded tensor generator
    K, N, G, M = 2048, 6144, 128, 1
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=0)
    x = orc.make_activations(M, K, seed=0)
    mod = AWQLinear_GEMM(4, G, K, N, False, "cpu")
    mod.qweight, mod.qzeros, mod.scales = (torch.from_numpy(qw), torch.from_numpy(qz),
                                           torch.from_numpy(sc))
    mod.impl_mode = "dequant_matmul"
    y = mod(torch.from_numpy(x))
    W = dequantize_gemm(mod.qweight, mod.qzeros, mod.scales, 4, G).numpy()
    np.savez_compressed(
        os.path.join(out_dir, "awq_config1_slice.npz"),
        y=y.numpy(), W_sha256=np.frombuffer(hashlib.sha256(W.tobytes()).digest(), dtype=np.uint8),
        W_cols_0_64=W[:, :64].copy(), qweight_sha256=np.frombuffer(
            hashlib.sha256(qw.tobytes()).digest(), dtype=np.uint8),
        K=np.int32(K), N=np.int32(N), M=np.int32(M), group_size=np.int32(G), seed=np.int32(0))
    print("golden fixtures written to", out_dir)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
