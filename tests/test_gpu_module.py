"""Module API and extension-function API on the GPU, against golden outputs of the
reference module and the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import awq_oracle as orc

pytestmark = pytest.mark.gpu
TOL = 2e-3


def _module(qw, qz, sc, G, bias=None):
    from llmrqt_sdv1_b200 import AWQLinear_GEMM
    K, N = qw.shape[0], qw.shape[1] * 8
    m = AWQLinear_GEMM(4, G, K, N, bias is not None, "cuda")
    sd = {"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": torch.from_numpy(sc)}
    if bias is not None:
        sd["bias"] = torch.from_numpy(bias)
    m.load_state_dict(sd)
    return m


def test_module_matches_reference_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "awq_bias_3d.npz"))
    m = _module(g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]), g["bias"])
    y3 = m(torch.from_numpy(g["x3"]).cuda())
    assert y3.shape == g["y3"].shape and y3.dtype == torch.float16
    assert orc.max_normalised_error(y3.cpu().numpy(), g["y3"]) <= TOL
    xbf = torch.from_numpy(g["xbf_as_f32"]).bfloat16().cuda()
    ybf = m(xbf)                                            # 2-D in -> [1, M, N] out, dtype restored
    assert tuple(ybf.shape) == tuple(g["ybf_shape"]) and ybf.dtype == torch.bfloat16
    assert orc.max_normalised_error(ybf.float().cpu().numpy(), g["ybf_as_f32"]) <= 1e-2   # bf16 output rounding
    assert m(torch.zeros(0, m.in_features, dtype=torch.float16, device="cuda")).shape == tuple(g["y_empty_shape"])
    m.impl_mode = "dequant_matmul"
    y3_ref_mode = m(torch.from_numpy(g["x3"]).cuda())
    assert orc.max_normalised_error(y3_ref_mode.cpu().numpy(), g["y3"]) <= TOL


def test_module_small_golden_and_modes(golden_dir):
    g = np.load(os.path.join(golden_dir, "awq_small.npz"))
    m = _module(g["qweight"], g["qzeros"], g["scales"], int(g["group_size"]))
    y = m(torch.from_numpy(g["x"]).cuda())
    assert y.shape == g["y"].shape
    assert orc.max_normalised_error(y.cpu().numpy(), g["y"]) <= TOL


def test_repack_follows_buffer_replacement():
    """q/k/v fusion replaces the buffers after load (utils/fused_utils.py:88-105): the
    cached kernel layout must follow."""
    K = 256
    a = orc.make_awq_tensors(K, 128, 128, seed=1)
    b = orc.make_awq_tensors(K, 64, 128, seed=2)
    ma, mb = _module(*a, 128), _module(*b, 128)
    x = torch.from_numpy(orc.make_activations(2, K, seed=0)).cuda()
    ya, yb = ma(x), mb(x)
    from llmrqt_sdv1_b200 import AWQLinear_GEMM
    fused = AWQLinear_GEMM(4, 128, K, 192, False, "cuda")
    fused.qweight = torch.cat([ma.qweight, mb.qweight], dim=1)
    fused.qzeros = torch.cat([ma.qzeros, mb.qzeros], dim=1)
    fused.scales = torch.cat([ma.scales, mb.scales], dim=1)
    yf = fused(x)
    assert torch.equal(yf[..., :128], ya) and torch.equal(yf[..., 128:], yb)
    # in-place overwrite (load_state_dict) must invalidate the cache too
    ma.load_state_dict({"qweight": torch.from_numpy(a[0]) ^ 0x11111111, "qzeros": torch.from_numpy(a[1]),
                        "scales": torch.from_numpy(a[2])})
    assert not torch.equal(ma(x), ya)


def test_extension_function_api():
    """The names and argument order the reference module calls (linear_awq.py:74-77,111-114)."""
    import runtime.sq_fp8_kernels as ext
    K, N = 512, 256
    qw, qz, sc = orc.make_awq_tensors(K, N, 128, seed=3)
    dq, dz, ds = (torch.from_numpy(t).cuda() for t in (qw, qz, sc))
    for M, fn in ((1, ext.awq_gemv), (7, lambda *a: ext.awq_gemv_coalesced(*a, 2)),
                  (8, lambda a, b, c, d, g: ext.awq_gemm_db(a, b, c, d, 8)),
                  (100, lambda a, b, c, d, g: ext.awq_gemm(a, b, c, d, 8)),
                  (40, lambda a, b, c, d, g: ext.awq_gemm_cutlass(a, b, c, d, 8))):
        x = orc.make_activations(M, K, seed=M)
        y = fn(torch.from_numpy(x).cuda(), dq, ds, dz, 128)
        assert y.shape == (M, N)
        assert orc.max_normalised_error(y.cpu().numpy(), orc.linear_forward(x, qw, qz, sc, 128)) <= TOL
    # the three non-AWQ names of the extension are real functions too (tests/test_gpu_q8.py covers their results)
    a = torch.zeros(2, 64, device="cuda").to(torch.float8_e4m3fn)
    b = torch.zeros(32, 64, device="cuda").to(torch.float8_e4m3fn)
    assert ext.cutlass_f8f8bf16_tensorwise_sm89(a, b.t(), None, 1.0, 1.0, "bfloat16").shape == (2, 32)
    assert ext.cutlass_f8f8bf16_rowwise_sm89(a, b.t(), None, torch.ones(2, 1, device="cuda"),
                                             torch.ones(1, 32, device="cuda"), True).dtype == torch.bfloat16
    assert ext.w8a8_int8_linear_bbf16_obf16_per_tensor(a.view(torch.int8), b.view(torch.int8).t(),
                                                       torch.zeros(32, device="cuda", dtype=torch.float16), 1.0, 1.0).dtype == torch.float16


def test_load_checkpoint_fills_and_repacks(tmp_path):
    """`checkpoint.load_checkpoint` into CUDA modules: buffers equal the file's tensors, the kernel layout is
    ready before the first forward, and the forward equals that of the module the file was saved from."""
    import os
    from llmrqt_sdv1_b200 import AWQLinear_GEMM, checkpoint, kernels, quantize

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = AWQLinear_GEMM(4, 128, 256, 512, True, "cuda")
            self.b = AWQLinear_GEMM(4, 128, 512, 256, False, "cuda")

        def forward(self, x):
            return self.b(self.a(x))

    src = Block()
    for i, m in enumerate((src.a, src.b)):
        m.qweight, m.qzeros, m.scales = quantize.random_awq_tensors(m.in_features, m.out_features, 128, seed=i, device="cuda")
    src.a.bias = (torch.randn(512, device="cuda") * 0.1).half()
    path = os.path.join(tmp_path, "block.safetensors")
    checkpoint.save_checkpoint(src.state_dict(), path)
    dst = Block()
    report = checkpoint.load_checkpoint(dst, path)
    assert sorted(report["loaded"]) == sorted(src.state_dict()) and not report["missing"]
    for k, v in src.state_dict().items():
        assert torch.equal(dst.state_dict()[k], v), k
    x = torch.randn((1, 5, 256), device="cuda").half()
    assert torch.equal(dst(x), src(x))
    assert kernels.gemv_status() == 0


def test_release_qweight_keeps_one_copy_and_state_dict_round_trips(tmp_path):
    """`release_qweight` frees the on-disk tensor (the module then holds the int4 weights once, in the kernel
    layout), forward results do not change, `state_dict()` still yields the on-disk tensors bit for bit, and a
    checkpoint loaded with `release_qweight=True` into a model built on the meta device ends up the same way."""
    import os
    from llmrqt_sdv1_b200 import AWQLinear_GEMM, checkpoint, kernels, quantize
    K, N = 2048, 4096
    torch.cuda.synchronize()
    base = torch.cuda.memory_allocated()
    m = AWQLinear_GEMM(4, 128, K, N, True, "cuda")
    m.qweight, m.qzeros, m.scales = quantize.random_awq_tensors(K, N, 128, seed=5, device="cuda")
    m.bias = (torch.randn(N, device="cuda") * 0.1).half()
    qweight = m.qweight.clone()
    x1, x9 = torch.randn((1, 1, K), device="cuda").half(), torch.randn((1, 9, K), device="cuda").half()
    y1, y9 = m(x1), m(x9)
    y9_bf16 = m(x9.to(torch.bfloat16))
    sd = {k: v.clone() for k, v in m.state_dict().items()}
    both = torch.cuda.memory_allocated()
    m.release_qweight()
    assert m.qweight.numel() == 0
    torch.cuda.synchronize()
    assert both - torch.cuda.memory_allocated() >= K * N // 2          # the on-disk copy is gone
    assert torch.equal(m(x1), y1) and torch.equal(m(x9), y9)
    assert torch.equal(m(x9.to(torch.bfloat16)), y9_bf16)           # other input dtypes: cast in, cast back
    for k, v in m.state_dict().items():
        assert torch.equal(v, sd[k]), k
    m.impl_mode = "dequant_matmul"                                      # needs the on-disk tensors: they come back
    yd = m(x9)
    assert torch.equal(m.qweight, qweight)
    assert float((yd.float() - y9.float()).abs().max() / y9.float().abs().max()) <= 2e-3
    m.impl_mode = "auto"
    m.release_qweight()
    m.load_state_dict(sd)                                               # loading restores, then overwrites
    assert torch.equal(m.qweight, qweight) and torch.equal(m(x1), y1)

    # a model built without storage, filled straight from the file
    class Block(torch.nn.Module):
        def __init__(self, dev):
            super().__init__()
            self.a = AWQLinear_GEMM(4, 128, K, N, True, dev)

    src = Block("cuda")
    src.a.load_state_dict(sd)
    path = os.path.join(tmp_path, "one.safetensors")
    checkpoint.save_checkpoint(src.state_dict(), path)
    del src, m, sd, qweight
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    dst = Block("meta")
    report = checkpoint.load_checkpoint(dst, path, device="cuda", release_qweight=True)
    assert not report["missing"] and not report["unexpected"]
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated() - before
    packed_bytes = K * N // 2
    extras = (K // 128) * N * 2 + (K // 128) * (N // 8) * 4 + N * 2     # scales, zeros, bias
    assert held <= packed_bytes + extras + (1 << 20), (held, packed_bytes, extras)
    assert dst.a.qweight.numel() == 0 and dst.a.qzeros.is_cuda
    assert torch.equal(dst.a(x1), y1)
    back = dst.state_dict()
    assert back["a.qweight"].shape == (K, N // 8)
    assert kernels.gemv_status() == 0
