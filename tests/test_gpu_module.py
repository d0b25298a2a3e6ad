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
    with pytest.raises(NotImplementedError):
        ext.cutlass_f8f8bf16_rowwise_sm89()


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
