"""Host-side logic of the module mirror (packing, construction, conventions).  CPU only."""
import os

import numpy as np
import pytest
import torch

from llmrqt_sdv1_b200 import AWQLinear_GEMM, WQLinear_GEMM, pack_awq_int4


def test_constructor_buffers():
    m = AWQLinear_GEMM(4, 128, 256, 64, True, "cpu")
    assert m.qweight.shape == (256, 8) and m.qweight.dtype == torch.int32
    assert m.qzeros.shape == (2, 8) and m.scales.shape == (2, 64) and m.scales.dtype == torch.float16
    assert m.bias.shape == (64,) and m.impl_mode == "auto"
    assert set(m.state_dict()) == {"qweight", "qzeros", "scales", "bias"}
    assert AWQLinear_GEMM(4, -1, 256, 64, False, "cpu").group_size == 256
    assert WQLinear_GEMM is AWQLinear_GEMM
    with pytest.raises(NotImplementedError):
        AWQLinear_GEMM(8, 128, 256, 64, False, "cpu")


def test_from_linear_matches_reference_packing(golden_dir):
    g = np.load(os.path.join(golden_dir, "awq_small.npz"))
    G = int(g["group_size"])
    N, K = g["w_fake"].shape
    lin = torch.nn.Linear(K, N, bias=False).half()
    lin.weight.data = torch.from_numpy(g["w_fake"])
    q = AWQLinear_GEMM.from_linear(lin, 4, G, scales=torch.from_numpy(g["scales_kn"]),
                                   zeros=torch.from_numpy(g["zeros_kn"]))
    assert np.array_equal(q.qweight.numpy(), g["qweight"])
    assert np.array_equal(q.qzeros.numpy(), g["qzeros"])
    assert np.array_equal(q.scales.numpy().view(np.uint16), g["scales"].view(np.uint16))


def test_pack_order():
    v = torch.arange(8).reshape(1, 8)
    w = int(pack_awq_int4(v)[0, 0]) & 0xFFFFFFFF
    assert [(w >> (4 * i)) & 0xF for i in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]


def test_empty_batch_and_no_cpu_fallback():
    m = AWQLinear_GEMM(4, 128, 128, 64, False, "cpu")
    assert m(torch.zeros(0, 128, dtype=torch.float16)).shape == (0, 64)
    with pytest.raises(RuntimeError):
        m(torch.zeros(2, 128, dtype=torch.float16))     # CPU tensors: the kernels refuse, nothing falls back
    m.impl_mode = "bogus"
    with pytest.raises(ValueError):
        m(torch.zeros(2, 128, dtype=torch.float16))


def test_torch_quantizer_matches_reference(golden_dir):
    from llmrqt_sdv1_b200.quantize import quantize_weight, rtn_quantize
    g = np.load(os.path.join(golden_dir, "awq_small.npz"))
    G = int(g["group_size"])
    w = torch.from_numpy(g["w"])
    fake, s, z = rtn_quantize(w, G)
    assert np.array_equal(fake.numpy().view(np.uint16), g["w_fake"].view(np.uint16))
    qw, qz, sc = quantize_weight(w, G)
    assert np.array_equal(qw.numpy(), g["qweight"]) and np.array_equal(qz.numpy(), g["qzeros"])
    assert np.array_equal(sc.numpy().view(np.uint16), g["scales"].view(np.uint16))


def test_fused_modules_have_no_cpu_path():
    """The two-launch MLP and the graphed step need the CUDA library's device code: on CPU tensors they
    raise instead of computing something else."""
    from llmrqt_sdv1_b200 import AWQGatedMLP, GraphedStep
    gate, up = AWQLinear_GEMM(4, 128, 128, 128, False, "cpu"), AWQLinear_GEMM(4, 128, 128, 128, False, "cpu")
    down = AWQLinear_GEMM(4, 128, 128, 128, False, "cpu")
    with pytest.raises(RuntimeError):
        AWQGatedMLP(gate, up, down)           # interleaving the columns is a device kernel
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError):
            GraphedStep(lambda x: x, (torch.zeros(4),))
    with pytest.raises(ValueError):
        AWQGatedMLP(gate, AWQLinear_GEMM(4, 128, 128, 64, False, "cpu"), down)


def test_out_tensor_is_validated_before_the_call():
    """`out` is written by the kernel as M x N contiguous fp16 elements: anything else must be refused on the
    host (it would be a stray write on the device).  The checks run before any CUDA call, so CPU tensors show
    them; a well-formed call with CPU tensors then still refuses to compute."""
    from llmrqt_sdv1_b200 import kernels
    K, N = 128, 64
    pw = kernels.PackedWeight(torch.zeros((1, N, 16), dtype=torch.int32), torch.zeros((1, N // 8), dtype=torch.int32),
                              torch.zeros((1, N), dtype=torch.float16), K, N, 128)
    x = torch.zeros((2, K), dtype=torch.float16)
    bad_outs = [torch.zeros((2, N), dtype=torch.float32),                 # wrong dtype
                torch.zeros((2, 2 * N), dtype=torch.float16)[:, ::2],     # strided view
                torch.zeros((1, N), dtype=torch.float16),                 # too short
                torch.zeros((3, N), dtype=torch.float16)]                 # too long
    for out in bad_outs:
        with pytest.raises(ValueError):
            kernels.linear(x, pw, out=out)
        with pytest.raises(ValueError):
            kernels.linear_fused(x, pw, out=out)
        with pytest.raises(ValueError):
            kernels.gemv(x, pw, out=out)
    with pytest.raises(ValueError):
        kernels.linear_fused(x, pw, gated=True, out=torch.zeros((2, N), dtype=torch.float16))   # gated: N / 2 columns
    with pytest.raises(ValueError):
        kernels.linear(x, pw, out_shape=(1, 2, N + 8))
    with pytest.raises(RuntimeError):
        kernels.linear(x, pw, out=torch.zeros((2, N), dtype=torch.float16))


def test_fp8_and_smoothquant_module_surface():
    """Names, shapes and dtypes of the parameters / buffers a reference checkpoint fills
    (LLMQRT/runtime_refact/nn_models/modules/linear/linear_fp8.py:134-454, linear_sq.py:44-147), the quant_method map
    of the reference's linear package, and no CPU fallback."""
    import llmrqt_sdv1_b200 as pkg
    assert sorted(pkg.method_to_linear) == ["awq", "fp8_dynamic_quant", "fp8_native_dynamic_quant",
                                            "fp8_native_static_quant", "fp8_static_quant", "sq"]
    assert pkg.get_concrete_linear_module("awq") is AWQLinear_GEMM
    d = pkg.FP8DynamicLinear(64, 32, True, dev="cpu", dtype=torch.bfloat16, per_tensor=True)
    assert d.weight.shape == (32, 64) and d.weight.dtype == torch.bfloat16 and d.weight_scale.shape == (1,)
    assert d.bias.shape == (32,) and d.bias.dtype == torch.bfloat16
    assert set(d.state_dict()) == {"weight", "weight_scale", "bias"}
    t = pkg.FP8DynamicLinear(64, 32, False, dev="cpu", per_tensor=False)
    assert t.weight_scale.shape == (32, 1) and t.bias is None
    s = pkg.FP8StaticLinear(64, 32, False, dev="cpu")
    assert set(s.state_dict()) == {"weight", "weight_scale", "input_scale", "output_scale"}
    n = pkg.FP8NativeStaticLinear(64, 32, False, dev="cpu")
    assert n.weight.dtype == torch.float8_e4m3fn
    lin = torch.nn.Linear(64, 32, bias=True)
    f = pkg.FP8NativeDynamicLinear.from_linear(lin, init_only=True, dtype=torch.float16, per_tensor=False)
    assert f.weight.dtype == torch.float8_e4m3fn and f.weight_scale.shape == (32, 1) and f.dtype == torch.float16
    with pytest.raises(AssertionError):
        pkg.FP8DynamicLinear.from_linear(lin, group_size=128)
    with pytest.raises(AssertionError):
        pkg.FP8DynamicLinear(64, 32, False, dev="cpu", impl_mode="other")
    q = pkg.SqW8A8BBF16OBF16PerTensor(8, 0, 64, 32, True, dev="cpu", dtype=torch.float16, weight_scale=0.02)
    assert q.qweight.shape == (32, 64) and q.qweight.dtype == torch.int8
    assert set(q.state_dict()) == {"qweight", "bias", "weight_scale", "input_scale"}
    assert abs(float(q.weight_scale) - 0.02) < 1e-8
    for mod in (d, q):
        with pytest.raises(RuntimeError, match="CUDA"):
            mod(torch.zeros(2, 64, dtype=mod.dtype))
