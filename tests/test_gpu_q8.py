"""8-bit quantized linears on the GPU against the CPU oracle (oracle/q8_oracle.c), through the C ABI:
INT8 bit-exact; FP8 within one output rounding step plus the fp32 accumulation bound; quantisers bit-exact, and
bit-exact against the reference's torch expressions run on the same GPU."""
import os

import numpy as np
import pytest
import torch

from oracle import q8_oracle as q8o

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def q8():
    from llmrqt_sdv1_b200 import q8 as mod
    return mod


def _bits(t):
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    return t.contiguous().view(torch.uint8).cpu().numpy()


def _f32(bits, bf16):
    return q8o.bf16_bits_to_f32(bits) if bf16 else bits.view(np.float16).astype(np.float32)


def _step(v, bf16):
    e = np.floor(np.log2(np.maximum(np.abs(v), 2.0 ** -14 if not bf16 else 2.0 ** -126)))
    return np.exp2(e - (7 if bf16 else 10))


def _rand_fp8(shape, seed, scale=1.0, dtype=torch.float8_e4m3fn):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ---------------------------------------------------------------------------------------------------------------
# INT8: exact
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (3, 300, 528), (32, 512, 1024), (33, 256, 128), (128, 1024, 512),
                                   (200, 777 + 7, 1040), (257, 512, 4096), (16, 128, 16), (64, 8192, 2048)])
@pytest.mark.parametrize("out_bf16", [False, True])
def test_int8_bit_exact(q8, M, N, K, out_bf16):
    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    dt = torch.bfloat16 if out_bf16 else torch.float16
    bias = torch.randn(N, generator=g).to(dt)
    alpha, beta = 3.1e-5, 1.0
    y = q8.gemm_tensorwise(x.cuda(), w.cuda().t(), bias.cuda(), alpha, beta, dt, int8=True)
    want = q8o.tensorwise(x.numpy(), w.numpy(), (_bits(bias), "bf16") if out_bf16 else bias.numpy(), alpha, beta,
                          out_bf16, kind=q8o.KIND_INT8)
    assert y.shape == (M, N) and y.dtype == dt
    assert np.array_equal(_bits(y), want)
    assert q8.status() == 0


def test_int8_golden_fixture(q8):
    g = np.load(os.path.join(GOLD, "q8_int8_gemm.npz"))
    x, w, bias = torch.from_numpy(g["x"]), torch.from_numpy(g["w"]), torch.from_numpy(g["bias"])
    from llmrqt_sdv1_b200 import sq_fp8_kernels as ext
    y = ext.w8a8_int8_linear_bbf16_obf16_per_tensor(x.cuda(), w.cuda().t(), bias.cuda(), float(g["alpha"][0]), 1.0)
    assert y.dtype == torch.float16
    want = q8o.tensorwise(g["x"], g["w"], g["bias"], float(g["alpha"][0]), 1.0, False, kind=q8o.KIND_INT8)
    assert np.array_equal(_bits(y), want)
    # the reference's unit test (unittest/test_sq_linear.py:37)
    assert torch.allclose(torch.from_numpy(g["y_fp16_linear"]), y.cpu(), atol=0.1)


def test_int8_extremes_and_device_alpha(q8):
    """All -128 x -128 (the largest products), K = 8192: the int32 sum 2^14 * 8192 = 2^27 is exact; alpha on the device."""
    M, N, K = 4, 256, 8192
    x = torch.full((M, K), -128, dtype=torch.int8)
    w = torch.full((N, K), -128, dtype=torch.int8)
    w[1::2] = 127
    bias = torch.zeros(N, dtype=torch.float16)
    a1 = torch.tensor([2.0 ** -20], device="cuda")
    a2 = torch.tensor([0.75], device="cuda")
    y = q8.gemm_tensorwise(x.cuda(), w.cuda().t(), bias.cuda(), a1, 1.0, torch.float16, alpha2=a2, int8=True)
    want = q8o.tensorwise(x.numpy(), w.numpy(), bias.numpy(), 0.75 * 2.0 ** -20, 1.0, False, kind=q8o.KIND_INT8)
    assert np.array_equal(_bits(y), want)


@pytest.mark.parametrize("M,N,K", [(1, 8192, 8192), (4, 1024, 28672), (32, 2048, 4096), (48, 4096, 8192), (128, 2048, 8192)])
def test_k_split_is_exact_for_int8_and_repeatable(q8, M, N, K):
    """Few rows: K is split over the CTAs of a cluster, which add the 32-bit partial sums over distributed shared
    memory.  INT8: the same bits as without the split and as the oracle.  FP8: the same bits on every call (the
    order of the additions is fixed), within the accumulation bound of the unsplit result."""
    from llmrqt_sdv1_b200._lib import lib
    assert lib.awq_b200_q8_splits(M, N, K) > 1                       # these shapes do split
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8).cuda()
    bias = torch.randn(N, generator=g).half().cuda()
    y0 = q8.gemm_tensorwise(x, w.t(), bias, 2e-5, 1.0, torch.float16, int8=True, split=False)
    y1 = q8.gemm_tensorwise(x, w.t(), bias, 2e-5, 1.0, torch.float16, int8=True)
    y2 = q8.gemm_tensorwise(x, w.t(), bias, 2e-5, 1.0, torch.float16, int8=True)
    assert torch.equal(y0, y1) and torch.equal(y1, y2)
    rows = slice(0, min(M, 4))
    want = q8o.tensorwise(x[rows].cpu().numpy(), w[:512].cpu().numpy(), bias[:512].cpu().numpy(), 2e-5, 1.0, False,
                          kind=q8o.KIND_INT8)
    assert np.array_equal(_bits(y1[rows, :512]), want)
    a = _rand_fp8((M, K), 3).cuda()
    b = _rand_fp8((N, K), 4).cuda()
    f0 = q8.gemm_tensorwise(a, b.t(), None, 1.0, 0.0, torch.bfloat16, split=False)
    f1 = q8.gemm_tensorwise(a, b.t(), None, 1.0, 0.0, torch.bfloat16)
    f2 = q8.gemm_tensorwise(a, b.t(), None, 1.0, 0.0, torch.bfloat16)
    assert torch.equal(f1, f2)
    want = q8o.tensorwise(_bits(a[rows]), _bits(b[:512]), None, 1.0, 0.0, True)
    slack = 2e-6 * q8o.gemm_abs(_bits(a[rows]), _bits(b[:512]), q8o.KIND_E4M3)
    _check_fp8(_bits(f1[rows, :512]), want, True, slack)
    _check_fp8(_bits(f0[rows, :512]), want, True, slack)
    assert q8.status() == 0


def test_pitched_operands(q8):
    """Row pitches larger than K (views into wider buffers), as the reference's checks allow (stride >= K)."""
    M, N, K, LD = 37, 320, 256, 384
    g = torch.Generator().manual_seed(5)
    xb = torch.randint(-128, 128, (M, LD), generator=g, dtype=torch.int8).cuda()
    wb = torch.randint(-128, 128, (N, LD), generator=g, dtype=torch.int8).cuda()
    x, w = xb[:, :K], wb[:, :K]
    bias = torch.randn(N, generator=g).half()
    y = q8.gemm_tensorwise(x, w.t(), bias.cuda(), 1e-4, 1.0, torch.float16, int8=True)
    want = q8o.tensorwise(x.cpu().numpy().copy(), w.cpu().numpy().copy(), bias.numpy(), 1e-4, 1.0, False, kind=q8o.KIND_INT8)
    assert np.array_equal(_bits(y), want)


# ---------------------------------------------------------------------------------------------------------------
# FP8
# ---------------------------------------------------------------------------------------------------------------
def _check_fp8(got_bits, want_bits, bf16, slack):
    got, want = _f32(got_bits, bf16), _f32(want_bits, bf16)
    assert not np.isnan(got).any()
    err = np.abs(got - want)
    assert np.all(err <= _step(want, bf16) + slack), float(np.max(err - _step(want, bf16) - slack))
    return float(np.mean(got != want))


@pytest.mark.parametrize("M,N,K", [(1, 256, 256), (5, 384, 272), (32, 512, 1024), (100, 768, 512), (128, 512, 256),
                                   (300, 1000, 2048), (64, 4096, 4096)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_fp8_tensorwise(q8, M, N, K, dt):
    a = _rand_fp8((M, K), M + K)
    b = _rand_fp8((N, K), N + K + 1)
    g = torch.Generator().manual_seed(3)
    bias = torch.randn(N, generator=g).to(dt)
    alpha, beta = 0.6, 1.0
    from llmrqt_sdv1_b200 import sq_fp8_kernels as ext
    y = ext.cutlass_f8f8bf16_tensorwise_sm89(a.cuda(), b.cuda().t(), bias.cuda(), alpha, beta,
                                             "bfloat16" if dt == torch.bfloat16 else "float16")
    bf = dt == torch.bfloat16
    want = q8o.tensorwise(_bits(a), _bits(b), (_bits(bias), "bf16") if bf else bias.numpy(), alpha, beta, bf)
    # fp32 accumulation of K exact products: error <= K * 2^-24 * sum|x||w| in the worst case; 2e-6 * sum covers the
    # tensor core's accumulation at these K with a wide margin and is ~1e-3 of one output step
    slack = 2e-6 * alpha * q8o.gemm_abs(_bits(a), _bits(b), q8o.KIND_E4M3)
    frac = _check_fp8(_bits(y), want, bf, slack)
    assert frac < 0.02, frac          # all but a few results are the correctly rounded ones
    assert q8.status() == 0


def test_fp8_golden_fixture_and_unit_test_tolerance(q8):
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    a = torch.from_numpy(g["a"]).view(torch.float8_e4m3fn).cuda()
    b = torch.from_numpy(g["b"]).view(torch.float8_e4m3fn).cuda()
    bias = torch.from_numpy(g["bias"].view(np.int16)).view(torch.bfloat16).cuda()
    from llmrqt_sdv1_b200 import sq_fp8_kernels as ext
    y = ext.cutlass_f8f8bf16_tensorwise_sm89(a, b.t(), bias, float(g["alpha"][0]), 1, "bfloat16")
    ref = torch.from_numpy(g["scaled_mm_bias"].view(np.int16)).view(torch.bfloat16)
    assert torch.allclose(y.cpu(), ref, atol=0.25)            # unittest/test_fp8_tensorwise_linear.py:54
    got, want = q8o.bf16_bits_to_f32(_bits(y)), q8o.bf16_bits_to_f32(g["scaled_mm_bias"])
    # what it actually is: the comparator rounds to bf16 before adding the bias, the kernel once, after
    assert np.all(np.abs(got - want) <= 2 * _step(np.maximum(np.abs(want), np.abs(want - q8o.bf16_bits_to_f32(g["bias"]))), True))
    # no bias (std::optional), rowwise
    sa = torch.from_numpy(g["row_sa"]).cuda()
    sb = torch.from_numpy(g["row_sb"]).cuda()
    y2 = ext.cutlass_f8f8bf16_rowwise_sm89(a, b.t(), None, sa, sb, True)
    got2 = q8o.bf16_bits_to_f32(_bits(y2))
    assert np.all(np.abs(got2 - g["row_f64"]) <= 0.51 * _step(g["row_f64"], True) + 2e-6 * np.abs(g["row_f64"]) + 1e-5)


@pytest.mark.parametrize("M,N,K,x_dtype,bias_dt", [(7, 256, 512, torch.float8_e4m3fn, None),
                                                   (64, 640, 1024, torch.float8_e4m3fn, torch.bfloat16),
                                                   (129, 512, 768, torch.float8_e5m2, torch.float32),
                                                   (32, 2048, 4096, torch.float8_e4m3fn, torch.float32)])
def test_fp8_rowwise(q8, M, N, K, x_dtype, bias_dt):
    a = _rand_fp8((M, K), 11 + M, dtype=x_dtype)
    b = _rand_fp8((N, K), 13 + N)
    g = torch.Generator().manual_seed(9)
    sa = torch.rand(M, 1, generator=g) + 0.1
    sb = torch.rand(1, N, generator=g) + 0.1
    bias = None if bias_dt is None else torch.randn(N, generator=g).to(bias_dt)
    y = q8.gemm_rowwise(a.cuda(), b.cuda().t(), None if bias is None else bias.cuda(), sa.cuda(), sb.cuda())
    kind = q8o.KIND_X_E5M2 if x_dtype == torch.float8_e5m2 else q8o.KIND_E4M3
    ob = None if bias is None else ((_bits(bias), "bf16") if bias_dt == torch.bfloat16 else bias.numpy())
    want = q8o.rowwise(_bits(a), _bits(b), ob, sa.numpy(), sb.numpy(), kind=kind)
    slack = 2e-6 * q8o.gemm_abs(_bits(a), _bits(b), kind) * sa.numpy() * sb.numpy()
    frac = _check_fp8(_bits(y), want, True, slack)
    assert frac < 0.02, frac


def test_fp8_linearity_at_full_size(q8):
    """Size-independent property at a full-size layer (8192 x 8192 weights, 4096 rows): doubling the activations
    (exact in e4m3 below the top binade) doubles every output exactly; and a sampled block matches the oracle."""
    M, N, K = 4096, 8192, 8192
    a = _rand_fp8((M, K), 21, scale=0.5).cuda()
    b = _rand_fp8((N, K), 22).cuda()
    a2 = (a.float() * 2).to(torch.float8_e4m3fn)
    assert torch.equal(a2.float(), a.float() * 2)
    y1 = q8.gemm_tensorwise(a, b.t(), None, 1.0, 0.0, torch.bfloat16)
    y2 = q8.gemm_tensorwise(a2, b.t(), None, 1.0, 0.0, torch.bfloat16)
    assert torch.equal(y2.float(), y1.float() * 2)
    rows, cols = slice(1000, 1016), slice(4000, 4128)
    want = q8o.tensorwise(_bits(a[rows]), _bits(b[cols]), None, 1.0, 0.0, True)
    slack = 2e-6 * q8o.gemm_abs(_bits(a[rows]), _bits(b[cols]), q8o.KIND_E4M3)
    _check_fp8(_bits(y1[rows, cols]), want, True, slack)
    assert q8.status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 57344, 8192), (16, 8192, 28672), (4096, 8192, 8192), (2048, 8192, 28672)])
def test_full_size_against_library_gemms_on_the_gpu(q8, M, N, K):
    """70B-class layers at full size, where the CPU oracle would take minutes: INT8 against the exact int32 product
    of the library (bit for bit: the scale is a power of two), FP8 against the library's FP8 GEMM within one output
    step plus the two kernels' accumulation bound."""
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    xi = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8, device="cuda")
    wi = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8, device="cuda")
    zero = torch.zeros(N, dtype=torch.float16, device="cuda")
    y = q8.gemm_tensorwise(xi, wi.t(), zero, 2.0 ** -18, 1.0, torch.float16, int8=True)
    rows = xi if M > 16 else torch.cat([xi, torch.zeros((32 - M, K), dtype=torch.int8, device="cuda")])
    acc = torch._int_mm(rows, wi.t())[:M]                       # int32, exact
    assert torch.equal(y, (acc.float() * 2.0 ** -18).half())
    xf = (torch.randn((M, K), generator=g, device="cuda") * 0.5).to(torch.float8_e4m3fn)
    wf = (torch.randn((N, K), generator=g, device="cuda") * 0.5).to(torch.float8_e4m3fn)
    yf = q8.gemm_tensorwise(xf, wf.t(), None, 1.0, 0.0, torch.bfloat16)
    one = torch.tensor(1.0, device="cuda")
    rowsf = xf if M >= 16 else torch.cat([xf, torch.zeros((16 - M, K), device="cuda").to(torch.float8_e4m3fn)])
    ref = torch._scaled_mm(rowsf, wf.t(), scale_a=one, scale_b=one, out_dtype=torch.float32)[:M]
    err = (yf.float() - ref).abs()
    # one bf16 step of the reference value + both kernels' fp32 accumulation noise (K products of magnitude <= ~1)
    bound = ref.abs().clamp_min(2.0 ** -126).log2().floor().exp2() * 2.0 ** -7 + 4e-6 * K ** 0.5 * 8
    assert bool((err <= bound).all()), float((err - bound).max())
    assert q8.status() == 0


# ---------------------------------------------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------------------------------------------
def _ref_per_tensor(t):
    finfo = torch.finfo(torch.float8_e4m3fn)
    mn, mx = t.aminmax()
    amax = torch.maximum(mn.abs(), mx.abs())
    scale = amax.clamp(min=1e-12) / finfo.max
    q = (t / scale).clamp(min=finfo.min, max=finfo.max).to(torch.float8_e4m3fn)
    return q, scale.float()


def _ref_per_token(t):
    finfo = torch.finfo(torch.float8_e4m3fn)
    amax = t.abs().amax(dim=-1, keepdim=True)
    scale = amax.clamp(min=1e-12) / finfo.max
    q = (t / scale).clamp(min=finfo.min, max=finfo.max).to(torch.float8_e4m3fn)
    return q, scale.float()


def _ref_sq(t):
    scales = t.abs().max()
    scales.clamp_(min=1e-5).div_(127)
    qt = t.div(scales).round().clamp(-128, 127).to(torch.int8)
    return qt, scales


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1, 64), (5, 4096), (3, 7, 256), (300, 1024)])
def test_quantisers_match_torch_on_gpu_and_oracle(q8, dt, shape):
    """The reference's expressions (linear_fp8.py:11-64, linear_sq.py:19-28), restated above, run with torch on
    the same GPU, must give the same bytes and scales as the fused kernels, and so must the oracle."""
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(shape, generator=g) * torch.rand(shape[:-1] + (1,), generator=g) * 8).to(dt).cuda()
    bf = dt == torch.bfloat16
    x2 = _bits(x).reshape(-1, shape[-1])

    q, s = q8.quantize(x, q8.QUANT_FP8_PER_TENSOR)
    rq, rs = _ref_per_tensor(x)
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8)) and float(s[0]) == float(rs)
    oq, os_ = q8o.quantize(x2, bf, q8o.QUANT_FP8_PER_TENSOR)
    assert np.array_equal(_bits(q).reshape(oq.shape), oq) and os_[0] == float(s[0])

    q, s = q8.quantize(x, q8.QUANT_FP8_PER_TOKEN)
    rq, rs = _ref_per_token(x)
    assert s.shape == rs.shape
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8)) and torch.equal(s, rs)
    oq, os_ = q8o.quantize(x2, bf, q8o.QUANT_FP8_PER_TOKEN)
    assert np.array_equal(_bits(q).reshape(oq.shape), oq) and np.array_equal(os_, s.cpu().numpy().ravel())

    sc = torch.tensor([0.0213], device="cuda")
    q, _ = q8.quantize(x, q8.QUANT_FP8_STATIC, static_scale=sc)
    rq = (x / sc).clamp(min=-448, max=448).to(torch.float8_e4m3fn)
    assert torch.equal(q.view(torch.uint8), rq.view(torch.uint8))
    oq, _ = q8o.quantize(x2, bf, q8o.QUANT_FP8_STATIC, static_scale=0.0213)
    assert np.array_equal(_bits(q).reshape(oq.shape), oq)

    q, s = q8.quantize(x, q8.QUANT_INT8_PER_TENSOR, weight_scale=0.0123)
    rq, rs = _ref_sq(x.clone())
    assert torch.equal(q, rq) and float(s[0]) == float(rs)
    assert float(s[1]) == float(rs * 0.0123)
    oq, os_ = q8o.quantize(x2, bf, q8o.QUANT_INT8_PER_TENSOR, weight_scale=0.0123)
    assert np.array_equal(q.cpu().numpy().view(np.uint8).reshape(oq.shape), oq) and np.array_equal(os_, s.cpu().numpy())


def test_quantiser_golden_fixture(q8):
    g = np.load(os.path.join(GOLD, "q8_quant.npz"))
    for tag, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        x = torch.from_numpy(g[f"x_{tag}"].view(np.int16)).view(dt).cuda()
        q, s = q8.quantize(x, q8.QUANT_FP8_PER_TOKEN)
        # made on a CPU (true division by 448); the two rules agree on this fixture's values
        assert np.array_equal(_bits(q), g[f"tok_q_{tag}"]) and np.array_equal(s.cpu().numpy().ravel(), g[f"tok_s_{tag}"])
        q, s = q8.quantize(x, q8.QUANT_INT8_PER_TENSOR, weight_scale=float(g["sq_weight_scale"][0]))
        assert np.array_equal(_bits(q), g[f"sq_q_{tag}"]) and float(s[1]) == float(g[f"sq_alpha_{tag}"][0])
        q, _ = q8.quantize(x, q8.QUANT_FP8_STATIC, static_scale=torch.from_numpy(g["static_scale"]).cuda())
        assert np.array_equal(_bits(q), g[f"st_q_{tag}"])


# ---------------------------------------------------------------------------------------------------------------
# modules
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("per_tensor", [True, False])
def test_fp8_dynamic_linear_module(per_tensor):
    from llmrqt_sdv1_b200.linear_fp8 import FP8DynamicLinear, FP8NativeDynamicLinear
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    kind = "tensor" if per_tensor else "token"
    b = torch.from_numpy(g["b"]).view(torch.float8_e4m3fn)
    bias = torch.from_numpy(g["bias"].view(np.int16)).view(torch.bfloat16)
    x = torch.from_numpy(g["mod_x"].view(np.int16)).view(torch.bfloat16).cuda()
    ws = torch.from_numpy(g[f"mod_ws_{kind}"])
    outs = []
    for cls in (FP8DynamicLinear, FP8NativeDynamicLinear):
        m = cls(256, 512, True, dev="cuda", dtype=torch.bfloat16, per_tensor=per_tensor)
        m.weight.data = b.cuda() if cls is FP8NativeDynamicLinear else b.to(torch.bfloat16).cuda()
        m.weight_scale.data = ws.cuda()
        m.bias.data = bias.cuda()
        y = m(x)
        assert y.shape == (2, 8, 512) and y.dtype == torch.bfloat16
        outs.append(y)
        # against the reference's own forward in its dequantise-and-matmul mode (CPU fixture): bf16 matmul there
        want = torch.from_numpy(g[f"mod_y_{kind}"].view(np.int16)).view(torch.bfloat16).float()
        err = (y.cpu().float() - want).abs().max() / want.abs().max()
        assert err < 2e-2, float(err)
        # against the oracle chain: quantise -> GEMM
        xq, s = q8o.quantize(_bits(x).reshape(-1, 256), True,
                             q8o.QUANT_FP8_PER_TENSOR if per_tensor else q8o.QUANT_FP8_PER_TOKEN)
        if per_tensor:
            o = q8o.tensorwise(xq, g["b"], (g["bias"], "bf16"), float(np.float32(ws[0]) * np.float32(s[0])), 1.0, True)
        else:
            o = q8o.rowwise(xq, g["b"], (g["bias"], "bf16"), s, ws.numpy().ravel())
        scale_bound = (float(ws.max()) * float(s.max())) * 2e-6 * q8o.gemm_abs(xq, g["b"], q8o.KIND_E4M3)
        _check_fp8(_bits(y).reshape(o.shape), o, True, scale_bound)
        # fp8_gemm mode is plain torch on the device
        m.impl_mode = "fp8_gemm"
        y3 = m(x)
        assert (y3.float() - y.float()).abs().max() / y.float().abs().max() < 2e-2
    assert torch.equal(outs[0], outs[1])                         # legacy (cast once) and native weights agree


def test_fp8_static_linear_module():
    from llmrqt_sdv1_b200.linear_fp8 import FP8NativeStaticLinear, FP8StaticLinear
    g = np.load(os.path.join(GOLD, "q8_fp8_gemm.npz"))
    b = torch.from_numpy(g["b"]).view(torch.float8_e4m3fn)
    x = torch.from_numpy(g["mod_x"].view(np.int16)).view(torch.bfloat16).cuda()
    m = FP8StaticLinear(256, 512, False, dev="cuda", dtype=torch.bfloat16)
    m.weight.data = b.to(torch.bfloat16).cuda()
    m.weight_scale.data = torch.tensor([0.02], device="cuda")
    m.input_scale.data = torch.tensor([0.03], device="cuda")
    y = m(x)
    xq, _ = q8o.quantize(_bits(x).reshape(-1, 256), True, q8o.QUANT_FP8_STATIC, static_scale=0.03)
    alpha = float(np.float32(0.02) * np.float32(0.03))
    o = q8o.tensorwise(xq, g["b"], None, alpha, 1.0, True)
    _check_fp8(_bits(y).reshape(o.shape), o, True, alpha * 2e-6 * q8o.gemm_abs(xq, g["b"], q8o.KIND_E4M3))
    n = FP8NativeStaticLinear(256, 512, False, dev="cuda", dtype=torch.bfloat16, quantize_output=True)
    n.weight.data = b.cuda()
    n.weight_scale.data, n.input_scale.data = m.weight_scale.data, m.input_scale.data
    n.output_scale.data = torch.tensor([0.05], device="cuda")
    y2 = n(x)
    want = (y / n.output_scale).clamp(-448, 448).to(torch.float8_e4m3fn).to(y.dtype) * n.output_scale
    assert torch.equal(y2, want)
    n.weight.data = n.weight.data.to(torch.bfloat16)
    with pytest.raises(RuntimeError, match="Native FP8 checkpoint weight was converted"):
        n(x)
    # empty batch (an expert that received no tokens)
    assert m(x[:0]).shape == (0, 8, 512)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("with_bias", [True, False])
def test_smoothquant_module(dt, with_bias):
    from llmrqt_sdv1_b200.linear_sq import SqW8A8BBF16OBF16PerTensor
    K, N = 512, 768
    g = torch.Generator().manual_seed(17)
    m = SqW8A8BBF16OBF16PerTensor(8, 0, K, N, with_bias, dev="cuda", dtype=dt, weight_scale=0.0123)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    m.qweight.copy_(w)
    bias = torch.randn(N, generator=g).to(dt)
    if with_bias:
        m.bias.copy_(bias)
    x = (torch.randn(3, 5, K, generator=g) * 2).to(dt).cuda()
    y = m(x)
    assert y.shape == (3, 5, N) and y.dtype == dt
    bf = dt == torch.bfloat16
    xq, s = q8o.quantize(_bits(x).reshape(-1, K), bf, q8o.QUANT_INT8_PER_TENSOR, weight_scale=0.0123)
    ob = (_bits(bias), "bf16") if bf else bias.numpy()
    if not with_bias:
        ob = (np.zeros(N, np.uint16), "bf16") if bf else np.zeros(N, np.float16)
    want = q8o.tensorwise(xq, w.numpy(), ob, float(s[1]), 1.0, bf, kind=q8o.KIND_INT8)
    assert np.array_equal(_bits(y).reshape(want.shape), want)            # whole forward bit-exact
    # dequantise-and-matmul mode of the reference as a loose cross-check
    m.impl_mode = "naive"
    y2 = m(x)
    assert (y2.float() - y.float()).abs().max() / y.float().abs().max() < 2e-2


# ---------------------------------------------------------------------------------------------------------------
# argument errors (the reference's TORCH_CHECKs surface as RuntimeError)
# ---------------------------------------------------------------------------------------------------------------
def test_argument_errors(q8):
    from llmrqt_sdv1_b200 import sq_fp8_kernels as ext
    a = _rand_fp8((4, 64), 1).cuda()
    b = _rand_fp8((32, 64), 2).cuda()
    with pytest.raises(RuntimeError, match="only support bf16 or fp16"):
        ext.cutlass_f8f8bf16_tensorwise_sm89(a, b.t(), None, 1.0, 1.0, "float32")
    with pytest.raises(RuntimeError, match="same as bias dtype"):
        ext.cutlass_f8f8bf16_tensorwise_sm89(a, b.t(), torch.zeros(32, device="cuda", dtype=torch.float16), 1.0, 1.0, "bfloat16")
    with pytest.raises(RuntimeError, match="stride"):
        ext.cutlass_f8f8bf16_tensorwise_sm89(a, b.t().contiguous(), None, 1.0, 1.0, "bfloat16")     # WQ not [1, K]-strided
    with pytest.raises(RuntimeError):
        ext.cutlass_f8f8bf16_tensorwise_sm89(a, _rand_fp8((32, 48), 2).cuda().t(), None, 1.0, 1.0, "bfloat16")   # K mismatch
    with pytest.raises(RuntimeError, match="x_scale must be"):
        ext.cutlass_f8f8bf16_rowwise_sm89(a, b.t(), None, torch.ones(4, device="cuda"), torch.ones(1, 32, device="cuda"))
    with pytest.raises(RuntimeError, match="bias is required"):
        ext.w8a8_int8_linear_bbf16_obf16_per_tensor(a.view(torch.int8), b.view(torch.int8).t(), None, 1.0, 1.0)
    with pytest.raises(ValueError):                                        # K = 24: row pitch not a multiple of 16 bytes
        q8.gemm_tensorwise(_rand_fp8((4, 24), 1).cuda(), _rand_fp8((32, 24), 2).cuda().t(), None, 1.0, 1.0, torch.bfloat16)
    # zero rows: an empty result, no launch
    y = ext.cutlass_f8f8bf16_tensorwise_sm89(a[:0], b.t(), None, 1.0, 1.0, "bfloat16")
    assert y.shape == (0, 32)
