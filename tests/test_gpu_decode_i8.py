"""The integer tensor-core decode kernel (1..8 rows, `awq_b200_decode_i8`) against the CPU oracle at oracle-sized
shapes and against device dequant + library matmul at full size; row results independent of the number of
rows; run-to-run identical; activations with outliers and extreme zero points."""
import numpy as np
import pytest
import torch

from oracle import awq_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 2e-3   # max|y - ref| / max|ref|


@pytest.fixture(scope="module")
def K_():
    from llmrqt_sdv1_b200 import kernels
    assert torch.cuda.is_available()
    return kernels


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _random_packed_inputs(K, N, G, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (K // G, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    sc = (torch.rand((K // G, N), device="cuda", generator=g) * 0.004 + 0.001).half()
    return qw, qz, sc


@pytest.mark.parametrize("K,N,G", [(128, 8, 128), (256, 264, 128), (1024, 1096, 128), (2048, 2048, 256),
                                   (6144, 2048, 128), (4096, 4096, 128), (512, 384, 512)])
def test_decode_i8_vs_oracle(K_, K, N, G):
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=K + N)
    x8 = orc.make_activations(8, K, seed=6)
    x = x8[:4]
    ref8 = orc.linear_forward(x8, qw, qz, sc, G)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    y4 = K_.decode_i8(dev(x), pw)
    assert y4.shape == (4, N) and y4.dtype == torch.float16
    assert orc.max_normalised_error(y4.cpu().numpy(), ref8[:4]) <= TOL
    for M in (1, 2, 3):
        yM = K_.decode_i8(dev(x[:M]), pw, overlap=(M % 2 == 1))
        assert torch.equal(yM, y4[:M]), f"rows differ between M={M} and M=4"
    assert torch.equal(K_.decode_i8(dev(x), pw), y4)          # run-to-run identical
    # 5..8 rows: the 8-row form behind the kernel that writes the activation planes once per call
    y8 = K_.decode_i8(dev(x8), pw)
    assert y8.shape == (8, N)
    assert orc.max_normalised_error(y8.cpu().numpy(), ref8) <= TOL
    assert torch.equal(y8[:4], y4), "rows differ between M=4 and M=8"
    for M in (5, 6, 7):
        yM = K_.decode_i8(dev(x8[:M]), pw, overlap=(M % 2 == 1))
        assert torch.equal(yM, y8[:M]), f"rows differ between M={M} and M=8"
    assert torch.equal(K_.decode_i8(dev(x8), pw, overlap=True), y8)
    assert K_.gemv_status() == 0


def test_decode_i8_bias_and_bounds(K_):
    K, N = 1024, 520
    qw, qz, sc = orc.make_awq_tensors(K, N, 128, seed=31)
    x = orc.make_activations(3, K, seed=32)
    bias = (np.random.default_rng(33).standard_normal(N) * 0.5).astype(np.float16)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.decode_i8(dev(x), pw, bias=dev(bias))
    ref = orc.linear_forward(x, qw, qz, sc, 128, bias=bias)
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    with pytest.raises(ValueError):
        K_.decode_i8(dev(orc.make_activations(9, K, seed=1)), pw)
    assert K_.gemv_status() == 0


def test_decode_i8_outliers_zero_rows_and_extreme_zero_points(K_):
    """Block-fixed-point activations: a block with one huge activation, an all-zero row, tiny activations
    and zero points 0 / 15 must all stay within the layer bound."""
    K, N = 2048, 512
    qw, qz, sc = orc.make_awq_tensors(K, N, 128, seed=3)
    qz = qz.copy()
    qz[:, : N // 16] = 0
    qz[:, N // 16: N // 8] = -1                # all nibbles 15
    rng = np.random.default_rng(4)
    x = rng.standard_normal((4, K)).astype(np.float32)
    x[0, 5] = 900.0                            # massive activation in one block
    x[0, 700] = -350.0
    x[1] = 0.0                                 # an all-zero row
    x[2] *= 1e-3                               # small activations (the output stays in fp16's normal range)
    x[3] = x[3] * 8.0 + 3.0                    # large and biased
    x = x.astype(np.float16)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.decode_i8(dev(x), pw).cpu().numpy()
    for m in range(4):
        ref = orc.linear_forward(x[m:m + 1], qw, qz, sc, 128)
        if m == 1:
            assert not y[m].any()
        else:
            assert orc.max_normalised_error(y[m:m + 1], ref) <= TOL, m
    assert K_.gemv_status() == 0


@pytest.mark.parametrize("K,N,M", [(8192, 57344, 1), (8192, 57344, 4), (28672, 8192, 4), (28672, 8192, 1),
                                   (8192, 7168, 3), (3584, 8192, 2), (2048, 12288, 2), (8192, 57344, 8),
                                   (28672, 8192, 5), (8192, 7168, 7), (7168, 8192, 6)])
def test_decode_i8_full_size_vs_device_dequant_matmul(K_, K, N, M):
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=K + N)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).half()
    W = K_.dequantize(qw, qz, sc, 128)
    ref = torch.matmul(x.float(), W.float())
    y = K_.decode_i8(x, pw)
    assert (y.float() - ref).abs().max() / ref.abs().max() <= TOL
    assert torch.equal(y, K_.decode_i8(x, pw))
    if M > 1:
        assert torch.equal(K_.decode_i8(x[:1].contiguous(), pw), y[:1])
    assert K_.gemv_status() == 0


def test_decode_i8_fused_epilogues_and_routing(K_):
    """Bias, SiLU(gate) * up over interleaved column pairs and the residual through `linear_fused` on a weight
    large enough to be routed here (64 MiB); `linear` picks this kernel for 1..8 rows, the exact-weight
    tensor-memory kernel for 9..16 rows, and the GEMV for every row count of a small weight."""
    import torch.nn.functional as F
    K, n = 8192, 8192
    gate = _random_packed_inputs(K, n, 128, seed=1)
    up = _random_packed_inputs(K, n, 128, seed=2)
    pw_gu = K_.make_gated_packed(gate, up, 128)               # [K, 2n]: 64 MiB
    x = torch.randn((16, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).half()
    x3 = x[:3].contiguous()
    res = torch.randn((3, n), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4)).half()
    bias = (torch.randn(2 * n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) * 0.1).half()
    plain = K_.decode_i8(x3, pw_gu, bias=bias)                # [3, 2n], bias added
    assert torch.equal(K_.linear(x3, pw_gu, bias=bias), plain)
    assert torch.equal(K_.linear(x[:1].contiguous(), pw_gu, bias=bias), plain[:1])
    want = F.silu(plain[:, 0::2]) * plain[:, 1::2] + res
    got = K_.linear_fused(x3, pw_gu, bias=bias, residual=res, gated=True)
    assert float((got.float() - want.float()).abs().max() / want.float().abs().max()) <= 2e-3
    res2 = torch.randn((3, 2 * n), device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)).half()
    assert torch.equal(K_.linear_fused(x3, pw_gu, bias=bias, residual=res2), plain + res2)   # exact: same roundings
    for M in (5, 8):
        xm = x[:M].contiguous()
        assert torch.equal(K_.linear(xm, pw_gu, bias=bias), K_.decode_i8(xm, pw_gu, bias=bias))
    x8 = x[:8].contiguous()
    res8 = torch.randn((8, n), device="cuda", generator=torch.Generator(device="cuda").manual_seed(7)).half()
    plain8 = K_.decode_i8(x8, pw_gu, bias=bias)
    want8 = F.silu(plain8[:, 0::2]) * plain8[:, 1::2] + res8
    got8 = K_.linear_fused(x8, pw_gu, bias=bias, residual=res8, gated=True)
    assert float((got8.float() - want8.float()).abs().max() / want8.float().abs().max()) <= 2e-3
    for M in (9, 16):
        xm = x[:M].contiguous()
        assert torch.equal(K_.linear(xm, pw_gu), K_.skinny(xm, pw_gu))
    K2, N2 = 2048, 8192                                        # 8 MiB: the GEMV at every row count
    qw, qz, sc = _random_packed_inputs(K2, N2, 128, seed=42)
    pw2 = K_.make_packed(qw, qz, sc, 128)
    x2 = torch.randn((8, K2), device="cuda", dtype=torch.float16)
    assert torch.equal(K_.linear(x2, pw2), K_.gemv(x2, pw2))
    assert torch.equal(K_.linear(x2[:2].contiguous(), pw2), K_.gemv(x2[:2].contiguous(), pw2))
    K3, N3 = 6144, 8192                                        # 24 MiB: this kernel at 1..4 rows
    qw, qz, sc = _random_packed_inputs(K3, N3, 128, seed=43)
    pw3 = K_.make_packed(qw, qz, sc, 128)
    x7 = torch.randn((7, K3), device="cuda", dtype=torch.float16)
    x4 = x7[:4].contiguous()
    y4 = K_.linear(x4, pw3)
    assert torch.equal(y4, K_.decode_i8(x4, pw3))
    assert torch.equal(K_.linear(x4[:1].contiguous(), pw3), y4[:1])       # decode and a short verification agree
    # one kernel for every call of fewer than 8 rows, as the reference dispatches: rows agree between 1, 2 and 7 rows
    y7 = K_.linear(x7, pw3, one_kernel_below_8=True)
    assert torch.equal(y7, K_.gemv(x7, pw3))
    for M in (1, 2, 5):
        assert torch.equal(K_.linear(x7[:M].contiguous(), pw3, one_kernel_below_8=True), y7[:M])
    assert torch.equal(K_.linear(x3, pw_gu, bias=bias, one_kernel_below_8=True), K_.gemv(x3, pw_gu, bias=bias))
    assert K_.gemv_status() == 0
