"""The tensor-memory decode kernel (1..16 rows, unscaled codes in tensor memory, `awq_b200_decode`) against the
CPU oracle at oracle-sized shapes and against device dequant + library matmul at full size; row results
independent of the number of rows; run-to-run identical; fused epilogues; routing by `awq_b200_linear`."""
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
def test_decode_vs_oracle(K_, K, N, G):
    """Ragged column counts (not a multiple of 32 or of the 256-column tile), one k block, groups of 256 and
    512, column tiles shared by several SMs and not; every row-count class of the kernel (1, 2, 4, 8, 16)."""
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=K + N)
    x = orc.make_activations(16, K, seed=6)
    ref = orc.linear_forward(x, qw, qz, sc, G)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    y16 = K_.decode(dev(x), pw)
    assert y16.shape == (16, N) and y16.dtype == torch.float16
    assert orc.max_normalised_error(y16.cpu().numpy(), ref) <= TOL
    for M in (1, 2, 3, 4, 5, 8, 9, 15):
        yM = K_.decode(dev(x[:M]), pw, overlap=(M % 2 == 1))
        assert torch.equal(yM, y16[:M]), f"rows differ between M={M} and M=16"
    assert torch.equal(K_.decode(dev(x), pw), y16)          # run-to-run identical
    assert K_.gemv_status() == 0


def test_decode_bias_and_bounds(K_):
    K, N = 1024, 520
    qw, qz, sc = orc.make_awq_tensors(K, N, 128, seed=31)
    x = orc.make_activations(5, K, seed=32)
    bias = (np.random.default_rng(33).standard_normal(N) * 0.5).astype(np.float16)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.decode(dev(x), pw, bias=dev(bias))
    ref = orc.linear_forward(x, qw, qz, sc, 128, bias=bias)
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    with pytest.raises(ValueError):
        K_.decode(dev(orc.make_activations(17, K, seed=1)), pw)
    assert K_.gemv_status() == 0


def test_decode_large_activations_and_extreme_zero_points(K_):
    """The constants carried by the codes (1024 / 64 per weight) are removed through the activation sums: the
    cancellation must hold for activations far from N(0, 1) and for columns whose zero point is 0 or 15."""
    K, N = 2048, 512
    qw, qz, sc = orc.make_awq_tensors(K, N, 128, seed=3)
    qz = qz.copy()
    qz[:, : N // 16] = 0                       # zero points 0
    qz[:, N // 16: N // 8] = -1                # all nibbles 15
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((4, K)) * 8.0 + 3.0).astype(np.float16)      # large, biased activations
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.decode(dev(x), pw)
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    assert K_.gemv_status() == 0


@pytest.mark.parametrize("K,N,M", [(8192, 57344, 1), (8192, 57344, 16), (28672, 8192, 16), (28672, 8192, 1),
                                   (8192, 7168, 3), (3584, 8192, 8), (2048, 12288, 4)])
def test_decode_full_size_vs_device_dequant_matmul(K_, K, N, M):
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=K + N)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).half()
    W = K_.dequantize(qw, qz, sc, 128)
    ref = torch.matmul(x.float(), W.float())
    y = K_.decode(x, pw)
    assert (y.float() - ref).abs().max() / ref.abs().max() <= TOL
    assert torch.equal(y, K_.decode(x, pw))
    if M > 1:
        assert torch.equal(K_.decode(x[:1].contiguous(), pw), y[:1])
    assert K_.gemv_status() == 0


def test_decode_fused_epilogues(K_):
    """Bias, SiLU(gate) * up over interleaved column pairs and the residual, as the other kernels do them:
    compared with the unfused kernel followed by the fp16 tensor operations."""
    import torch.nn.functional as F
    K, n = 4096, 4096
    gate = _random_packed_inputs(K, n, 128, seed=1)
    up = _random_packed_inputs(K, n, 128, seed=2)
    pw_gu = K_.make_gated_packed(gate, up, 128)               # [K, 2n]: 32 MiB, routed to the decode kernel
    x = torch.randn((3, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).half()
    res = torch.randn((3, n), device="cuda", generator=torch.Generator(device="cuda").manual_seed(4)).half()
    bias = (torch.randn(2 * n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) * 0.1).half()
    plain = K_.decode(x, pw_gu, bias=bias)                    # [3, 2n], bias added
    assert torch.equal(K_.linear(x, pw_gu, bias=bias), plain)
    want = F.silu(plain[:, 0::2]) * plain[:, 1::2] + res
    got = K_.linear_fused(x, pw_gu, bias=bias, residual=res, gated=True)
    diff = (got.float() - want.float()).abs()
    assert float(diff.max() / want.float().abs().max()) <= 2e-3
    # the residual-only epilogue is exact: fp16(acc) + bias + residual in the same order
    res2 = torch.randn((3, 2 * n), device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)).half()
    got2 = K_.linear_fused(x, pw_gu, bias=bias, residual=res2)
    assert torch.equal(got2, plain + res2)
    assert K_.gemv_status() == 0


def test_linear_routes_by_weight_size(K_):
    """From 16 MiB of packed weights `linear` uses the decode kernel for every M <= 16 (one kernel for all
    small row counts of a shape, so rows stay independent of the batch), the GEMV below that."""
    K, N = 4096, 8192                       # 16 MiB
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=41)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((16, K), device="cuda", dtype=torch.float16)
    y16 = K_.linear(x, pw)
    assert torch.equal(y16, K_.decode(x, pw))
    for M in (1, 8, 9):
        assert torch.equal(K_.linear(x[:M].contiguous(), pw), y16[:M])
    K2, N2 = 2048, 8192                     # 8 MiB
    qw, qz, sc = _random_packed_inputs(K2, N2, 128, seed=42)
    pw2 = K_.make_packed(qw, qz, sc, 128)
    x2 = torch.randn((8, K2), device="cuda", dtype=torch.float16)
    assert torch.equal(K_.linear(x2, pw2), K_.gemv(x2, pw2))
    assert K_.gemv_status() == 0
