"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the
reference-generated golden fixtures.  Needs a B200."""
import os

import numpy as np
import pytest
import torch

from oracle import awq_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 2e-3   # max|y - ref| / max|ref|, the layer-output bound of the parity contract


@pytest.fixture(scope="module")
def K_():
    from llmrqt_sdv1_b200 import kernels
    assert torch.cuda.is_available()
    return kernels


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


_cache = {}


def tensors(K, N, G=128, seed=0):
    key = (K, N, G, seed)
    if key not in _cache:
        _cache[key] = orc.make_awq_tensors(K, N, G, seed)
    return _cache[key]


# --------------------------------------------------------------------------- dequant
def test_dequant_golden_all_pairs(K_, golden_dir):
    g = np.load(os.path.join(golden_dir, "awq_all_pairs.npz"))
    G = int(g["group_size"])
    W = K_.dequantize(dev(g["qweight"]), dev(g["qzeros"]), dev(g["scales"]), G)
    assert np.array_equal(bits(W), g["W_bits"])            # incl. subnormals, inf, -0
    pw = K_.make_packed(dev(g["qweight"]), dev(g["qzeros"]), dev(g["scales"]), G)
    assert np.array_equal(bits(K_.dequantize_packed(pw)), g["W_bits"])


def test_dequant_golden_small(K_, golden_dir):
    g = np.load(os.path.join(golden_dir, "awq_small.npz"))
    W = K_.dequantize(dev(g["qweight"]), dev(g["qzeros"]), dev(g["scales"]), int(g["group_size"]))
    assert np.array_equal(bits(W), g["W"].view(np.uint16))


@pytest.mark.parametrize("K,N,G", [(128, 8, 128), (256, 72, 128), (512, 128, 256), (2048, 6144, 128),
                                   (384, 64, 384)])
def test_dequant_and_repack_vs_oracle(K_, K, N, G):
    qw, qz, sc = tensors(K, N, G, seed=5)
    ref = orc.dequantize(qw, qz, sc, G).view(np.uint16)
    dqw, dqz, dsc = dev(qw), dev(qz), dev(sc)
    assert np.array_equal(bits(K_.dequantize(dqw, dqz, dsc, G)), ref)
    pw = K_.make_packed(dqw, dqz, dsc, G)
    assert pw.packed.numel() * 4 == K * N // 2
    assert np.array_equal(bits(K_.dequantize_packed(pw)), ref)
    assert torch.equal(K_.unpack(pw.packed), dqw)          # exact inverse


def test_dequant_random_bits(K_):
    """Arbitrary int32 patterns (sign bit set, all nibble values) and random fp16 scale bits."""
    rng = np.random.default_rng(11)
    K, N, G = 256, 256, 128
    qw = rng.integers(-2**31, 2**31, size=(K, N // 8), dtype=np.int64).astype(np.int32)
    qz = rng.integers(-2**31, 2**31, size=(K // G, N // 8), dtype=np.int64).astype(np.int32)
    sb = rng.integers(0, 2**16, size=(K // G, N), dtype=np.int64).astype(np.uint16)
    sb[(sb & 0x7C00) == 0x7C00] &= 0x83FF        # no inf/nan scales (nan payloads are not pinned)
    sc = sb.view(np.float16)
    ref = orc.dequantize(qw, qz, sc, G)
    got = K_.dequantize(dev(qw), dev(qz), dev(sc), G)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    got_p = K_.dequantize_packed(pw)
    finite = np.isfinite(ref)
    assert np.array_equal(bits(got)[finite], ref.view(np.uint16)[finite])
    assert np.array_equal(bits(got_p), bits(got))
    assert np.array_equal(np.isinf(got.cpu().numpy()), np.isinf(ref))


# --------------------------------------------------------------------------- GEMV
GEMV_SHAPES = [(128, 8), (256, 72), (2048, 2048), (2048, 6144), (6144, 2048), (1024, 1000 * 8)]


@pytest.mark.parametrize("K,N", GEMV_SHAPES)
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 23, 40, 64])
def test_gemv_vs_oracle(K_, K, N, M):
    qw, qz, sc = tensors(K, N, 128, seed=1)
    x = orc.make_activations(M, K, seed=M)
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.gemv(dev(x), pw)
    assert y.shape == (M, N) and y.dtype == torch.float16
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL


def test_gemv_config1_golden(K_, golden_dir):
    """Config 1 (M=1, K=2048, N=6144, seed 0) against the reference's own forward output."""
    g = np.load(os.path.join(golden_dir, "awq_config1_slice.npz"))
    K, N, G = int(g["K"]), int(g["N"]), int(g["group_size"])
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=0)
    x = orc.make_activations(1, K, seed=0)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    y = K_.linear(dev(x), pw).cpu().numpy()
    assert orc.max_normalised_error(y, g["y"][0]) <= TOL
    W = K_.dequantize_packed(pw)
    assert np.array_equal(bits(W[:, :64]), g["W_cols_0_64"].view(np.uint16))


@pytest.mark.parametrize("ntw", [2, 4])
@pytest.mark.parametrize("kw", [1, 2, 4, 8, 104, 108, 116])   # 1xx = 16 compute warps per CTA
@pytest.mark.parametrize("bps", [1, 2, 3, 5, 16])
def test_gemv_every_decomposition(K_, ntw, kw, bps):
    K, N, M = 2048, 1096, 5                       # N/8 = 137 tiles: ragged for every ntw
    qw, qz, sc = tensors(K, N, 128, seed=2)
    x = orc.make_activations(M, K, seed=3)
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.gemv_plan(dev(x), pw, ntw, bps, kw=kw)
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    y2 = K_.gemv_plan(dev(x), pw, ntw, bps, kw=kw)      # counters were left clean: second call identical
    assert torch.equal(y, y2)
    # split partials added over distributed shared memory (cluster) or through the workspace: same bits
    y3 = K_.gemv_plan(dev(x), pw, ntw, bps, kw=kw, no_cluster=True)
    y4 = K_.gemv_plan(dev(x), pw, ntw, bps, kw=kw, overlap=True)
    assert torch.equal(y, y3) and torch.equal(y, y4)
    assert K_.gemv_status() == 0


@pytest.mark.parametrize("kw", [1, 2, 4, 8, 104, 108, 116])   # 1xx = 16 compute warps per CTA
@pytest.mark.parametrize("K,N", [(2048, 1096), (1024, 264), (6144, 2048), (4096, 11008)])
def test_gemv_stream_every_decomposition(K_, kw, K, N):
    """The persistent stream variant: every in-CTA k split, ragged column counts, column groups that
    straddle CTAs (partials + last-arriver reduction) and ones that do not; deterministic; a row's
    bits independent of the row count (which switches the kernel to two passes per segment)."""
    qw, qz, sc = tensors(K, N, 128, seed=K + N)
    x = orc.make_activations(16, K, seed=5)
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y16 = K_.gemv_plan(dev(x), pw, 0, 0, kw=kw, mode="stream")
    assert orc.max_normalised_error(y16.cpu().numpy(), ref) <= TOL
    assert torch.equal(y16, K_.gemv_plan(dev(x), pw, 0, 0, kw=kw, mode="stream", overlap=True))
    for M in (1, 5, 8, 9):
        yM = K_.gemv_plan(dev(x[:M]), pw, 0, 0, kw=kw, mode="stream")
        assert torch.equal(yM, y16[:M]), f"rows differ between M={M} and M=16"
    for ntw in (2, 4):     # column tiles per warp never change the order of additions
        assert torch.equal(K_.gemv_plan(dev(x[:3]), pw, ntw, 0, kw=kw, mode="stream"), y16[:3])
    assert K_.gemv_status() == 0


def test_gemv_stream_and_per_split_agree(K_):
    """The two ways of handing out the work group a column's k blocks differently, so they agree
    to fp32 rounding; both stay within the tolerance of the oracle."""
    K, N, M = 8192, 4096, 4
    qw, qz, sc = tensors(K, N, 128, seed=21)
    x = orc.make_activations(M, K, seed=22)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    a = K_.gemv(dev(x), pw, mode="stream").float()
    b = K_.gemv(dev(x), pw, mode="per_split").float()
    assert ((a - b).abs().max() / b.abs().max()).item() <= 1e-3
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    assert orc.max_normalised_error(a.cpu().numpy(), ref) <= TOL
    with pytest.raises(ValueError):
        K_.gemv(dev(x), pw, mode="bogus")


def test_gemv_row_result_independent_of_batch(K_):
    """A row's bits must not depend on M (decode q_len=1 and verify q_len=2 must agree,
    LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:161-166) nor on the run."""
    K, N = 2048, 4096
    qw, qz, sc = tensors(K, N, 128, seed=4)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    x64 = dev(orc.make_activations(64, K, seed=9))
    y64 = K_.gemv(x64, pw)
    x16, y16 = x64[:16].contiguous(), y64[:16]
    for M in (1, 2, 7, 8, 9, 15, 16, 17, 33):
        yM = K_.gemv(x64[:M].contiguous(), pw)
        assert torch.equal(yM, y64[:M]), f"rows differ between M={M} and M=64"
    for r in (3, 12):
        assert torch.equal(K_.gemv(x16[r:r + 1].contiguous(), pw)[0], y16[r])
    for _ in range(50):
        assert torch.equal(K_.gemv(x16, pw), y16)


def test_gemv_bias_group256_and_linearity(K_):
    K, N, G = 1024, 512, 256
    qw, qz, sc = tensors(K, N, G, seed=6)
    rng = np.random.default_rng(0)
    bias = rng.standard_normal(N).astype(np.float16)
    x = orc.make_activations(4, K, seed=1)
    ref = orc.linear_forward(x, qw, qz, sc, G, bias)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    y = K_.gemv(dev(x), pw, bias=dev(bias))
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    # y(2x) == 2 y(x) exactly in binary floating point (no bias)
    y1 = K_.gemv(dev(x), pw)
    y2 = K_.gemv(dev((x * np.float16(2)).astype(np.float16)), pw)
    assert torch.equal(y2, y1 * 2)


def test_gemv_rejects_bad_arguments(K_):
    qw, qz, sc = tensors(256, 72, 128, seed=5)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    with pytest.raises(ValueError):
        K_.gemv(torch.zeros(65, 256, dtype=torch.float16, device="cuda"), pw)
    with pytest.raises(ValueError):
        K_.gemv(torch.zeros(1, 128, dtype=torch.float16, device="cuda"), pw)
    with pytest.raises(ValueError):
        K_.make_packed(dev(qw), dev(qz), dev(sc), 64)


# --------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,K,N", [(17, 128, 128), (64, 256, 256), (128, 512, 384), (200, 1024, 72),
                                   (256, 4096, 256), (300, 2048, 1000 * 8), (512, 4096, 4096),
                                   (1000, 1024, 640)])
def test_gemm_vs_oracle(K_, M, K, N):
    qw, qz, sc = tensors(K, N, 128, seed=7)
    x = orc.make_activations(M, K, seed=M)
    ref = orc.linear_forward(x, qw, qz, sc, 128)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.gemm(dev(x), pw)
    torch.cuda.synchronize()
    assert K_.gemm_status() == 0
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    # both tensor-core kernels (weights staged in shared memory / in tensor memory, every row tile)
    # multiply the same fp16 weights in the same k order: identical bits as long as one CTA finishes a tile;
    # where the tensor-memory kernel cuts tiles along k (long k, SMs otherwise idle) the fp32 partial sums
    # are added in k order instead: equal to fp32 rounding, and the same bits on every call
    ys = K_.gemm_smem(dev(x), pw)
    scale = float(ys.float().abs().max())
    assert float((y.float() - ys.float()).abs().max()) <= 1e-3 * scale
    for mt in (64, 128, 192):
        assert torch.equal(K_.gemm_wtm_unsplit(dev(x), pw, m_tile=mt), ys)
        ym = K_.gemm_wtm(dev(x), pw, m_tile=mt)
        assert float((ym.float() - ys.float()).abs().max()) <= 1e-3 * scale
        assert torch.equal(ym, K_.gemm_wtm(dev(x), pw, m_tile=mt))
    assert K_.gemm_status() == 0


def test_gemm_bias_group_and_small_m(K_):
    K, N, G = 1024, 512, 512
    qw, qz, sc = tensors(K, N, G, seed=8)
    rng = np.random.default_rng(1)
    bias = rng.standard_normal(N).astype(np.float16)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    for M in (1, 16, 33, 129):
        x = orc.make_activations(M, K, seed=M)
        ref = orc.linear_forward(x, qw, qz, sc, G, bias)
        y = K_.gemm(dev(x), pw, bias=dev(bias))
        assert K_.gemm_status() == 0
        assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL


def test_gemm_matches_gemv_rows(K_):
    """The two kernels multiply the same fp16 weights with fp32 accumulation."""
    K, N = 2048, 2048
    qw, qz, sc = tensors(K, N, 128, seed=1)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    x = dev(orc.make_activations(16, K, seed=2))
    a, b = K_.gemv(x, pw).float(), K_.gemm(x, pw).float()
    assert (a - b).abs().max() / b.abs().max() <= 1e-3


# --------------------------------------------------------------------------- full-size properties
@pytest.mark.parametrize("K,N,G", [(128, 8, 128), (256, 264, 128), (1024, 1096, 128), (2048, 2048, 256),
                                   (6144, 2048, 128), (4096, 4096, 128)])
def test_skinny_vs_oracle(K_, K, N, G):
    """The tensor-memory split-K kernel for 1..64 rows: ragged column counts (not a multiple of 32 or
    of the 256-column tile), one k block, group 256, column tiles shared by several SMs and not."""
    qw, qz, sc = tensors(K, N, G, seed=K + N)
    x = orc.make_activations(64, K, seed=6)
    ref = orc.linear_forward(x, qw, qz, sc, G)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    y64 = K_.skinny(dev(x), pw)
    assert y64.shape == (64, N) and y64.dtype == torch.float16
    assert orc.max_normalised_error(y64.cpu().numpy(), ref) <= TOL
    for M in (1, 3, 16, 17, 33):
        yM = K_.skinny(dev(x[:M]), pw, overlap=(M % 2 == 1))
        assert torch.equal(yM, y64[:M]), f"rows differ between M={M} and M=64"
    assert K_.gemv_status() == 0


def test_skinny_bias_and_bounds(K_):
    K, N = 1024, 520
    qw, qz, sc = tensors(K, N, 128, seed=31)
    x = orc.make_activations(5, K, seed=32)
    bias = (np.random.default_rng(33).standard_normal(N) * 0.5).astype(np.float16)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), 128)
    y = K_.skinny(dev(x), pw, bias=dev(bias))
    ref = orc.linear_forward(x, qw, qz, sc, 128, bias=bias)
    assert orc.max_normalised_error(y.cpu().numpy(), ref) <= TOL
    # same weights as the GEMM path: identical dequantised operands, fp32 accumulation
    yg = K_.gemm(dev(x), pw, bias=dev(bias))
    assert ((y.float() - yg.float()).abs().max() / yg.float().abs().max()).item() <= 1e-3
    with pytest.raises(ValueError):
        K_.skinny(dev(orc.make_activations(65, K, seed=1)), pw)


def test_linear_routes_mid_row_counts_to_skinny(K_):
    """17..64 rows of a matrix with few column tiles and a long k go to the exact-weight tensor-memory kernel."""
    K, N = 12288, 8192                      # 48 MiB packed, 32 column tiles, 96 k blocks
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=40)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((40, K), device="cuda", dtype=torch.float16)
    y40 = K_.linear(x, pw)
    assert torch.equal(y40, K_.skinny(x, pw))
    assert torch.equal(K_.linear(x[:17].contiguous(), pw), y40[:17])
    W = K_.dequantize_packed(pw)
    ref = x.float() @ W.float()
    assert ((y40.float() - ref).abs().max() / ref.abs().max()).item() <= TOL
    assert K_.gemv_status() == 0


def test_gemm_tail_split(K_):
    """176 tiles of 192 x 256 on 148 SMs: the 28 tiles of the last wave are cut along k, shared by all
    SMs and finished through fp32 partial tiles.  Same result to fp32 rounding as one CTA per tile,
    deterministic, counters left clean (second call identical)."""
    M, K, N = 2048, 4096, 4096
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=77)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(3)).half()
    bias = (torch.randn(N, device="cuda") * 0.1).half()
    y = K_.gemm_wtm(x, pw, bias=bias, m_tile=192)
    y_again = K_.gemm_wtm(x, pw, bias=bias, m_tile=192)
    y_unsplit = K_.gemm_wtm_unsplit(x, pw, bias=bias, m_tile=192)
    assert K_.gemm_status() == 0
    assert torch.equal(y, y_again)
    ref = torch.matmul(x, K_.dequantize(qw, qz, sc, 128)).float() + bias.float()
    scale = ref.abs().max()
    assert (y.float() - ref).abs().max() / scale <= TOL
    assert (y.float() - y_unsplit.float()).abs().max() / scale <= 1e-3
    assert torch.equal(y_unsplit, K_.gemm_smem(x, pw, bias=bias))
    # fewer tiles than SMs: every tile is cut along k and all SMs work
    M3, N3 = 300, 1024
    qw, qz, sc = _random_packed_inputs(K, N3, 128, seed=79)
    pw3 = K_.make_packed(qw, qz, sc, 128)
    for mt in (64, 128, 192):
        y3 = K_.gemm_wtm(x[:M3].contiguous(), pw3, m_tile=mt)
        y3u = K_.gemm_wtm_unsplit(x[:M3].contiguous(), pw3, m_tile=mt)
        ref3 = torch.matmul(x[:M3], K_.dequantize(qw, qz, sc, 128)).float()
        assert (y3.float() - ref3).abs().max() / ref3.abs().max() <= TOL
        assert (y3.float() - y3u.float()).abs().max() / ref3.abs().max() <= 1e-3
        assert torch.equal(y3, K_.gemm_wtm(x[:M3].contiguous(), pw3, m_tile=mt))
    # ragged rows and columns through the shared tiles as well
    M2, N2 = 2000, 4040
    qw, qz, sc = _random_packed_inputs(K, N2, 128, seed=78)
    pw2 = K_.make_packed(qw, qz, sc, 128)
    y2 = K_.gemm_wtm(x[:M2].contiguous(), pw2, m_tile=192)
    ref2 = torch.matmul(x[:M2], K_.dequantize(qw, qz, sc, 128)).float()
    assert (y2.float() - ref2).abs().max() / ref2.abs().max() <= TOL
    assert K_.gemm_status() == 0


def _random_packed_inputs(K, N, G, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (K // G, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    sc = (torch.rand((K // G, N), device="cuda", generator=g) * 0.004 + 0.001).half()
    return qw, qz, sc


@pytest.mark.parametrize("K,N,M", [(8192, 57344, 1), (28672, 8192, 16), (2048, 12288, 4)])
def test_gemv_full_size_vs_device_dequant_matmul(K_, K, N, M):
    """Full-size decode linears (70B-class and Qwen3 shapes): the kernel against dequant (proved bit-exact above)
    followed by a library fp16 matmul on the same device, plus the unpack round trip."""
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=K + N)
    pw = K_.make_packed(qw, qz, sc, 128)
    assert torch.equal(K_.unpack(pw.packed), qw)
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).half()
    W = K_.dequantize(qw, qz, sc, 128)
    ref = torch.matmul(x.float(), W.float())
    y = K_.gemv(x, pw).float()
    assert (y - ref).abs().max() / ref.abs().max() <= TOL
    assert torch.equal(K_.dequantize_packed(pw), W)


@pytest.mark.parametrize("K,N,M", [(4096, 28672, 2048), (14336, 4096, 2048), (4096, 6144, 8192)])
def test_gemm_full_size_vs_device_dequant_matmul(K_, K, N, M):
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed=K + N + M)
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(2)).half()
    W = K_.dequantize(qw, qz, sc, 128)
    ref = torch.matmul(x, W).float()
    y = K_.gemm(x, pw)
    assert K_.gemm_status() == 0
    assert (y.float() - ref).abs().max() / ref.abs().max() <= TOL


# --------------------------------------------------------------------------- group sizes 32 and 64
@pytest.mark.parametrize("G", [32, 64])
@pytest.mark.parametrize("K,N", [(256, 264), (1024, 1096), (4096, 512)])
def test_small_groups_every_row_count(K_, K, N, G):
    """The reference module takes any group size that divides K (linear_awq.py:228-236).  Groups of 32 and 64
    put several scale rows into one 128-k block: the kernels that build the exact fp16 weight per element serve
    them (dequant bit-exact; the split-K tensor-memory kernel up to 64 rows, the GEMMs beyond), and `linear`
    routes there for every row count."""
    qw, qz, sc = tensors(K, N, G, seed=K + N + G)
    pw = K_.make_packed(dev(qw), dev(qz), dev(sc), G)
    assert np.array_equal(bits(K_.dequantize_packed(pw)), orc.dequantize(qw, qz, sc, G).view(np.uint16))
    assert np.array_equal(bits(K_.dequantize(dev(qw), dev(qz), dev(sc), G)), orc.dequantize(qw, qz, sc, G).view(np.uint16))
    x = orc.make_activations(300, K, seed=G)
    ref = orc.linear_forward(x, qw, qz, sc, G)
    for M in (1, 8, 16, 40, 64, 65, 300):
        y = K_.linear(dev(x[:M]), pw)
        assert orc.max_normalised_error(y.cpu().numpy(), ref[:M]) <= TOL, (M, G)
    ys = K_.skinny(dev(x[:33]), pw)
    assert torch.equal(ys, K_.linear(dev(x[:33]), pw))
    for fn in (K_.gemm, K_.gemm_smem, K_.gemm_wtm):
        yg = fn(dev(x), pw)
        assert orc.max_normalised_error(yg.cpu().numpy(), ref) <= TOL, (fn.__name__, G)
    assert torch.equal(K_.gemm_smem(dev(x), pw), K_.gemm_wtm_unsplit(dev(x), pw))
    with pytest.raises(ValueError):
        K_.gemv(dev(x[:1]), pw)            # the per-block decode kernels need whole 128-k groups
    with pytest.raises(ValueError):
        K_.decode_i8(dev(x[:1]), pw)
    assert K_.gemm_status() == 0 and K_.gemv_status() == 0


def test_small_groups_through_the_module(K_):
    from llmrqt_sdv1_b200 import AWQLinear_GEMM
    K, N, G = 512, 384, 64
    qw, qz, sc = tensors(K, N, G, seed=77)
    m = AWQLinear_GEMM(4, G, K, N, False, "cuda")
    m.load_state_dict({"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": torch.from_numpy(sc)})
    for M in (1, 70):
        x = orc.make_activations(M, K, seed=M)
        y = m(dev(x))[0].cpu().numpy()
        assert orc.max_normalised_error(y, orc.linear_forward(x, qw, qz, sc, G)) <= TOL
