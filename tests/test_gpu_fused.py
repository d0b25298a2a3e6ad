"""The fused epilogues (bias, SiLU(gate) * up over interleaved column pairs, residual add) of every
kernel behind `awq_b200_linear_fused`, against the unfused kernel followed by the separate fp16 tensor
operations, and against the CPU oracle.  Needs a B200."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import awq_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 2e-3


@pytest.fixture(scope="module")
def K_():
    from llmrqt_sdv1_b200 import kernels
    assert torch.cuda.is_available()
    return kernels


def _random_awq(K, N, G, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (K // G, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    sc = (torch.rand((K // G, N), device="cuda", generator=g) * 0.004 + 0.001).half()
    return qw, qz, sc


def _places(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in fp16 representable values."""
    def line(t):
        u = t.contiguous().view(torch.int16).to(torch.int32)
        mag = u & 0x7FFF
        return torch.where(u < 0, -mag, mag)
    return (line(a) - line(b)).abs()


def test_interleave_matches_oracle_and_dequant(K_):
    K, n, G = 256, 72, 128
    gq, gz, gs = orc.make_awq_tensors(K, n, G, seed=1)
    uq, uz, us = orc.make_awq_tensors(K, n, G, seed=2)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = K_.interleave_columns(dev(gq), dev(uq))
    assert np.array_equal(out.cpu().numpy(), orc.interleave_columns(gq, uq))
    assert np.array_equal(K_.interleave_columns(dev(gz), dev(uz)).cpu().numpy(), orc.interleave_columns(gz, uz))
    pw = K_.make_gated_packed((dev(gq), dev(gz), dev(gs)), (dev(uq), dev(uz), dev(us)), G)
    W = K_.dequantize_packed(pw).cpu().numpy()
    assert np.array_equal(W[:, 0::2].view(np.uint16), orc.dequantize(gq, gz, gs, G).view(np.uint16))
    assert np.array_equal(W[:, 1::2].view(np.uint16), orc.dequantize(uq, uz, us, G).view(np.uint16))


def test_gated_vs_oracle_small(K_):
    """One small gated MLP front half end to end against the numpy oracle (separate gate and up linears,
    SiLU * up, residual)."""
    K, n, G = 512, 192, 128
    gq, gz, gs = orc.make_awq_tensors(K, n, G, seed=3)
    uq, uz, us = orc.make_awq_tensors(K, n, G, seed=4)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    pw = K_.make_gated_packed((dev(gq), dev(gz), dev(gs)), (dev(uq), dev(uz), dev(us)), G)
    for M in (1, 7, 16, 40, 200):
        x = orc.make_activations(M, K, seed=M)
        res = orc.make_activations(M, n, seed=100 + M)
        ref = orc.add_residual(orc.silu_mul(orc.linear_forward(x, gq, gz, gs, G), orc.linear_forward(x, uq, uz, us, G)), res)
        y = K_.linear_fused(dev(x), pw, residual=dev(res), gated=True).cpu().numpy()
        assert y.shape == (M, n)
        assert orc.max_normalised_error(y, ref) <= TOL, M
    assert K_.gemv_status() == 0 and K_.gemm_status() == 0


def _check_against_unfused(K_, M, K, n, flags, seed, with_bias=True):
    """Fused result against the same kernel without epilogue (same decomposition, hence the same fp32 sums)
    followed by the separate fp16 tensor operations."""
    G = 128
    gate, up = _random_awq(K, n, G, seed), _random_awq(K, n, G, seed + 1)
    pw = K_.make_gated_packed(gate, up, G)
    gen = torch.Generator(device="cuda").manual_seed(seed + 2)
    x = torch.randn((M, K), device="cuda", generator=gen).half()
    bias = (torch.randn(2 * n, device="cuda", generator=gen) * 0.5).half() if with_bias else None
    res_half = torch.randn((M, n), device="cuda", generator=gen).half()
    res_full = torch.randn((M, 2 * n), device="cuda", generator=gen).half()
    y_plain = K_.linear_fused(x, pw, bias=bias, flags=flags)                      # [M, 2n], bias only
    # residual only: exact
    y_res = K_.linear_fused(x, pw, bias=bias, residual=res_full, flags=flags)
    assert torch.equal(y_res, y_plain + res_full)
    # gated (+ residual): SiLU may differ in its last place on a few elements
    ref = F.silu(y_plain[:, 0::2]) * y_plain[:, 1::2]
    y_gated = K_.linear_fused(x, pw, bias=bias, gated=True, flags=flags)
    assert y_gated.shape == (M, n)
    d = _places(y_gated, ref)
    assert int(d.max()) <= 2 and float((d != 0).float().mean()) < 2e-3
    y_both = K_.linear_fused(x, pw, bias=bias, residual=res_half, gated=True, flags=flags)
    exact = d == 0
    assert torch.equal(y_both[exact], (ref + res_half)[exact])
    # in place on the residual buffer (the decoder layer's `h = h + ...`)
    h = res_half.clone()
    K_.linear_fused(x, pw, bias=bias, residual=h, gated=True, out=h, flags=flags)
    assert torch.equal(h, y_both)
    # and the unfused result itself is right
    W = K_.dequantize_packed(pw)
    full = torch.matmul(x, W).float() + (bias.float() if bias is not None else 0.0)
    assert (y_plain.float() - full).abs().max() / full.abs().max() <= TOL
    assert K_.gemv_status() == 0 and K_.gemm_status() == 0


@pytest.mark.parametrize("M", [1, 5, 16])
@pytest.mark.parametrize("K,n,mode", [
    (128, 64, "per_split"),                 # one split: finished through a single partial
    (2048, 1024, "per_split"),              # a few splits (cluster reduction where it applies)
    (2048, 1024, "per_split_no_cluster"),   # the same through the global partials
    (6144, 1024, "per_split"),
    (2048, 2048, "stream"),                 # persistent stream, segments with one and with several contributors
    (2048, 6144, None),                     # the library's own choice for the gate_up shape of the decode config
    (4096, 72, None),                       # ragged: N = 144 is not a multiple of the column tile
])
def test_decode_kernels_fused(K_, M, K, n, mode):
    from llmrqt_sdv1_b200 import _lib
    flags = {"per_split": _lib.GEMV_PER_SPLIT, "per_split_no_cluster": _lib.GEMV_PER_SPLIT | _lib.NO_CLUSTER,
             "stream": _lib.GEMV_STREAM, None: 0}[mode]
    _check_against_unfused(K_, M, K, n, flags, seed=K + n + M)


@pytest.mark.parametrize("M,K,n", [(24, 4096, 1024), (64, 4096, 520), (3, 8192, 6144), (16, 8192, 6144)])
def test_split_k_tensor_memory_kernel_fused(K_, M, K, n):
    """17..64 rows of a narrow matrix, and few rows of a 48 MiB weight: the split-K tensor-memory kernel."""
    _check_against_unfused(K_, M, K, n, 0, seed=K + n + M)


@pytest.mark.parametrize("M,K,n,smem", [(300, 4096, 512, False),     # fewer tiles than SMs: tiles cut along k, fix-up kernel
                                         (2048, 1024, 1024, False),  # whole tiles, weights in tensor memory
                                         (2048, 1024, 1024, True),   # weights in shared memory
                                         (1000, 512, 1016, False),   # ragged rows and columns
                                         (1000, 512, 1016, True)])
def test_gemm_kernels_fused(K_, M, K, n, smem):
    from llmrqt_sdv1_b200 import _lib
    _check_against_unfused(K_, M, K, n, _lib.GEMM_SMEM if smem else 0, seed=K + n + M, with_bias=(M != 300))


def test_fused_argument_checks(K_):
    qw, qz, sc = _random_awq(256, 72, 128, seed=9)       # N = 72: not a multiple of 16
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((2, 256), device="cuda").half()
    with pytest.raises(ValueError):
        K_.linear_fused(x, pw, gated=True)
    with pytest.raises(ValueError):
        K_.linear_fused(x, pw, residual=torch.zeros((2, 8), device="cuda").half())
    y = K_.linear_fused(x, pw)                            # no epilogue at all = the plain linear
    assert torch.equal(y, K_.linear(x, pw))


def _module(K, N, seed, bias=False):
    from llmrqt_sdv1_b200 import AWQLinear_GEMM
    qw, qz, sc = _random_awq(K, N, 128, seed)
    m = AWQLinear_GEMM(4, 128, K, N, bias, "cuda")
    m.qweight, m.qzeros, m.scales = qw, qz, sc
    if bias:
        m.bias = (torch.randn(N, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed)) * 0.2).half()
    return m


@pytest.mark.parametrize("shape", [(1, 1, 2048), (1, 7, 2048), (2, 100, 2048), (300, 2048)])
@pytest.mark.parametrize("bias", [False, True])
def test_gated_mlp_module(K_, shape, bias):
    """`AWQGatedMLP` against the three-module form it replaces (different column counts may pick different
    k-splits, so the comparison is the layer-output bound, not bit equality), with and without residual,
    and against its own `dequant_matmul` mode."""
    from llmrqt_sdv1_b200 import AWQGatedMLP
    hidden, inter = 2048, 1536
    gate, up, down = _module(hidden, inter, 1, bias), _module(hidden, inter, 2, bias), _module(inter, hidden, 3, bias)
    mlp = AWQGatedMLP(gate, up, down)
    x = torch.randn(shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).half() * 4
    res = torch.randn(shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)).half()
    ref = down(F.silu(gate(x)) * up(x)).reshape(shape)          # AWQLinear_GEMM hands 2-D input back 3-D
    y = mlp(x)
    assert y.shape == tuple(shape) and y.dtype == torch.float16
    scale = ref.float().abs().max()
    assert (y.float() - ref.float()).abs().max() / scale <= TOL
    y_res = mlp(x, residual=res)
    assert torch.equal(y_res, y + res)
    mlp.impl_mode = "dequant_matmul"
    y_dm = mlp(x, residual=res)
    assert (y_dm.float() - y_res.float()).abs().max() / (ref.float() + res.float()).abs().max() <= TOL
    # the plain module's residual argument
    o = down(torch.randn(shape[:-1] + (inter,), device="cuda").half())
    x_d = torch.randn(shape[:-1] + (inter,), device="cuda", generator=torch.Generator(device="cuda").manual_seed(8)).half()
    assert torch.equal(down(x_d, residual=res).reshape(shape), down(x_d).reshape(shape) + res)
    assert o.shape[-1] == hidden
    assert K_.gemv_status() == 0 and K_.gemm_status() == 0


def test_gated_mlp_state_dict_and_dtype(K_):
    from llmrqt_sdv1_b200 import AWQGatedMLP
    mlp = AWQGatedMLP(_module(256, 128, 1), _module(256, 128, 2), _module(128, 256, 3))
    names = set(mlp.state_dict().keys())
    assert {"gate_up_qweight", "gate_up_qzeros", "gate_up_scales", "down_proj.qweight"} <= names
    assert mlp.gate_up_qweight.shape == (256, 32) and mlp.gate_up_scales.shape == (2, 256)
    x = torch.randn((3, 256), device="cuda").bfloat16()
    y = mlp(x)
    assert y.dtype == torch.bfloat16 and y.shape == (3, 256)
    assert mlp(torch.zeros((0, 256), device="cuda").half()).shape == (0, 256)
    with pytest.raises(ValueError):
        AWQGatedMLP(_module(256, 128, 1), _module(256, 64, 2), _module(128, 256, 3))


def test_graphed_step_matches_eager(K_):
    """A chain of modules (plain, gated MLP with residual) captured once and replayed: same bits as the eager
    calls, also for new inputs given from pinned host memory."""
    from llmrqt_sdv1_b200 import AWQGatedMLP, GraphedStep
    qkv, o = _module(512, 1024, 11, bias=True), _module(1024, 512, 12)
    mlp = AWQGatedMLP(_module(512, 768, 13), _module(512, 768, 14), _module(768, 512, 15))

    def chain(x):
        a = qkv(x)
        h = o(a, residual=x)
        return mlp(h, residual=h), a

    gen = torch.Generator(device="cuda").manual_seed(21)
    x0 = torch.randn((1, 3, 512), device="cuda", generator=gen).half()
    step = GraphedStep(chain, (x0,))
    y_g, a_g = step(x0)
    y_e, a_e = chain(x0)
    assert torch.equal(y_g, y_e) and torch.equal(a_g, a_e)
    x1 = torch.randn((1, 3, 512), generator=torch.Generator().manual_seed(22)).half().pin_memory()
    y_g, _ = step(x1)
    y_e, _ = chain(x1.cuda())
    assert torch.equal(y_g, y_e)
    assert len(step.static_outputs) == 2
    assert step.status() == 0
    with pytest.raises(ValueError):
        step(torch.zeros((1, 4, 512), dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        step(x0, x0)


def test_workspace_growth_keeps_a_captured_graph_valid(K_):
    """A graph captured by the caller holds the address of the stream's workspace; a later call that needs a larger
    workspace gets a new one, and the old one stays allocated: the replay is still correct."""
    from llmrqt_sdv1_b200 import quantize
    side = torch.cuda.Stream()
    qw, qz, sc = quantize.random_awq_tensors(512, 1024, 128, seed=31, device="cuda")
    pw = K_.make_packed(qw, qz, sc, 128)
    x = torch.randn((2, 512), device="cuda", generator=torch.Generator(device="cuda").manual_seed(32)).half()
    y = torch.empty((2, 1024), dtype=torch.float16, device="cuda")
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            K_.linear(x, pw, out=y)
        side.synchronize()
        want = y.clone()
        key = (x.device.index, side.cuda_stream, "awq_b200_linear")
        before = K_._workspaces[key]
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            K_.linear(x, pw, out=y)
        # a weight whose few-row kernel shares column tiles between CTAs through partial sums: a larger workspace
        qw2, qz2, sc2 = quantize.random_awq_tensors(8192, 8192, 128, seed=33, device="cuda")
        pw2 = K_.make_packed(qw2, qz2, sc2, 128)
        x2 = torch.randn((64, 8192), device="cuda").half()
        assert K_.lib.awq_b200_linear_workspace_bytes(64, 8192, 8192) > before.numel()
        K_.linear(x2, pw2)
        after = K_._workspaces[key]
        assert after.data_ptr() != before.data_ptr() and any(t is before for t in K_._retired_workspaces)
        junk = [torch.full((1 << 20,), 7, dtype=torch.uint8, device="cuda") for _ in range(8)]   # would reuse freed memory
        y.zero_()
        g.replay()
        side.synchronize()
    torch.cuda.current_stream().wait_stream(side)
    assert torch.equal(y, want)
    del junk
    assert K_.gemv_status() == 0
