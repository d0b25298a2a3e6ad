"""The two decode-time plumbing kernels (`awq_b200_qk_norm_rope_cache`, `awq_b200_attn_decode`) against the
tensor operations they replace: Hugging Face-style per-head RMSNorm + rotary embedding + cache write, and
scaled-dot-product attention of one query token over the cached positions."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).half()


def _hf_rms(x, w, eps):
    v = x.float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return w * v.to(x.dtype)


def _rotate_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


@pytest.mark.parametrize("H,KV,D,with_norm", [(16, 8, 128, True), (32, 8, 128, False), (8, 2, 64, True)])
def test_qk_norm_rope_cache(H, KV, D, with_norm):
    from llmrqt_sdv1_b200 import kernels
    max_len, eps = 96, 1e-6
    qkv = _rand((1, 1, (H + 2 * KV) * D), 1)
    qw, kw = (_rand((D,), 2, 0.3) + 1.0, _rand((D,), 3, 0.3) + 1.0) if with_norm else (None, None)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos, sin = torch.cat((ang.cos(), ang.cos()), -1).half().contiguous(), torch.cat((ang.sin(), ang.sin()), -1).half().contiguous()
    k_cache = torch.zeros((KV, max_len, D), dtype=torch.float16, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    q_out = torch.empty((H, D), dtype=torch.float16, device="cuda")
    for p in (0, 37, max_len - 1):
        pos = torch.tensor([p], dtype=torch.long, device="cuda")
        kernels.qk_norm_rope_cache(qkv, qw, kw, eps, cos, sin, pos, q_out, k_cache, v_cache)
        row = qkv.view(-1)
        q = row[:H * D].view(H, D)
        k = row[H * D:(H + KV) * D].view(KV, D)
        v = row[(H + KV) * D:].view(KV, D)
        if with_norm:
            q, k = _hf_rms(q, qw, eps), _hf_rms(k, kw, eps)
        q_ref = q * cos[p] + _rotate_half(q) * sin[p]
        k_ref = k * cos[p] + _rotate_half(k) * sin[p]
        torch.cuda.synchronize()
        # same roundings as the fp16 tensor operations; the sum of squares may be added in another order, which
        # can move a normalised value by one fp16 place
        assert (q_out.float() - q_ref.float()).abs().max() <= 2e-3 * q_ref.float().abs().max()
        assert (k_cache[:, p].float() - k_ref.float()).abs().max() <= 2e-3 * k_ref.float().abs().max()
        assert torch.equal(v_cache[:, p], v)
        if not with_norm:
            assert torch.equal(q_out, q_ref) and torch.equal(k_cache[:, p], k_ref)
    assert int((k_cache.abs().sum(-1) != 0).sum()) == 3 * KV          # only the three rows were written
    # a position outside the cache writes nothing
    before = k_cache.clone()
    kernels.qk_norm_rope_cache(qkv, qw, kw, eps, cos, sin, torch.tensor([max_len], dtype=torch.long, device="cuda"),
                               q_out, k_cache, v_cache)
    torch.cuda.synchronize()
    assert torch.equal(before, k_cache)


@pytest.mark.parametrize("H,KV,D", [(16, 8, 128), (32, 8, 128), (8, 8, 64)])
def test_attn_decode(H, KV, D):
    from llmrqt_sdv1_b200 import kernels
    max_len = 300
    k_cache, v_cache = _rand((KV, max_len, D), 5), _rand((KV, max_len, D), 6)
    q = _rand((H, D), 7)
    out = torch.empty((1, 1, H * D), dtype=torch.float16, device="cuda")
    scale = D ** -0.5
    for p in (0, 1, 7, 130, max_len - 1):
        pos = torch.tensor([p], dtype=torch.long, device="cuda")
        kernels.attn_decode(q, k_cache, v_cache, pos, out, scale)
        ref = F.scaled_dot_product_attention(q.view(1, H, 1, D).float(), k_cache[None, :, :p + 1].float(),
                                             v_cache[None, :, :p + 1].float(), enable_gqa=(H != KV), scale=scale)
        torch.cuda.synchronize()
        err = (out.view(H, D).float() - ref.view(H, D)).abs().max() / ref.abs().max()
        assert err <= 2e-3, (p, float(err))


@pytest.mark.parametrize("H,KV,D", [(16, 8, 128), (64, 8, 128), (8, 8, 64), (4, 4, 128)])
def test_attn_decode_long_context_in_chunks(H, KV, D):
    """Beyond 256 positions the cached positions are cut into chunks, one CTA per (head, chunk), merged by the
    last CTA of a head: against torch's attention, against the one-CTA-per-head form, run to run identical, and
    identical to it up to 256 positions."""
    from llmrqt_sdv1_b200 import kernels
    max_len = 4200
    k_cache, v_cache = _rand((KV, max_len, D), 15), _rand((KV, max_len, D), 16)
    q = _rand((H, D), 17, 2.0)
    out = torch.empty((H * D,), dtype=torch.float16, device="cuda")
    one = torch.empty_like(out)
    scale = D ** -0.5
    for p in (0, 200, 255, 256, 257, 511, 512, 1000, 1023, 1024, 2049, 4095, max_len - 1):
        pos = torch.tensor([p], dtype=torch.long, device="cuda")
        kernels.attn_decode(q, k_cache, v_cache, pos, out, scale)
        kernels.attn_decode(q, k_cache, v_cache, pos, one, scale, split=False)
        ref = F.scaled_dot_product_attention(q.view(1, H, 1, D).float(), k_cache[None, :, :p + 1].float(),
                                             v_cache[None, :, :p + 1].float(), enable_gqa=(H != KV), scale=scale)
        scale_ref = ref.abs().max()
        assert (out.view(H, D).float() - ref.view(H, D)).abs().max() / scale_ref <= 2e-3, p
        assert (one.view(H, D).float() - ref.view(H, D)).abs().max() / scale_ref <= 2e-3, p
        if p < 256:
            assert torch.equal(out, one), p
        again = torch.empty_like(out)
        kernels.attn_decode(q, k_cache, v_cache, pos, again, scale)
        assert torch.equal(out, again), p
    # the arrival counters are left at zero
    ws = kernels._workspaces[(0, torch.cuda.current_stream().cuda_stream, "awq_b200_attn")]
    torch.cuda.synchronize()
    assert not ws[:256].any()


@pytest.mark.parametrize("H,KV,D,with_norm", [(16, 8, 128, True), (32, 8, 128, False), (8, 2, 64, True), (4, 4, 128, True)])
def test_attn_step_equals_the_two_kernel_sequence(H, KV, D, with_norm):
    """`awq_b200_attn_step` (one launch per layer) against `qk_norm_rope_cache` followed by `attn_decode`: the same
    output bits and the same cache contents, token after token, including position 0 and the last cache row; a
    position outside the cache changes nothing."""
    from llmrqt_sdv1_b200 import kernels
    max_len, eps, scale = 1400, 1e-6, D ** -0.5
    qw, kw = (_rand((D,), 2, 0.3) + 1.0, _rand((D,), 3, 0.3) + 1.0) if with_norm else (None, None)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    ang = torch.arange(max_len, device="cuda").float()[:, None] * inv[None, :]
    cos = torch.cat((ang.cos(), ang.cos()), -1).half().contiguous()
    sin = torch.cat((ang.sin(), ang.sin()), -1).half().contiguous()
    caches = [[_rand((KV, max_len, D), 5, 0.5), _rand((KV, max_len, D), 6, 0.5)] for _ in range(2)]   # same prefill in both
    q_buf = torch.empty((H, D), dtype=torch.float16, device="cuda")
    out_a = torch.empty((H * D,), dtype=torch.float16, device="cuda")
    out_b = torch.empty_like(out_a)
    for step, p in enumerate([0, 1, 2, 3, 4, 63, 64, 65, 128, 255, 256, 257, 700, 1024, max_len - 1]):
        pos = torch.tensor([p], dtype=torch.long, device="cuda")
        qkv = _rand((1, 1, (H + 2 * KV) * D), 10 + step)
        kernels.qk_norm_rope_cache(qkv, qw, kw, eps, cos, sin, pos, q_buf, caches[0][0], caches[0][1])
        kernels.attn_decode(q_buf, caches[0][0], caches[0][1], pos, out_a, scale)
        kernels.attn_step(qkv, qw, kw, eps, cos, sin, pos, caches[1][0], caches[1][1], out_b, scale)
        assert torch.equal(out_a, out_b), f"position {p}"
        assert torch.equal(caches[0][0], caches[1][0]) and torch.equal(caches[0][1], caches[1][1]), f"position {p}"
    before = (caches[1][0].clone(), caches[1][1].clone(), out_b.clone())
    kernels.attn_step(qkv, qw, kw, eps, cos, sin, torch.tensor([max_len], dtype=torch.long, device="cuda"),
                      caches[1][0], caches[1][1], out_b, scale)
    torch.cuda.synchronize()
    assert torch.equal(caches[1][0], before[0]) and torch.equal(caches[1][1], before[1]) and torch.equal(out_b, before[2])


@pytest.mark.parametrize("shape", [(1, 1, 2048), (1, 128, 2048), (7, 4096), (3, 130)])
def test_rmsnorm_against_torch(shape):
    """`awq_b200_rmsnorm`: fp32 arithmetic, one rounding - within one fp16 step of torch.nn.functional.rms_norm (the
    order in which the squares are added is not part of either contract), and of a float64 evaluation."""
    from llmrqt_sdv1_b200 import kernels
    x = _rand(shape, 1, 2.0)
    w = _rand((shape[-1],), 2, 0.2) + 1.0
    y = kernels.rmsnorm(x, w, 1e-6)
    ref = F.rms_norm(x, (shape[-1],), w, 1e-6)
    v = x.double()
    exact = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * w.double())
    step = exact.abs().clamp_min(2.0 ** -14).log2().floor().exp2() * 2.0 ** -10
    assert bool(((y.double() - exact).abs() <= 0.51 * step + 1e-6 * exact.abs()).all())
    assert bool(((y.double() - ref.double()).abs() <= step).all())
    assert float((y != ref).float().mean()) < 0.01
