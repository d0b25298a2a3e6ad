"""Every cell of the benchmark configurations at full size, through the dispatcher the module calls
(`kernels.linear`), against device dequantisation (bit-exact to the reference's `dequantize_gemm`, checked
in test_gpu_parity.py) followed by a library matmul on the same device.

  decode linears   Qwen3-1.7B shapes x M in {1, 4, 8, 16}
  prefill GEMMs    Llama-3-8B shapes x M in {512, 2048, 8192}
  sharded FFN      70B-class gate_up column shards / down row shards at tp in {1, 2, 4, 8} x M in {1, 16, 4096}
                   (a shard is just a smaller linear, so one GPU checks every shard shape)
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-3   # max|y - ref| / max|ref|


def _random_packed_inputs(K, N, G, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    qw = torch.randint(-2**31, 2**31 - 1, (K, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    qz = torch.randint(-2**31, 2**31 - 1, (K // G, N // 8), dtype=torch.int64, device="cuda", generator=g).to(torch.int32)
    sc = (torch.rand((K // G, N), device="cuda", generator=g) * 0.004 + 0.001).half()
    return qw, qz, sc


def _check(K, N, Ms, seed):
    from llmrqt_sdv1_b200 import kernels
    qw, qz, sc = _random_packed_inputs(K, N, 128, seed)
    pw = kernels.make_packed(qw, qz, sc, 128)
    W = kernels.dequantize(qw, qz, sc, 128)
    del qw
    for M in Ms:
        x = torch.randn((M, K), device="cuda", generator=torch.Generator(device="cuda").manual_seed(M)).half()
        y = kernels.linear(x, pw)
        again = kernels.linear(x, pw)
        ref = torch.matmul(x, W).float()       # fp16 inputs, fp32 accumulation inside the library
        err = float((y.float() - ref).abs().max() / ref.abs().max())
        assert err <= TOL, f"M={M} K={K} N={N}: {err}"
        assert torch.equal(y, again), f"M={M} K={K} N={N}: two calls differ"
        del x, y, again, ref
    torch.cuda.synchronize()
    assert kernels.gemm_status() == 0 and kernels.gemv_status() == 0
    del W, pw
    torch.cuda.empty_cache()


@pytest.mark.parametrize("K,N", [(2048, 6144), (2048, 4096), (2048, 2048), (2048, 12288), (6144, 2048)])
def test_decode_cells(K, N):
    _check(K, N, (1, 4, 8, 16), seed=K + N)


@pytest.mark.parametrize("K,N", [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)])
def test_prefill_cells(K, N):
    _check(K, N, (512, 2048, 8192), seed=K + N + 1)


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_sharded_ffn_cells(tp):
    _check(8192, 57344 // tp, (1, 16, 4096), seed=100 + tp)     # gate_up, column shard
    _check(28672 // tp, 8192, (1, 16, 4096), seed=200 + tp)     # down, row shard (the partial sum of one rank)
