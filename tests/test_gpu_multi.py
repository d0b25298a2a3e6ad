"""Two-GPU tests of the row-parallel path: the one-shot all-reduce over peer memory against an fp32 sum
of the gathered partials, and RowParallelAWQLinear with it against the NCCL all-reduce.  Skipped on
boxes with fewer than two GPUs.  NVLS is switched off in the child processes (plain peer loads only)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from llmrqt_sdv1_b200 import quantize
        from llmrqt_sdv1_b200.sharded import PeerSum, RowParallelAWQLinear
        ok, status = True, 0
        for mode in ("push", "pull"):
            ok_mode, st = _check_mode(mode, rank, world, dev, dist, quantize, PeerSum, RowParallelAWQLinear)
            ok, status = ok and ok_mode, status | st
        results[rank] = (ok, status)
    finally:
        dist.destroy_process_group()


def _check_mode(mode, rank, world, dev, dist, quantize, PeerSum, RowParallelAWQLinear):
    if True:
        ps = PeerSum(16 * 4096, dev, mode=mode)
        ok = True
        for (M, N) in [(1, 4096), (5, 2048), (16, 4096)]:
            for it in range(4):            # the same buffers carry new data every call
                g = torch.Generator(device=dev).manual_seed(10 * it + rank)
                part = torch.randn((M, N), device=dev, generator=g).half()
                ps.partial(M, N).copy_(part)
                y = ps.reduce(M, N)
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                ref = torch.stack([p.float() for p in parts]).sum(0).half()
                ys = [torch.empty_like(y) for _ in range(world)]
                dist.all_gather(ys, y)
                ok = ok and torch.equal(y, ref) and all(torch.equal(ys[0], t) for t in ys)
        # bias is added after the sum
        bias = torch.randn(4096, device=dev, generator=torch.Generator(device=dev).manual_seed(5)).half()
        ps.partial(2, 4096).fill_(0.5)
        yb = ps.reduce(2, 4096, bias=bias)
        ok = ok and torch.equal(yb, (torch.full((2, 4096), 0.5 * world, device=dev).half() + bias))
        # the module: peer sum and NCCL all-reduce agree (fp32 sum of fp16 partials vs fp16 ring adds)
        K, N = 1024, 2048
        qw, qz, sc = quantize.random_awq_tensors(K // world, N, 128, seed=3 + rank, device=dev)
        mod = RowParallelAWQLinear.from_local(qw, qz, sc, None, 128)
        x = torch.randn((3, K // world), device=dev, generator=torch.Generator(device=dev).manual_seed(rank)).half()
        y_nccl = mod(x)
        mod.use_peer_sum(ps)
        y_peer = mod(x)
        rel = ((y_peer.float() - y_nccl.float()).abs().max() / y_nccl.float().abs().max()).item()
        ok = ok and y_peer.shape == y_nccl.shape and rel <= 2e-3
        # many rows (prefill), optional form: GEMM and NCCL all-reduce in pieces of rows, each piece's exchange behind
        # the next piece's GEMM - the same bits as one GEMM followed by one all-reduce (two ranks: one addition per element)
        if mode == "push":
            K3, N3 = 1024 * world, 2048
            qw, qz, sc = quantize.random_awq_tensors(K3 // world, N3, 128, seed=11 + rank, device=dev)
            mod3 = RowParallelAWQLinear.from_local(qw, qz, sc, None, 128)
            x3 = torch.randn((2 * 1024 + 192, K3 // world), device=dev,
                             generator=torch.Generator(device=dev).manual_seed(30 + rank)).half()
            mod3.prefill_chunk_rows = 1024
            y_pieces = mod3(x3)
            mod3.prefill_chunk_rows = 0
            y_whole = mod3(x3)
            ok = ok and y_pieces.shape == y_whole.shape and torch.equal(y_pieces, y_whole)
            ys = [torch.empty_like(y_pieces) for _ in range(world)]
            dist.all_gather(ys, y_pieces.contiguous())
            ok = ok and all(torch.equal(ys[0], t) for t in ys)
        # the exchange inside the decode kernel's epilogue: same bits as decode kernel + push kernel, and the two
        # forms may alternate (one call counter)
        if mode == "push":
            from llmrqt_sdv1_b200 import kernels
            K2, N2 = 4096 * world, 8192                                  # 16 MiB per rank
            qw, qz, sc = quantize.random_awq_tensors(K2 // world, N2, 128, seed=7 + rank, device=dev)
            bias = torch.randn(N2, device=dev, generator=torch.Generator(device=dev).manual_seed(8)).half()
            mod2 = RowParallelAWQLinear.from_local(qw, qz, sc, bias, 128)
            mod2.use_peer_sum(ps)
            pw2 = mod2.packed()
            ok = ok and not ps.can_fuse(6, pw2)                          # 5..8 rows: fused from 48 MiB per rank only
            ps.FUSED_MIN_PACKED_BYTES_5_TO_8 = 12 << 20                  # (here: the 8-row form on this shard all the same)
            for M2 in (1, 4, 2, 6, 8):
                x2 = torch.randn((M2, K2 // world), device=dev, generator=torch.Generator(device=dev).manual_seed(20 + rank + M2)).half()
                ok = ok and ps.can_fuse(M2, pw2)
                mod2.fuse_exchange = True
                y_fused = mod2(x2).view(M2, N2)
                kernels.decode_i8(x2, pw2, bias=mod2.linear.bias, out=ps.partial(M2, N2))
                y_two = ps.reduce(M2, N2)
                ok = ok and torch.equal(y_fused, y_two)
                ys = [torch.empty_like(y_fused) for _ in range(world)]
                dist.all_gather(ys, y_fused)
                ok = ok and all(torch.equal(ys[0], t) for t in ys)
            # in a graph, alternating with the standalone form
            x2 = torch.randn((1, K2 // world), device=dev, generator=torch.Generator(device=dev).manual_seed(40 + rank)).half()
            o1 = torch.empty((1, N2), dtype=torch.float16, device=dev)
            o2 = torch.empty((1, N2), dtype=torch.float16, device=dev)
            def both():
                ps.linear_push(x2, pw2, bias=mod2.linear.bias, out=o1)
                kernels.decode_i8(x2, pw2, bias=mod2.linear.bias, out=ps.partial(1, N2))
                ps.reduce(1, N2, out=o2)
            both()
            gr2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr2):
                both()
                both()
                ps.linear_push(x2, pw2, bias=mod2.linear.bias, out=o1)
            for _ in range(3):
                gr2.replay()
            torch.cuda.synchronize()
            ok = ok and torch.equal(o1, o2)
        # a graph with an odd number of calls replays correctly (the epoch, and with it the receive slot in
        # use, lives in device memory)
        outs = [torch.empty((1, 4096), dtype=torch.float16, device=dev) for _ in range(3)]
        ps.partial(1, 4096).fill_(float(rank + 1))
        for o in outs:
            ps.reduce(1, 4096, out=o)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for o in outs:
                ps.reduce(1, 4096, out=o)
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        expect = float(sum(range(1, world + 1)))
        ok = ok and all(bool((o == expect).all()) for o in outs)
        return ok, ps.status()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_allreduce_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok, status = results[rank]
        assert ok, f"rank {rank} saw a wrong sum"
        assert status == 0, f"rank {rank}: a wait on a peer expired (status {status})"
