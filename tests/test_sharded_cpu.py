"""Host logic of the tensor-parallel linears on CPU ranks (gloo, world_size 2):
slicing rules, the row-parallel all-reduce, bias placement, fused-part handling,
and that a rank failing before the collective surfaces as an exception on its
peer instead of a hang.  The local matmul of each rank is done by the oracle
(the product has no CPU kernel), so this checks everything around the kernel."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import awq_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_forward(lin):
    def fwd(x):
        b = lin.bias.numpy() if lin.bias is not None else None
        y = orc.linear_forward(x.numpy(), lin.qweight.numpy(), lin.qzeros.numpy(), lin.scales.numpy(),
                               lin.group_size, b)
        return torch.from_numpy(y)
    return fwd


def _worker(rank, world, port, case, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from llmrqt_sdv1_b200.sharded import ColumnParallelAWQLinear, RowParallelAWQLinear
    K, N, G = 512, 256, 128
    qw, qz, sc = (torch.from_numpy(t) for t in orc.make_awq_tensors(K, N, G, seed=3))
    bias = torch.from_numpy(np.random.default_rng(0).standard_normal(N).astype(np.float16))
    x = torch.from_numpy(orc.make_activations(3, K, seed=1))
    try:
        if case == "column":
            m = ColumnParallelAWQLinear(qw, qz, sc, bias, G, parts=[128, 128], gather_output=True)
            m.linear.forward = _oracle_forward(m.linear)
            y = m(x)
            # gathered layout is [rank0: gate-half, up-half | rank1: ...]; undo the fused interleave
            w = N // 2 // world
            cols = [y[..., r * 2 * w + p * w: r * 2 * w + (p + 1) * w] for p in range(2) for r in range(world)]
            y = torch.cat(cols, dim=-1)
        elif case == "row":
            m = RowParallelAWQLinear(qw, qz, sc, bias, G, input_is_parallel=False)
            assert (m.linear.bias is not None) == (rank == 0)
            m.linear.forward = _oracle_forward(m.linear)
            y = m(x)
        elif case == "row_peer_fails":
            m = RowParallelAWQLinear(qw, qz, sc, None, G, input_is_parallel=False)
            m.linear.forward = _oracle_forward(m.linear)
            if rank == 1:
                raise RuntimeError("injected failure before the collective")
            try:
                m(x)
                outcome = "completed"
            except Exception as e:   # peer is gone: gloo reports it, nothing hangs
                outcome = "raised:" + type(e).__name__
            open(os.path.join(out_dir, "outcome.txt"), "w").write(outcome)
            return
        if rank == 0:
            np.save(os.path.join(out_dir, f"{case}.npy"), y.numpy())
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(case, tmp_path, expect_ok=True):
    port = _free_port()
    ctx = mp.spawn(_worker, args=(2, port, case, str(tmp_path)), nprocs=2, join=False)
    try:
        while not ctx.join(timeout=60):
            pass
    except Exception:
        if expect_ok:
            raise


def _reference(bias=True):
    K, N, G = 512, 256, 128
    qw, qz, sc = orc.make_awq_tensors(K, N, G, seed=3)
    b = np.random.default_rng(0).standard_normal(N).astype(np.float16) if bias else None
    x = orc.make_activations(3, K, seed=1)
    return orc.linear_forward(x, qw, qz, sc, G, b)


def test_column_parallel_two_ranks(tmp_path):
    _run("column", tmp_path)
    y = np.load(tmp_path / "column.npy")
    assert np.array_equal(y.view(np.uint16), _reference().view(np.uint16))   # no reduction: bit-equal


def test_row_parallel_two_ranks(tmp_path):
    _run("row", tmp_path)
    y = np.load(tmp_path / "row.npy")
    assert orc.max_normalised_error(y, _reference()) <= 2e-3   # two fp16 partials added: within the layer bound


def test_row_parallel_peer_failure_does_not_hang(tmp_path):
    _run("row_peer_fails", tmp_path, expect_ok=False)
    outcome = (tmp_path / "outcome.txt").read_text()
    assert outcome.startswith("raised:"), outcome


def test_shard_validation():
    from llmrqt_sdv1_b200.sharded import column_shard, row_shard
    qw, qz, sc = (torch.from_numpy(t) for t in orc.make_awq_tensors(256, 64, 128, seed=0))
    with pytest.raises(ValueError):
        row_shard(qw, qz, sc, 128, 0, 4)          # 64 rows per rank: below the 128-row group
    with pytest.raises(ValueError):
        column_shard(qw, qz, sc, None, 0, 2, parts=[40, 24])
    a, b, c, _ = column_shard(qw, qz, sc, None, 1, 2)
    assert a.shape == (256, 4) and b.shape == (2, 4) and c.shape == (2, 32)
    assert torch.equal(c, sc[:, 32:])
