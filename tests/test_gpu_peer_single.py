"""The one-shot peer all-reduce on ONE GPU, with the peer played by the host.

Two kernels that wait for each other must not run as separate launches on one GPU (nothing makes them
run at the same time), so the second rank is not a kernel here: the test itself writes what rank 1 would
have sent (wire-format words or flags) into rank 0's memory BEFORE rank 0's call is launched, and checks
afterwards what rank 0 sent to rank 1's area.  Every launched kernel therefore finds its data present and
never waits - except in the expiry tests, where nothing is written, the wait limit is set to about a
millisecond, and the kernel must come back with the status word set (no fault, no hang).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

WORLD = 2
STATUS, LIMIT = 34, 37          # AWQ_B200_PEER_STATUS_WORD / AWQ_B200_PEER_WAIT_LIMIT_WORD


class _Rig:
    """Rank 0's view of a two-rank exchange whose buffers all live on this GPU."""

    def __init__(self, slot_elems: int):
        from llmrqt_sdv1_b200 import _lib
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        self.dev, self.slot_elems = dev, slot_elems
        nflag = _lib.lib.awq_b200_peer_allreduce_flag_bytes() // 4
        self.flags = [torch.zeros(nflag, dtype=torch.int32, device=dev) for _ in range(WORLD)]
        # push form: per rank 2 parities x WORLD slots x slot_elems elements x 4 bytes
        self.recv = [torch.zeros(2 * WORLD * slot_elems, dtype=torch.int32, device=dev) for _ in range(WORLD)]
        # pull form: one partial buffer per rank
        self.bufs = [torch.zeros(slot_elems, dtype=torch.float16, device=dev) for _ in range(WORLD)]
        self.flags_tab = torch.tensor([t.data_ptr() for t in self.flags], dtype=torch.int64, device=dev)
        self.recv_tab = torch.tensor([t.data_ptr() for t in self.recv], dtype=torch.int64, device=dev)
        self.bufs_tab = torch.tensor([t.data_ptr() for t in self.bufs], dtype=torch.int64, device=dev)

    def slot(self, rank: int, parity: int, sender: int) -> torch.Tensor:
        w = self.slot_elems          # int32 words per slot: 4 bytes per fp16 element
        at = (parity * WORLD + sender) * w
        return self.recv[rank][at:at + w]

    def peer_pushes(self, part: torch.Tensor, epoch: int) -> None:
        """What rank 1's call `epoch` stores into rank 0's receive slot: {payload word, epoch} pairs."""
        payload = part.contiguous().view(-1).view(torch.int32)
        wire = torch.stack((payload, torch.full_like(payload, epoch)), dim=1).reshape(-1)
        self.slot(0, epoch & 1, 1)[:wire.numel()].copy_(wire)

    def sent_by_rank0(self, count: int, epoch: int):
        """Decode what rank 0 pushed into rank 1's slot: (payload as fp16, all counters equal `epoch`)."""
        wire = self.slot(1, epoch & 1, 0)[:count].view(-1, 2)
        return wire[:, 0].contiguous().view(torch.float16), bool((wire[:, 1] == epoch).all())

    def reset(self) -> None:
        torch.cuda.synchronize()
        for f in self.flags:
            limit = f[LIMIT].clone()
            f.zero_()
            f[LIMIT] = limit
        for r in self.recv:
            r.zero_()

    def push(self, part, M, N, out=None, bias=None):
        from llmrqt_sdv1_b200 import kernels
        return kernels.peer_allreduce_push(part, self.recv_tab.data_ptr(), self.flags_tab.data_ptr(),
                                           self.slot_elems, M, N, 0, WORLD, out=out, bias=bias)

    def pull(self, M, N, out=None, bias=None):
        from llmrqt_sdv1_b200 import kernels
        return kernels.peer_allreduce(self.bufs_tab.data_ptr(), self.flags_tab.data_ptr(), self.bufs[0], M, N, 0,
                                      WORLD, out=out, bias=bias)


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, device="cuda", generator=g).half()


def _fp32_sum(a, b):
    return (a.float() + b.float()).half()


def test_push_wire_format_and_slot_parity_over_calls():
    rig = _Rig(16 * 4096)
    epoch = 0
    for call, (M, N) in enumerate([(1, 4096), (1, 4096), (5, 2048), (16, 4096), (3, 1024), (1, 8192), (1, 4096)]):
        epoch += 1
        mine, theirs = _rand((M, N), 2 * call), _rand((M, N), 2 * call + 1)
        rig.peer_pushes(theirs, epoch)
        y = rig.push(mine, M, N)
        torch.cuda.synchronize()
        assert torch.equal(y, _fp32_sum(mine, theirs)), f"call {call}: wrong sum"
        sent, counters_ok = rig.sent_by_rank0(M * N, epoch)
        assert counters_ok and torch.equal(sent.view(M, N), mine), f"call {call}: wire words sent to the peer are wrong"
    assert int(rig.flags[0][STATUS].item()) == 0
    assert int(rig.flags[0][35].item()) == epoch        # the call counter lives in device memory


def test_push_bias_is_added_after_the_sum():
    rig = _Rig(4096)
    mine, theirs, bias = _rand((2, 2048), 1), _rand((2, 2048), 2), _rand((2048,), 3)
    rig.peer_pushes(theirs, 1)
    y = rig.push(mine, 2, 2048, bias=bias)
    torch.cuda.synchronize()
    assert torch.equal(y, _fp32_sum(mine, theirs) + bias)


def test_push_inside_a_replayed_graph():
    """Two calls per replay use the two slot parities; the host rewrites both slots between replays."""
    rig = _Rig(4096)
    mine = [_rand((1, 4096), 10), _rand((1, 4096), 11)]
    outs = [torch.empty((1, 4096), dtype=torch.float16, device="cuda") for _ in range(2)]
    epoch = 0

    def fill(seed):
        theirs = [_rand((1, 4096), seed), _rand((1, 4096), seed + 1)]
        for j, t in enumerate(theirs):
            rig.peer_pushes(t, epoch + 1 + j)
        return theirs

    fill(100)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for j in range(2):                     # warm-up outside the capture, consumes epochs 1 and 2
            rig.push(mine[j], 1, 4096, out=outs[j])
        side.synchronize()
        epoch = 2
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for j in range(2):
                rig.push(mine[j], 1, 4096, out=outs[j])
    torch.cuda.current_stream().wait_stream(side)
    for replay in range(3):
        theirs = fill(200 + 10 * replay)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        epoch += 2
        for j in range(2):
            assert torch.equal(outs[j], _fp32_sum(mine[j], theirs[j])), f"replay {replay}, call {j}"
    assert int(rig.flags[0][STATUS].item()) == 0


def test_push_wait_runs_out_sets_status_and_reset_recovers():
    rig = _Rig(4096)
    rig.flags[0][LIMIT] = 2000                  # 2000 x 1024 cycles: about a millisecond
    mine, theirs = _rand((1, 4096), 1), _rand((1, 4096), 2)
    rig.push(mine, 1, 4096)                     # nobody pushed: the wait must give up and the kernel return
    torch.cuda.synchronize()
    assert int(rig.flags[0][STATUS].item()) == 3
    rig.reset()
    assert int(rig.flags[0][STATUS].item()) == 0 and int(rig.flags[0][LIMIT].item()) == 2000
    rig.peer_pushes(theirs, 1)                  # counters start again at 1 after a reset
    y = rig.push(mine, 1, 4096)
    torch.cuda.synchronize()
    assert torch.equal(y, _fp32_sum(mine, theirs))
    assert int(rig.flags[0][STATUS].item()) == 0


def test_pull_form_with_flags_set_by_the_host():
    rig = _Rig(16 * 4096)
    epoch = 0
    for call, (M, N) in enumerate([(1, 4096), (4, 2048), (16, 4096), (1, 4096), (2, 1024)]):
        epoch += 1
        mine, theirs = _rand((M, N), 50 + 2 * call), _rand((M, N), 51 + 2 * call)
        rig.bufs[0][:M * N].copy_(mine.view(-1))
        rig.bufs[1][:M * N].copy_(theirs.view(-1))
        rig.flags[0][1] = epoch                 # rank 1: "my partial is written"
        rig.flags[0][17] = epoch                # rank 1: "I have read yours"
        y = rig.pull(M, N)
        torch.cuda.synchronize()
        assert torch.equal(y, _fp32_sum(mine, theirs)), f"call {call}"
        assert int(rig.flags[1][0].item()) == epoch and int(rig.flags[1][16].item()) == epoch   # what rank 0 told rank 1
    assert int(rig.flags[0][STATUS].item()) == 0


def test_pull_wait_runs_out_sets_status():
    rig = _Rig(4096)
    rig.flags[0][LIMIT] = 2000
    rig.bufs[0].fill_(1.0)
    rig.pull(1, 4096)                           # rank 1 never signals
    torch.cuda.synchronize()
    assert int(rig.flags[0][STATUS].item()) in (1, 2)
    rig.reset()
    rig.bufs[1].fill_(2.0)
    rig.flags[0][1] = 1
    rig.flags[0][17] = 1
    y = rig.pull(1, 4096)
    torch.cuda.synchronize()
    assert bool((y == 3.0).all()) and int(rig.flags[0][STATUS].item()) == 0
