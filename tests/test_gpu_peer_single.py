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

    def fused(self, x, pw, out=None, bias=None, overlap=False):
        """Rank 0's row shard through the decode kernel whose epilogue does the push exchange itself."""
        from llmrqt_sdv1_b200 import kernels
        return kernels.decode_i8_push(x, pw, self.recv_tab.data_ptr(), self.flags_tab.data_ptr(), self.slot_elems, 0,
                                      WORLD, bias=bias, out=out, overlap=overlap)

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


# ---------------------------------------------------------------------------------------------------------------
# The decode kernel that performs the push exchange in its epilogue (awq_b200_decode_i8_push)
# ---------------------------------------------------------------------------------------------------------------
def _packed(K, N, seed):
    from llmrqt_sdv1_b200 import kernels, quantize
    qw, qz, sc = quantize.random_awq_tensors(K, N, 128, seed=seed, device="cuda")
    return kernels.make_packed(qw, qz, sc, 128)


@pytest.mark.parametrize("K,N", [(1024, 2048),        # 8 column tiles x 8 blocks = 64 units: one CTA per unit, shared tiles
                                 (8192, 8192),        # 32 tiles x 64 blocks: several CTAs per tile, all through partials
                                 (128, 80 * 256)])    # 80 tiles x 1 block: every CTA owns its tile (direct stores)
def test_fused_exchange_equals_decode_then_push(K, N):
    """Same bits as the decode kernel into a partial followed by the push kernel; the words sent to the peer are
    this rank's partial in wire format; the call counter advances once per call; bias goes into the partial."""
    from llmrqt_sdv1_b200 import kernels
    pw = _packed(K, N, seed=K + N)
    rig = _Rig(8 * N)
    epoch = 0
    for call, M in enumerate((1, 2, 4, 3, 8, 5, 1)):
        epoch += 1
        x = _rand((M, K), 50 + call)
        bias = _rand((N,), 60 + call) if call % 2 else None
        theirs = _rand((M, N), 70 + call)
        mine = kernels.decode_i8(x, pw, bias=bias)                 # what the unfused path would push
        rig.peer_pushes(theirs, epoch)
        y = rig.fused(x, pw, bias=bias, overlap=(call % 2 == 0))
        torch.cuda.synchronize()
        assert torch.equal(y, _fp32_sum(mine, theirs)), f"call {call}: wrong sum"
        sent, counters_ok = rig.sent_by_rank0(M * N, epoch)
        assert counters_ok and torch.equal(sent.view(M, N), mine), f"call {call}: wire words sent to the peer are wrong"
        assert int(rig.flags[0][35].item()) == epoch
    # the standalone push kernel continues the same call sequence (shared counter and slots)
    epoch += 1
    mine, theirs = _rand((1, N), 1), _rand((1, N), 2)
    rig.peer_pushes(theirs, epoch)
    assert torch.equal(rig.push(mine, 1, N), _fp32_sum(mine, theirs))
    torch.cuda.synchronize()
    assert int(rig.flags[0][STATUS].item()) == 0
    assert kernels.gemv_status() == 0


@pytest.mark.parametrize("M", [1, 4, 7])       # from 3 rows: the forms behind the kernel that writes the activation planes
def test_fused_exchange_inside_a_replayed_graph(M):
    from llmrqt_sdv1_b200 import kernels
    K, N = 4096, 4096
    pw = _packed(K, N, seed=9)
    rig = _Rig(M * N)
    x = [_rand((M, K), 20), _rand((M, K), 21), _rand((M, K), 22)]
    mine = [kernels.decode_i8(xi, pw) for xi in x]
    outs = [torch.empty((M, N), dtype=torch.float16, device="cuda") for _ in x]
    epoch = 0

    def fill(seed):
        theirs = [_rand((M, N), seed + j) for j in range(3)]
        # three calls per replay: the third reuses the parity of the first, so the host writes it after the
        # first two slots have been consumed - here all three are written up front into distinct epochs' words
        for j, t in enumerate(theirs[:2]):
            rig.peer_pushes(t, epoch + 1 + j)
        return theirs

    theirs = fill(200)
    for o, xi in zip(outs[:2], x[:2]):
        rig.fused(xi, pw, out=o)
    torch.cuda.synchronize()
    epoch += 2
    for j in range(2):
        assert torch.equal(outs[j], _fp32_sum(mine[j], theirs[j]))
    g = torch.cuda.CUDAGraph()
    theirs = fill(300)
    with torch.cuda.graph(g):
        for o, xi in zip(outs[:2], x[:2]):
            rig.fused(xi, pw, out=o)
    for rep in range(3):
        theirs = fill(400 + 10 * rep)
        g.replay()
        torch.cuda.synchronize()
        epoch += 2
        for j in range(2):
            assert torch.equal(outs[j], _fp32_sum(mine[j], theirs[j])), f"replay {rep}, call {j}"
    assert int(rig.flags[0][35].item()) == epoch and int(rig.flags[0][STATUS].item()) == 0


def test_fused_exchange_refuses_more_than_eight_rows():
    pw = _packed(1024, 2048, seed=1)
    rig = _Rig(16 * 2048)
    with pytest.raises(ValueError):
        rig.fused(_rand((9, 1024), 1), pw)
    torch.cuda.synchronize()
    assert int(rig.flags[0][35].item()) == 0 and int(rig.flags[0][STATUS].item()) == 0


def test_fused_exchange_wait_runs_out_sets_status_and_reset_recovers():
    """Nothing arrives from the peer and the limit is ~1 ms: the kernel returns, status 3, the context stays usable;
    after a reset the next matched call is correct."""
    from llmrqt_sdv1_b200 import kernels
    K, N = 2048, 4096
    pw = _packed(K, N, seed=3)
    rig = _Rig(N)
    rig.flags[0][LIMIT] = 2000                      # x 1024 cycles: about a millisecond
    x = _rand((1, K), 5)
    rig.fused(x, pw)
    torch.cuda.synchronize()
    assert int(rig.flags[0][STATUS].item()) == 3
    rig.reset()
    theirs = _rand((1, N), 6)
    rig.peer_pushes(theirs, 1)
    y = rig.fused(x, pw)
    torch.cuda.synchronize()
    assert torch.equal(y, _fp32_sum(kernels.decode_i8(x, pw), theirs))
    assert int(rig.flags[0][STATUS].item()) == 0
