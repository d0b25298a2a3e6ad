"""Tensor-parallel AWQ linears for weights too large for one GPU.

The reference runtime is single-GPU (LLMQRT/runtime_refact/core/base.py:44 pins
CUDA_VISIBLE_DEVICES=0); the only tensor-parallel precedent in its repository
is the fp16 Column/Merged/Row-parallel linears of
spec-decoding-src-code/eagle_ssd/ssd/layers/linear.py:68-199, whose slicing
rules these classes follow for the AWQ tensors:

* column-sharded (gate/up/qkv): rank r keeps output columns
  [r*N/tp, (r+1)*N/tp) of qweight / qzeros / scales (for a fused tensor, that
  slice of EACH fused part); activations are replicated; no collective.
* row-sharded (down/o): rank r keeps input rows [r*K/tp, (r+1)*K/tp) of
  qweight and the matching group rows of qzeros / scales; the input is the
  matching K-slice; outputs are summed with ONE all-reduce; bias is added on
  rank 0 only, before the reduction.

One process per GPU; `torch.distributed` (NCCL over NVLink on GPUs, gloo on CPU
for the host-logic tests) provides the collective.  The all-reduce runs on the
fp16 outputs; each rank's fp16 partial was rounded once from an fp32
accumulator, so tp roundings plus tp-1 fp16 additions enter the result (within
the 2e-3 layer-output bound for tp <= 8 at the tested shapes).
"""
from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .linear_awq import AWQLinear_GEMM

PACK = 8


def column_shard(qweight, qzeros, scales, bias, rank: int, world: int, parts: Sequence[int] | None = None):
    """Slice the on-disk tensors along N.  `parts` lists the widths of fused
    sub-matrices (e.g. [gate, up] or [q, k, v]); each is sliced separately and
    the slices are concatenated, so every rank holds matching pieces of all."""
    N = scales.shape[1]
    parts = list(parts) if parts else [N]
    if sum(parts) != N:
        raise ValueError(f"parts {parts} do not add up to out_features {N}")
    qw, qz, sc, bs = [], [], [], []
    start = 0
    for width in parts:
        if width % (world * PACK) != 0:
            raise ValueError(f"fused part of width {width} cannot be split {world} ways on an 8-column boundary")
        w = width // world
        lo = start + rank * w
        qw.append(qweight[:, lo // PACK:(lo + w) // PACK])
        qz.append(qzeros[:, lo // PACK:(lo + w) // PACK])
        sc.append(scales[:, lo:lo + w])
        if bias is not None:
            bs.append(bias[lo:lo + w])
        start += width
    cat = lambda xs, d: torch.cat(xs, dim=d).contiguous()
    return cat(qw, 1), cat(qz, 1), cat(sc, 1), (cat(bs, 0) if bias is not None else None)


def row_shard(qweight, qzeros, scales, group_size: int, rank: int, world: int):
    """Slice the on-disk tensors along K on a group (and 128-row) boundary."""
    K = qweight.shape[0]
    if K % world != 0 or (K // world) % group_size != 0 or (K // world) % 128 != 0:
        raise ValueError(f"in_features {K} cannot be split {world} ways on a group / 128-row boundary")
    k = K // world
    g = k // group_size
    return (qweight[rank * k:(rank + 1) * k].contiguous(), qzeros[rank * g:(rank + 1) * g].contiguous(),
            scales[rank * g:(rank + 1) * g].contiguous())


def _world(group):
    if not dist.is_available() or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def _local_linear(qw, qz, sc, bias, group_size, device) -> AWQLinear_GEMM:
    K, n = qw.shape[0], sc.shape[1]
    lin = AWQLinear_GEMM(4, group_size, K, n, bias is not None, device)
    lin.qweight.copy_(qw)
    lin.qzeros.copy_(qz)
    lin.scales.copy_(sc)
    if bias is not None:
        lin.bias.copy_(bias)
    return lin


def _packed(lin: AWQLinear_GEMM):
    return lin.packed()


class ColumnParallelAWQLinear(nn.Module):
    """y_local = x . W[:, shard]; optionally all-gathers the shards along N."""

    def __init__(self, qweight, qzeros, scales, bias, group_size: int, parts: Sequence[int] | None = None,
                 gather_output: bool = False, group=None, device=None):
        super().__init__()
        self.group = group
        self.rank, self.world = _world(group)
        self.gather_output = gather_output
        qw, qz, sc, b = column_shard(qweight, qzeros, scales, bias, self.rank, self.world, parts)
        self.linear = _local_linear(qw, qz, sc, b, group_size, device if device is not None else qweight.device)
        self.out_features = scales.shape[1]

    @classmethod
    def from_local(cls, qweight, qzeros, scales, bias, group_size: int, gather_output: bool = False, group=None):
        """Wrap tensors that already are this rank's column shard."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.group, self.gather_output = group, gather_output
        self.rank, self.world = _world(group)
        self.linear = _local_linear(qweight, qzeros, scales, bias, group_size, qweight.device)
        self.out_features = scales.shape[1] * self.world
        return self

    def packed(self):
        return _packed(self.linear)

    def forward(self, x):
        y = self.linear(x)
        if self.gather_output and self.world > 1:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            y = torch.cat(parts, dim=-1)
        return y


class PeerSum:
    """One-shot sum of small row-parallel partial outputs over peer memory (NVLink), for CUDA ranks of
    one node.  Each rank writes its fp16 partial into `partial(M, N)`; `reduce` launches the library's peer
    all-reduce kernel, which adds the ranks' partials in rank order in fp32 and writes the fp16 result
    locally (identical bits on every rank).  Replaces an NCCL all-reduce whose cost at these sizes
    (16 KB ... 1 MB) is all latency.  One instance serves any number of layers on a stream.

    mode "push" (default): every rank stores its partial into a receive slot on each peer in a wire format
    that carries its own flag; a rank waits for one one-way trip, polling its own memory.  mode "pull": every rank publishes a flag
    and reads the peers' partials with peer loads, then waits until all peers have read its own."""

    def __init__(self, max_elems: int, device, group=None, mode: str = "push"):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        if mode not in ("push", "pull"):
            raise ValueError(f"mode must be 'push' or 'pull', got {mode!r}")
        group = group if group is not None else dist.group.WORLD
        self.group, self.mode = group, mode
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.max_elems = (int(max_elems) + 7) // 8 * 8
        self.buf = symm_mem.empty(self.max_elems, dtype=torch.float16, device=device)
        self.flags = symm_mem.empty(_lib.lib.awq_b200_peer_allreduce_flag_bytes() // 4, dtype=torch.int32, device=device)
        self.flags.zero_()
        self._h_buf = symm_mem.rendezvous(self.buf, group)
        self._h_flags = symm_mem.rendezvous(self.flags, group)
        if mode == "push":
            # wire format: 4 bytes per fp16 element, two parities, one slot per rank
            self.recv = symm_mem.empty(4 * self.world * self.max_elems, dtype=torch.float16, device=device)
            self.recv.zero_()
            self._h_recv = symm_mem.rendezvous(self.recv, group)
        torch.cuda.synchronize(device)
        dist.barrier(group)            # every rank's flags are zero before anyone signals

    def fits(self, M: int, N: int) -> bool:
        return M * N <= self.max_elems and (M * N) % 8 == 0

    def partial(self, M: int, N: int) -> torch.Tensor:
        return self.buf[:M * N].view(M, N)

    def reduce(self, M: int, N: int, out: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> torch.Tensor:
        from . import kernels
        if self.mode == "push":
            return kernels.peer_allreduce_push(self.buf, self._h_recv.buffer_ptrs_dev, self._h_flags.buffer_ptrs_dev,
                                               self.max_elems, M, N, self.rank, self.world, out=out, bias=bias)
        return kernels.peer_allreduce(self._h_buf.buffer_ptrs_dev, self._h_flags.buffer_ptrs_dev, self.buf,
                                      M, N, self.rank, self.world, out=out, bias=bias)

    # The fused form: one to four rows of a shard whose weights are large enough for the integer decode kernel
    # (about what that kernel needs to beat the GEMV plus a separate exchange launch); five to eight rows from
    # the size at which the dispatcher gives them to that kernel anyway.
    FUSED_MAX_ROWS, FUSED_MIN_PACKED_BYTES = 8, 12 << 20
    FUSED_MIN_PACKED_BYTES_5_TO_8 = 48 << 20

    def can_fuse(self, M: int, pw) -> bool:
        """Whether `linear_push` serves M rows of this packed shard (push mode, 2..8 ranks, group size >= 128)."""
        need = self.FUSED_MIN_PACKED_BYTES if M <= 4 else self.FUSED_MIN_PACKED_BYTES_5_TO_8
        return (self.mode == "push" and 2 <= self.world <= 8 and 1 <= M <= self.FUSED_MAX_ROWS
                and pw.group_size % 128 == 0 and pw.K * pw.N // 2 >= need and self.fits(M, pw.N))

    def linear_push(self, x2d: torch.Tensor, pw, bias=None, out: torch.Tensor | None = None,
                    overlap: bool = False) -> torch.Tensor:
        """This rank's row shard times its activations AND the sum over the ranks, in one launch: the decode
        kernel's epilogue pushes each finished pair of results to the peers and collects theirs.  Same bits as
        `kernels.decode_i8` into `partial()` followed by `reduce()`; counts as one call of the exchange."""
        from . import kernels
        return kernels.decode_i8_push(x2d, pw, self._h_recv.buffer_ptrs_dev, self._h_flags.buffer_ptrs_dev,
                                      self.max_elems, self.rank, self.world, bias=bias, out=out, overlap=overlap)

    STATUS_WORD, WAIT_LIMIT_WORD = 34, 37      # AWQ_B200_PEER_STATUS_WORD / AWQ_B200_PEER_WAIT_LIMIT_WORD

    def status(self) -> int:
        """0, or which wait expired in some call (1: peers' partials, 2: peers' reads, 3: peers' pushes).
        Sticky until `reset`.  Synchronises."""
        return int(self.flags[self.STATUS_WORD].item())

    def check(self) -> None:
        """Raise if a wait on a peer has expired since the last reset (the outputs of that call and of
        every later call are invalid: the ranks' call counters no longer agree)."""
        st = self.status()
        if st != 0:
            raise RuntimeError(f"peer all-reduce: a wait on a peer expired (status {st}); call reset() on every rank")

    def set_wait_limit(self, seconds: float | None, sm_clock_hz: float = 1.9e9) -> None:
        """How long one call may wait for its peers before it gives up and sets the status word
        (None = the library's default of about 2 s).  Takes effect with the next launch."""
        kcycles = 0 if seconds is None else max(1, min(0xFFFFFFFF, int(seconds * sm_clock_hz / 1024)))
        self.flags[self.WAIT_LIMIT_WORD] = kcycles if kcycles < 2 ** 31 else kcycles - 2 ** 32

    def reset(self) -> None:
        """Collective: bring every rank's call counters, flags, status word and receive slots back to their
        initial state after an expired wait or a mismatched number of calls.  All ranks must call it, with
        no exchange in flight; the wait limit is kept."""
        torch.cuda.synchronize(self.flags.device)
        dist.barrier(self.group)           # nobody is still pushing into a slot that is about to be cleared
        limit = self.flags[self.WAIT_LIMIT_WORD].clone()
        self.flags.zero_()
        self.flags[self.WAIT_LIMIT_WORD] = limit
        if self.mode == "push":
            self.recv.zero_()
        torch.cuda.synchronize(self.flags.device)
        dist.barrier(self.group)


# Rows per piece when a row-parallel linear of many rows is cut so that the all-reduce of one piece may run while
# the GEMM of the next does; 0 = one GEMM, then one all-reduce.  Off by default: the GEMM is a persistent kernel on
# every SM, so NCCL's kernel mostly waits for it anyway, and smaller GEMMs fill their last wave worse (70B down
# projection, 4096 rows, 8 layers: 20.9 against 21.1 ms in pieces of 1024 rows on 2 GPUs, 7.37 against 6.94 ms on 8).
PREFILL_CHUNK_ROWS = 0


def linear_all_reduce(x2d: torch.Tensor, pw, bias=None, out: torch.Tensor | None = None, group=None,
                      chunk_rows: int = PREFILL_CHUNK_ROWS) -> torch.Tensor:
    """Row-parallel linear of many rows (prefill): y = all_reduce_sum(x2d . W_shard (+ bias)).

    With `chunk_rows` > 0 the rows are cut into pieces; each piece's NCCL all-reduce is started asynchronously
    right behind its GEMM (on NCCL's stream) and may run while the next piece's GEMM does.  `chunk_rows <= 0` or
    fewer than two pieces: one GEMM, one all-reduce.
    Returns after making the current stream wait for every piece."""
    from . import kernels
    rows, N = x2d.shape[0], pw.N
    if out is None:
        out = torch.empty((rows, N), dtype=torch.float16, device=x2d.device)
    pieces = 1 if chunk_rows <= 0 else rows // chunk_rows
    if pieces < 2:
        kernels.linear(x2d, pw, bias=bias, out=out)
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out
    works = []
    for c in range(pieces):
        r0 = c * chunk_rows
        r1 = rows if c == pieces - 1 else r0 + chunk_rows
        piece = out[r0:r1]
        kernels.linear(x2d[r0:r1], pw, bias=bias, out=piece)
        works.append(dist.all_reduce(piece, op=dist.ReduceOp.SUM, group=group, async_op=True))
    for w in works:
        w.wait()
    return out


class RowParallelAWQLinear(nn.Module):
    """y = all_reduce_sum( x[..., shard] . W[shard, :] ) (+ bias on rank 0)."""

    def __init__(self, qweight, qzeros, scales, bias, group_size: int, input_is_parallel: bool = True,
                 group=None, device=None):
        super().__init__()
        self.group = group
        self.rank, self.world = _world(group)
        self.input_is_parallel = input_is_parallel
        G = qweight.shape[0] if group_size == -1 else group_size
        qw, qz, sc = row_shard(qweight, qzeros, scales, G, self.rank, self.world)
        self.linear = _local_linear(qw, qz, sc, bias if self.rank == 0 else None, G,
                                    device if device is not None else qweight.device)
        self.in_features = qweight.shape[0]
        self.k_local = qw.shape[0]

    @classmethod
    def from_local(cls, qweight, qzeros, scales, bias, group_size: int, input_is_parallel: bool = True, group=None):
        """Wrap tensors that already are this rank's row shard (bias is kept on rank 0 only)."""
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        self.group, self.input_is_parallel = group, input_is_parallel
        self.rank, self.world = _world(group)
        G = qweight.shape[0] if group_size == -1 else group_size
        self.linear = _local_linear(qweight, qzeros, scales, bias if self.rank == 0 else None, G, qweight.device)
        self.k_local = qweight.shape[0]
        self.in_features = self.k_local * self.world
        return self

    def packed(self):
        return _packed(self.linear)

    def use_peer_sum(self, peer_sum: PeerSum | None) -> None:
        """Sum small outputs with `peer_sum` (shared between layers) instead of an NCCL all-reduce."""
        self.peer_sum = peer_sum

    def forward(self, x):
        if not self.input_is_parallel:
            x = x[..., self.rank * self.k_local:(self.rank + 1) * self.k_local]
        ps = getattr(self, "peer_sum", None)
        if ps is not None and self.world > 1 and x.is_cuda and x.dtype == torch.float16:
            rows = x.numel() // x.shape[-1]
            N = self.linear.out_features
            if ps.fits(rows, N):
                from . import kernels
                pw = self.packed()
                overlap, pw.fresh = not pw.fresh, False     # first call after a repack: no weight prefetch
                if getattr(self, "fuse_exchange", True) and ps.can_fuse(rows, pw):
                    y = ps.linear_push(x.reshape(rows, -1), pw, bias=self.linear.bias, overlap=overlap)
                    return y.view(*x.shape[:-1], N) if x.dim() > 2 else y.view(1, rows, N)
                kernels.linear(x.reshape(rows, -1), pw, bias=self.linear.bias, out=ps.partial(rows, N),
                               overlap=overlap)
                y = ps.reduce(rows, N)
                return y.view(*x.shape[:-1], N) if x.dim() > 2 else y.view(1, rows, N)
        if self.world > 1 and x.is_cuda and x.dtype == torch.float16:
            rows = x.numel() // x.shape[-1]
            chunk = getattr(self, "prefill_chunk_rows", PREFILL_CHUNK_ROWS)
            if chunk > 0 and rows >= 2 * chunk:
                pw = self.packed()
                pw.fresh = False
                y = linear_all_reduce(x.reshape(rows, -1), pw, bias=self.linear.bias, group=self.group, chunk_rows=chunk)
                return y.view(*x.shape[:-1], -1) if x.dim() > 2 else y.view(1, rows, -1)
        y = self.linear(x)
        if self.world > 1:
            y = y.contiguous()
            dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y
