"""Torch-level wrappers over the C ABI: they allocate outputs and workspaces
with torch, pass raw device pointers plus the current stream, and turn status
codes into exceptions.  No arithmetic happens here."""
from __future__ import annotations

from ctypes import addressof as _addressof

import torch

from . import _lib
from ._lib import check, lib

GEMV_MAX_ROWS = lib.awq_b200_gemv_max_rows()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


# The raw handle of the current stream without building a torch.cuda.Stream object (2 us cheaper per call).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _prep(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    if dev.type != "cuda":
        raise RuntimeError("llmrqt_sdv1_b200 kernels need CUDA tensors; there is no CPU fallback")
    for t in tensors:
        if t is not None and t.device != dev:
            raise RuntimeError("all tensors of one call must be on the same device")
    _lib.set_device(dev.index if dev.index is not None else torch.cuda.current_device())
    return dev


def _kn(qweight: torch.Tensor) -> tuple[int, int]:
    if qweight.dtype != torch.int32 or qweight.dim() != 2:
        raise ValueError("qweight must be int32 [K, N/8]")
    return qweight.shape[0], qweight.shape[1] * 8


class PackedWeight:
    """Kernel-layout weight of one linear: packed nibbles plus the on-disk
    scales / qzeros it is used with."""
    __slots__ = ("packed", "qzeros", "scales", "K", "N", "group_size", "fresh", "_ptrs", "_ws_need")

    def __init__(self, packed, qzeros, scales, K, N, group_size, fresh=False):
        self.packed, self.qzeros, self.scales = packed, qzeros, scales
        self.K, self.N, self.group_size = K, N, group_size
        # per-call constants of the hot wrapper: raw pointers (the tensors above keep them alive) and
        # the workspace size per row count
        self._ptrs = (packed.data_ptr(), scales.data_ptr(), qzeros.data_ptr(), packed.device)
        self._ws_need = {}
        # True while the repack kernel that produced `packed` may still be queued: the first
        # compute call must then not prefetch the weights ahead of the previous kernel.
        self.fresh = fresh


def repack(qweight: torch.Tensor) -> torch.Tensor:
    """On-disk qweight int32 [K, N/8] -> packed int32 [K/128, N, 16] (same bytes)."""
    K, N = _kn(qweight)
    qweight = qweight.contiguous()
    _prep(qweight)
    if K % 128 != 0:
        raise ValueError(f"in_features must be a multiple of 128, got {K}")
    packed = torch.empty((K // 128, N, 16), dtype=torch.int32, device=qweight.device)
    check(lib.awq_b200_repack(qweight.data_ptr(), packed.data_ptr(), K, N, _stream(qweight)), "awq_b200_repack")
    return packed


def unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of `repack`."""
    nblk, N, _ = packed.shape
    K = nblk * 128
    _prep(packed)
    qweight = torch.empty((K, N // 8), dtype=torch.int32, device=packed.device)
    check(lib.awq_b200_unpack(packed.data_ptr(), qweight.data_ptr(), K, N, _stream(packed)), "awq_b200_unpack")
    return qweight


def make_packed(qweight, qzeros, scales, group_size) -> PackedWeight:
    K, N = _kn(qweight)
    G = K if group_size == -1 else group_size
    if scales.dtype != torch.float16 or tuple(scales.shape) != (K // G, N):
        raise ValueError("scales must be fp16 [K/G, N]")
    if qzeros.dtype != torch.int32 or tuple(qzeros.shape) != (K // G, N // 8):
        raise ValueError("qzeros must be int32 [K/G, N/8]")
    return PackedWeight(repack(qweight), qzeros.contiguous(), scales.contiguous(), K, N, G, fresh=True)


def dequantize(qweight, qzeros, scales, group_size) -> torch.Tensor:
    """fp16 [K, N], bit-identical to the reference's dequantize_gemm."""
    K, N = _kn(qweight)
    qweight, qzeros, scales = qweight.contiguous(), qzeros.contiguous(), scales.contiguous()
    _prep(qweight, qzeros, scales)
    W = torch.empty((K, N), dtype=torch.float16, device=qweight.device)
    check(lib.awq_b200_dequant(qweight.data_ptr(), qzeros.data_ptr(), scales.data_ptr(), W.data_ptr(), K, N,
                               K if group_size == -1 else group_size, _stream(W)), "awq_b200_dequant")
    return W


def dequantize_packed(pw: PackedWeight) -> torch.Tensor:
    _prep(pw.packed, pw.qzeros, pw.scales)
    W = torch.empty((pw.K, pw.N), dtype=torch.float16, device=pw.packed.device)
    check(lib.awq_b200_dequant_packed(pw.packed.data_ptr(), pw.qzeros.data_ptr(), pw.scales.data_ptr(),
                                      W.data_ptr(), pw.K, pw.N, pw.group_size, _stream(W)),
          "awq_b200_dequant_packed")
    return W


# One zero-initialised workspace per (device, stream, entry point): calls that
# share a workspace must not overlap on the GPU (calls on one stream never do),
# and the entry points lay their workspace out differently.
_workspaces: dict[tuple[int, int, str], torch.Tensor] = {}


_retired_workspaces: list[torch.Tensor] = []


def _workspace(dev: torch.device, stream: int, nbytes: int, kind: str) -> torch.Tensor:
    """The zero-initialised scratch of one (device, stream, entry point).  When a call needs more than the buffer
    holds, a larger one takes its place (at least 1.5 x, so few are ever made) and the old one is kept allocated:
    a CUDA graph captured earlier still holds its address."""
    key = (dev.index, stream, kind)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired_workspaces.append(ws)
            nbytes = max(nbytes, ws.numel() * 3 // 2)
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def _check_out(out, out_shape, M: int, ncols: int, dev: torch.device) -> None:
    """The kernels write M * ncols contiguous fp16 elements at `out`: anything else (a strided view, a
    shorter tensor, another dtype) would be an out-of-bounds or misplaced write on the device, so it is
    refused here, before the call."""
    if out is not None:
        if out.dtype != torch.float16 or not out.is_contiguous() or out.numel() != M * ncols:
            raise ValueError(f"out must be a contiguous fp16 tensor of {M} x {ncols} elements, got {out.dtype} "
                             f"{tuple(out.shape)} (contiguous: {out.is_contiguous()})")
        if out.device != dev:
            raise RuntimeError("all tensors of one call must be on the same device")
    elif out_shape is not None:
        n = 1
        for d in out_shape:
            n *= int(d)
        if n != M * ncols:
            raise ValueError(f"out_shape {tuple(out_shape)} does not hold {M} x {ncols} elements")


def _check_x(x: torch.Tensor, pw: PackedWeight) -> torch.Tensor:
    if x.dtype != torch.float16 or x.dim() != 2 or x.shape[1] != pw.K:
        raise ValueError(f"x must be fp16 [M, {pw.K}], got {x.dtype} {tuple(x.shape)}")
    return x.contiguous()


def _run(fn, name, x, pw, bias, ws_bytes, out=None, extra=()):
    x = _check_x(x, pw)
    M = x.shape[0]
    _check_out(out, None, M, pw.N, x.device)
    dev = _prep(x, pw.packed, pw.qzeros, pw.scales, bias)
    y = out if out is not None else torch.empty((M, pw.N), dtype=torch.float16, device=dev)
    stream = _stream(x)
    ws = _workspace(dev, stream, ws_bytes, name)
    check(fn(x.data_ptr(), pw.packed.data_ptr(), pw.scales.data_ptr(), pw.qzeros.data_ptr(),
             bias.data_ptr() if bias is not None else None, y.data_ptr(), M, pw.K, pw.N, pw.group_size,
             ws.data_ptr(), ws.numel(), stream, *extra), name)
    return y


def _gemv_flags(overlap: bool, no_cluster: bool, mode) -> int:
    if mode not in (None, "stream", "per_split"):
        raise ValueError(f"mode must be None, 'stream' or 'per_split', got {mode!r}")
    return ((_lib.OVERLAP_PREVIOUS if overlap else 0) | (_lib.NO_CLUSTER if no_cluster else 0) |
            (_lib.GEMV_STREAM if mode == "stream" else 0) | (_lib.GEMV_PER_SPLIT if mode == "per_split" else 0))


def gemv(x, pw: PackedWeight, bias=None, out=None, overlap: bool = False, no_cluster: bool = False,
         mode=None) -> torch.Tensor:
    """Decode kernel, 1 <= M <= 64 (8 rows per CTA).  `overlap=True` lets the kernel prefetch its weights while the
    previous kernel of the stream drains; pass it only when the weights are not being written by
    work still queued on that stream (i.e. not right after `repack`).  `mode` forces the persistent
    stream ("stream") or the one-CTA-per-split grid ("per_split"); None lets the library choose."""
    M = max(x.shape[0], 1)
    ws = (lib.awq_b200_gemv_workspace_bytes(M, pw.K, pw.N) if mode is None
          else lib.awq_b200_gemv_workspace_bytes_max(M, pw.K, pw.N))
    return _run(lib.awq_b200_gemv_ex, "awq_b200_gemv", x, pw, bias, ws, out, (_gemv_flags(overlap, no_cluster, mode),))


def gemv_plan(x, pw: PackedWeight, ntw: int, bps: int, bias=None, out=None, overlap: bool = False,
              no_cluster: bool = False, kw: int = 0, mode=None) -> torch.Tensor:
    """Decode kernel with a forced decomposition (tuning and tests)."""
    return _run(lib.awq_b200_gemv_plan, "awq_b200_gemv_plan", x, pw, bias,
                lib.awq_b200_gemv_workspace_bytes_max(max(x.shape[0], 1), pw.K, pw.N), out,
                (ntw, kw, bps, _gemv_flags(overlap, no_cluster, mode)))


def skinny(x, pw: PackedWeight, bias=None, out=None, overlap: bool = False) -> torch.Tensor:
    """Few rows (1 <= M <= 64) on the tensor-memory path with split-K over all SMs."""
    return _run(lib.awq_b200_skinny, "awq_b200_skinny", x, pw, bias,
                lib.awq_b200_skinny_workspace_bytes(max(x.shape[0], 1), pw.K, pw.N), out,
                (_lib.OVERLAP_PREVIOUS if overlap else 0,))


def decode_i8(x, pw: PackedWeight, bias=None, out=None, overlap: bool = False) -> torch.Tensor:
    """Decode rows (1 <= M <= 8) on the integer tensor-core path (packed bytes x block-fixed-point activations)."""
    return _run(lib.awq_b200_decode_i8, "awq_b200_decode", x, pw, bias,
                lib.awq_b200_decode_workspace_bytes(max(x.shape[0], 1), pw.K, pw.N), out,
                (_lib.OVERLAP_PREVIOUS if overlap else 0,))


def gemm(x, pw: PackedWeight, bias=None, out=None) -> torch.Tensor:
    """Prefill kernel (tcgen05), any M >= 1."""
    return _run(lib.awq_b200_gemm, "awq_b200_gemm", x, pw, bias,
                lib.awq_b200_gemm_workspace_bytes(x.shape[0], pw.K, pw.N), out)


def gemm_smem(x, pw: PackedWeight, bias=None, out=None) -> torch.Tensor:
    """Prefill kernel, dequantised-weights-in-shared-memory variant only."""
    return _run(lib.awq_b200_gemm_smem, "awq_b200_gemm", x, pw, bias,
                lib.awq_b200_gemm_workspace_bytes(x.shape[0], pw.K, pw.N), out)


def gemm_wtm_unsplit(x, pw: PackedWeight, bias=None, out=None, m_tile: int = 0) -> torch.Tensor:
    """`gemm_wtm` with a workspace too small for partial tiles: every tile is finished by one CTA
    (the bits of the shared-memory variant).  For tests."""
    return _run(lib.awq_b200_gemm_wtm_tile, "awq_b200_gemm_unsplit", x, pw, bias, 256, out, (m_tile,))


def gemm_wtm(x, pw: PackedWeight, bias=None, out=None, m_tile: int = 0) -> torch.Tensor:
    """Prefill kernel, weights-in-tensor-memory variant, any M >= 1 (`m_tile` forces the row tile)."""
    return _run(lib.awq_b200_gemm_wtm_tile, "awq_b200_gemm", x, pw, bias,
                lib.awq_b200_gemm_workspace_bytes(x.shape[0], pw.K, pw.N), out, (m_tile,))


def linear(x, pw: PackedWeight, bias=None, out=None, overlap: bool = False, out_shape=None,
           one_kernel_below_8: bool = False) -> torch.Tensor:
    """The library's dispatcher (decode GEMV, split-K tensor-memory kernel or GEMM by rows and shape).
    `overlap` as in `gemv`.  `one_kernel_below_8` serves every call of fewer than 8 rows with the GEMV, so that
    decode and speculative verification add in the same order (the reference's rule, linear_awq.py:161-166).  `x` is fp16 [..., K]; its leading dimensions are the rows.  The result is
    `out`, or a new tensor of `out_shape` (default [M, N]).  This is the per-token call of the module, so
    the wrapper keeps its own work to a minimum: cached pointers and workspace sizes, one ctypes call."""
    wp, sp, zp, dev = pw._ptrs
    if x.dtype != torch.float16 or x.dim() < 2 or x.shape[-1] != pw.K:
        raise ValueError(f"x must be fp16 [..., {pw.K}], got {x.dtype} {tuple(x.shape)}")
    if x.device != dev:
        if x.device.type != "cuda":
            raise RuntimeError("llmrqt_sdv1_b200 kernels need CUDA tensors; there is no CPU fallback")
        raise RuntimeError("all tensors of one call must be on the same device")
    if bias is not None and bias.device != dev:
        raise RuntimeError("all tensors of one call must be on the same device")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.numel() // pw.K
    if out is not None or out_shape is not None:
        _check_out(out, out_shape, M, pw.N, dev)
    if dev.type != "cuda":
        raise RuntimeError("llmrqt_sdv1_b200 kernels need CUDA tensors; there is no CPU fallback")
    index = dev.index
    _lib.set_device(index)
    need = pw._ws_need.get(M)
    if need is None:
        need = pw._ws_need[M] = lib.awq_b200_linear_workspace_bytes(max(M, 1), pw.K, pw.N)
    stream = _raw_stream(index) if _raw_stream is not None else torch.cuda.current_stream(dev).cuda_stream
    ws = _workspaces.get((index, stream, "awq_b200_linear"))
    if ws is None or ws.numel() < need:
        ws = _workspace(dev, stream, need, "awq_b200_linear")
    if out is not None:
        y = out
    else:
        y = torch.empty(out_shape if out_shape is not None else (M, pw.N), dtype=torch.float16, device=dev)
    st = lib.awq_b200_linear_ex(x.data_ptr(), wp, sp, zp, bias.data_ptr() if bias is not None else None,
                                y.data_ptr(), M, pw.K, pw.N, pw.group_size, ws.data_ptr(), ws.numel(), stream,
                                (_lib.OVERLAP_PREVIOUS if overlap else 0) |
                                (_lib.ONE_KERNEL_BELOW_8 if one_kernel_below_8 else 0))
    if st != 0:
        check(st, "awq_b200_linear")
    return y


def interleave_columns(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Two AWQ int4 tensors of equal shape (qweight [K, n/8] or qzeros [K/G, n/8], int32) -> [rows, 2n/8]
    with column 2j from `a` and column 2j+1 from `b`."""
    if a.dtype != torch.int32 or b.dtype != torch.int32 or a.dim() != 2 or a.shape != b.shape:
        raise ValueError("interleave_columns needs two int32 [rows, words] tensors of equal shape")
    a, b = a.contiguous(), b.contiguous()
    _prep(a, b)
    out = torch.empty((a.shape[0], 2 * a.shape[1]), dtype=torch.int32, device=a.device)
    check(lib.awq_b200_interleave_columns(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.shape[0], a.shape[1],
                                          _stream(a)), "awq_b200_interleave_columns")
    return out


def make_gated_packed(gate, up, group_size) -> PackedWeight:
    """One kernel-layout weight [K, 2n] from the (qweight, qzeros, scales) of a gate and an up projection
    [K, n] each, columns interleaved (gate j, up j) as the gated epilogue of `linear_fused` expects."""
    (gq, gz, gs), (uq, uz, us) = gate, up
    if gs.shape != us.shape or gs.dtype != torch.float16 or us.dtype != torch.float16:
        raise ValueError("gate and up scales must be fp16 tensors of equal shape")
    scales = torch.stack((gs, us), dim=-1).reshape(gs.shape[0], 2 * gs.shape[1])
    return make_packed(interleave_columns(gq, uq), interleave_columns(gz, uz), scales, group_size)


def interleave_bias(gate_bias: torch.Tensor, up_bias: torch.Tensor) -> torch.Tensor:
    """The bias of a `make_gated_packed` weight: [2n] in the packed column order."""
    return torch.stack((gate_bias, up_bias), dim=-1).reshape(-1).contiguous()


def linear_fused(x, pw: PackedWeight, bias=None, residual=None, gated: bool = False, out=None,
                 overlap: bool = False, out_shape=None, flags: int = 0) -> torch.Tensor:
    """`linear` with the elementwise work that follows it done in the kernel's epilogue: bias, then with
    `gated` SiLU(gate) * up over the (gate, up) column pairs of a `make_gated_packed` weight (the result
    has N / 2 columns), then `+ residual` (fp16, the shape of the result).  Every step rounds to fp16 as
    the separate fp16 tensor operations would."""
    wp, sp, zp, dev = pw._ptrs
    if x.dtype != torch.float16 or x.dim() < 2 or x.shape[-1] != pw.K:
        raise ValueError(f"x must be fp16 [..., {pw.K}], got {x.dtype} {tuple(x.shape)}")
    for t in (x, bias, residual, out):
        if t is not None and t.device != dev:
            if t.device.type != "cuda":
                raise RuntimeError("llmrqt_sdv1_b200 kernels need CUDA tensors; there is no CPU fallback")
            raise RuntimeError("all tensors of one call must be on the same device")
    if not x.is_contiguous():
        x = x.contiguous()
    M = x.numel() // pw.K
    ncols = pw.N // 2 if gated else pw.N
    if residual is not None:
        if residual.dtype != torch.float16 or residual.numel() != M * ncols:
            raise ValueError(f"residual must be fp16 with {M} x {ncols} elements")
        if not residual.is_contiguous():
            residual = residual.contiguous()
    if out is not None or out_shape is not None:
        _check_out(out, out_shape, M, ncols, dev)
    if dev.type != "cuda":
        raise RuntimeError("llmrqt_sdv1_b200 kernels need CUDA tensors; there is no CPU fallback")
    index = dev.index
    _lib.set_device(index)
    need = pw._ws_need.get(M)
    if need is None:
        need = pw._ws_need[M] = lib.awq_b200_linear_workspace_bytes(max(M, 1), pw.K, pw.N)
    stream = _raw_stream(index) if _raw_stream is not None else torch.cuda.current_stream(dev).cuda_stream
    ws = _workspaces.get((index, stream, "awq_b200_linear"))
    if ws is None or ws.numel() < need:
        ws = _workspace(dev, stream, need, "awq_b200_linear")
    if out is not None:
        y = out
    else:
        y = torch.empty(out_shape if out_shape is not None else (M, ncols), dtype=torch.float16, device=dev)
    epi = _lib.Epilogue(bias.data_ptr() if bias is not None else None,
                        residual.data_ptr() if residual is not None else None, 1 if gated else 0)
    st = lib.awq_b200_linear_fused(x.data_ptr(), wp, sp, zp, _addressof(epi), y.data_ptr(), M, pw.K, pw.N,
                                   pw.group_size, ws.data_ptr(), ws.numel(), stream,
                                   (_lib.OVERLAP_PREVIOUS if overlap else 0) | flags)
    if st != 0:
        check(st, "awq_b200_linear_fused")
    return y


def peer_allreduce(bufs_dev: int, flags_dev: int, local_buf: torch.Tensor, M: int, N: int, rank: int, world: int,
                   out: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> torch.Tensor:
    """Sum of the ranks' [M, N] fp16 partials held in symmetric memory (see `sharded.PeerSum`).
    `bufs_dev` / `flags_dev` are device arrays of per-rank pointers."""
    dev = local_buf.device
    _check_out(out, None, M, N, dev)
    _lib.set_device(dev.index)
    y = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=dev)
    check(lib.awq_b200_peer_allreduce(bufs_dev, flags_dev, y.data_ptr(), bias.data_ptr() if bias is not None else None,
                                      M * N, N, rank, world, _stream(local_buf)), "awq_b200_peer_allreduce")
    return y


def peer_allreduce_push(partial: torch.Tensor, recv_dev: int, flags_dev: int, slot_elems: int, M: int, N: int,
                        rank: int, world: int, out: torch.Tensor | None = None,
                        bias: torch.Tensor | None = None) -> torch.Tensor:
    """`peer_allreduce` with the partials pushed into the peers' receive slots (see `sharded.PeerSum`)."""
    dev = partial.device
    _check_out(out, None, M, N, dev)
    _lib.set_device(dev.index)
    y = out if out is not None else torch.empty((M, N), dtype=torch.float16, device=dev)
    check(lib.awq_b200_peer_allreduce_push(partial.data_ptr(), recv_dev, flags_dev, y.data_ptr(),
                                           bias.data_ptr() if bias is not None else None, M * N, N, slot_elems,
                                           rank, world, _stream(partial)), "awq_b200_peer_allreduce_push")
    return y


def decode_i8_push(x, pw: PackedWeight, recv_dev: int, flags_dev: int, slot_elems: int, rank: int, world: int,
                   bias=None, out=None, overlap: bool = False) -> torch.Tensor:
    """`decode_i8` on this rank's row shard with the push form of the peer exchange done by the kernel's epilogue:
    returns the SUM over the ranks (see `sharded.PeerSum.linear_push`).  1 <= M <= 8, 2 <= world <= 8."""
    x = _check_x(x, pw)
    M = x.shape[0]
    _check_out(out, None, M, pw.N, x.device)
    dev = _prep(x, pw.packed, pw.qzeros, pw.scales, bias)
    y = out if out is not None else torch.empty((M, pw.N), dtype=torch.float16, device=dev)
    stream = _stream(x)
    ws = _workspace(dev, stream, lib.awq_b200_decode_workspace_bytes(max(M, 1), pw.K, pw.N), "awq_b200_decode")
    check(lib.awq_b200_decode_i8_push(x.data_ptr(), pw.packed.data_ptr(), pw.scales.data_ptr(), pw.qzeros.data_ptr(),
                                      bias.data_ptr() if bias is not None else None, y.data_ptr(), M, pw.K, pw.N,
                                      pw.group_size, ws.data_ptr(), ws.numel(), recv_dev, flags_dev, slot_elems, rank,
                                      world, stream, _lib.OVERLAP_PREVIOUS if overlap else 0), "awq_b200_decode_i8_push")
    return y


def qk_norm_rope_cache(qkv, q_weight, k_weight, eps, cos_tab, sin_tab, pos, q_out, k_cache, v_cache) -> None:
    """One token's fused qkv row -> q (normalised per head, rotated) into `q_out` [H, D], k (likewise) and v into row
    `pos` of `k_cache` / `v_cache` [KV, max_len, D].  `pos` is an int64 tensor on the device (one element)."""
    KV, max_len, D = k_cache.shape[-3], k_cache.shape[-2], k_cache.shape[-1]
    H = q_out.numel() // D
    for t in (qkv, cos_tab, sin_tab, q_out, k_cache, v_cache):
        if t.dtype != torch.float16 or not t.is_contiguous():
            raise ValueError("qk_norm_rope_cache needs contiguous fp16 tensors")
    if qkv.numel() != (H + 2 * KV) * D or v_cache.shape != k_cache.shape or pos.dtype != torch.int64:
        raise ValueError("qk_norm_rope_cache: inconsistent shapes")
    if tuple(cos_tab.shape) != (max_len, D) or tuple(sin_tab.shape) != (max_len, D):
        raise ValueError(f"rotary tables must be [{max_len}, {D}]")
    dev = _prep(qkv, cos_tab, sin_tab, pos, q_out, k_cache, v_cache)
    check(lib.awq_b200_qk_norm_rope_cache(
        qkv.data_ptr(), q_weight.data_ptr() if q_weight is not None else None,
        k_weight.data_ptr() if k_weight is not None else None, float(eps), cos_tab.data_ptr(), sin_tab.data_ptr(),
        pos.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), H, KV, D, max_len,
        torch.cuda.current_stream(dev).cuda_stream), "awq_b200_qk_norm_rope_cache")


def _attn_workspace(dev, H: int, D: int, split: bool):
    """(pointer, bytes) of the per-stream scratch of the attention kernels; (None, 0) makes them never split."""
    if not split:
        return None, 0
    need = lib.awq_b200_attn_workspace_bytes(H, D)
    ws = _workspace(dev, torch.cuda.current_stream(dev).cuda_stream, need, "awq_b200_attn")
    return ws.data_ptr(), ws.numel()


def attn_decode(q, k_cache, v_cache, pos, out, scale: float, split: bool = True) -> None:
    """`out` [H * D] = attention of one query token `q` [H, D] over rows 0..pos of the caches [KV, max_len, D].
    `split=False`: one CTA per head whatever the position (beyond 256 positions the default cuts the positions
    into chunks, one CTA each)."""
    KV, max_len, D = k_cache.shape[-3], k_cache.shape[-2], k_cache.shape[-1]
    H = q.numel() // D
    for t in (q, k_cache, v_cache, out):
        if t.dtype != torch.float16 or not t.is_contiguous():
            raise ValueError("attn_decode needs contiguous fp16 tensors")
    if out.numel() != H * D or v_cache.shape != k_cache.shape or pos.dtype != torch.int64:
        raise ValueError("attn_decode: inconsistent shapes")
    dev = _prep(q, k_cache, v_cache, pos, out)
    ws, ws_bytes = _attn_workspace(dev, H, D, split)
    check(lib.awq_b200_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                   H, KV, D, max_len, float(scale), ws, ws_bytes,
                                   torch.cuda.current_stream(dev).cuda_stream),
          "awq_b200_attn_decode")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm over the last dimension of fp16 `x` times `weight` (fp32 arithmetic, one rounding), one launch."""
    D = x.shape[-1]
    if x.dtype != torch.float16 or weight.dtype != torch.float16 or not x.is_contiguous() or weight.numel() != D:
        raise ValueError("rmsnorm needs contiguous fp16 x [..., D] and an fp16 weight [D]")
    dev = _prep(x, weight)
    y = out if out is not None else torch.empty_like(x)
    if y.dtype != torch.float16 or not y.is_contiguous() or y.numel() != x.numel():
        raise ValueError("rmsnorm: out must be a contiguous fp16 tensor of x's size")
    if x.numel() == 0:
        return y
    check(lib.awq_b200_rmsnorm(x.data_ptr(), weight.data_ptr(), float(eps), y.data_ptr(), x.numel() // D, D,
                               torch.cuda.current_stream(dev).cuda_stream), "awq_b200_rmsnorm")
    return y


def attn_step(qkv, q_weight, k_weight, eps, cos_tab, sin_tab, pos, k_cache, v_cache, out, scale: float,
              split: bool = True) -> None:
    """`qk_norm_rope_cache` + `attn_decode` in one launch: the fused qkv row in, the attention output [H * D] out,
    row `pos` of the caches appended.  Same bits as the two calls (with the same `split`)."""
    KV, max_len, D = k_cache.shape[-3], k_cache.shape[-2], k_cache.shape[-1]
    H = out.numel() // D
    for t in (qkv, cos_tab, sin_tab, out, k_cache, v_cache):
        if t.dtype != torch.float16 or not t.is_contiguous():
            raise ValueError("attn_step needs contiguous fp16 tensors")
    if qkv.numel() != (H + 2 * KV) * D or v_cache.shape != k_cache.shape or pos.dtype != torch.int64:
        raise ValueError("attn_step: inconsistent shapes")
    if tuple(cos_tab.shape) != (max_len, D) or tuple(sin_tab.shape) != (max_len, D):
        raise ValueError(f"rotary tables must be [{max_len}, {D}]")
    dev = _prep(qkv, cos_tab, sin_tab, pos, out, k_cache, v_cache)
    ws, ws_bytes = _attn_workspace(dev, H, D, split)
    check(lib.awq_b200_attn_step(
        qkv.data_ptr(), q_weight.data_ptr() if q_weight is not None else None,
        k_weight.data_ptr() if k_weight is not None else None, float(eps), cos_tab.data_ptr(), sin_tab.data_ptr(),
        pos.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), H, KV, D, max_len, float(scale),
        ws, ws_bytes, torch.cuda.current_stream(dev).cuda_stream), "awq_b200_attn_step")


def gemv_status(dev: torch.device | None = None) -> int:
    """Status word of the decode kernels (GEMV and split-K tensor-memory kernel) in this stream's workspaces (0 = no device-side wait expired).
    Synchronises."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = 0
    for kind, off in (("awq_b200_gemv", 0), ("awq_b200_gemv_plan", 0), ("awq_b200_skinny", 0), ("awq_b200_decode", 0),
                      ("awq_b200_linear", 256)):
        ws = _workspaces.get((dev.index, stream, kind))
        if ws is not None:
            status |= int(ws[off + 4095 * 4: off + 4096 * 4].view(torch.int32).item())
    return status


def gemm_status(dev: torch.device | None = None) -> int:
    """Status word the GEMM kernel leaves in this stream's workspace (0 = every
    device-side wait completed).  Synchronises."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    status = 0
    for kind in ("awq_b200_gemm", "awq_b200_linear"):
        ws = _workspaces.get((dev.index, stream, kind))
        if ws is not None:
            status |= int(ws[:4].view(torch.int32).item())
    return status
