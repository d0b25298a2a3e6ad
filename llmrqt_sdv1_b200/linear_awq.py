"""`AWQLinear_GEMM`: the reference runtime's AWQ W4A16 linear module
(LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:216-414) with the
same constructor, buffer names / shapes / dtypes, `from_linear`, `impl_mode`
and forward conventions, so reference checkpoints, `load_state_dict`, and the
q/k/v fusion that concatenates buffers along N work unchanged.  The forward
runs the sm_100a kernels; the kernel-layout repack of `qweight` happens lazily
on the first forward after the buffers last changed (or eagerly via `prepare`).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.autograd import Function

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)


_KERNELS = None


def _kernels():
    # Imported on first use so that host-only helpers (packing, sharding plans)
    # stay importable for inspection; any compute call still fails loudly
    # without the CUDA library.
    global _KERNELS
    if _KERNELS is None:
        from . import kernels, sq_fp8_kernels
        _KERNELS = (kernels, sq_fp8_kernels)
    return _KERNELS


def pack_awq_int4(values: torch.Tensor) -> torch.Tensor:
    """int tensor [R, C] with entries 0..15 -> int32 [R, C/8]; slot i of a word holds
    column 8c + AWQ_ORDER[i] (linear_awq.py:333-346, vectorised)."""
    R, Cc = values.shape
    v = values.to(torch.int32).reshape(R, Cc // 8, 8)
    out = torch.zeros((R, Cc // 8), dtype=torch.int32, device=values.device)
    for slot, logical in enumerate(AWQ_ORDER):
        out |= v[:, :, logical] << (4 * slot)
    return out


class AWQLinearMMFunction(Function):
    """Same positional signature as the reference function (linear_awq.py:128-212)."""

    @staticmethod
    def forward(ctx, x, qweight, qzeros, scales, w_bit=4, group_size=128, bias=None, out_features=0,
                impl_mode="auto"):
        out_shape = x.shape[:-1] + (out_features,)
        if x.shape[0] == 0 or x.numel() == 0:
            return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        if impl_mode not in {"auto", "dequant_matmul"}:
            raise ValueError(f"AWQ impl_mode must be 'auto' or 'dequant_matmul', got {impl_mode!r}")
        kernels, ext = _kernels()
        if impl_mode == "dequant_matmul":
            # Explicit reference path: materialise the fp16 weight, then a library matmul.
            out = torch.matmul(x, kernels.dequantize(qweight, qzeros, scales, group_size))
        else:
            pw = ext.packed_for(qweight, qzeros, scales, group_size)
            overlap, pw.fresh = not pw.fresh, False   # first call after a repack: no weight prefetch
            # the bias is added inside the kernel: fp16(acc), then fp16(y + bias) - the two roundings of the
            # reference's `out + bias` on fp16 tensors (linear_awq.py:205)
            # 2-D input comes back 3-D, as from the reference (linear_awq.py:209-210)
            shape3 = (1,) + tuple(out_shape) if len(out_shape) == 2 else out_shape
            return kernels.linear(x if x.dim() >= 2 else x.unsqueeze(0), pw, bias=bias, overlap=overlap,
                                  out_shape=shape3)
        out = out + bias if bias is not None else out
        if out.dim() == 2:          # the reference always hands back a 3-D tensor
            out = out.unsqueeze(0)
        return out


class AWQLinear_GEMM(nn.Module):
    def __init__(self, w_bit, group_size, in_features, out_features, bias, dev, training=False):
        super().__init__()
        if w_bit not in [4]:
            raise NotImplementedError("Only 4-bit are supported for now.")
        self.in_features = in_features
        self.out_features = out_features
        self.w_bit = w_bit
        self.group_size = group_size if group_size != -1 else in_features
        self.training = training
        self.impl_mode = "auto"     # or "dequant_matmul"
        # True: every call of fewer than 8 rows takes one kernel whatever the weight's size, so decode (1 row) and
        # speculative verification (2..7 rows) add in the same order (the reference's rule, linear_awq.py:161-166).
        # False (default): rows 1..4 share a kernel, rows 5..8 share a kernel, large weights take the faster ones.
        self.one_kernel_below_8 = False
        assert self.in_features % self.group_size == 0
        assert out_features % (32 // self.w_bit) == 0
        pack = 32 // self.w_bit
        self.register_buffer("qweight", torch.zeros((in_features, out_features // pack), dtype=torch.int32, device=dev))
        self.register_buffer("qzeros", torch.zeros((in_features // self.group_size, out_features // pack),
                                                   dtype=torch.int32, device=dev))
        self.register_buffer("scales", torch.zeros((in_features // self.group_size, out_features),
                                                   dtype=torch.float16, device=dev))
        if bias:
            self.register_buffer("bias", torch.zeros((out_features,), dtype=torch.float16, device=dev))
        else:
            self.bias = None
        self._released = None       # the kernel-layout weight while `qweight` is released

    @classmethod
    def from_linear(cls, linear, w_bit, group_size, init_only=False, dtype=torch.bfloat16, scales=None,
                    zeros=None, per_tensor=False):
        """Build from an nn.Linear holding the fake-quantised fp16 weight plus its
        `scales` / `zeros` [K/G, N] (linear_awq.py:274-363).  Same arithmetic as the
        reference's per-column loop, done on whole tensors."""
        awq_linear = cls(w_bit, group_size, linear.in_features, linear.out_features,
                         linear.bias is not None, linear.weight.device)
        if init_only:
            return awq_linear
        assert scales is not None and zeros is not None
        G = awq_linear.group_size
        scale_zeros = zeros * scales
        awq_linear.scales = scales.clone().half()
        if linear.bias is not None:
            awq_linear.bias = linear.bias.clone().half()
        w_t = linear.weight.data.t()                                             # [K, N]
        intweight = torch.round((w_t + scale_zeros.repeat_interleave(G, dim=0))
                                / awq_linear.scales.repeat_interleave(G, dim=0)).to(torch.int32)
        awq_linear.qweight = pack_awq_int4(intweight.contiguous())
        awq_linear.qzeros = pack_awq_int4(zeros.to(torch.int32))
        return awq_linear

    def prepare(self):
        """Repack now instead of on the first forward (call after any buffer surgery)."""
        if getattr(self, "_released", None) is not None:
            return self
        _, ext = _kernels()
        ext.packed_for(self.qweight, self.qzeros, self.scales, self.group_size)
        return self

    def packed(self):
        """The kernel-layout weight of this module (repacked on first use, or the one kept by `release_qweight`)."""
        pw = getattr(self, "_released", None)
        if pw is not None:
            return pw
        _, ext = _kernels()
        return ext.packed_for(self.qweight, self.qzeros, self.scales, self.group_size)

    # The kernels read the repacked weight only.  A module that serves and is not being edited can therefore
    # give the on-disk `qweight` back: `release_qweight` keeps the kernel-layout copy alone (half the int4
    # bytes of a layer that otherwise holds both), and `state_dict()` / `restore_qweight` rebuild the on-disk
    # tensor bit for bit with the inverse repack (awq_b200_unpack) whenever it is asked for.
    def release_qweight(self):
        """Free the on-disk `qweight` buffer; forward keeps working from the kernel-layout weight."""
        if getattr(self, "_released", None) is not None:
            return self
        _, ext = _kernels()
        pw = ext.packed_for(self.qweight, self.qzeros, self.scales, self.group_size)
        self._released = pw
        self.qweight = torch.empty((0, self.out_features // (32 // self.w_bit)), dtype=torch.int32,
                                   device=pw.packed.device)
        return self

    def adopt_packed(self, pw):
        """Take a kernel-layout weight built elsewhere (a loader that repacks straight from the file) as this
        module's weight, with `qweight` released.  `pw.qzeros` / `pw.scales` become the module's buffers."""
        if (pw.K, pw.N, pw.group_size) != (self.in_features, self.out_features, self.group_size):
            raise ValueError("packed weight does not match the module's shape / group size")
        self.qzeros, self.scales = pw.qzeros, pw.scales
        self._released = pw
        self.qweight = torch.empty((0, self.out_features // (32 // self.w_bit)), dtype=torch.int32,
                                   device=pw.packed.device)
        return self

    def restore_qweight(self):
        """Bring the on-disk `qweight` buffer back (needed before editing buffers, e.g. q/k/v fusion)."""
        pw = getattr(self, "_released", None)
        if pw is not None:
            kernels, _ = _kernels()
            self.qweight = kernels.unpack(pw.packed)
            self._released = None
        return self

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        pw = getattr(self, "_released", None)
        if pw is not None:       # the checkpoint format is the on-disk one, whatever the module holds
            kernels, _ = _kernels()
            destination[prefix + "qweight"] = kernels.unpack(pw.packed)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        if getattr(self, "_released", None) is not None and prefix + "qweight" in state_dict:
            self.restore_qweight()
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def forward(self, x, residual=None):
        """`residual` (optional, not in the reference's signature): a tensor of the result's shape that the
        kernel's epilogue adds after the bias, as `residual + forward(x)` on fp16 tensors would."""
        buffers = self._buffers
        qweight, qzeros, scales = buffers["qweight"], buffers["qzeros"], buffers["scales"]
        dev = qweight.device
        assert x.device == dev, "when awq linear fwd, input and qweight must be same device!"
        assert qzeros.device == dev, "when awq linear fwd, qzeros and qweight must be same device!"
        assert scales.device == dev, "when awq linear fwd, scales and qweight must be same device!"
        released = self.__dict__.get("_released")
        if released is not None and self.impl_mode != "auto":
            # the explicit reference path materialises the fp16 weight from the on-disk tensors
            self.restore_qweight()
            qweight, released = self._buffers["qweight"], None
        if x.dtype == torch.float16 and self.impl_mode == "auto" and x.dim() >= 2 and x.numel() != 0:
            # The per-token path: straight to the library's dispatcher.  Nothing here records autograd
            # state (the result is a fresh tensor written by the kernel), so no no_grad block is needed.
            kernels, ext = _kernels()
            pw = released if released is not None else ext.packed_for(qweight, qzeros, scales, self.group_size)
            overlap, pw.fresh = not pw.fresh, False   # first call after a repack: no weight prefetch
            shape = x.shape[:-1] + (self.out_features,)
            shape = (1,) + tuple(shape) if len(shape) == 2 else shape
            if residual is None:
                return kernels.linear(x, pw, bias=self.bias, overlap=overlap, out_shape=shape,
                                      one_kernel_below_8=self.one_kernel_below_8)
            return kernels.linear_fused(x, pw, bias=self.bias, residual=residual, overlap=overlap, out_shape=shape)
        out_shape = x.shape[:-1] + (self.out_features,)
        if x.shape[0] == 0:
            return torch.zeros(out_shape, dtype=x.dtype, device=x.device)
        if released is not None:
            if self.impl_mode not in {"auto", "dequant_matmul"}:
                raise ValueError(f"AWQ impl_mode must be 'auto' or 'dequant_matmul', got {self.impl_mode!r}")
            x16 = x.to(torch.float16)
            y = self.forward(x16 if x16.dim() >= 2 else x16.unsqueeze(0),
                             residual.to(torch.float16) if residual is not None else None)
            y = y if x.dim() >= 2 else y.reshape(out_shape)
            return y if x.dtype == torch.float16 else y.to(x.dtype)
        input_dtype = x.dtype
        if input_dtype != torch.float16:
            x = x.to(torch.float16)
        with torch.no_grad():
            # The reference goes through AWQLinearMMFunction.apply (linear_awq.py:385-395); under
            # no_grad that is the same computation plus ~10 us of autograd bookkeeping per call.
            out = AWQLinearMMFunction.forward(None, x, qweight, qzeros, scales, self.w_bit,
                                              self.group_size, self.bias, self.out_features, self.impl_mode)
        if residual is not None:
            out = residual.to(torch.float16).reshape(out.shape) + out
        if input_dtype != torch.float16:
            out = out.to(dtype=input_dtype)
        return out

    def extra_repr(self) -> str:
        return "in_features={}, out_features={}, bias={}, w_bit={}, group_size={}".format(
            self.in_features, self.out_features, self.bias is not None, self.w_bit, self.group_size)


# Older names kept by the reference (linear_awq.py:412-414).
WQLinear_GEMM = AWQLinear_GEMM
WQLinearMMFunction = AWQLinearMMFunction
