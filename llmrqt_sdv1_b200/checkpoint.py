"""Checkpoint tensors <-> quantized-linear modules, without `accelerate`.

The reference fills its `AWQLinear_GEMM` buffers with `accelerate.load_checkpoint_and_dispatch`
(LLMQRT/runtime_refact/core/base.py:143-151) from the `.safetensors` files its quantizer wrote
(`qweight` int32 [K, N/8], `qzeros` int32 [K/G, N/8], `scales` fp16 [K/G, N], optional `bias`, all under the
module's name).  `load_checkpoint` does the same job for a model on one GPU: it maps the files, copies every
tensor whose name matches a parameter or buffer of the model straight to its device, and repacks the AWQ
weights into the kernel layout right away, so the first forward does no set-up work.  `save_checkpoint` is
the inverse (`state_dict()` round trip) and writes the same file format.

The safetensors container is read and written here directly (8-byte little-endian header length, a JSON
header with dtype / shape / byte range per tensor, then the raw little-endian data): mapping the file gives
zero-copy CPU views, so a tensor goes disk -> page cache -> GPU with no intermediate host copy.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Dict, Iterable, Iterator, Tuple

import numpy as np
import torch

from .linear_awq import AWQLinear_GEMM

# safetensors dtype tag -> (numpy dtype used for the mapped view, torch dtype of the result)
_DTYPES = {
    "F64": (np.float64, torch.float64), "F32": (np.float32, torch.float32), "F16": (np.float16, torch.float16),
    "BF16": (np.int16, torch.bfloat16), "I64": (np.int64, torch.int64), "I32": (np.int32, torch.int32),
    "I16": (np.int16, torch.int16), "I8": (np.int8, torch.int8), "U8": (np.uint8, torch.uint8),
    "BOOL": (np.bool_, torch.bool),
}
_TAGS = {t: tag for tag, (_, t) in _DTYPES.items()}


def read_header(path: str) -> Tuple[Dict[str, dict], int]:
    """({name: {"dtype", "shape", "data_offsets"}}, offset of the data section) of one .safetensors file."""
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", raw)
        size = os.path.getsize(path)
        if n > size - 8:
            raise ValueError(f"{path}: header length {n} exceeds the file size")
        header = json.loads(f.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    for name, meta in header.items():
        lo, hi = meta["data_offsets"]
        if meta["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {meta['dtype']}")
        itemsize = np.dtype(_DTYPES[meta["dtype"]][0]).itemsize
        if lo > hi or 8 + n + hi > size or hi - lo != itemsize * int(np.prod(meta["shape"], dtype=np.int64)):
            raise ValueError(f"{path}: tensor {name!r} has an inconsistent byte range")
    return header, 8 + n


def iter_tensors(path: str, names: Iterable[str] | None = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, CPU tensor) for the tensors of one file; the tensors are read-only views of the mapped file."""
    header, start = read_header(path)
    wanted = None if names is None else set(names)
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    for name, meta in header.items():
        if wanted is not None and name not in wanted:
            continue
        np_dtype, torch_dtype = _DTYPES[meta["dtype"]]
        lo, hi = meta["data_offsets"]
        arr = np.frombuffer(mm, dtype=np_dtype, count=(hi - lo) // np.dtype(np_dtype).itemsize, offset=start + lo)
        t = torch.from_numpy(arr.reshape(meta["shape"])) if arr.size else torch.empty(meta["shape"], dtype=torch_dtype)
        if torch_dtype == torch.bfloat16 and arr.size:
            t = t.view(torch.bfloat16)
        yield name, t


def checkpoint_files(path: str) -> list[str]:
    """A .safetensors file, or every .safetensors file of a directory in name order."""
    if os.path.isdir(path):
        files = sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
        if not files:
            raise FileNotFoundError(f"no .safetensors files in {path}")
        return files
    return [path]


def _assign(model: torch.nn.Module, name: str, tensor: torch.Tensor) -> None:
    """Replace the parameter or buffer `name` of `model` by `tensor` (used for destinations on the meta device)."""
    mod_name, _, leaf = name.rpartition(".")
    mod = model.get_submodule(mod_name) if mod_name else model
    if leaf in mod._parameters:
        mod._parameters[leaf] = torch.nn.Parameter(tensor, requires_grad=False)
    else:
        mod._buffers[leaf] = tensor


@torch.no_grad()
def load_checkpoint(model: torch.nn.Module, path: str, strict: bool = True, prepare: bool = True,
                    device: torch.device | str | None = None, release_qweight: bool = False) -> dict:
    """Copy every checkpoint tensor that names a parameter or buffer of `model` into it, then repack each
    `AWQLinear_GEMM` into the kernel layout.  Shapes and dtypes must match, except that floating tensors are
    cast to the destination's dtype.  A destination that lives on the meta device (a model built without
    storage, as the reference builds it under `init_empty_weights`, LLMQRT/runtime_refact/core/base.py:132-151)
    is created on `device`; every other destination is filled where it already lives.

    `release_qweight=True` repacks every quantized linear as soon as its three tensors are in and gives its
    on-disk `qweight` back at once, so the device never holds more than one layer's int4 weights twice: after
    the load it holds 1.0 x the packed bytes plus scales and zeros (`state_dict()` still returns the on-disk
    tensors, rebuilt on demand by the inverse repack).

    Returns {"loaded": [...], "missing": [...], "unexpected": [...]}; with `strict`, missing or unexpected
    names raise."""
    import warnings
    dest = dict(model.named_parameters())
    dest.update(dict(model.named_buffers()))
    target = torch.device(device) if device is not None else None
    awq_modules = {n: m for n, m in model.named_modules() if isinstance(m, AWQLinear_GEMM)}
    pending = {n: {"qweight", "qzeros", "scales"} for n in awq_modules} if release_qweight else {}
    loaded, unexpected = [], []
    with warnings.catch_warnings():
        warnings.filterwarnings("ignore", message=".*not writable.*")
        for file in checkpoint_files(path):
            for name, src in iter_tensors(file):
                d = dest.get(name)
                if d is None:
                    unexpected.append(name)
                    continue
                if tuple(d.shape) != tuple(src.shape):
                    raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} != module shape {tuple(d.shape)}")
                if d.dtype != src.dtype and not (d.dtype.is_floating_point and src.dtype.is_floating_point):
                    raise ValueError(f"{name}: checkpoint dtype {src.dtype} cannot fill a {d.dtype} tensor")
                if d.device.type == "meta":
                    if target is None:
                        raise ValueError(f"{name} lives on the meta device: pass device= to say where to create it")
                    _assign(model, name, src.to(device=target, dtype=d.dtype))
                else:
                    d.copy_(src)      # pageable host memory -> device: one staged copy, cast on the device side
                loaded.append(name)
                mod_name, _, leaf = name.rpartition(".")
                todo = pending.get(mod_name)
                if todo is not None:
                    todo.discard(leaf)
                    m = awq_modules[mod_name]
                    if not todo and m.qweight.is_cuda:
                        m.release_qweight()          # repack now, keep the kernel layout only
                        del pending[mod_name]
    missing = sorted(set(dest) - set(loaded))
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint does not match the model: missing {missing[:8]}{'...' if len(missing) > 8 else ''}, "
                       f"unexpected {unexpected[:8]}{'...' if len(unexpected) > 8 else ''}")
    if prepare:
        for m in model.modules():
            if isinstance(m, AWQLinear_GEMM) and m.qweight.is_cuda:
                m.prepare()
    return {"loaded": loaded, "missing": missing, "unexpected": unexpected}


def save_checkpoint(state: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] | None = None) -> None:
    """Write `state` (e.g. `model.state_dict()`) as one .safetensors file: tensors in name order, data
    8-byte aligned, header padded with spaces as the format asks."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(state)
    arrays = []
    for name in order:
        t = state[name].detach()
        if t.dtype not in _TAGS:
            raise ValueError(f"{name}: dtype {t.dtype} cannot be stored")
        t = t.contiguous().cpu()
        raw = (t.view(torch.int16) if t.dtype == torch.bfloat16 else t).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _TAGS[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        arrays.append(raw)
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for raw in arrays:
            f.write(raw)
    os.replace(tmp, path)
