"""`GraphedStep`: a fixed sequence of quantized-linear calls (one decode step of a model, or any part of
it with static shapes) captured once in a CUDA graph and replayed per token.

At decode sizes a linear is a few microseconds of device time, less than the host needs to get through
one Python module call (the reference's wrapper costs about 70 us per call in its own profile,
LLMQRT/runtime_refact/nn_models/modules/linear/linear_awq.py:128-212; this package's about 13 us).  Replaying
a captured step removes the per-call host work altogether: the 112 linears of a 28-layer step become one
graph launch.  The kernels are capture-safe as they are: no allocation, no synchronisation, workspaces
reached through pointers that stay valid (they are created during the warm-up calls before the capture).

    step = GraphedStep(lambda x: [m(x) for m in modules][-1], example_inputs=(x,))
    y = step(x_new)            # copies x_new into the captured input, replays, returns the captured output

Inputs may live on the host (pinned memory makes the copy asynchronous).  The returned tensors are the
graph's own output buffers: they are overwritten by the next call.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


def _flatten(out):
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, (list, tuple)):
        flat = []
        for o in out:
            flat.extend(_flatten(o))
        return flat
    raise TypeError(f"a graphed step must return tensors (or lists / tuples of them), got {type(out).__name__}")


class GraphedStep:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], device: torch.device | str | None = None,
                 warmup: int = 3):
        """`fn(*inputs)` must launch the same kernels on the same shapes every time it is called and must not
        synchronise.  `example_inputs` fix the shapes and dtypes (their values are used for the warm-up calls,
        which also let every module repack its weights and size its workspace before the capture)."""
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device; there is no CPU fallback")
        if device is None:
            on_device = [t.device for t in example_inputs if t.is_cuda]
            device = on_device[0] if on_device else torch.device("cuda", torch.cuda.current_device())
        self.device = torch.device(device)
        self.fn = fn
        self.static_inputs = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in example_inputs]
        for s, t in zip(self.static_inputs, example_inputs):
            s.copy_(t)
        self.graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side), torch.no_grad():
            # warm-up on the capture stream: workspaces are per stream, and the first call after a repack
            # must not run inside the graph
            for _ in range(max(warmup, 2)):
                fn(*self.static_inputs)
            side.synchronize()
            with torch.cuda.graph(self.graph, stream=side):
                self._out = fn(*self.static_inputs)
        torch.cuda.current_stream(self.device).wait_stream(side)
        self.static_outputs = _flatten(self._out)
        # The captured kernels hold raw pointers into the capture stream's workspaces: keep those alive.
        from . import kernels
        self._stream = side
        self._workspaces = {key[2]: ws for key, ws in kernels._workspaces.items()
                            if key[0] == self.device.index and key[1] == side.cuda_stream}

    def status(self) -> int:
        """0, or the code a device-side wait left behind in one of the captured kernels' workspaces
        (the outputs of that replay are then invalid).  Synchronises."""
        status = 0
        ws = self._workspaces.get("awq_b200_linear")
        if ws is not None:
            status |= int(ws[:4].view(torch.int32).item())
            status |= int(ws[256 + 4095 * 4: 256 + 4096 * 4].view(torch.int32).item())
        return status

    def replay(self):
        """Replay on the current stream with whatever the captured input buffers hold."""
        self.graph.replay()
        return self._out

    def __call__(self, *inputs: torch.Tensor):
        if len(inputs) != len(self.static_inputs):
            raise ValueError(f"expected {len(self.static_inputs)} inputs, got {len(inputs)}")
        for s, t in zip(self.static_inputs, inputs):
            if t.shape != s.shape or t.dtype != s.dtype:
                raise ValueError(f"input of shape {tuple(t.shape)} / {t.dtype} does not match the captured "
                                 f"{tuple(s.shape)} / {s.dtype}")
            if t.data_ptr() != s.data_ptr():
                s.copy_(t, non_blocking=True)
        self.graph.replay()
        return self._out
