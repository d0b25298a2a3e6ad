#!/usr/bin/env python
"""Benchmark of the AWQ W4A16 quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One JSON line on stdout (rank 0).  Workloads:

  ffn70b_tp     (default at every N)  the 70B-class FFN linears, M=1, tensor-parallel over
                the N ranks (N = 1: unsharded): gate_up 8192->57344 column-sharded, down
                28672->8192 row-sharded + one all-reduce (the library's one-shot peer
                all-reduce for small outputs, NCCL timed beside it); one step = 8 layers with
                their own weights (2.9 GB per step over all ranks, larger than L2).  The
                1/2/4/8-GPU series is this one workload (strong scaling).  At N = 1 the line
                also carries the block `qwen3_decode` and the per-shape tables.
  qwen3_decode  the Qwen3-1.7B-shaped decode linears, M=1: one step =
                28 layers x {qkv 2048->4096, o 2048->2048, gate_up 2048->12288,
                down 6144->2048}, every layer with its own weights (734 MB per step,
                larger than the 126 MB L2, so no flush is needed between steps).
  qwen3_e2e     a random-init Qwen3-1.7B-architecture model, 128 prompt + 128 greedy tokens.

Any device-side wait that expired (status words of the kernels' workspaces and of the peer all-reduce)
makes the run exit 1 instead of printing a number.

`value` times the kernels alone (inputs resident in HBM, one CUDA graph per step);
`e2e` times the module API (`AWQLinear_GEMM.forward`) with the activations starting in
pinned host memory and the result read back to the host every step.  `--impl reference`
times the CPU dequant+matmul path (the oracle's C restatement, all host threads) on
a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GROUP = 128
QWEN3_LAYERS = 28
QWEN3_LINEARS = [("qkv", 2048, 4096), ("o", 2048, 2048), ("gate_up", 2048, 12288), ("down", 6144, 2048)]
FFN70B_LAYERS = 8
FFN70B = {"gate_up": (8192, 57344), "down": (28672, 8192)}
PREFILL_SHAPES = [(4096, 6144), (4096, 4096), (4096, 28672), (14336, 4096)]

# dram__bytes_read.sum + dram__bytes_write.sum per launch of a decode kernel, from one ncu capture of that
# kernel on that shape (None where no capture exists).
NCU_TRAFFIC_BYTES = {"gemv_2048x12288_m1": 13_117_440, "decode_8192x57344_m1": 248_161_280}


def gemv_bytes(M, K, N, G=GROUP):
    """Algorithmic bytes of one decode linear: packed weights + scales + zeros + x + y."""
    return K * N // 2 + (K // G) * N * 2 + (K // G) * N // 2 + 2 * M * K + 2 * M * N


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting"}

    def __init__(self, index):
        self.ok = False
        self.sm, self.bits = [], 0
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_sm = None

    def sample(self):
        if not self.ok:
            return
        try:
            self.sm.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            fn = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
            self.bits |= int(fn(self.h))
        except Exception:
            pass

    def wait_and_sample(self, end_event):
        self.sample()
        while not end_event.query():
            self.sample()
            time.sleep(0.001)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.max_sm, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.sm), "sm_max_mhz": self.max_sm,
                "reasons": [n for b, n in self.REASONS.items() if self.bits & b], "samples": len(self.sm)}


# ----------------------------------------------------------------------------- reference / CPU arm
# The CPU legs time the C restatement of the reference's dequant + matmul path with OpenMP on every host
# core.  Launchers such as torchrun export OMP_NUM_THREADS=1 to their ranks; the baseline ignores that and
# asks for all cores, and reports the count it got.
CPU_SAMPLES = {
    # name -> (shapes, description).  A GB/s rate does not depend on how much of the workload is sampled.
    "ffn70b_tp": ([("gate_up", 8192, 7168), ("down", 3584, 8192)],
                  "one eighth of a 70B FFN layer per step (gate_up 8192x7168 and down 3584x8192, the tp=8 shard "
                  "of the GPU arm's layer; 44 MB of int4 weights) at M=1"),
    "qwen3_decode": ([(n, K, N) for (n, K, N) in QWEN3_LINEARS],
                     "one Qwen3-1.7B layer's four decode linears at M=1 per step (1/28 of the GPU arm's step)"),
}


def cpu_threads_all():
    from oracle import c_oracle
    return c_oracle.use_all_cores()


def cpu_layer_tensors(shapes, seed=0):
    """Random int4 codes, zero points and scales of the given shapes (numpy, seeded).  The timed C code does
    the same work whatever the values are, so the tensors are drawn directly instead of being quantised from
    a random fp16 weight (which takes numpy longer than the whole measurement)."""
    import numpy as np
    out = []
    for i, (_, K, N) in enumerate(shapes):
        rng = np.random.default_rng(seed + i)
        qw = rng.integers(0, 1 << 32, size=(K, N // 8), dtype=np.uint32).view(np.int32)
        qz = rng.integers(0, 1 << 32, size=(K // GROUP, N // 8), dtype=np.uint32).view(np.int32)
        sc = (rng.random((K // GROUP, N), dtype=np.float32) * 0.004 + 0.002).astype(np.float16)
        x = rng.standard_normal((1, K), dtype=np.float32).astype(np.float16)
        out.append((K, N, qw, qz, sc, x))
    return out


def cpu_time_decode_layers(layer, repeats):
    """Seconds per pass of the reference CPU path (dequant + matmul, C restatement) over `layer`."""
    from oracle import c_oracle
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for (K, N, qw, qz, sc, x) in layer:
            c_oracle.linear_forward(x, qw, qz, sc, GROUP)
        times.append(time.perf_counter() - t0)
    return times


def cpu_baseline(workload, passes):
    """The `cpu_baseline` object of a GPU-arm line: a bounded sample of `workload` on the host cores."""
    cores = cpu_threads_all()
    shapes, sample = CPU_SAMPLES[workload]
    layer = cpu_layer_tensors(shapes)
    cpu_time_decode_layers(layer, 2)
    t = cpu_time_decode_layers(layer, passes)
    sec = sum(t) / len(t)
    nbytes = sum(gemv_bytes(1, K, N) for (K, N, *_r) in layer)
    return {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{sample}, {passes} passes, C restatement of dequant+matmul with OpenMP", "ms_per_pass": sec * 1e3}


def run_reference(args, rank):
    """`--impl reference`: the CPU dequant+matmul path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    cores = cpu_threads_all()
    workload = args.workload if args.workload in CPU_SAMPLES else "ffn70b_tp"
    shapes, sample = CPU_SAMPLES[workload]
    layer = cpu_layer_tensors(shapes)
    nbytes = sum(gemv_bytes(1, K, N) for (K, N, *_r) in layer)
    cpu_time_decode_layers(layer, max(args.warmup, 1))
    times = cpu_time_decode_layers(layer, args.steps)
    sec = sum(times) / len(times)
    gbs = nbytes / sec / 1e9
    line = {
        "impl": "reference", "metric": "W4A16 GEMV HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong" if workload == "ffn70b_tp" else "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic", "config": {"workload": workload, "M": 1, "group_size": GROUP,
                                        "bytes_per_step": nbytes, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm helpers
def _dist():
    import torch.distributed as dist
    return dist if (dist.is_available() and dist.is_initialized()) else None


def time_graph(torch, fn, iters, warmup=3, reps=3, min_ms=4.0):
    """Median ms per call of `fn` (a sequence of launches on the current stream), graph-replayed.
    `iters` is raised until one repetition lasts at least `min_ms` (short repetitions are measured while
    the clocks are still ramping).  With several ranks every rank must replay the graph the same number of
    times (the graph may contain an exchange that waits for the peers), so the estimate the count is derived
    from is the maximum over the ranks."""
    for _ in range(warmup):
        fn()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    est = max(a.elapsed_time(b) / 3, 1e-3)
    dist = _dist()
    if dist is not None and dist.get_world_size() > 1:
        t = torch.tensor([est], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        est = float(t.item())
    iters = max(iters, min(2000, int(min_ms / est) + 1))
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / iters)
    return statistics.median(out)


def require_clean(torch, phase, **words):
    """Every status word must be zero on every rank; otherwise all ranks stop with exit code 1 and no
    benchmark line is printed (a number measured around an expired device-side wait means nothing)."""
    bad = {k: int(v) for k, v in words.items() if v is not None and int(v) != 0}
    flag = 1 if bad else 0
    dist = _dist()
    if dist is not None and dist.get_world_size() > 1:
        t = torch.tensor([flag], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        flag = int(t.item())
    if flag:
        sys.stderr.write(json.dumps({"error": "a device-side wait expired", "phase": phase, "status": bad,
                                     "rank": int(os.environ.get("RANK", "0"))}) + "\n")
        sys.stderr.flush()
        if dist is not None:
            try:
                dist.destroy_process_group()
            except Exception:
                pass
        sys.exit(1)


def decode_detail(torch, kernels, quantize, peaks):
    """Per-shape decode table: GB/s at M in {1,4,8,16}, weights rotated over > 2x L2."""
    rows = []
    shapes = [(n, K, N) for (n, K, N) in QWEN3_LINEARS] + [("gate", 2048, 6144)] + \
             [("70b_gate_up", *FFN70B["gate_up"]), ("70b_down", *FFN70B["down"])]
    for name, K, N in shapes:
        per = K * N // 2
        copies = max(2, min(64, (300 << 20) // per + 1))
        qw, qz, sc = quantize.random_awq_tensors(K, N, GROUP, seed=K + N, device="cuda")
        base = kernels.make_packed(qw, qz, sc, GROUP)
        pws = [base] + [kernels.PackedWeight(base.packed.clone(), qz.clone(), sc.clone(), K, N, GROUP)
                        for _ in range(copies - 1)]
        for M in (1, 4, 8, 16):
            x = torch.randn((M, K), device="cuda").half()
            ys = [torch.empty((M, N), dtype=torch.float16, device="cuda") for _ in range(copies)]

            def fn():
                for pw, y in zip(pws, ys):
                    kernels.linear(x, pw, out=y, overlap=True)
            ms = time_graph(torch, fn, iters=5) / copies
            gbs = gemv_bytes(M, K, N) / (ms * 1e-3) / 1e9
            rows.append({"linear": name, "K": K, "N": N, "M": M, "us": round(ms * 1e3, 3), "gbs": round(gbs, 1),
                         "frac_measured": round(gbs / peaks["hbm_gbs"], 4), "frac_nominal_8tbs": round(gbs / 8000.0, 4)})
        del pws, base
    return rows


def q8_detail(torch, peaks):
    """The other quantized linears of the reference extension (FP8 e4m3, SmoothQuant INT8) on 70B-sized layers.
    Decode rows (M in {1, 16}) against the HBM peak: bytes = 8-bit weights + activations + 16-bit output, weights
    rotated over more than 2x L2.  Prefill rows (M in {2048, 8192}) in TFLOP/s; MEASURED_PEAKS holds no 8-bit
    figure, so the fraction is of twice the measured bf16 burst (the ratio of the two nominal dense peaks), with
    the library's own FP8 GEMM (torch._scaled_mm) timed beside it.  `module_us` is a whole FP8DynamicLinear forward
    (activation quantisation + GEMM)."""
    from llmrqt_sdv1_b200 import q8
    from llmrqt_sdv1_b200.linear_fp8 import FP8NativeDynamicLinear
    rows = []
    one = torch.tensor(1.0, device="cuda")
    for name, N, K in (("qkvo", 8192, 8192), ("gate_up", 57344, 8192), ("down", 8192, 28672)):
        copies = max(2, min(8, (300 << 20) // (N * K) + 1))
        wf = [torch.randn(N, K, device="cuda").mul_(0.5).to(torch.float8_e4m3fn) for _ in range(copies)]
        wi = [w.view(torch.int8) for w in wf]
        mod = FP8NativeDynamicLinear(K, N, False, dev="cuda", dtype=torch.bfloat16)
        mod.weight.data = wf[0]
        mod.weight_scale.data.fill_(0.01)
        for M in (1, 16, 2048, 8192):
            xb = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            xf = xb.to(torch.float8_e4m3fn)
            xi = xf.view(torch.int8)
            ob = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            oh = torch.empty(M, N, device="cuda", dtype=torch.float16)
            bias = torch.zeros(N, device="cuda", dtype=torch.float16)
            min_ms = 50.0 if M >= 2048 else 20.0

            def run_fp8():
                for w in wf:
                    q8.gemm_tensorwise(xf, w.t(), None, 0.5, 1.0, torch.bfloat16, out=ob)

            def run_int8():
                for w in wi:
                    q8.gemm_tensorwise(xi, w.t(), bias, 1e-4, 1.0, torch.float16, int8=True, out=oh)

            def run_lib():
                for w in wf:
                    torch._scaled_mm(xf, w.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            if M == 1:
                time_graph(torch, run_fp8, iters=3, min_ms=min_ms)      # first pass over freshly written weights: discarded
            t_f = time_graph(torch, run_fp8, iters=3, min_ms=min_ms) / copies
            t_i = time_graph(torch, run_int8, iters=3, min_ms=min_ms) / copies
            t_m = time_graph(torch, lambda: mod(xb), iters=3, min_ms=min_ms)
            try:
                t_l = time_graph(torch, run_lib, iters=3, min_ms=min_ms) / copies if M >= 16 else None
            except Exception:
                t_l = None
            flops, nbytes = 2.0 * M * N * K, N * K + M * K + 2 * M * N
            row = {"linear": name, "N": N, "K": K, "M": M, "fp8_us": round(t_f * 1e3, 2), "int8_us": round(t_i * 1e3, 2),
                   "module_us": round(t_m * 1e3, 2), "scaled_mm_us": round(t_l * 1e3, 2) if t_l else None}
            if M <= 16:
                row.update(fp8_gbs=round(nbytes / t_f / 1e6, 1), int8_gbs=round(nbytes / t_i / 1e6, 1),
                           fp8_frac_hbm=round(nbytes / t_f / 1e6 / peaks["hbm_gbs"], 4))
            else:
                row.update(fp8_tflops=round(flops / t_f / 1e9, 1), int8_tops=round(flops / t_i / 1e9, 1),
                           scaled_mm_tflops=round(flops / t_l / 1e9, 1) if t_l else None,
                           fp8_frac_2x_bf16_burst=round(flops / t_f / 1e9 / (2 * peaks["tflops"]), 4))
            rows.append(row)
        require_clean(torch, "q8_detail", q8=q8.status())
        del wf, wi, mod
        torch.cuda.empty_cache()
    return rows


def mlp_fusion_detail(torch, kernels, quantize):
    """The MLP of the decode configuration (hidden 2048, intermediate 6144) over 28 layers of distinct weights
    (0.5 GB > L2), `h = h + down(silu(gate(h)) * up(h))`, as the three linears plus separate elementwise
    kernels the reference's layer runs, and as two launches with fused epilogues.  us per layer, CUDA graph."""
    import torch.nn.functional as F
    hidden, inter, layers = 2048, 6144, 28
    sep, fused = [], []
    for layer in range(layers):
        gate = quantize.random_awq_tensors(hidden, inter, GROUP, seed=10 * layer, device="cuda")
        up = quantize.random_awq_tensors(hidden, inter, GROUP, seed=10 * layer + 1, device="cuda")
        down = quantize.random_awq_tensors(inter, hidden, GROUP, seed=10 * layer + 2, device="cuda")
        pw_d = kernels.make_packed(*down, GROUP)
        sep.append((kernels.make_packed(*gate, GROUP), kernels.make_packed(*up, GROUP), pw_d))
        fused.append((kernels.make_gated_packed(gate, up, GROUP), pw_d))
    out = {}
    for M in (1, 16):
        h = torch.randn((M, hidden), device="cuda").half()
        g, u, a = (torch.empty((M, inter), dtype=torch.float16, device="cuda") for _ in range(3))
        d = torch.empty((M, hidden), dtype=torch.float16, device="cuda")

        def step_separate():
            for pw_g, pw_u, pw_d in sep:
                kernels.linear(h, pw_g, out=g, overlap=True)
                kernels.linear(h, pw_u, out=u, overlap=True)
                torch.mul(F.silu(g), u, out=a)
                kernels.linear(a, pw_d, out=d, overlap=True)
                h.add_(d)

        def step_fused():
            for pw_gu, pw_d in fused:
                kernels.linear_fused(h, pw_gu, gated=True, out=a, overlap=True)
                kernels.linear_fused(a, pw_d, residual=h, out=h, overlap=True)
        t_sep = time_graph(torch, step_separate, iters=10) / layers
        h.normal_()
        t_fused = time_graph(torch, step_fused, iters=10) / layers
        out["M%d" % M] = {"separate_us_per_layer": round(t_sep * 1e3, 2), "fused_us_per_layer": round(t_fused * 1e3, 2),
                          "launches_per_layer": {"separate": 6, "fused": 2}}
    return out


def prefill_detail(torch, kernels, quantize, peaks):
    """Config 3: every (K, N, M) cell, each timed in repetitions of at least 50 ms of back-to-back launches (so
    under the power cap), with the SM clock sampled during the cell: `us_x_ghz` (time x median clock) tells a
    slower kernel from a lower clock when two runs of one cell differ."""
    rows = []
    for K, N in PREFILL_SHAPES:
        qw, qz, sc = quantize.random_awq_tensors(K, N, GROUP, seed=K + N, device="cuda")
        pw = kernels.make_packed(qw, qz, sc, GROUP)
        for M in (512, 2048, 8192):
            x = torch.randn((M, K), device="cuda").half()
            y = torch.empty((M, N), dtype=torch.float16, device="cuda")
            sampler = ClockSampler(0)
            stop = {"done": False}
            import threading

            def poll():
                while not stop["done"]:
                    sampler.sample()
                    time.sleep(0.002)
            th = threading.Thread(target=poll, daemon=True)
            th.start()
            ms = time_graph(torch, lambda: kernels.gemm(x, pw, out=y), iters=10, min_ms=50.0)
            stop["done"] = True
            th.join()
            mhz = sampler.summary()["sm_mhz"]
            tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
            rows.append({"K": K, "N": N, "M": M, "us": round(ms * 1e3, 2), "tflops": round(tf, 1),
                         "frac_measured": round(tf / peaks["tflops"], 4),
                         "frac_sustained": round(tf / peaks["tflops_sustained"], 4),
                         "frac_nominal_2250": round(tf / 2250.0, 4), "sm_mhz": mhz,
                         "us_x_ghz": (round(ms * 1e3 * mhz / 1e3, 1) if mhz else None)})
        require_clean(torch, "prefill_detail", gemm=kernels.gemm_status())
    return rows


def qwen3_decode_measure(args, torch, peaks):
    """The Qwen3-1.7B decode step (28 layers x 4 linears, M = 1): device time of the 112 dispatcher calls in one
    CUDA graph, the same step end to end through the module API with host buffers, and parity of what was timed."""
    from llmrqt_sdv1_b200 import AWQLinear_GEMM, kernels, quantize
    from llmrqt_sdv1_b200.sq_fp8_kernels import packed_for
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    M = 1
    modules, pws, xs, ys = [], [], {}, []
    for K in (2048, 6144):
        xs[K] = torch.randn((M, K), device=dev).half()
    for layer in range(QWEN3_LAYERS):
        for i, (name, K, N) in enumerate(QWEN3_LINEARS):
            qw, qz, sc = quantize.random_awq_tensors(K, N, GROUP, seed=layer * 16 + i, device=dev)
            m = AWQLinear_GEMM(4, GROUP, K, N, False, dev)
            m.qweight, m.qzeros, m.scales = qw, qz, sc
            m.prepare()
            modules.append(m)
            pws.append(packed_for(m.qweight, m.qzeros, m.scales, GROUP))
            ys.append(torch.empty((M, N), dtype=torch.float16, device=dev))
    step_bytes = sum(gemv_bytes(M, pw.K, pw.N) for pw in pws)
    launches_per_step = len(pws)

    def step():
        for pw, y in zip(pws, ys):
            kernels.linear(xs[pw.K], pw, out=y, overlap=True)

    for _ in range(max(args.warmup, 3)):
        step()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        graph.replay()
    b.record()
    sampler.wait_and_sample(b)
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    value = step_bytes / (ms * 1e-3) / 1e9
    require_clean(torch, "qwen3_decode timed region", gemv=kernels.gemv_status(), gemm=kernels.gemm_status())

    # ---- end to end through the module API, host buffers ---------------------------------
    hx = {K: torch.randn((1, M, K)).half().pin_memory() for K in (2048, 6144)}
    dx = {K: torch.empty((1, M, K), dtype=torch.float16, device=dev) for K in (2048, 6144)}
    hy = torch.empty((1, M, QWEN3_LINEARS[-1][2]), dtype=torch.float16).pin_memory()

    def e2e_step():
        for K in dx:
            dx[K].copy_(hx[K], non_blocking=True)
        y = None
        for m in modules:
            y = m(dx[m.in_features])
        hy.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        e2e_step()
    a2, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a2.record()
    for _ in range(args.steps):
        e2e_step()
    b2.record()
    torch.cuda.synchronize()
    e2e_ms = a2.elapsed_time(b2) / args.steps
    eager = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "ms_per_step": e2e_ms,
             "api": "AWQLinear_GEMM.forward x 112 per step, no graph"}
    nbytes_in = sum(t.numel() * 2 for t in hx.values())
    graphed = None
    try:
        # The same step as the package's decode API runs it: the 112 module calls captured once in a CUDA graph
        # (GraphedStep), per step the host->device copies of the inputs, one replay, the device->host copy.
        from llmrqt_sdv1_b200 import GraphedStep

        def all_modules(x2048, x6144):
            by_k = {2048: x2048, 6144: x6144}
            y = None
            for m in modules:
                y = m(by_k[m.in_features])
            return y
        graphed = GraphedStep(all_modules, (dx[2048], dx[6144]))

        def e2e_graphed_step():
            y = graphed(hx[2048], hx[6144])
            hy.copy_(y, non_blocking=True)
            torch.cuda.synchronize()

        for _ in range(max(args.warmup, 3)):
            e2e_graphed_step()
        y_graphed = hy.clone()
        e2e_step()
        graphed_equal = bool(torch.equal(y_graphed, hy))
        a3, b3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a3.record()
        for _ in range(args.steps):
            e2e_graphed_step()
        b3.record()
        torch.cuda.synchronize()
        g_ms = a3.elapsed_time(b3) / args.steps
        e2e = {"value": step_bytes / (g_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": g_ms,
               "h2d_bytes_per_step": nbytes_in, "d2h_bytes_per_step": hy.numel() * 2,
               "api": "GraphedStep over AWQLinear_GEMM.forward x 112: host inputs copied in, one graph replay, result copied out",
               "same_bits_as_eager": graphed_equal, "eager": eager}
    except Exception as exc:   # the eager number stands if the capture is refused on this box
        e2e = dict(eager, unit="GB/s", h2d_bytes_per_step=nbytes_in, d2h_bytes_per_step=hy.numel() * 2,
                   graphed_unavailable=f"{type(exc).__name__}: {exc}")
    require_clean(torch, "qwen3_decode end to end", gemv=kernels.gemv_status(), gemm=kernels.gemm_status(),
                  graphed=(graphed.status() if graphed is not None else 0))

    # ---- parity of what was just timed, against dequant + library matmul on the device ----
    pw0, m0 = pws[2], modules[2]
    W = kernels.dequantize(m0.qweight, m0.qzeros, m0.scales, GROUP)
    ref = torch.matmul(xs[pw0.K].float(), W.float())
    err = float((ys[2].float() - ref).abs().max() / ref.abs().max())
    parity = {"dequant_bit_exact": bool(torch.equal(kernels.dequantize_packed(pw0), W)), "max_norm_err": err,
              "tolerance": 2e-3}
    return {"ms_per_step": ms, "value": value, "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
            "frac_of_nominal_8tbs": value / 8000.0, "launches_per_step": launches_per_step,
            "avg_launch_us": ms * 1e3 / launches_per_step, "bytes_per_step": step_bytes, "e2e": e2e,
            "parity": parity, "clocks": sampler.summary(),
            "traffic_gate_up_launch": NCU_TRAFFIC_BYTES["gemv_2048x12288_m1"]}


def detail_tables(line, args, torch, peaks):
    """Per-shape tables of the single-GPU line (configs 2 and 3 of the baseline, the MLP fusion, config 5)."""
    from llmrqt_sdv1_b200 import kernels, quantize
    line["decode_detail"] = decode_detail(torch, kernels, quantize, peaks)
    require_clean(torch, "decode_detail", gemv=kernels.gemv_status(), gemm=kernels.gemm_status())
    line["prefill_detail"] = prefill_detail(torch, kernels, quantize, peaks)
    line["mlp_fusion"] = mlp_fusion_detail(torch, kernels, quantize)
    line["q8_detail"] = q8_detail(torch, peaks)
    require_clean(torch, "prefill_detail / mlp_fusion", gemv=kernels.gemv_status(), gemm=kernels.gemm_status())
    best = max(line["prefill_detail"], key=lambda r: r["tflops"])
    # Each shape is timed in repetitions of back-to-back launches, i.e. under the power cap: the sustained
    # library figure is the matching denominator; the burst figure is given beside it.
    line["roofline_gemm"] = {"bound": "tensor", "achieved": best["tflops"], "peak": peaks["tflops_sustained"],
                             "unit": "TFLOP/s", "frac": best["tflops"] / peaks["tflops_sustained"],
                             "peak_burst": peaks["tflops"], "frac_of_burst": best["tflops"] / peaks["tflops"],
                             "frac_of_nominal_2250": best["tflops"] / 2250.0, "traffic": None,
                             "peak_source": peaks["source"], "kernel": "awq::wtm_kernel",
                             "shape": {k: best[k] for k in ("M", "K", "N")}}


def run_qwen3_decode(args, torch, peaks):
    """`--workload qwen3_decode`: the Qwen3-1.7B decode step as the headline of its own line."""
    blk = qwen3_decode_measure(args, torch, peaks)
    line = {
        "metric": "W4A16 GEMV HBM GB/s", "value": blk["value"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": blk["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "qwen3_decode: Qwen3-1.7B decode linears (qkv, o, gate_up, down) x 28 layers, M=1, "
                               "W4A16 g128", "M": 1, "group_size": GROUP, "launches_per_step": blk["launches_per_step"],
                   "bytes_per_step": blk["bytes_per_step"], "l2": "inputs larger than L2 (734 MB of weights per step, no flush)",
                   "timing": "one CUDA graph per step, CUDA events on the launching stream"},
        "roofline": {"bound": "hbm", "achieved": blk["value"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": blk["frac"], "traffic": blk["traffic_gate_up_launch"],
                     "peak_source": peaks["source"], "kernel": "awq::gemv_kernel",
                     "avg_launch_us": blk["avg_launch_us"], "frac_of_nominal_8tbs": blk["frac_of_nominal_8tbs"]},
        "e2e": blk["e2e"], "gpu_launches": blk["launches_per_step"] * args.steps, "clocks": blk["clocks"],
        "parity": blk["parity"],
    }
    if not args.no_detail:
        detail_tables(line, args, torch, peaks)
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline("qwen3_decode", 28 * 3)
    print(json.dumps(line), flush=True)


def run_ffn70b_tp(args, torch, peaks, rank, world, local_rank):
    """The headline workload at every N: 8 layers of the 70B-class FFN linears at M = 1, tensor-parallel over
    `world` ranks (unsharded at world = 1)."""
    import torch.distributed as dist
    from llmrqt_sdv1_b200 import kernels, quantize
    from llmrqt_sdv1_b200.sharded import ColumnParallelAWQLinear, RowParallelAWQLinear
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    M = 1
    Kg, Ng = FFN70B["gate_up"]
    Kd, Nd = FFN70B["down"]
    ng_local, kd_local = Ng // world, Kd // world
    gate_up, down, y_g, y_d = [], [], [], []
    for layer in range(FFN70B_LAYERS):
        # A rank's shard of a seeded full matrix is itself a seeded matrix (RTN groups never straddle a
        # shard boundary), so the shards are generated directly.
        qw, qz, sc = quantize.random_awq_tensors(Kg, ng_local, GROUP, seed=1000 * layer + rank, device=dev)
        gate_up.append(ColumnParallelAWQLinear.from_local(qw, qz, sc, None, GROUP))
        qw, qz, sc = quantize.random_awq_tensors(kd_local, Nd, GROUP, seed=1000 * layer + 500 + rank, device=dev)
        down.append(RowParallelAWQLinear.from_local(qw, qz, sc, None, GROUP))
        del qw, qz, sc
        y_g.append(torch.empty((M, ng_local), dtype=torch.float16, device=dev))
        y_d.append(torch.empty((M, Nd), dtype=torch.float16, device=dev))
    x_g = torch.randn((M, Kg), device=dev).half()
    x_d = torch.randn((M, kd_local), device=dev).half()
    pw_g = [m.packed() for m in gate_up]
    pw_d = [m.packed() for m in down]
    step_bytes_total = FFN70B_LAYERS * (gemv_bytes(M, Kg, Ng) + gemv_bytes(M, Kd, Nd))

    # Row-parallel partial outputs are summed by the library's one-shot peer all-reduce (every rank reads
    # all partials over NVLink); the NCCL all-reduce is timed beside it.
    peers, peer, peer_error = {}, None, None
    if world > 1:
        from llmrqt_sdv1_b200.sharded import PeerSum
        try:
            peers = {"peer_push": PeerSum(64 * Nd, dev, mode="push"), "peer_pull": PeerSum(64 * Nd, dev, mode="pull")}
        except Exception as e:          # no symmetric memory on this box: every rank falls back to NCCL
            peer_error = f"{type(e).__name__}: {e}"[:200]
        flag = torch.tensor([0 if peers else 1], device=dev)
        dist.all_reduce(flag)           # all ranks must agree, or the exchanges would not match
        if int(flag.item()) != 0:
            peers = {}

    def statuses():
        st = {"gemv": kernels.gemv_status(dev), "gemm": kernels.gemm_status(dev)}
        for name, ps in peers.items():
            st[name] = ps.status()
        return st

    fused = False          # the down kernel's epilogue does the push exchange itself (one launch less per layer)

    def step():
        for i in range(FFN70B_LAYERS):
            kernels.linear(x_g, pw_g[i], out=y_g[i], overlap=True)
            if peer is not None and fused:
                peer.linear_push(x_d, pw_d[i], out=y_d[i], overlap=True)
            elif peer is not None:
                kernels.linear(x_d, pw_d[i], out=peer.partial(M, Nd), overlap=True)
                peer.reduce(M, Nd, out=y_d[i])
            else:
                kernels.linear(x_d, pw_d[i], out=y_d[i], overlap=True)
                if world > 1:
                    dist.all_reduce(y_d[i])

    def step_nccl():
        for i in range(FFN70B_LAYERS):
            kernels.linear(x_g, pw_g[i], out=y_g[i], overlap=True)
            kernels.linear(x_d, pw_d[i], out=y_d[i], overlap=True)
            if world > 1:
                dist.all_reduce(y_d[i])

    # Which exchange the timed step uses: all are timed briefly first (device time, max over ranks, and the
    # same number of replays on every rank) and the fastest is the configuration that is measured.
    allreduce, calib = "none", {}
    if world > 1:
        names = list(peers) + ["nccl"]
        if "peer_push" in peers and peers["peer_push"].can_fuse(M, pw_d[0]):
            names.insert(0, "peer_push_fused")
        for name in names:
            peer = peers.get("peer_push" if name == "peer_push_fused" else name)
            fused = name == "peer_push_fused"
            dist.barrier()
            tc = torch.tensor([time_graph(torch, step_nccl if name == "nccl" else step, iters=5)], device=dev)
            dist.all_reduce(tc, op=dist.ReduceOp.MAX)
            calib[name] = float(tc.item())
            require_clean(torch, f"calibration of {name}", **statuses())
        allreduce = min(calib, key=calib.get)
        fused = allreduce == "peer_push_fused"
        peer = peers.get("peer_push" if fused else allreduce)
        if peer is not None:
            for m in down:
                m.use_peer_sum(peer)
                m.fuse_exchange = fused
    step_timed = step_nccl if allreduce == "nccl" else step
    # the exchange that is timed against the library collective on the same partials (fp32 sum of fp16
    # partials vs NCCL's fp16 additions: equal to a few fp16 places)
    agrees = None
    if world > 1 and peer is not None:
        step()
        y_peer = y_d[-1].float().clone()
        step_nccl()
        scale = y_d[-1].float().abs().max().clamp_min(1e-6)
        bad = torch.tensor([float(((y_peer - y_d[-1].float()).abs().max() / scale) > 2e-3)], device=dev)
        dist.all_reduce(bad)
        agrees = bool(bad.item() == 0)
    for _ in range(max(args.warmup, 3)):
        step_timed()
    torch.cuda.synchronize()
    graphed = True
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step_timed()
        run = graph.replay
    except Exception:
        graphed, run = False, step_timed
    if world > 1:                       # every rank replays, or none does
        gflag = torch.tensor([0 if graphed else 1], device=dev)
        dist.all_reduce(gflag)
        if int(gflag.item()) != 0:
            graphed, run = False, step_timed
    for _ in range(max(args.warmup, 3)):
        run()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)      # set up before the barrier: its start-up time differs between ranks
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    # One more untimed step right before the timed ones: the step's own exchange lines the ranks up, so
    # that the timed region does not begin with one rank waiting for another to leave the barrier.
    run()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(args.steps):
        run()
    b.record()
    sampler.wait_and_sample(b)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    require_clean(torch, "timed region", **statuses())

    # parity of what was just timed (this rank's gate_up shard) against dequant + library matmul on the device
    m0 = gate_up[0].linear
    W = kernels.dequantize(m0.qweight, m0.qzeros, m0.scales, GROUP)
    ref = torch.matmul(x_g.float(), W.float())
    parity = {"dequant_bit_exact": bool(torch.equal(kernels.dequantize_packed(pw_g[0]), W)),
              "max_norm_err": float((y_g[0].float() - ref).abs().max() / ref.abs().max()), "tolerance": 2e-3,
              "checked": "layer 0 gate_up shard of rank 0 against device dequant (bit-exact) + fp32 matmul"}
    del W, ref

    # end to end: module API, activations from pinned host memory, result read back
    hxg, hxd = torch.randn((1, M, Kg)).half().pin_memory(), torch.randn((1, M, kd_local)).half().pin_memory()
    dxg, dxd = torch.empty_like(hxg, device=dev), torch.empty_like(hxd, device=dev)
    hy = torch.empty((1, M, Nd), dtype=torch.float16).pin_memory()

    def e2e_step():
        dxg.copy_(hxg, non_blocking=True)
        dxd.copy_(hxd, non_blocking=True)
        y = None
        for i in range(FFN70B_LAYERS):
            gate_up[i](dxg)
            y = down[i](dxd)
        hy.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    def time_e2e(fn):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        a2, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a2.record()
        for _ in range(args.steps):
            fn()
        b2.record()
        torch.cuda.synchronize()
        t2 = torch.tensor([a2.elapsed_time(b2) / args.steps], device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        return float(t2.item())

    e2e_eager_ms = time_e2e(e2e_step)
    e2e_ms, e2e_api = e2e_eager_ms, "ColumnParallelAWQLinear / RowParallelAWQLinear forward"
    # The same module calls captured once (GraphedStep) where the exchange is the library's own kernel: per step
    # the host inputs are copied in, the graph is replayed, the result is copied out.  Every rank must take the
    # same route, so a rank that cannot capture sends all of them back to the eager calls.
    graphed_step = None
    if world == 1 or allreduce.startswith("peer"):
        try:
            from llmrqt_sdv1_b200 import GraphedStep

            def module_chain(xg, xd):
                y = None
                for i in range(FFN70B_LAYERS):
                    gate_up[i](xg)
                    y = down[i](xd)
                return y
            graphed_step = GraphedStep(module_chain, (dxg, dxd))
        except Exception:
            graphed_step = None
        ok_flag = torch.tensor([0 if graphed_step is not None else 1], device=dev)
        if world > 1:
            dist.all_reduce(ok_flag)
        if int(ok_flag.item()) == 0:
            def e2e_graphed():
                y = graphed_step(hxg, hxd)
                hy.copy_(y, non_blocking=True)
                torch.cuda.synchronize()
            e2e_ms = time_e2e(e2e_graphed)
            e2e_api = "GraphedStep over ColumnParallelAWQLinear / RowParallelAWQLinear forward: host inputs copied in, one graph replay, result copied out"
        else:
            graphed_step = None
    require_clean(torch, "end to end", graphed=(graphed_step.status() if graphed_step is not None else 0), **statuses())

    # The same M = 1 step without the all-reduce (what the collective costs): device time, max over ranks.
    ms_local = None
    if world > 1:
        def step_local():
            for i in range(FFN70B_LAYERS):
                kernels.linear(x_g, pw_g[i], out=y_g[i], overlap=True)
                kernels.linear(x_d, pw_d[i], out=y_d[i], overlap=True)
        t3 = torch.tensor([time_graph(torch, step_local, iters=max(args.steps, 5))], device=dev)
        dist.all_reduce(t3, op=dist.ReduceOp.MAX)
        ms_local = float(t3.item())

    # The other row counts of the sharded configuration: M = 16 (decode batch) and M = 4096 (prefill),
    # same layers, same all-reduce, device time, max over ranks.
    tp_detail = []
    for Md in (16, 4096):
        xg = torch.randn((Md, Kg), device=dev).half()
        xd = torch.randn((Md, kd_local), device=dev).half()
        yg = torch.empty((Md, ng_local), dtype=torch.float16, device=dev)
        yd = torch.empty((Md, Nd), dtype=torch.float16, device=dev)

        ov = Md <= 64     # the decode batch prefetches its weights behind the previous launch, as the M = 1 step does

        def step_m():
            for i in range(FFN70B_LAYERS):
                kernels.linear(xg, pw_g[i], out=yg, overlap=ov)
                if peer is not None and peer.fits(Md, Nd):
                    kernels.linear(xd, pw_d[i], out=peer.partial(Md, Nd), overlap=ov)
                    peer.reduce(Md, Nd, out=yd)
                else:
                    kernels.linear(xd, pw_d[i], out=yd, overlap=ov)
                    if world > 1:
                        dist.all_reduce(yd)
        if world > 1:
            dist.barrier()
        if Md <= 64:
            # decode batch: replayed as a CUDA graph like the M = 1 step (eager launches would be host-bound)
            tm = torch.tensor([time_graph(torch, step_m, iters=5)], device=dev)
        else:
            for _ in range(3):
                step_m()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(2):
                step_m()
            e1.record()
            torch.cuda.synchronize()
            tm = torch.tensor([e0.elapsed_time(e1) / 2], device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms_m = float(tm.item())
        require_clean(torch, f"tp_detail M={Md}", **statuses())
        flops = 2.0 * Md * (Kg * Ng + Kd * Nd) * FFN70B_LAYERS
        row = {"M": Md, "ms_per_step": round(ms_m, 4)}
        if Md <= 64:
            gb = FFN70B_LAYERS * (gemv_bytes(Md, Kg, Ng) + gemv_bytes(Md, Kd, Nd)) / (ms_m * 1e-3) / 1e9
            row.update({"gbs_all_ranks": round(gb, 1), "frac_measured_per_gpu": round(gb / world / peaks["hbm_gbs"], 4)})
        else:
            tf = flops / (ms_m * 1e-3) / 1e12
            row.update({"tflops_all_ranks": round(tf, 1),
                        "frac_measured_per_gpu": round(tf / world / peaks["tflops"], 4),
                        "frac_nominal_per_gpu": round(tf / world / 2250.0, 4)})
        tp_detail.append(row)
        del xg, xd, yg, yd
    final_status = statuses()
    if rank != 0:
        return
    value = step_bytes_total / (ms * 1e-3) / 1e9
    per_gpu = value / world
    launches_per_layer = 2 if (fused or not allreduce.startswith("peer")) else 3
    exchange = ("push exchange over peer memory (NVLink) inside the down kernel's epilogue" if fused
                else "one-shot all-reduce over peer memory (NVLink)" if allreduce.startswith("peer")
                else ("NCCL all-reduce" if world > 1 else "no exchange (one GPU)"))
    line = {
        "metric": "W4A16 GEMV HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "ffn70b_tp: 70B-class FFN linears, gate_up 8192->57344 column-sharded, down "
                               "28672->8192 row-sharded + " + exchange + ", M=1, W4A16 g128, 8 layers per step",
                   "M": M, "tp": world, "group_size": GROUP, "bytes_per_step_all_ranks": step_bytes_total,
                   "launches_per_step": launches_per_layer * FFN70B_LAYERS,
                   "l2": "inputs larger than L2 (8 distinct layers per step, 2.9 GB over all ranks)",
                   "timing": "one CUDA graph per step, CUDA events on the launching stream, max over ranks",
                   "cuda_graph": graphed},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": per_gpu / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["decode_8192x57344_m1"],
                     "traffic_of": "one launch of the decode kernel on the unsharded gate_up (8192 x 57344, M = 1)",
                     "peak_source": peaks["source"], "frac_of_nominal_8tbs": per_gpu / 8000.0,
                     "kernel": ("awq::decode_i8_kernel" if world <= 2 else "awq::decode_i8_kernel / awq::gemv_kernel by shard size")
                               + (" (+ the all-reduce named in allreduce.used)" if world > 1 else ""),
                     "algorithmic_bytes_per_launch": gemv_bytes(M, Kg, Ng),
                     "per_gpu": True},
        "e2e": {"value": step_bytes_total / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": (hxg.numel() + hxd.numel()) * 2, "d2h_bytes_per_step": hy.numel() * 2,
                "api": e2e_api, "eager_ms_per_step": e2e_eager_ms},
        "gpu_launches": launches_per_layer * FFN70B_LAYERS * args.steps, "clocks": sampler.summary(),
        "parity": parity, "tp_detail": tp_detail, "status": final_status,
    }
    if world > 1:
        line["without_allreduce"] = {"ms_per_step": ms_local, "value": step_bytes_total / (ms_local * 1e-3) / 1e9,
                                     "unit": "GB/s"}
        line["allreduce"] = {"used": allreduce, "calibration_ms_per_step": calib, "peer_unavailable": peer_error,
                             "agrees_with_nccl": agrees}
    else:
        # One GPU: the Qwen3-1.7B decode step (the small shapes, where per-launch latency decides), the per-shape
        # tables and the whole-model leg ride on the same line.
        if not args.headline_only:
            line["qwen3_decode"] = qwen3_decode_measure(args, torch, peaks)
        if not args.no_detail and not args.headline_only:
            detail_tables(line, args, torch, peaks)
            try:
                line["config5"] = config5_block(torch)
            except Exception as exc:
                line["config5"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline("ffn70b_tp", 100)
    print(json.dumps(line), flush=True)


def config5_measure(torch, new_tokens=128):
    """Config 5: a random-init Qwen3-1.7B-architecture model whose decoder linears are AWQ W4A16 linears on
    the library's kernels (q/k/v fused into one linear of 4096 columns as the reference's fuser does,
    LLMQRT/runtime_refact/nn_models/models/qwen3.py:97-164; gate/up/down with fused epilogues), batch 1, a
    128-token prompt of uniform random ids, `new_tokens` greedy tokens.  Hugging Face's attention stands in
    for the reference's attention module (the reference tree is not present where this runs).  Decoding
    runs through `decoder.GraphedDecoder` (one CUDA graph per token) and, for comparison, through Hugging
    Face's `generate`; parity is against the same model with every linear in `dequant_matmul` mode."""
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from llmrqt_sdv1_b200 import kernels
    from llmrqt_sdv1_b200.hf_adapter import fuse_mlp_, fuse_qkv_, quantize_model_, set_impl_mode
    torch.cuda.set_device(0)
    # The cuDNN attention backend rebuilds its plan for every new KV length (milliseconds of host time per
    # decode step); the flash / math backends do not.
    torch.backends.cuda.enable_cudnn_sdp(False)
    cfg = Qwen3Config(hidden_size=2048, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                      head_dim=128, intermediate_size=6144, vocab_size=151936, max_position_embeddings=4096,
                      tie_word_embeddings=False)
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = Qwen3ForCausalLM(cfg).half().eval()
    n_lin = quantize_model_(model, GROUP)
    g = torch.Generator(device="cuda").manual_seed(0)
    prompt = torch.randint(0, 151936, (1, 128), device="cuda", generator=g)
    out = {"linears_quantized": n_lin, "prompt_tokens": 128, "new_tokens": new_tokens}

    def hf_run(tag):
        model.generate(prompt, max_new_tokens=8, do_sample=False)      # warm-up (also repacks once)
        torch.cuda.synchronize()
        t0 = time.perf_counter(); model(prompt, use_cache=True); torch.cuda.synchronize()
        prefill_ms = (time.perf_counter() - t0) * 1e3
        t0 = time.perf_counter()
        seq = model.generate(prompt, max_new_tokens=new_tokens, min_new_tokens=new_tokens, do_sample=False)
        torch.cuda.synchronize()
        total_ms = (time.perf_counter() - t0) * 1e3
        out[tag] = {"prefill_ms": prefill_ms, "generate_ms": total_ms,
                    "decode_tok_s": new_tokens / max((total_ms - prefill_ms) * 1e-3, 1e-9)}
        return seq

    with torch.no_grad():
        set_impl_mode(model, "dequant_matmul")
        seq_ref = hf_run("hf_generate_dequant_matmul")
        logits_ref = model(seq_ref).logits.float()
        set_impl_mode(model, "auto")
        seq_auto = hf_run("hf_generate_separate_linears")
        logits_auto = model(seq_ref).logits.float()
        out["parity_separate_linears"] = {
            "greedy_tokens_equal": sum(int(a == b) for a, b in zip(seq_auto[0, 128:].tolist(), seq_ref[0, 128:].tolist())),
            "of": new_tokens,
            "teacher_forced_logit_err": float((logits_auto - logits_ref).abs().max() / logits_ref.abs().max())}
        # the fused form: q/k/v as one linear, gate/up/down as two launches with fused epilogues
        out["fused"] = {"qkv": fuse_qkv_(model), "mlp": fuse_mlp_(model)}
        seq_fused = hf_run("hf_generate_fused")
        logits_fused = model(seq_ref).logits.float()
        out["teacher_forced_logit_err"] = float((logits_fused - logits_ref).abs().max() / logits_ref.abs().max())
        out["greedy_tokens_equal_to_dequant_matmul"] = sum(
            int(a == b) for a, b in zip(seq_fused[0, 128:].tolist(), seq_ref[0, 128:].tolist()))
        # one CUDA graph per token
        try:
            from llmrqt_sdv1_b200.decoder import GraphedDecoder
            dec = GraphedDecoder(model, max_len=128 + new_tokens + 8)
            dec.generate(prompt, 8)
            torch.cuda.synchronize()
            t0 = time.perf_counter(); dec.prefill(prompt); torch.cuda.synchronize()
            prefill_ms = (time.perf_counter() - t0) * 1e3
            t0 = time.perf_counter()
            seq_g = dec.generate(prompt, new_tokens)
            torch.cuda.synchronize()
            total_ms = (time.perf_counter() - t0) * 1e3
            decode_ms = max(total_ms - prefill_ms, 1e-6)
            lin_ms = dec.time_linears_only()
            out["graphed_decoder"] = {
                "prefill_ms": prefill_ms, "generate_ms": total_ms, "decode_tok_s": new_tokens / (decode_ms * 1e-3),
                "ms_per_token": decode_ms / new_tokens, "awq_linears_ms_per_token": lin_ms,
                "share_of_step_in_awq_linears": lin_ms / (decode_ms / new_tokens),
                "greedy_tokens_equal_to_hf_generate": sum(int(a == b) for a, b in zip(seq_g[0, 128:].tolist(),
                                                                                     seq_fused[0, 128:].tolist())),
                "teacher_forced_logit_err_vs_hf": dec.teacher_forced_error(seq_ref, logits_fused)}
            out["decode_tok_s"] = out["graphed_decoder"]["decode_tok_s"]
            out["prefill_ms"] = prefill_ms
            # the same step deep into a long context: attention over the cache split into chunks of positions
            # (one CTA per head and chunk) against one CTA per head
            del dec
            long_ctx = {"max_len": 4096, "positions": [200, 1000, 4000]}
            for name, split in (("ms_per_token", True), ("ms_per_token_one_cta_per_head", False)):
                dec_l = GraphedDecoder(model, max_len=4096, attn_split=split)
                long_ctx[name] = [round(dec_l.time_step_at(p), 4) for p in long_ctx["positions"]]
                del dec_l
            out["graphed_decoder"]["long_context"] = long_ctx
            out["share_of_step_in_awq_linears"] = out["graphed_decoder"]["share_of_step_in_awq_linears"]
        except Exception as exc:
            out["graphed_decoder"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
            out["decode_tok_s"] = out["hf_generate_fused"]["decode_tok_s"]
            out["prefill_ms"] = out["hf_generate_fused"]["prefill_ms"]
    out["status"] = {"gemm": kernels.gemm_status(), "gemv": kernels.gemv_status()}
    del model
    torch.cuda.empty_cache()
    return out


def config5_block(torch):
    blk = config5_measure(torch)
    require_clean(torch, "config5", **blk["status"])
    return blk


def run_qwen3_e2e(args, torch, peaks):
    """`--workload qwen3_e2e`: config 5 as the headline of its own line."""
    blk = config5_block(torch)
    line = {"metric": "decode tokens/s (config 5)", "value": blk["decode_tok_s"], "unit": "tok/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "qwen3_e2e: random-init Qwen3-1.7B architecture, 28 layers, AWQ W4A16 linears "
                                   "(fused qkv, fused MLP epilogues), HF attention, bs=1, 128 prompt + 128 greedy tokens"},
            "config5": blk}
    print(json.dumps(line), flush=True)


def run_profile_case(args, torch):
    """Small, self-terminating cases for `ncu` captures (a few launches, a few hundred MB)."""
    from llmrqt_sdv1_b200 import kernels, quantize
    torch.cuda.set_device(0)
    if args.profile_case.startswith("q8"):
        # q8_decode: fp8 57344 x 8192 weights (470 MB > L2), 16 rows, three launches (two CTAs per SM, no K split)
        # q8_decode_split: fp8 8192 x 28672 weights (235 MB), 16 rows, three launches (clusters of four along K)
        # q8_prefill: fp8 8192 x 8192 weights, 4096 rows, three launches
        from llmrqt_sdv1_b200 import q8
        M, N, K = {"q8_decode": (16, 57344, 8192), "q8_decode_split": (16, 8192, 28672)}.get(args.profile_case, (4096, 8192, 8192))
        w = torch.randn(N, K, device="cuda").mul_(0.5).to(torch.float8_e4m3fn)
        x = torch.randn(M, K, device="cuda").to(torch.float8_e4m3fn)
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            q8.gemm_tensorwise(x, w.t(), None, 0.5, 1.0, torch.bfloat16, out=y)
        torch.cuda.synchronize()
        assert q8.status() == 0
    elif args.profile_case.startswith(("gemv", "skinny", "decode")):
        # gemv / gemv16: 24 distinct 2048x12288 weights (13 MB each, 314 MB > L2), two passes
        # gemv70b / skinny70b[_m16] / decode70b[_m4, _m8]: one 8192x57344 weight (235 MB > L2), three launches
        M = 16 if args.profile_case in ("gemv16", "skinny70b_m16") else {"decode70b_m4": 4, "decode70b_m8": 8}.get(args.profile_case, 1)
        fn = (kernels.skinny if args.profile_case.startswith("skinny") else
              kernels.decode_i8 if args.profile_case.startswith("decode") else kernels.gemv)
        K, N, copies, passes = (8192, 57344, 1, 3) if "70b" in args.profile_case else (2048, 12288, 24, 2)
        qw, qz, sc = quantize.random_awq_tensors(K, N, GROUP, seed=1, device="cuda")
        base = kernels.make_packed(qw, qz, sc, GROUP)
        pws = [base] + [kernels.PackedWeight(base.packed.clone(), qz, sc, K, N, GROUP) for _ in range(copies - 1)]
        x = torch.randn((M, K), device="cuda").half()
        y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        for _ in range(passes):
            for pw in pws:
                fn(x, pw, out=y)
    else:
        M, K, N = {"gemm_large": (8192, 4096, 28672), "gemm_m64": (64, 4096, 28672)}.get(args.profile_case, (2048, 4096, 6144))
        qw, qz, sc = quantize.random_awq_tensors(K, N, GROUP, seed=1, device="cuda")
        pw = kernels.make_packed(qw, qz, sc, GROUP)
        x = torch.randn((M, K), device="cuda").half()
        y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        for _ in range(4):
            kernels.gemm(x, pw, out=y)
        torch.cuda.synchronize()
        assert kernels.gemm_status() == 0
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": args.profile_case, "ok": True}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, "qwen3_decode", "ffn70b_tp", "qwen3_e2e"])
    ap.add_argument("--no-detail", action="store_true", help="skip the per-shape decode / prefill tables")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--headline-only", action="store_true",
                    help="time the headline workload only (no qwen3_decode block, no tables): for launch-list captures")
    ap.add_argument("--profile-case", default=None, choices=["gemv", "gemv16", "gemv70b", "skinny70b", "skinny70b_m16", "decode70b", "decode70b_m4", "decode70b_m8",
                                                       "q8_decode", "q8_decode_split", "q8_prefill",
                             "gemm", "gemm_large", "gemm_m64"],
                    help="run a small fixed case of one kernel (for ncu) and exit")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload is None:
        args.workload = "ffn70b_tp"
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback for the product path")
    if args.profile_case:
        run_profile_case(args, torch)
        return
    peaks = load_peaks()
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "qwen3_e2e":
            if rank == 0:
                run_qwen3_e2e(args, torch, peaks)
        elif args.workload == "qwen3_decode":
            if rank == 0:
                run_qwen3_decode(args, torch, peaks)
        else:
            run_ffn70b_tp(args, torch, peaks, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
