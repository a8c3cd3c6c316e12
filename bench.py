#!/usr/bin/env python
"""Benchmark of the NanoQuant quantised-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch T] [--impl reference]

Workload (``config.workload``): the quantised linears of a Qwen3-8B-shaped decoder at 0.8 bpw —
36 layers x {q, k, v, o, gate, up, down}, ranks from the reference's rank formula, random ±1
factors and scales ``(U[0,1)+0.5)*0.01``, synthetic N(0,1) activations — executed for one decode
step of ``--batch`` tokens (default 1).  A *step* is one pass over all 252 linears, i.e. the
hot-path work of one generated token per sequence.  Per layer the launches are q/k/v (one group),
o, gate/up (one group), down: 4 launches of the group GEMV kernel, 144 per step, captured in a
CUDA graph.  The packed factors (690 MB) exceed L2, so every step streams them from HBM.

* ``value``      tokens/s of the device-resident step (CUDA events around K graph replays).
* ``e2e``        the same through host buffers: per step the activations are copied from pinned
                 host memory, the step runs, and the last projection's output is copied back.
* ``roofline``   algorithmic bytes of a step / step time against the measured HBM copy peak.
* ``cpu_baseline`` the reference's PyTorch dequantise-then-matmul path (torch CPU, bf16 as the
                 reference module keeps its parameters) timed on this host on a bounded sample
                 (one decoder layer), extrapolated to the 36 layers.

``--impl reference`` times only that CPU path and prints the same JSON line with
``"impl": "reference"``.  With N > 1 (launched by torchrun) every rank runs an independent replica
of the step (data-parallel decode streams, no data-path collective): weak scaling.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, LAYERS, KV = 4096, 12288, 36, 1024
BPW = 0.8
WORKLOAD = "qwen3-8b"
GEMM_MIN_TOKENS = 0   # --gemm-min-tokens: decode batches from this size on use the group GEMM (0: the library's dispatch limit)
# name -> (hidden, intermediate, layers, kv width, bits per weight); the first one is the headline workload
WORKLOADS = {"qwen3-8b": (4096, 12288, 36, 1024, 0.8), "llama-3.2-1b": (2048, 8192, 16, 512, 1.0)}
L2_BYTES = 126e6


def set_workload(name):
    global HIDDEN, INTER, LAYERS, KV, BPW, WORKLOAD
    HIDDEN, INTER, LAYERS, KV, BPW = WORKLOADS[name]
    WORKLOAD = name


def packed_bytes_per_step():
    return sum(R * (N + M) // 8 for (_, N, R, M, _, _) in layer_linears()) * LAYERS


def weight_copies():
    """Copies of the decoder's weights that a timed replay cycles through: 1 when one copy already
    exceeds L2 by a wide margin, otherwise enough of them that no replay finds its weights in L2."""
    b = packed_bytes_per_step()
    return 1 if b > 2.5 * L2_BYTES else int(2.5 * L2_BYTES // b) + 1


def rank_for_bits(in_f, out_f, bits):
    """Rank of a layer at a bit budget: floor((bits*in*out/(in+out) - 16) / 32) * 32, the
    reference's two-scale formula (src/nanoquant/utils/utils.py:132-159)."""
    r = int(in_f * out_f * bits / (in_f + out_f) - 16) // 32 * 32
    return max(32, min(r, in_f, out_f))


def layer_linears():
    """(name, N, R, M, input buffer, launch group) of the 7 quantised linears of a layer."""
    spec = [("q", HIDDEN, HIDDEN, "h", 0), ("k", HIDDEN, KV, "h", 0), ("v", HIDDEN, KV, "h", 0),
            ("o", HIDDEN, HIDDEN, "h", 1), ("gate", HIDDEN, INTER, "h", 2), ("up", HIDDEN, INTER, "h", 2),
            ("down", INTER, HIDDEN, "i", 3)]
    return [(n, N, rank_for_bits(N, M, BPW), M, src, grp) for (n, N, M, src, grp) in spec]


def algorithmic_bytes(N, R, M, T, e=2):
    """Packed factors + scales + activations in and out; the rank-R intermediate stays on chip / in L2."""
    return R * (N + M) // 8 + e * (N + R + M) + e * T * (N + M)


# --------------------------------------------------------------------------------------------
# clocks sampling
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for n, v in zip(names, p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# CPU reference arm
# --------------------------------------------------------------------------------------------
class CpuLayer:
    """One decoder layer (7 quantised linears) of the reference's PyTorch dequantise-then-matmul
    path on the host cores: dense +-1 matrices in bf16, as the reference module keeps them
    (src/nanoquant/modules/linear.py:69-76,90).  When the reference's own module has been staged
    (oracle/make_ref.py -> oracle/_ref), its `forward` (PyTorch branch, linear.py:143-150) is what runs
    (`kind` "reference"); otherwise the oracle's restatement of those four lines (`kind` "port")."""

    def __init__(self, T):
        import torch
        from oracle import nanoquant_oracle as oc
        self.torch, self.oc = torch, oc
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        g = torch.Generator().manual_seed(0)
        dt = torch.bfloat16
        ref = None
        try:
            from oracle import make_ref
            if make_ref.load() is not None:
                import importlib
                ref = importlib.import_module("nanoquant_ref.modules.linear")
        except Exception:
            ref = None
        self.kind = "reference" if ref is not None else "port"
        self.layers = []
        for (_, N, R, M, _, _) in layer_linears():
            V = (torch.randint(0, 2, (R, N), generator=g) * 2 - 1).to(dt)
            U = (torch.randint(0, 2, (M, R), generator=g) * 2 - 1).to(dt)
            sc = lambda n: ((torch.rand(n, generator=g) + 0.5) * 0.01).to(dt)
            x, a, b, c = torch.randn(T, N, generator=g).to(dt), sc(N), sc(R), sc(M)
            if ref is not None:
                lin = torch.nn.Linear(N, M, bias=False)
                lin.__class__ = ref.NanoQuantLinear           # the reference loader's class swap
                lin.init_for_inference(rank=R, has_scale_mid=True)
                with torch.no_grad():
                    lin.V.copy_(V); lin.U.copy_(U)
                    lin.scale_pre.copy_(a[None]); lin.scale_mid.copy_(b[None]); lin.scale_post.copy_(c[None])
                self.layers.append((x, lin))
            else:
                self.layers.append((x, V, U, a, b, c))

    def run_once(self):
        with self.torch.no_grad():
            t0 = time.perf_counter()
            if self.kind == "reference":
                for (x, lin) in self.layers:
                    lin(x)
            else:
                for (x, V, U, a, b, c) in self.layers:
                    self.oc.torch_cpu_forward(x, V, U, a, b, c)
            return time.perf_counter() - t0

    def timed(self, budget_s, min_reps=5, max_reps=2000):
        for _ in range(3):
            self.run_once()
        times, t_end = [], time.perf_counter() + budget_s
        while len(times) < min_reps or (time.perf_counter() < t_end and len(times) < max_reps):
            times.append(self.run_once())
        return statistics.median(times), len(times)


def cpu_sample_text(T, reps, kind="port"):
    what = ("the reference's NanoQuantLinear.forward, PyTorch branch" if kind == "reference"
            else "oracle restatement of the reference's PyTorch branch")
    return (f"1 of {LAYERS} decoder layers (7 linears, {what}, dense +-1 bf16 matmuls, T={T}), "
            f"median of {reps} runs, x{LAYERS} layers")


def reference_arm(args):
    """Each step is one pass over the bounded sample (one decoder layer); the step time reported is
    that pass scaled to the 36 layers of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    T = args.batch
    cpu = CpuLayer(T)
    for _ in range(max(args.warmup, 3)):
        cpu.run_once()
    times, t_stop = [], time.perf_counter() + 150.0
    for _ in range(args.steps):
        times.append(cpu.run_once())
        if time.perf_counter() > t_stop:
            break
    step_s = statistics.median(times) * LAYERS
    value = T / step_s
    out = {
        "impl": "reference", "metric": "decode tok/s (quantised linears of one decode step)", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(times), "warmup": max(args.warmup, 3),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": workload_config(T),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cpu.cores, "kind": cpu.kind,
                         "sample": cpu_sample_text(T, len(times), cpu.kind)},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out), flush=True)


def workload_config(T):
    mb, c = packed_bytes_per_step() / 1e6, weight_copies()
    l2 = (f"packed factors ({mb:.0f} MB per step) exceed L2; no flush needed" if c == 1 else
          f"packed factors are {mb:.0f} MB per step: consecutive steps cycle through {c} separate copies of the "
          f"weights ({c * mb:.0f} MB), so no step finds its weights in L2")
    return {"workload": f"{WORKLOAD}-shaped decoder, all {7 * LAYERS} quantised linears at {BPW} bpw, decode batch {T}",
            "hidden": HIDDEN, "intermediate": INTER, "layers": LAYERS, "batch": T,
            "ranks": {n: r for (n, _, r, _, _, _) in layer_linears()}, "l2": l2}


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def dram_traffic_ratio():
    """dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the captured decode launches, read
    from the line `traffic_ratio: <x>` of the tracked ncu summary of this kernel; None when there is none."""
    path = os.path.join(ROOT, "profiles", "gemv_group_kernel_qwen3_8b_decode.md")
    try:
        for line in open(path):
            if line.strip().startswith("traffic_ratio:"):
                return float(line.split(":", 1)[1].split()[0])
    except (OSError, ValueError):
        pass
    return None


class Step:
    """Device-resident weights of the decoder layers and the launch list of one decode step."""

    def __init__(self, T, dtype, device, layers=None):
        import torch
        layers = LAYERS if layers is None else layers
        from nanoquant_b200 import _lib
        self.torch, self.lib, self.L = torch, _lib, _lib.lib()
        self.T, self.dtype, self.device = T, dtype, device
        self.dt_id = _lib.NQ_BF16 if dtype == torch.bfloat16 else _lib.NQ_F16
        g = torch.Generator(device=device).manual_seed(0)
        rnd_bits = lambda rows, cols: torch.randint(-2**31, 2**31 - 1, ((rows + 15) // 16, (cols + 255) // 256, 128),
                                                    generator=g, device=device, dtype=torch.int32)
        scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
        self.x = {"h": torch.randn(T, HIDDEN, generator=g, device=device).to(dtype),
                  "i": torch.randn(T, INTER, generator=g, device=device).to(dtype)}
        self.keep, self.launches, self.bytes = [], [], 0
        scratch_bytes = 0
        # more tokens than one decode launch takes: the groups go through nq_gemm_group_fwd (split-K GEMM)
        self.per_linear = T >= (GEMM_MIN_TOKENS or self.L.nq_gemv_max_tokens() + 1)
        self.n_linears = 0
        for _ in range(layers):
            groups = {}
            for (name, N, R, M, src, grp) in layer_linears():
                t = dict(v=rnd_bits(R, N), u=rnd_bits(M, R), s_in=scale(N), s_mid=scale(R), s_out=scale(M),
                         y=torch.empty(T, M, device=device, dtype=dtype))
                self.keep.append(t)
                d = _lib.LinearDesc(self.x[src].data_ptr(), t["s_in"].data_ptr(), t["v"].data_ptr(),
                                    t["s_mid"].data_ptr(), t["u"].data_ptr(), t["s_out"].data_ptr(),
                                    t["y"].data_ptr(), N, R, M, N, M)
                groups.setdefault(grp, []).append(d)
                self.bytes += algorithmic_bytes(N, R, M, T)
                self.n_linears += 1
            for grp in sorted(groups):
                arr = (_lib.LinearDesc * len(groups[grp]))(*groups[grp])
                size_fn = self.L.nq_gemm_group_scratch_bytes if self.per_linear else self.L.nq_gemv_group_scratch_bytes
                scratch_bytes = max(scratch_bytes, size_fn(arr, len(arr), T))
                self.launches.append(arr)
        self.last_y = self.keep[-1]["y"]
        self.scratch = torch.zeros(scratch_bytes, dtype=torch.uint8, device=device)
        self.kernels_per_step = (2 if self.per_linear else 1) * len(self.launches)
        self.kernel_name = "gemm_stage_kernel (split-K)" if self.per_linear else "gemv_group_kernel"
        self.graph = None

    def run(self):
        st = self.torch.cuda.current_stream(self.device).cuda_stream
        if self.per_linear:
            for arr in self.launches:
                rc = self.L.nq_gemm_group_fwd(arr, len(arr), self.T, self.dt_id, self.scratch.data_ptr(),
                                              self.scratch.numel(), st)
                self.lib.check(rc, "nq_gemm_group_fwd")
            return
        for arr in self.launches:
            rc = self.L.nq_gemv_group_fwd(arr, len(arr), self.T, self.dt_id, self.scratch.data_ptr(),
                                          self.scratch.numel(), st)
            self.lib.check(rc, "nq_gemv_group_fwd")

    def capture(self):
        torch = self.torch
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.run()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=s):
                self.run()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)

    def capture_e2e(self, hx, hy):
        """The step with its host traffic as ONE graph: the activations copied in from the pinned host tensors `hx`,
        the launches, the last output copied out to the pinned host tensor `hy` (what a serving loop replays per token)."""
        torch = self.torch
        s = torch.cuda.Stream(self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.e2e_graph, stream=s):
                for k in hx:
                    self.x[k].copy_(hx[k], non_blocking=True)
                self.run()
                hy.copy_(self.last_y, non_blocking=True)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)

    def status(self):
        return self.L.nq_scratch_status(self.scratch.data_ptr(), self.torch.cuda.current_stream(self.device).cuda_stream)


class StepCycle:
    """The decode step on `weight_copies()` separate copies of the weights, replayed in turn, so that a
    decoder whose packed factors fit L2 still streams them from HBM in every timed step."""

    def __init__(self, T, dtype, device, layers=None):
        n = weight_copies() if layers in (None, LAYERS) else 1
        self.steps = [Step(T, dtype, device, layers) for _ in range(n)]
        self.i = 0
        s0 = self.steps[0]
        self.bytes, self.kernels_per_step = s0.bytes, s0.kernels_per_step
        self.per_linear, self.kernel_name = s0.per_linear, s0.kernel_name

    def capture(self):
        for st in self.steps:
            st.capture()

    def current(self):
        return self.steps[self.i % len(self.steps)]

    def replay(self):
        self.current().graph.replay()
        self.i += 1

    def status(self):
        return max(st.status() for st in self.steps)


def check_step(T, dtype, device):
    """The launch structure of the timed step on ONE decoder layer with real factors: seeded +-1 matrices packed on
    the GPU (nq_pack_rows, nq_rows_to_tiles), the same four group launches (q/k/v, o, gate/up, down), every output
    against the fp64 oracle.  Outside the timed region; returns (max |y - y64| / max |y64|, the same with half a unit
    in the last place of the output type taken off every element's error) over the 7 linears, and stops the
    benchmark when the second exceeds the tests' bar of 2e-3."""
    import numpy as np
    import torch
    from nanoquant_b200 import _lib
    from nanoquant_b200.kernel import utils as ku
    from oracle import nanoquant_oracle as oc
    L = _lib.lib()
    g = torch.Generator(device=device).manual_seed(1234)
    scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
    x = {"h": torch.randn(T, HIDDEN, generator=g, device=device).to(dtype),
         "i": torch.randn(T, INTER, generator=g, device=device).to(dtype)}
    signs = lambda r, c: (torch.randint(0, 2, (r, c), generator=g, device=device, dtype=torch.int8) * 2 - 1)
    tiles = lambda w: ku.pack_tiles(ku.pack_binary_gemv(w, method="half2"), tuple(w.shape), "half2")
    groups, keep = {}, []
    for (name, N, R, M, src, grp) in layer_linears():
        V, U = signs(R, N), signs(M, R)
        t = dict(V=V, U=U, v=tiles(V), u=tiles(U), s_in=scale(N), s_mid=scale(R), s_out=scale(M),
                 y=torch.empty(T, M, device=device, dtype=dtype), x=x[src], name=name)
        keep.append(t)
        groups.setdefault(grp, []).append(
            _lib.LinearDesc(x[src].data_ptr(), t["s_in"].data_ptr(), t["v"].data_ptr(), t["s_mid"].data_ptr(),
                            t["u"].data_ptr(), t["s_out"].data_ptr(), t["y"].data_ptr(), N, R, M, N, M))
    use_gemm = T >= (GEMM_MIN_TOKENS or L.nq_gemv_max_tokens() + 1)
    fwd = L.nq_gemm_group_fwd if use_gemm else L.nq_gemv_group_fwd
    size_fn = L.nq_gemm_group_scratch_bytes if use_gemm else L.nq_gemv_group_scratch_bytes
    st = torch.cuda.current_stream(device).cuda_stream
    for grp in sorted(groups):
        arr = (_lib.LinearDesc * len(groups[grp]))(*groups[grp])
        nb = size_fn(arr, len(arr), T)
        scratch = torch.zeros(nb, dtype=torch.uint8, device=device)
        _lib.check(fwd(arr, len(arr), T, _lib.NQ_BF16 if dtype == torch.bfloat16 else _lib.NQ_F16,
                       scratch.data_ptr(), nb, st), "check launch")
        if L.nq_scratch_status(scratch.data_ptr(), st) != 0:
            raise SystemExit("bench.py --check: a device-side wait timed out")
    worst, beyond = 0.0, 0.0
    f64 = lambda t_: t_.float().cpu().numpy().astype(np.float64)
    bits = 8 if dtype == torch.bfloat16 else 11     # significant bits of the output type
    for t in keep:
        y64 = oc.forward_fp64(f64(t["x"]), t["V"].cpu().numpy(), t["U"].cpu().numpy(), f64(t["s_in"]), f64(t["s_mid"]),
                              f64(t["s_out"]))
        y = f64(t["y"])
        worst = max(worst, oc.rel_err(y, y64))
        # the parity bar of the tests: |y - y64| <= 2e-3 * max|y64| + half a unit in the last place at that element
        mag = np.maximum(np.maximum(np.abs(y64), np.abs(y)), 2.0 ** -126)
        half_ulp = 2.0 ** (np.floor(np.log2(mag)) - bits)
        beyond = max(beyond, float(np.max(np.abs(y - y64) - half_ulp) / np.max(np.abs(y64))))
    if beyond > 2e-3:
        raise SystemExit(f"bench.py: output check failed: an element is {beyond:.3e} of the maximum off the oracle beyond "
                         f"its own rounding (bar 2e-3)")
    return worst, beyond


VOCAB = {"qwen3-8b": 151936, "llama-3.2-1b": 128256}


def measure_head(device, dtype, T, step_ms=None, vocab=None, steps=20, profile=False):
    """The un-quantised ``lm_head`` of the workload's model ([vocab, hidden] in the model dtype, larger than L2)
    as one ``nq_dense_gemv_fwd`` launch per decode step: time, algorithmic GB/s against the measured HBM peak,
    and, given the time of the decoder's linears, the decode rate with the head included."""
    import torch
    from nanoquant_b200 import ops
    V = vocab or VOCAB[WORKLOAD]
    g = torch.Generator(device=device).manual_seed(3)
    W = (torch.randn((V, HIDDEN), generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    x = torch.randn((T, HIDDEN), generator=g, device=device, dtype=torch.float32).to(dtype)
    for _ in range(3):
        ops.dense_gemv_forward(x, W)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    if profile:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(steps):
        ops.dense_gemv_forward(x, W)
    e1.record()
    torch.cuda.synchronize(device)
    if profile:
        torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / steps
    nbytes = 2 * (V * HIDDEN + T * (HIDDEN + V))
    out = {"value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms": ms, "kernel": "dense_gemv_kernel",
           "shape": [V, HIDDEN], "hbm_frac": nbytes / (ms * 1e-3) / 1e9 / hbm_peak()[0]}
    if step_ms is not None:
        out["decode_tokens_per_s_with_head"] = T / ((step_ms + ms) * 1e-3)
    return out


def side_numbers(device, dtype, step_ms):
    """Short measurements of the workload's other operating points (decode batches 4 and 16, one prefill GEMM
    size), reported beside the headline line; same kernels, same synthetic weights, CUDA events."""
    import torch
    out = {}
    for T in (4, 16):
        step = StepCycle(T, dtype, device)
        step.capture()
        for _ in range(3):
            step.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(device)
        e0.record()
        for _ in range(10):
            step.replay()
        e1.record()
        torch.cuda.synchronize(device)
        if step.status() != 0:
            raise SystemExit("bench.py: a device-side wait timed out")
        ms = e0.elapsed_time(e1) / 10
        out[f"decode_batch{T}"] = {"value": T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                                   "kernel": step.kernel_name, "hbm_frac": step.bytes / (ms * 1e-3) / 1e9 / hbm_peak()[0]}
        del step
        torch.cuda.empty_cache()
    for T in (1, 4):   # the reference's CUDA GEMV on the same GPU and linears, when its library was built
        try:
            r = measure_refkernel(T, LAYERS, 10, 3, device)
        except (RuntimeError, OSError) as e:   # e.g. a library built against another torch: a side number, not the line
            r = {"unavailable": str(e).splitlines()[0][:200]}
        if r is not None:
            out[f"reference_cuda_gemv_decode_batch{T}"] = r
        torch.cuda.empty_cache()
    out["lm_head_gemv"] = measure_head(device, dtype, 1, step_ms)
    for model in ("llama-2-7b", "qwen3-8b"):
        for tokens in (2048, 512, 128):
            tf, ms, _, _, _ = measure_prefill(tokens, 4, 5, 3, device, model=model)
            out[f"prefill_{tokens}_tokens_{model}"] = {"value": tf, "unit": "TFLOP/s", "ms_per_step": ms,
                                                       "frac_of_sustained_bf16_peak": tf / tensor_peak()[0]}
    return out


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def hbm_peak():
    p = _peaks()
    return (float(p.get("hbm_gbs", 6650.0)),
            "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in p else "fallback 6650 GB/s")


def tensor_peak():
    p = _peaks()
    return (float(p.get("bf16_tflops_sustained", 1400.0)),
            "measured (MEASURED_PEAKS.json bf16_tflops_sustained)" if "bf16_tflops_sustained" in p else "fallback 1400")


def gpu_arm(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    T = args.batch
    dtype = torch.bfloat16
    # the launches that are about to be timed, on real factors, against the oracle (bf16 outputs: 2e-3 + half an ulp)
    check_err = check_step(T, dtype, device) if (rank == 0 and not args.no_check) else None
    step = StepCycle(T, dtype, device, args.layers)
    step.capture()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(local)
    for _ in range(max(args.warmup, 3)):
        step.replay()
    barrier()
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.profiler.start()   # lets `ncu --profile-from-start off` see exactly the timed region
    e0.record()
    for _ in range(args.steps):
        step.replay()
    e1.record()
    barrier()
    torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1)
    # keep the clocks sample meaningful for short runs: load for at least ~1 s in total
    t_extra = time.perf_counter() + max(0.0, 1.0 - ms * 1e-3)
    while time.perf_counter() < t_extra:
        step.replay()
        torch.cuda.synchronize(device)
    clocks = sampler.stop() if rank == 0 else None
    if step.status() != 0:
        raise SystemExit("bench.py: a device-wide wait timed out inside the GEMV kernel")

    # end to end through host buffers
    hx = {k: v.cpu().pin_memory() for k, v in step.current().x.items()}
    hy = torch.empty_like(step.current().last_y, device="cpu").pin_memory()
    for st_ in step.steps:
        st_.capture_e2e(hx, hy)

    def e2e_step():   # host -> device copies, the step, device -> host copy: one graph launch and one wait per token
        step.current().e2e_graph.replay()
        step.i += 1
        torch.cuda.current_stream(device).synchronize()
    for _ in range(3):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1)

    times = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    # N > 1: the replicas above are the weak-scaling value; the sharded configuration (tensor parallelism over the
    # GPUs of this run) is measured beside it, every rank taking part
    tp = tp_record(args, device, world, rank) if (world > 1 and not args.no_side_numbers) else None
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_src = hbm_peak()
    ratio = dram_traffic_ratio()
    step_s = ms * 1e-3 / args.steps
    achieved = step.bytes / step_s / 1e9
    if args.layers != LAYERS:   # profiling aid: fewer layers resident; report per-step numbers of what ran
        out_note = f"{args.layers} of {LAYERS} layers timed (profiling run, not a benchmark value)"
    else:
        out_note = None
    launch_us = step_s / step.kernels_per_step * 1e6
    out = {
        "metric": "decode tok/s (quantised linears of one decode step)", "value": world * T / step_s,
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("bf16 tcgen05 mma / f32 accumulate; bf16 in/out" if step.per_linear
                  else "s8 mma / s32 accumulate on 16-bit fixed point; bf16 in/out"), "data": "synthetic",
        "config": workload_config(T),
        "parallelism": "single gpu" if world == 1 else f"{world} independent replicas",
        "layers_timed": args.layers,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (step.bytes / step.kernels_per_step * ratio if (ratio and not step.per_linear) else None),
                     "traffic_source": ("dram__bytes_read+write over algorithmic bytes of three launches captured with ncu, "
                                        "scaled to the average launch" if (ratio and not step.per_linear) else None),
                     "kernel": step.kernel_name,
                     "bytes_per_launch": step.bytes / step.kernels_per_step, "us_per_launch": launch_us,
                     "peak_source": peak_src},
        "e2e": {"value": world * T / (e2e_ms * 1e-3 / args.steps), "unit": "tokens/s",
                "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in hx.values()),
                "d2h_bytes_per_step": hy.numel() * hy.element_size()},
        "gpu_launches": step.kernels_per_step * args.steps,
        "checked": check_err is not None, "max_rel_err": check_err[0] if check_err else None,
        "max_err_beyond_output_rounding": check_err[1] if check_err else None,
        "parity_bar": "2e-3 * max|y64| + half ulp of the output type at the element",
        "clocks": clocks,
    }
    if out_note:
        out["note"] = out_note
    if world == 1 and T == 1 and args.layers == LAYERS and WORKLOAD == "qwen3-8b" and not args.no_side_numbers:
        del step
        torch.cuda.empty_cache()
        out["other_operating_points"] = side_numbers(device, dtype, step_s * 1e3)
    if tp is not None:
        out["tp"] = tp
    if not args.no_cpu_baseline and world == 1:   # the CPU baseline is reported on rank 0 of a single-GPU run only
        cpu = CpuLayer(T)
        t_layer, reps = cpu.timed(budget_s=12.0)
        out["cpu_baseline"] = {"value": T / (t_layer * LAYERS), "unit": "tokens/s", "cores": cpu.cores,
                               "kind": cpu.kind, "sample": cpu_sample_text(T, reps, cpu.kind)}
    print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()



# --------------------------------------------------------------------------------------------
# tensor-parallel arm (--mode tp): Llama-3-70B-shaped linears, U split by output rows, NCCL all-gather
# --------------------------------------------------------------------------------------------
TP_HIDDEN, TP_INTER, TP_LAYERS, TP_KV = 8192, 28672, 80, 1024


def tp_layer_linears():
    spec = [("q", TP_HIDDEN, TP_HIDDEN, "h", 0), ("k", TP_HIDDEN, TP_KV, "h", 0), ("v", TP_HIDDEN, TP_KV, "h", 0),
            ("o", TP_HIDDEN, TP_HIDDEN, "h", 1), ("gate", TP_HIDDEN, TP_INTER, "h", 2), ("up", TP_HIDDEN, TP_INTER, "h", 2),
            ("down", TP_INTER, TP_HIDDEN, "i", 3)]
    return [(n, N, rank_for_bits(N, M, BPW), M, src, grp) for (n, N, M, src, grp) in spec]


def measure_tp(T, layers, steps, warmup, collective, device, world, rank, shard=True):
    """One decode (or prefill) step of `layers` Llama-3-70B-shaped layers with every U sharded by output rows over the
    ranks: per launch group the local kernel(s), then one all-gather of the group's [T, sum(M/G)] shards.  With
    shard=False the same step runs unsharded on this GPU alone (the one-GPU figure the sharded ones are compared
    with).  Needs an initialised process group when world > 1.  Returns a dict (times are the max over ranks)."""
    import torch
    import torch.distributed as dist
    from nanoquant_b200 import _lib
    L = _lib.lib()
    G = world if shard else 1
    dtype = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(0)   # same seed on every rank: replicated tensors agree
    rnd_bits = lambda rows, cols: torch.randint(-2**31, 2**31 - 1, ((rows + 15) // 16, (cols + 255) // 256, 128),
                                                generator=g, device=device, dtype=torch.int32)
    scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
    x = {"h": torch.randn(T, TP_HIDDEN, generator=g, device=device).to(dtype),
         "i": torch.randn(T, TP_INTER, generator=g, device=device).to(dtype)}
    keep, steps_, nbytes, scratch_bytes = [], [], 0, 0
    # collective: "peer" = nq_allgather_push on symmetric memory (one kernel per gather, graph-capturable),
    # "nccl" = all_gather_into_tensor, issued eagerly
    peer = None
    if G > 1 and collective == "peer":
        from nanoquant_b200 import tp as nq_tp
        esz = 2
        gathered = sum(G * T * sum(M // G for (_, _, _, M, _, g_) in tp_layer_linears() if g_ == grp) * esz + 256
                       for grp in range(4)) * layers
        try:
            peer = nq_tp.PeerGather(gathered + 4096)
            ok = torch.ones(1, device=device)
        except Exception as e:   # no symmetric memory on this system: every rank falls back to NCCL together
            print(f"bench.py: peer-memory all-gather unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr)
            peer, ok = None, torch.zeros(1, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            peer = None
    use_gemm = T > L.nq_gemv_max_tokens()   # more tokens than a decode launch takes: the group GEMM (two launches)
    group_fwd = L.nq_gemm_group_fwd if use_gemm else L.nq_gemv_group_fwd
    group_bytes = L.nq_gemm_group_scratch_bytes if use_gemm else L.nq_gemv_group_scratch_bytes
    for _ in range(layers):
        groups = {}
        for spec in tp_layer_linears():
            groups.setdefault(spec[5], []).append(spec)
        for grp in sorted(groups):
            # The shards of a launch group (q/k/v, gate/up) are written side by side into one [T, sum(M/G)]
            # buffer, so one all-gather per group brings every rank's block: the gathered layout is
            # [rank][T][q_r | k_r | v_r].
            width = sum(M // G for (_, _, _, M, _, _) in groups[grp])
            ybuf = torch.empty(T, width, device=device, dtype=dtype)
            full = (peer.region((T, width), dtype) if peer is not None
                    else torch.empty(G * T, width, device=device, dtype=dtype))
            descs, col = [], 0
            for (name, N, R, M, src, _) in groups[grp]:
                m = M // G
                t = dict(v=rnd_bits(R, N), u=rnd_bits(m, R), s_in=scale(N), s_mid=scale(R), s_out=scale(m))
                keep.append(t)
                yptr = ybuf.data_ptr() + col * ybuf.element_size()
                descs.append(_lib.LinearDesc(x[src].data_ptr(), t["s_in"].data_ptr(), t["v"].data_ptr(),
                                             t["s_mid"].data_ptr(), t["u"].data_ptr(), t["s_out"].data_ptr(),
                                             yptr, N, R, m, N, width))
                col += m
                nbytes += R * N // 8 + R * m // 8 + 2 * (N + R + m) + 2 * T * (N + m)
            arr = (_lib.LinearDesc * len(descs))(*descs)
            scratch_bytes = max(scratch_bytes, group_bytes(arr, len(arr), T))
            steps_.append((arr, ybuf, full))
    scratch = torch.zeros(scratch_bytes, dtype=torch.uint8, device=device)
    launches_per_step = (2 if use_gemm else 1) * len(steps_)

    def run():
        st = torch.cuda.current_stream(device).cuda_stream
        for arr, ybuf, full in steps_:
            _lib.check(group_fwd(arr, len(arr), T, _lib.NQ_BF16, scratch.data_ptr(), scratch.numel(), st), "group_fwd")
            if peer is not None:
                peer.gather(ybuf, full)
            elif G > 1:
                dist.all_gather_into_tensor(full, ybuf)

    # One GPU, or the peer-memory collective: the step is replayed as a CUDA graph.  With NCCL the launches
    # and the collectives are issued eagerly in stream order: a captured NCCL collective runs on a stream of
    # its own beside the next cooperative launch, which cannot become resident while the collective's CTAs hold
    # SMs and wait for a peer that is itself waiting for its cooperative launch: that combination can deadlock
    # and is not used.
    graph = None
    for _ in range(2):
        run()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    if G == 1 or peer is not None:
        s = torch.cuda.Stream(device)
        s.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(s):
            run()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                run()
        torch.cuda.current_stream(device).wait_stream(s)
        torch.cuda.synchronize(device)
    replay = graph.replay if graph is not None else run

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)
    for _ in range(max(warmup, 3)):
        replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        replay()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if L.nq_scratch_status(scratch.data_ptr(), torch.cuda.current_stream(device).cuda_stream) != 0:
        raise SystemExit("bench.py: a device-wide wait timed out inside the GEMV kernel")
    if peer is not None and peer.status() != 0:
        raise SystemExit("bench.py: a wait for a peer's shard timed out inside the all-gather kernel")
    step_s = ms.item() * 1e-3 / steps * (TP_LAYERS / layers)
    per_gpu = nbytes * (TP_LAYERS / layers) / step_s / 1e9
    res = {"tokens_per_s": T / step_s, "ms_per_step": step_s * 1e3, "per_gpu_gbs": per_gpu,
           "hbm_frac_per_gpu": per_gpu / hbm_peak()[0], "gpus": G, "batch": T, "layers_timed": layers,
           "collective": ("none" if G == 1 else "peer-memory kernel, CUDA graph" if peer is not None else "NCCL, eager"),
           "kernel": "gemm_stage_kernel" if use_gemm else "gemv_group_kernel", "launches_per_step": launches_per_step}
    del keep, steps_, scratch, graph, peer
    torch.cuda.empty_cache()
    return res


def tp_record(args, device, world, rank):
    """The sharded 70B-shaped step at this number of GPUs beside the same step on one GPU: decode batch 1 and 16
    and a 512-token prefill, 8 of 80 layers timed and scaled.  Per-GPU roofline bytes: R*N/8 + R*M/(8G) + scales +
    activations (the rank-R stage is replicated by design)."""
    out = {"workload": f"llama-3-70b-shaped decoder linears at {BPW} bpw, U split by output rows over {world} GPUs, "
                       "one all-gather per launch group", "scaling": "strong"}
    for T in (1, 16, 512):
        steps = 10 if T <= 16 else 3
        sharded = measure_tp(T, 8, steps, 3, args.tp_collective, device, world, rank, shard=True)
        single = measure_tp(T, 8, steps, 3, args.tp_collective, device, world, rank, shard=False)
        sharded["speedup_over_one_gpu"] = sharded["tokens_per_s"] / single["tokens_per_s"]
        out[f"batch{T}" if T <= 16 else f"prefill{T}"] = {"sharded": sharded, "one_gpu": single}
    return out


def tp_arm(args):
    """`--mode tp`: the sharded step alone (strong scaling), one JSON line."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    T = args.batch
    r = measure_tp(T, args.tp_layers, args.steps, args.warmup, args.tp_collective, device, world, rank)
    if rank == 0:
        print(json.dumps({
            "mode": "tp", "metric": "decode tok/s (quantised linears of one decode step)", "value": r["tokens_per_s"],
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": ("bf16 tcgen05 mma / f32 accumulate; bf16 in/out" if r["kernel"].startswith("gemm")
                      else "s8 mma / s32 accumulate; bf16 in/out"),
            "data": "synthetic",
            "config": {"workload": f"llama-3-70b-shaped decoder linears at {BPW} bpw, decode batch {T}, U split by output "
                                   f"rows over {world} GPUs + one all-gather per launch group ({r['collective']})",
                       "layers_timed": args.tp_layers, "layers": TP_LAYERS, "parallelism": f"tp{world}"},
            "roofline": {"bound": "hbm", "achieved": r["per_gpu_gbs"], "peak": hbm_peak()[0], "unit": "GB/s per GPU",
                         "frac": r["hbm_frac_per_gpu"], "traffic": None},
            "gpu_launches": r["launches_per_step"] * args.steps}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# prefill arm (--mode prefill): Llama-2-7B-shaped layer GEMMs at 1.0 bpw, T tokens per GEMM
# --------------------------------------------------------------------------------------------
PREFILL_SHAPES = {   # name -> (hidden, intermediate, kv width, bits per weight)
    "llama-2-7b": (4096, 11008, 4096, 1.0),
    "qwen3-8b": (4096, 12288, 1024, 0.8),
}


def measure_prefill(T, layers, steps, warmup, device, profile=False, min_seconds=0.0, e2e=False, model="llama-2-7b",
                    grouped=True):
    """TFLOP/s of the GEMM path on the 7 linears of `layers` decoder layers of `model`'s shape (ranks from the rank
    formula at its bit budget), T tokens per GEMM.  `grouped`: q/k/v and gate/up go through nq_gemm_group_fwd as one
    launch group each (what `LinearGroup` issues for a decoder layer, as in the decode step); otherwise one
    nq_gemm_fwd per linear.  Returns (TFLOP/s, ms per step, launches per step, clock record or None, end-to-end
    record or None)."""
    import torch
    from nanoquant_b200 import _lib
    L = _lib.lib()
    dtype = torch.bfloat16
    H, I, KVW, bpw = PREFILL_SHAPES[model]
    shapes = [(H, H), (H, KVW), (H, KVW), (H, H), (H, I), (H, I), (I, H)]
    g = torch.Generator(device=device).manual_seed(0)
    rnd_bits = lambda rows, cols: torch.randint(-2**31, 2**31 - 1, ((rows + 15) // 16, (cols + 255) // 256, 128),
                                                generator=g, device=device, dtype=torch.int32)
    scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
    xs = {H: torch.randn(T, H, generator=g, device=device).to(dtype), I: torch.randn(T, I, generator=g, device=device).to(dtype)}
    calls, flops, scratch_bytes = [], 0.0, 0
    group_of = [0, 0, 0, 1, 2, 2, 3] if grouped else list(range(7))
    for _ in range(layers):
        members = {}
        for (N, M), gi in zip(shapes, group_of):
            R = rank_for_bits(N, M, bpw)
            t = dict(v=rnd_bits(R, N), u=rnd_bits(M, R), a=scale(N), b=scale(R), c=scale(M),
                     y=torch.empty(T, M, device=device, dtype=dtype))
            members.setdefault(gi, []).append((t, N, R, M))
            flops += 2.0 * T * R * (N + M)
        for gi in sorted(members):
            descs = [_lib.LinearDesc(xs[N].data_ptr(), t["a"].data_ptr(), t["v"].data_ptr(), t["b"].data_ptr(), t["u"].data_ptr(),
                                     t["c"].data_ptr(), t["y"].data_ptr(), N, R, M, N, M) for (t, N, R, M) in members[gi]]
            arr = (_lib.LinearDesc * len(descs))(*descs)
            calls.append((arr, len(descs), members[gi]))
            scratch_bytes = max(scratch_bytes, L.nq_gemm_group_scratch_bytes(arr, len(descs), T))
    scratch = torch.zeros(scratch_bytes, dtype=torch.uint8, device=device)
    st = torch.cuda.current_stream(device).cuda_stream

    def run():
        for (arr, n, _) in calls:
            _lib.check(L.nq_gemm_group_fwd(arr, n, T, _lib.NQ_BF16, scratch.data_ptr(), scratch.numel(), st),
                       "nq_gemm_group_fwd")
    for _ in range(max(warmup, 3)):
        run()
    torch.cuda.synchronize(device)
    sampler = None
    if min_seconds > 0:
        sampler = ClockSampler(device.index)
        sampler.start()
        time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if profile:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    torch.cuda.synchronize(device)
    if profile:
        torch.cuda.profiler.stop()
    ms = e0.elapsed_time(e1) / steps
    t_end = time.perf_counter() + max(0.0, min_seconds - ms * steps * 1e-3)
    while time.perf_counter() < t_end:   # keeps the clock record meaningful for short runs
        run()
        torch.cuda.synchronize(device)
    clocks = sampler.stop() if sampler else None
    e2e_info = None
    if e2e:   # the same step with the activations copied from pinned host memory and the last output read back
        hx = {k: v.cpu().pin_memory() for k, v in xs.items()}
        last_y = calls[-1][2][-1][0]["y"]
        hy = torch.empty_like(last_y, device="cpu").pin_memory()

        def e2e_step():
            for k in hx:
                xs[k].copy_(hx[k], non_blocking=True)
            run()
            hy.copy_(last_y, non_blocking=True)
            torch.cuda.current_stream(device).synchronize()
        for _ in range(2):
            e2e_step()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(steps):
            e2e_step()
        f1.record()
        torch.cuda.synchronize(device)
        e2e_ms = f0.elapsed_time(f1) / steps
        e2e_info = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": sum(v.numel() * v.element_size() for v in hx.values()),
                    "d2h_bytes_per_step": hy.numel() * hy.element_size()}
    if L.nq_scratch_status(scratch.data_ptr(), st) != 0:
        raise SystemExit("bench.py: a device-side wait timed out inside the GEMM kernel")
    return flops / (ms * 1e-3) / 1e12, ms, 2 * len(calls), clocks, e2e_info


def prefill_arm(args):
    """`--mode prefill`: the tcgen05 GEMM path at `--tokens` tokens per GEMM."""
    import torch
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    T = args.tokens
    layers = args.layers if args.layers != LAYERS else 4
    model = args.prefill_model
    tf, ms, launches, clocks, e2e = measure_prefill(T, layers, args.steps, args.warmup, device, profile=True,
                                                    min_seconds=1.0, e2e=True, model=model, grouped=not args.no_groups)
    peak, peak_src = tensor_peak()
    print(json.dumps({
        "mode": "prefill", "metric": "prefill TFLOP/s (quantised linears, 2*T*R*(N+M) flops)", "value": tf,
        "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"{model}-shaped layer GEMMs at {PREFILL_SHAPES[model][3]} bpw, {T} tokens per GEMM, "
                               f"{layers} layers; " + ("one launch per linear and stage" if args.no_groups else
                                                       "q/k/v and gate/up as launch groups (8 launches per layer)"),
                   "tokens": T},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                     "traffic": None, "kernel": "gemm_stage_kernel", "peak_source": peak_src},
        "e2e": e2e,
        "tokens_per_s": T / (ms * 1e-3),   # T tokens through the GEMMs of `layers` layers per step
        "gpu_launches": launches * args.steps, "clocks": clocks}), flush=True)


# --------------------------------------------------------------------------------------------
# single launch group (--mode linear): one linear or one launch group, rotated over copies larger than L2
# --------------------------------------------------------------------------------------------
GROUP_SHAPES = {   # name -> [(N, R, M)] of one launch
    "config1": [(4096, 1536, 4096)],                       # 4096 -> 4096, r = 1536 (0.75 bpw)
    "qwen3-qkv": [(4096, 1600, 4096), (4096, 608, 1024), (4096, 608, 1024)],
    "qwen3-o": [(4096, 1600, 4096)],
    "qwen3-gate-up": [(4096, 2432, 12288)] * 2,
    "qwen3-down": [(12288, 2432, 4096)],
    "llama70b-qkv": [(8192, 3232, 8192), (8192, 704, 1024), (8192, 704, 1024)],
    "llama70b-o": [(8192, 3232, 8192)],
    "llama70b-gate-up": [(8192, 5056, 28672)] * 2,
    "llama70b-down": [(28672, 5056, 8192)],
}


def measure_group(shapes, T, dtype, device, steps, resident, profile=False, max_copies=0):
    """Time of one launch group (us), over `copies` separate weight sets replayed from one CUDA graph (rotated: more
    than 2 x L2 of packed factors, so every launch streams from HBM) or over one set (L2-resident when it fits)."""
    import torch
    from nanoquant_b200 import _lib
    L = _lib.lib()
    dt_id = _lib.NQ_BF16 if dtype == torch.bfloat16 else _lib.NQ_F16
    g = torch.Generator(device=device).manual_seed(0)
    rnd_bits = lambda rows, cols: torch.randint(-2**31, 2**31 - 1, ((rows + 15) // 16, (cols + 255) // 256, 128),
                                                generator=g, device=device, dtype=torch.int32)
    scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
    packed = sum(R * (N + M) // 8 for (N, R, M) in shapes)
    copies = 1 if resident else max(2, int(2 * L2_BYTES // packed) + 1)
    if max_copies:
        copies = min(copies, max_copies)
    use_gemm = T > L.nq_gemv_max_tokens()
    fwd = L.nq_gemm_group_fwd if use_gemm else L.nq_gemv_group_fwd
    size_fn = L.nq_gemm_group_scratch_bytes if use_gemm else L.nq_gemv_group_scratch_bytes
    xs = {N: torch.randn(T, N, generator=g, device=device).to(dtype) for N in {n for (n, _, _) in shapes}}
    keep, arrs = [], []
    for _ in range(copies):
        ds = []
        for (N, R, M) in shapes:
            t = dict(v=rnd_bits(R, N), u=rnd_bits(M, R), a=scale(N), b=scale(R), c=scale(M),
                     y=torch.empty(T, M, device=device, dtype=dtype))
            keep.append(t)
            ds.append(_lib.LinearDesc(xs[N].data_ptr(), t["a"].data_ptr(), t["v"].data_ptr(), t["b"].data_ptr(),
                                      t["u"].data_ptr(), t["c"].data_ptr(), t["y"].data_ptr(), N, R, M, N, M))
        arrs.append((_lib.LinearDesc * len(ds))(*ds))
    nbytes = size_fn(arrs[0], len(shapes), T)
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    reps = 1 if copies > 1 else 8

    def run():
        st = torch.cuda.current_stream(device).cuda_stream
        for _ in range(reps):
            for a in arrs:
                _lib.check(fwd(a, len(shapes), T, dt_id, scratch.data_ptr(), nbytes, st), "group launch")
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        run()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=s):
            run()
    torch.cuda.current_stream(device).wait_stream(s)
    torch.cuda.synchronize(device)
    for _ in range(3):
        graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    if profile:
        torch.cuda.profiler.start()
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    if profile:
        torch.cuda.profiler.stop()
    if L.nq_scratch_status(scratch.data_ptr(), torch.cuda.current_stream(device).cuda_stream) != 0:
        raise SystemExit("bench.py: a device-side wait timed out")
    us = e0.elapsed_time(e1) * 1e3 / (steps * copies * reps)
    return us, copies, (2 if use_gemm else (T + 3) // 4)


def linear_arm(args):
    """`--mode linear --shape NAME --batch T`: one launch group alone, HBM-streamed (rotated copies) and L2-resident."""
    import torch
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    dtype = torch.float16 if args.dtype == "f16" else torch.bfloat16
    shapes, T = GROUP_SHAPES[args.shape], args.batch
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    us, copies, launches = measure_group(shapes, T, dtype, device, args.steps, resident=False, profile=True,
                                         max_copies=args.copies)
    clocks = sampler.stop()
    us_l2, _, _ = measure_group(shapes, T, dtype, device, args.steps, resident=True)
    nbytes = sum(algorithmic_bytes(N, R, M, T) for (N, R, M) in shapes)
    flops = sum(2.0 * T * R * (N + M) for (N, R, M) in shapes)
    gemm = T > 4
    peak, peak_src = (tensor_peak() if gemm else hbm_peak())
    achieved = flops / us / 1e6 if gemm else nbytes / us / 1e3
    print(json.dumps({
        "mode": "linear", "metric": ("launch group TFLOP/s (2*T*R*(N+M))" if gemm else
                                     "launch group GB/s (algorithmic bytes: packed factors + scales + activations)"),
        "value": achieved, "unit": "TFLOP/s" if gemm else "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": 3,
        "us_per_group": us, "us_per_group_l2_resident": us_l2, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"{args.shape} {shapes}, {T} token(s); {copies} weight sets replayed in turn "
                               f"({copies * sum(R * (N + M) // 8 for (N, R, M) in shapes) / 1e6:.0f} MB of packed factors)",
                   "launches_per_group": launches},
        "roofline": {"bound": "tensor" if gemm else "hbm", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s" if gemm else "GB/s", "frac": achieved / peak, "traffic": None,
                     "bytes_per_group": nbytes, "peak_source": peak_src,
                     "l2_resident_achieved": (flops / us_l2 / 1e6 if gemm else nbytes / us_l2 / 1e3)},
        "gpu_launches": launches * copies * args.steps, "clocks": clocks}), flush=True)


def pack_arm(args):
    """`--mode pack`: the pack / layout kernels on a 12288 x 4096 matrix, GB/s of algorithmic bytes against the measured
    HBM peak.  Inputs are rotated over enough separate matrices to exceed 2 x L2."""
    import torch
    from nanoquant_b200 import _lib
    L = _lib.lib()
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    rows, cols = 12288, 4096
    st = torch.cuda.current_stream(device).cuda_stream
    g = torch.Generator(device=device).manual_seed(0)
    n_dense = max(2, int(2 * L2_BYTES // (rows * cols)) + 1)            # 1 byte per weight
    n_packed = max(2, int(2 * L2_BYTES // (rows * cols // 8 * 2)) + 1)  # 1/8 byte per weight, read + written
    dense = [(torch.randint(0, 2, (rows, cols), generator=g, device=device, dtype=torch.int8) * 2 - 1) for _ in range(n_dense)]
    words = [torch.randint(-2**31, 2**31 - 1, (rows, cols // 32), generator=g, device=device, dtype=torch.int32)
             for _ in range(n_packed)]
    out_words = torch.empty(rows, cols // 32, dtype=torch.int32, device=device)
    out_dense = torch.empty(rows, cols, dtype=torch.int8, device=device)
    out_marlin = torch.empty(cols // 16, rows // 2, dtype=torch.int32, device=device)
    out_tiles = torch.empty(L.nq_tiles_bytes(rows, cols), dtype=torch.uint8, device=device)
    W = rows * cols
    cases = [
        ("nq_pack_rows", W + W / 8, n_dense, lambda i: L.nq_pack_rows(dense[i].data_ptr(), out_words.data_ptr(), rows, cols, _lib.NQ_HALF2, st)),
        ("nq_unpack_rows", W / 8 + W, n_packed, lambda i: L.nq_unpack_rows(words[i].data_ptr(), out_dense.data_ptr(), rows, cols, _lib.NQ_LSB_FIRST, st)),
        ("nq_pack_marlin", W + W / 8, n_dense, lambda i: L.nq_pack_marlin(dense[i].data_ptr(), out_marlin.data_ptr(), rows, cols, st)),
        ("nq_rows_to_tiles", W / 8 + W / 8, n_packed, lambda i: L.nq_rows_to_tiles(words[i].data_ptr(), out_tiles.data_ptr(), rows, cols, _lib.NQ_LSB_FIRST, st)),
        ("nq_reorder_words", W / 8 + W / 8, n_packed, lambda i: L.nq_reorder_words(words[i].data_ptr(), out_words.data_ptr(), rows * (cols // 32), _lib.NQ_LSB_FIRST, _lib.NQ_HALF2, st)),
    ]
    # the word-to-word kernels again on a 70B-sized factor (28672 x 8192: 59 MB read + written per launch): at
    # 12288 x 4096 they move 12.6 MB, which the memory system delivers in 2 us, less than a launch takes to ramp up
    rows2, cols2 = 28672, 8192
    W2 = rows2 * cols2
    words2 = [torch.randint(-2**31, 2**31 - 1, (rows2, cols2 // 32), generator=g, device=device, dtype=torch.int32)
              for _ in range(5)]
    out_words2 = torch.empty(rows2, cols2 // 32, dtype=torch.int32, device=device)
    out_tiles2 = torch.empty(L.nq_tiles_bytes(rows2, cols2), dtype=torch.uint8, device=device)
    cases += [
        ("nq_rows_to_tiles 28672x8192", W2 / 4, 5, lambda i: L.nq_rows_to_tiles(words2[i].data_ptr(), out_tiles2.data_ptr(), rows2, cols2, _lib.NQ_LSB_FIRST, st)),
        ("nq_reorder_words 28672x8192", W2 / 4, 5, lambda i: L.nq_reorder_words(words2[i].data_ptr(), out_words2.data_ptr(), rows2 * (cols2 // 32), _lib.NQ_LSB_FIRST, _lib.NQ_HALF2, st)),
    ]
    peak, peak_src = hbm_peak()
    res = {}
    stream = torch.cuda.Stream(device)
    for name, nbytes, n, fn in cases:
        # one rotation over the inputs as a CUDA graph: the kernels take 2-15 us, less than a launch from Python
        with torch.cuda.stream(stream):
            st = stream.cuda_stream
            for i in range(n):
                _lib.check(fn(i), name)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n):
                    _lib.check(fn(i), name)
            graph.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            stream.synchronize()
            e0.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (args.steps * n)
        res[name] = {"us": us, "GBps": nbytes / us / 1e3, "hbm_frac": nbytes / us / 1e3 / peak, "algorithmic_bytes": nbytes}
    top = res["nq_rows_to_tiles"]
    print(json.dumps({
        "mode": "pack", "metric": "pack / layout kernels, GB/s of algorithmic bytes", "value": top["GBps"], "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": 1, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 / u32 bit operations", "data": "synthetic",
        "config": {"workload": f"{rows} x {cols} +-1 matrix; {n_dense} dense / {n_packed} packed inputs in rotation (> 2 x L2)"},
        "roofline": {"bound": "hbm", "achieved": top["GBps"], "peak": peak, "unit": "GB/s", "frac": top["hbm_frac"],
                     "traffic": None, "kernel": "rows_to_tiles_kernel", "peak_source": peak_src},
        "kernels": res, "gpu_launches": args.steps * (3 * n_packed + 2 * n_dense + 10)}), flush=True)


def head_arm(args):
    """`--mode head`: the dense GEMV of the un-quantised `lm_head` alone (`--vocab` rows, `--batch` tokens)."""
    import torch
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    h = measure_head(device, torch.bfloat16, args.batch, vocab=args.vocab or None, steps=args.steps, profile=True)
    clocks = sampler.stop()
    peak, peak_src = hbm_peak()
    print(json.dumps({
        "mode": "head", "metric": "lm_head GEMV GB/s (algorithmic bytes: weights once + x + y)", "value": h["value"],
        "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": 3, "ms_per_step": h["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": f"{WORKLOAD} lm_head {h['shape'][0]} x {h['shape'][1]}, {args.batch} token(s)",
                   "l2": "weights larger than L2" if 2 * h["shape"][0] * h["shape"][1] > 2 * L2_BYTES else "weights may fit L2"},
        "roofline": {"bound": "hbm", "achieved": h["value"], "peak": peak, "unit": "GB/s", "frac": h["value"] / peak,
                     "traffic": None, "kernel": "dense_gemv_kernel", "peak_source": peak_src},
        "gpu_launches": args.steps, "clocks": clocks}), flush=True)


REF_KERNEL_LIB = os.path.join(ROOT, "baseline", "_ref", "libnq_reference_kernels.so")
# the launch parameters the reference's module passes (src/nanoquant/modules/linear.py:175-184)
REF_GEMV_KWARGS = dict(num_thread_stage1=128, num_thread_stage2=128, num_row_per_warp_stage1=2, num_row_per_warp_stage2=2,
                       num_acc_stage1=1, num_acc_stage2=1, num_pipeline_stage1=8, num_pipeline_stage2=8)


def measure_refkernel(T, layers_timed, steps, warmup, device):
    """The REFERENCE's own decode GEMV (its `gemv_kernel.cu`, compiled for sm_100 by `baseline/build_ref_kernels.py`) on
    the linears of the decode step, one operator call per linear (two kernel launches each) replayed from a CUDA graph
    as the reference's decode benchmark does (`kernel/test_decode.py:385-417`).  Returns a record, or None when the
    library is not built."""
    import torch
    if not os.path.exists(REF_KERNEL_LIB):
        return None
    torch.ops.load_library(REF_KERNEL_LIB)
    op = torch.ops.nq_reference.nanoquant_dyn_forward
    dtype = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(0)
    words = lambda rows, cols: torch.randint(-2**31, 2**31 - 1, (rows, cols // 32), generator=g, device=device, dtype=torch.int32)
    scale = lambda n: ((torch.rand(n, generator=g, device=device) + 0.5) * 0.01).to(dtype)
    xs = {"h": torch.randn(T, HIDDEN, generator=g, device=device).to(dtype),
          "i": torch.randn(T, INTER, generator=g, device=device).to(dtype)}
    layers = []
    for _ in range(layers_timed):
        layers.append([(src, scale(N), words(R, N), scale(R), words(M, R), scale(M)) for (_, N, R, M, src, _) in layer_linears()])

    # one linear against the oracle first: the operands are in the reference's `half2` row layout
    err = None
    try:
        from oracle import nanoquant_oracle as oc
        import numpy as np
        d = oc.synth_linear(1024, 256, 512, T, seed=5)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a).astype(np.float32)).to(dtype).to(device)
        bits = lambda w: torch.from_numpy(oc.pack_rows(w, "half2")).to(device)
        xq, a, b, c = to(d["x"]), to(d["s_pre"]), to(d["s_mid"]), to(d["s_post"])
        y = op(xq, a, bits(d["V"]), b, bits(d["U"]), c, **REF_GEMV_KWARGS)
        f = lambda t: t.float().cpu().numpy().astype(np.float64)
        err = float(oc.rel_err(f(y), oc.forward_fp64(f(xq), d["V"], d["U"], f(a), f(b), f(c))))
    except ImportError:
        pass

    def run():
        out = None
        for lay in layers:
            for (src, a, v, b, u, c) in lay:
                out = op(xs[src], a, v, b, u, c, **REF_GEMV_KWARGS)
        return out
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(3):
            run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        for _ in range(max(warmup, 3)):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / steps * (LAYERS / layers_timed)
    nbytes = sum(algorithmic_bytes(N, R, M, T) for (_, N, R, M, _, _) in layer_linears()) * LAYERS
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"value": T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "hbm_gbs": gbs, "hbm_frac": gbs / hbm_peak()[0],
            "launches_per_step": 2 * 7 * LAYERS, "layers_timed": layers_timed, "max_rel_err_vs_oracle": err,
            "what": "the reference's own gemv_kernel.cu built for sm_100, one call per linear, CUDA-graph replay, same GPU"}


def refkernel_arm(args):
    """`--mode refkernel`: a same-GPU kernel-against-kernel figure beside the default line (not the `--impl reference`
    arm, which is the reference's CPU path)."""
    import torch
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    r = measure_refkernel(args.batch, args.layers, args.steps, args.warmup, device)
    clocks = sampler.stop()
    if r is None:
        print(json.dumps({"mode": "refkernel", "unavailable": "baseline/_ref/libnq_reference_kernels.so is not built "
                          "(python baseline/build_ref_kernels.py needs the reference checkout)"}), flush=True)
        return
    peak, peak_src = hbm_peak()
    print(json.dumps({
        "mode": "refkernel", "impl": "reference CUDA kernels (gemv_kernel.cu, sm_100 build)",
        "metric": "decode tok/s (quantised linears of one decode step)", "value": r["value"], "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "dtype": "bf16 (half2-style accumulation in the I/O type)", "data": "synthetic",
        "config": workload_config(args.batch),
        "roofline": {"bound": "hbm", "achieved": r["hbm_gbs"], "peak": peak, "unit": "GB/s", "frac": r["hbm_frac"],
                     "traffic": None, "peak_source": peak_src},
        "gpu_launches": 2 * 7 * args.layers * args.steps, "layers_timed": args.layers,
        "max_rel_err_vs_oracle": r["max_rel_err_vs_oracle"], "clocks": clocks}), flush=True)


def probe_arm(args):
    """`--mode probe`: the library's measurement probes.  `chain_us` is the time per launch of a decode launch's
    dependent chain with the arithmetic taken out (the floor of the launch structure) for several CTA counts;
    `loop_gbs` is the rate of the GEMV's item loop fed from shared memory only, a cp.async ring, or registers."""
    import ctypes
    import torch
    from nanoquant_b200 import _lib
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    torch.zeros(1, device=device)   # primary context
    L = _lib.lib()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    out = ctypes.c_float()
    chain = {}
    for ctas in sorted({sms, sms * 7 // 8, sms * 13 // 20, sms * 3 // 5, sms // 2, sms // 4}):
        for rank in (1600, 2432):
            _lib.check(L.nq_probe_chain(ctas, rank, 0, ctypes.byref(out)), "nq_probe_chain")
            chain[f"{ctas} CTAs, rank {rank}"] = round(out.value, 3)
    loop = {}
    for mode, name in enumerate(("shared memory only", "cp.async ring", "registers")):
        _lib.check(L.nq_probe_loop(mode, 256, ctypes.byref(out)), "nq_probe_loop")
        loop[name] = round(out.value, 1)
    peak, peak_src = hbm_peak()
    print(json.dumps({"mode": "probe", "chain_us_per_launch": chain, "loop_gbs": loop, "hbm_peak_gbs": peak,
                      "peak_source": peak_src, "n_gpus": 1}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--batch", type=int, default=1, help="tokens per decode step (1, 4 or 16 in the workload)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="qwen3-8b", choices=sorted(WORKLOADS),
                    help="decoder shape of the decode step (qwen3-8b is the headline workload)")
    ap.add_argument("--gemm-min-tokens", type=int, default=0,
                    help="decode batches of at least this many tokens run the group GEMM instead of the GEMV (0: library default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the output check of the launch structure against the oracle")
    ap.add_argument("--no-side-numbers", action="store_true",
                    help="skip the short batch-4 / batch-16 / prefill measurements added to the default line")
    ap.add_argument("--mode", default="replica", choices=["replica", "tp", "prefill", "head", "linear", "pack", "probe", "refkernel"],
                    help="replica: the decode step (N > 1: independent replicas); tp: 70B-shaped TP decode step; "
                         "prefill: GEMM TFLOP/s on Llama-2-7B-shaped layers")
    ap.add_argument("--shape", default="config1", choices=sorted(GROUP_SHAPES), help="launch group of --mode linear")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16"], help="I/O type of --mode linear")
    ap.add_argument("--copies", type=int, default=0, help="--mode linear: cap on the weight sets (0: enough for 2 x L2)")
    ap.add_argument("--vocab", type=int, default=0, help="rows of the head in --mode head (0: the workload's vocabulary)")
    ap.add_argument("--tokens", type=int, default=2048, help="tokens per GEMM in --mode prefill")
    ap.add_argument("--prefill-model", default="llama-2-7b", choices=sorted(PREFILL_SHAPES),
                    help="layer shapes of --mode prefill")
    ap.add_argument("--precise-intermediate", action="store_true",
                    help="bf16 GEMM path: keep the rank-R intermediate as scaled fp16 (nq_gemm_set_precise_intermediate)")
    ap.add_argument("--no-groups", action="store_true",
                    help="--mode prefill: one GEMM call per linear instead of launch groups for q/k/v and gate/up")
    ap.add_argument("--layers", type=int, default=LAYERS, help="decoder layers resident (fewer only for profiling)")
    ap.add_argument("--tp-layers", type=int, default=TP_LAYERS, help="layers actually timed in --mode tp")
    ap.add_argument("--tp-collective", default="peer", choices=["peer", "nccl"],
                    help="--mode tp with several GPUs: all-gather by the peer-memory kernel (graph replay) or by NCCL (eager)")
    args = ap.parse_args()
    global GEMM_MIN_TOKENS
    GEMM_MIN_TOKENS = args.gemm_min_tokens
    set_workload(args.workload)
    if args.layers == WORKLOADS["qwen3-8b"][2]:   # the default of --layers means "all layers of the workload"
        args.layers = LAYERS
    if args.precise_intermediate and args.impl != "reference":
        from nanoquant_b200 import _lib
        _lib.lib().nq_gemm_set_precise_intermediate(1)
    if args.impl == "reference":
        reference_arm(args)
    elif args.mode == "tp":
        tp_arm(args)
    elif args.mode == "prefill":
        prefill_arm(args)
    elif args.mode == "head":
        head_arm(args)
    elif args.mode == "linear":
        linear_arm(args)
    elif args.mode == "pack":
        pack_arm(args)
    elif args.mode == "probe":
        probe_arm(args)
    elif args.mode == "refkernel":
        refkernel_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
