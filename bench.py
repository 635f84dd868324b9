#!/usr/bin/env python
"""Benchmark of the B200 map / reduce / contraction path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line. A step is one pass of the hot path over one batch of
seeded synthetic input. The default workload is the row-softmax chain
(fp32 [16384, 4096]); the other configurations are reported under
"other_workloads" of the same line (kernel-only numbers, fewer steps) and can be
made the headline with --workload.

Multi-GPU (launched by torchrun, one rank per GPU): every workload shards along
its independent axis with no data-path collective, so each rank runs the full
per-GPU batch on its own block of a global batch N times as large (weak
scaling); the reported value is the work of all ranks over the slowest rank's
device time.

--impl reference times the CPU oracle (a restatement of the reference's naive
fp32 loops; the reference itself is Go and cannot be built in this image) on the
host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of each workload's kernel, from the ncu
# captures summarised under profiles/ (mean of the two captured launches).
NCU_TRAFFIC_BYTES = {
    "softmax_rows_f32_16384x4096": 482008320,      # read 268.4 MB + write 213.4 MB (the rest of y still in L2)
    "layernorm_rows_bf16_65536x8192": 2097942000,
    "reduce_outer_f32_256x1024x1024": 1078629812,
    "map_rowsum_f32_4096x1024": 16784000,
    "gemm_bias_relu_bf16_8192": 1000201344,
    "softmax_rows_f32_8192x16384": 1015706112,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------
class Workload:
    """One benchmark configuration: seeded inputs, the C-ABI call, its algorithmic work."""
    name = ""
    dtype = ""
    bound = "hbm"          # roofline that bounds the kernel
    unit = "GB/s"
    metric = "hbm_gbs"
    shape = ""
    launches_per_step = 1

    def work(self) -> float:           # algorithmic bytes (or flops) of one step on one GPU
        raise NotImplementedError

    def e2e_work(self) -> float:       # algorithmic work of one end-to-end step (defaults to a full step)
        return self.work()

    def make(self, dev, seed):         # device-resident inputs and outputs
        raise NotImplementedError

    def step(self):                    # one pass of the hot path (asynchronous)
        raise NotImplementedError

    def host_inputs(self):             # pinned host copies for the end-to-end leg
        raise NotImplementedError

    def e2e_step(self):                # H2D of the inputs, the call, D2H of the result
        raise NotImplementedError

    def e2e_join(self):                # the current stream waits for every chunk the end-to-end steps enqueued
        pipe = getattr(self, "pipe", None)
        if pipe is not None:
            pipe.join()

    def cpu_sample(self, oracle):      # -> (one pass as a callable, work per pass, description)
        raise NotImplementedError

    def check(self, oracle):           # sampled parity against the oracle (raises on mismatch)
        pass


class SoftmaxRows(Workload):
    name = "softmax_rows_f32_16384x4096"
    dtype = "f32"
    rows, cols = 16384, 4096
    shape = "x fp32 [16384, 4096] ~ 4*N(0,1) -> y fp32 [16384, 4096]"

    def work(self):
        return 2.0 * self.rows * self.cols * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = 4 * torch.randn((self.rows, self.cols), generator=g, device=dev)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.softmax_rows(self.x, out=self.y)

    def host_inputs(self):
        from tcacomp_b200.pipeline import RowPipeline
        self.hx = self.x.cpu().pin_memory()
        self.hy = torch.empty_like(self.hx).pin_memory()
        self.h2d = self.hx.numel() * 4
        self.d2h = self.hy.numel() * 4
        self.pipe = RowPipeline(self.x.device, self.rows // 8, (self.cols,), torch.float32,
                                {"y": ((self.cols,), torch.float32)})

    def e2e_step(self):
        self.pipe.run(self.hx, {"y": self.hy}, lambda din, dout: self.T.softmax_rows(din, out=dout["y"]), join=False)

    def cpu_sample(self, oracle):
        x = self.x.cpu().numpy()
        return (lambda: oracle.softmax_rows(x)), self.work(), f"all {self.rows} rows per pass"

    def check(self, oracle):
        idx = torch.tensor([0, 77, self.rows - 1], device=self.x.device)
        from oracle import checks
        assert checks.softmax_close(self.y[idx].cpu().numpy(), self.x[idx].cpu().numpy()), \
            "softmax parity check failed"


class LayernormRows(Workload):
    name = "layernorm_rows_bf16_65536x8192"
    dtype = "bf16"
    rows, cols = 65536, 8192
    shape = "x bf16 [65536, 8192] ~ N(0,1), gamma/beta bf16 [8192] -> y bf16 [65536, 8192]"

    def work(self):
        return 2.0 * self.rows * self.cols * 2 + 2 * self.cols * 2

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.empty((self.rows, self.cols), device=dev, dtype=torch.bfloat16)
        for lo in range(0, self.rows, 8192):  # generate in slabs: no 2 GB fp32 temporary
            self.x[lo:lo + 8192] = torch.randn((8192, self.cols), generator=g, device=dev).to(torch.bfloat16)
        self.gamma = (1 + 0.1 * torch.randn(self.cols, generator=g, device=dev)).to(torch.bfloat16)
        self.beta = (0.1 * torch.randn(self.cols, generator=g, device=dev)).to(torch.bfloat16)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.layernorm_rows(self.x, self.gamma, self.beta, 1e-5, out=self.y)

    def host_inputs(self):
        from tcacomp_b200.pipeline import RowPipeline
        self.hx = self.x.cpu().pin_memory()
        self.hy = torch.empty_like(self.hx).pin_memory()
        self.h2d = self.hx.numel() * 2
        self.d2h = self.hy.numel() * 2
        self.pipe = RowPipeline(self.x.device, self.rows // 8, (self.cols,), torch.bfloat16,
                                {"y": ((self.cols,), torch.bfloat16)})

    def e2e_step(self):
        self.pipe.run(self.hx, {"y": self.hy},
                      lambda din, dout: self.T.layernorm_rows(din, self.gamma, self.beta, 1e-5, out=dout["y"]), join=False)

    def cpu_sample(self, oracle):
        rows = 8192
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)  # noqa: E731
        x, g, b = bits(self.x[:rows]), bits(self.gamma), bits(self.beta)
        return ((lambda: oracle.layernorm_rows_bf16(x, g, b, 1e-5)), 2.0 * rows * self.cols * 2,
                f"first {rows} of {self.rows} rows per pass")

    def check(self, oracle):
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)  # noqa: E731
        idx = torch.tensor([0, 4099, self.rows - 1], device=self.x.device)
        from oracle import checks
        assert checks.layernorm_bf16_close(bits(self.y[idx]), bits(self.x[idx]), bits(self.gamma), bits(self.beta)), \
            "layernorm parity check failed"


class ReduceOuter(Workload):
    name = "reduce_outer_f32_256x1024x1024"
    dtype = "f32"
    nb, nk, nc = 256, 1024, 1024
    shape = "t fp32 [256, 1024, 1024] ~ U(-100,100) -> sum f32, max f32, argmax i32 [256, 1024] in one pass"

    def work(self):
        return self.nb * self.nk * self.nc * 4.0 + 3.0 * self.nb * self.nc * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.t = torch.rand((self.nb, self.nk, self.nc), generator=g, device=dev) * 200 - 100
        self.out = {"sum": torch.empty((self.nb, self.nc), device=dev),
                    "max": torch.empty((self.nb, self.nc), device=dev),
                    "argmax": torch.empty((self.nb, self.nc), device=dev, dtype=torch.int32)}

    def step(self):
        self.T.reduce_outer(self.t, out=self.out)

    def host_inputs(self):
        self.ht = self.t.cpu().pin_memory()
        self.ho = {k: torch.empty_like(v, device="cpu").pin_memory() for k, v in self.out.items()}
        self.h2d = self.ht.numel() * 4
        self.d2h = 3 * self.nb * self.nc * 4
        from tcacomp_b200.pipeline import RowPipeline
        self.pipe = RowPipeline(self.t.device, self.nb // 8, (self.nk, self.nc), torch.float32,
                                {"sum": ((self.nc,), torch.float32), "max": ((self.nc,), torch.float32),
                                 "argmax": ((self.nc,), torch.int32)})

    def e2e_step(self):
        self.pipe.run(self.ht, self.ho, lambda din, dout: self.T.reduce_outer(din, out=dout), join=False)

    def cpu_sample(self, oracle):
        nb = 32
        t = self.t[:nb].cpu().numpy()
        return ((lambda: oracle.reduce_outer(t)), nb * self.nk * self.nc * 4.0 + 3.0 * nb * self.nc * 4,
                f"first {nb} of {self.nb} batches per pass")

    def check(self, oracle):
        s, m, a = oracle.reduce_outer(self.t[:2].cpu().numpy())
        assert np.array_equal(self.out["argmax"][:2].cpu().numpy(), a), "argmax parity check failed"
        assert np.array_equal(self.out["max"][:2].cpu().numpy(), m), "max parity check failed"
        assert np.abs(self.out["sum"][:2].cpu().numpy() - s).max() <= 1e-5 * 51200, "sum parity check failed"


class MapRowsum(Workload):
    name = "map_rowsum_f32_4096x1024"
    dtype = "f32"
    rows, cols = 4096, 1024
    copies = 16  # distinct input buffers, one launch each per step: 256 MiB in total, larger than L2
    launches_per_step = 16
    shape = ("x fp32 [4096, 1024] ~ U(-1,1) -> y[i] = sum_j (0.5*x+0.25)^2 fp32 [4096]; one step = a CUDA graph "
             "of 16 launches over 16 distinct inputs (a single 16 MB launch is launch-latency bound and L2-resident)")
    EXPR = "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)"

    def work(self):
        return self.copies * (self.rows * self.cols * 4.0 + self.rows * 4)

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.xs = [torch.rand((self.rows, self.cols), generator=g, device=dev) * 2 - 1 for _ in range(self.copies)]
        self.ys = [torch.empty((self.rows,), device=dev) for _ in range(self.copies)]
        self.y = self.ys[0]
        self._launch_all()              # first calls outside capture (occupancy queries are cached)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._launch_all()

    def _launch_all(self):
        for x, y in zip(self.xs, self.ys):
            self.T.chain_reduce([x], self.EXPR, out=y)

    def step(self):
        self.graph.replay()

    def e2e_work(self):
        return self.work() / self.copies   # the end-to-end step moves and reduces ONE [4096, 1024] input

    def host_inputs(self):
        self.hx = self.xs[0].cpu().pin_memory()
        self.hy = torch.empty((self.rows,)).pin_memory()
        self.h2d = self.hx.numel() * 4
        self.d2h = self.rows * 4

    def e2e_step(self):
        self.xs[0].copy_(self.hx, non_blocking=True)
        self.T.chain_reduce([self.xs[0]], self.EXPR, out=self.y)
        self.hy.copy_(self.y, non_blocking=True)

    def cpu_sample(self, oracle):
        x = self.xs[0].cpu().numpy()
        return (lambda: oracle.map_rowsum_affine_sq(x)), self.work() / self.copies, "the full [4096, 1024] input per pass"

    def check(self, oracle):
        self.T.chain_reduce([self.xs[0]], self.EXPR, out=self.y)
        from oracle import checks
        assert checks.rowsum_close(self.y.cpu().numpy(), self.xs[0].cpu().numpy()), "rowsum parity check failed"


class GemmBiasRelu(Workload):
    name = "gemm_bias_relu_bf16_8192"
    dtype = "bf16"
    bound = "tensor"
    unit = "TFLOP/s"
    metric = "bf16_tflops"
    m = n = k = 8192
    shape = "a, b bf16 [8192, 8192] ~ N(0,1)/sqrt(8192), bias fp32 [8192] -> c = relu(a@b+bias) bf16, fp32 accumulate"

    def work(self):
        return 2.0 * self.m * self.n * self.k

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        sc = 1.0 / np.sqrt(self.k)
        self.a = (torch.randn((self.m, self.k), generator=g, device=dev) * sc).to(torch.bfloat16)
        self.b = (torch.randn((self.k, self.n), generator=g, device=dev) * sc).to(torch.bfloat16)
        self.bias = torch.randn((self.n,), generator=g, device=dev) * 0.02
        self.c = torch.empty((self.m, self.n), device=dev, dtype=torch.bfloat16)

    def step(self):
        self.T.gemm_bias_act(self.a, self.b, self.bias, "relu", out=self.c)

    def host_inputs(self):
        self.ha = self.a.cpu().pin_memory()
        self.hc = torch.empty_like(self.c, device="cpu").pin_memory()
        self.h2d = self.ha.numel() * 2   # a is the per-step input; b and bias are weights resident in HBM
        self.d2h = self.hc.numel() * 2

    def e2e_step(self):
        if not hasattr(self, "pipe"):
            from tcacomp_b200.pipeline import RowPipeline
            self.pipe = RowPipeline(self.a.device, self.m // 8, (self.k,), torch.bfloat16,
                                    {"c": ((self.n,), torch.bfloat16)})
        self.pipe.run(self.ha, {"c": self.hc},
                      lambda din, dout: self.T.gemm_bias_act(din, self.b, self.bias, "relu", out=dout["c"]), join=False)

    def cpu_sample(self, oracle):
        rows = 64
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)  # noqa: E731
        a, b, bias = bits(self.a[:rows]), bits(self.b), self.bias.cpu().numpy()
        return ((lambda: oracle.gemm_bias_act_bf16(a, b, bias, "relu")), 2.0 * rows * self.n * self.k,
                f"first {rows} of {self.m} rows of a (all of b) per pass")

    def check(self, oracle):
        bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)  # noqa: E731
        rows = 8
        want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(bits(self.a[:rows]), bits(self.b),
                                                            self.bias.cpu().numpy(), "relu"))
        got = self.c[:rows].float().cpu().numpy()
        err = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
        assert err <= 1e-3, f"gemm parity check failed: relative Frobenius error {err}"


class SoftmaxLongRows(SoftmaxRows):
    """Rows too long for a CTA's registers (the shared-memory row kernel); selectable, not part of the default line."""
    name = "softmax_rows_f32_8192x16384"
    rows, cols = 8192, 16384
    shape = "x fp32 [8192, 16384] ~ 4*N(0,1) -> y fp32 [8192, 16384]"


WORKLOADS = {w.name: w for w in (SoftmaxRows, LayernormRows, ReduceOuter, MapRowsum, GemmBiasRelu)}
SELECTABLE = dict(WORKLOADS, **{SoftmaxLongRows.name: SoftmaxLongRows})
DEFAULT = SoftmaxRows.name


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU through NVML (read-only) from a
    thread, every 10 ms, so that even a timed region of a few milliseconds gets samples."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
               0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.index = index
        self.samples = []   # (perf_counter, sm_mhz, reasons bitmask)
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            # NVML enumerates physical GPUs; map the CUDA ordinal through the device's UUID
            uuid = torch.cuda.get_device_properties(self.index).uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}".encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # no NVML: report it, never fail the benchmark
            self.error = f"{type(exc).__name__}: {exc}"[:120]
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    why = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    why = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.samples.append((time.perf_counter(), mhz, why))
            except Exception as exc:
                self.error = f"{type(exc).__name__}: {exc}"[:120]
                return
            time.sleep(0.01)

    def stop(self, t0: float, t1: float):
        """Summary over the samples taken in [t0, t1] (the load window around the timed region)."""
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        win = [s for s in self.samples if t0 <= s[0] <= t1]
        if not win:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0,
                    "reasons": [self.error or "no sample fell inside the load window"]}
        mask = 0
        for _, _, why in win:
            mask |= why
        return {"sm_mhz": statistics.median(s[1] for s in win), "sm_max_mhz": self.max_mhz,
                "samples": len(win), "reasons": sorted(v for k, v in self.REASONS.items() if mask & k)}


# ----------------------------------------------------------------------------
# timing
# ----------------------------------------------------------------------------
def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def barrier(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int, dev) -> float:
    if world == 1:
        return ms
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def timed(fn, steps: int, warmup: int, world: int, dev, after=None) -> float:
    """Device time in ms of exactly `steps` calls of fn on the current stream, max over ranks. `after` runs once
    after the last call, inside the timed region (a pipeline's join)."""
    for _ in range(warmup):
        fn()
    if after is not None:
        after()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if after is not None:
        after()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world, dev)


def per_step_ms(fn, steps: int) -> dict:
    """Median and minimum device time of single steps (this rank), from one event pair per step, taken in a pass
    of its own so that the extra event records do not sit inside the region `value` is computed from."""
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        fn()
        marks[i + 1].record()
    torch.cuda.synchronize()
    t = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    return {"median": t[len(t) // 2], "min": t[0], "max": t[-1], "steps": steps}


def measure(wl, steps, warmup, world, dev, peaks, peak_src):
    """Kernel-only throughput of one workload with inputs resident in HBM."""
    ms = timed(wl.step, steps, warmup, world, dev)
    per_gpu = wl.work() * steps / (ms * 1e-3)               # bytes/s or flop/s of one GPU
    scale = 1e9 if wl.bound == "hbm" else 1e12
    key = "hbm_gbs" if wl.bound == "hbm" else "bf16_tflops_sustained"
    peak = peaks.get(key) or peaks["bf16_tflops"]
    roofline = {"bound": wl.bound, "achieved": per_gpu / scale, "peak": peak, "unit": wl.unit,
                "frac": per_gpu / scale / peak, "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                "peak_source": f"{peak_src}:{key}", "algorithmic_per_launch": wl.work() / wl.launches_per_step,
                "avg_launch_ms": ms / (steps * wl.launches_per_step)}
    return ms, per_gpu * world / scale, roofline


def run_ours(args) -> dict:
    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    import tcacomp_b200 as T
    from oracle import binding as oracle  # checker and CPU baseline only

    peaks, peak_src = load_peaks()
    wl = SELECTABLE[args.workload]()
    wl.make(dev, seed=1234 + rank)

    # correctness of what is about to be timed (sampled rows against the oracle)
    wl.step()
    torch.cuda.synchronize()
    wl.check(oracle)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        wl.step()
    # keep the GPU under the same load for a moment before timing, so that the clocks have settled
    # and the sampler sees them under load even when the timed region lasts a few milliseconds
    t_load0 = time.perf_counter()
    while time.perf_counter() - t_load0 < args.preload_ms * 1e-3:
        for _ in range(8):
            wl.step()
        torch.cuda.synchronize()
    n0 = T.launch_count()
    ms, value, roofline = measure(wl, args.steps, 0, world, dev, peaks, peak_src)
    launches = T.launch_count() - n0
    roofline["step_ms"] = per_step_ms(wl.step, max(20, args.steps))
    if hasattr(wl, "graph"):  # launches replayed from a CUDA graph do not pass through the library's counter
        launches = args.steps * wl.launches_per_step
    clocks = sampler.stop(t_load0, time.perf_counter()) if rank == 0 else None

    # end to end: pinned host inputs -> H2D -> the call -> D2H of the result, every step
    wl.host_inputs()
    e2e_steps = max(2, min(args.steps, 10))
    # batches stream through the pipeline back to back; one join ends the warm-up and one the timed region
    e2e_ms = timed(wl.e2e_step, e2e_steps, 1, world, dev, after=wl.e2e_join)
    scale = 1e9 if wl.bound == "hbm" else 1e12
    e2e = {"value": wl.e2e_work() * e2e_steps * world / (e2e_ms * 1e-3) / scale, "unit": wl.unit,
           "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "steps": e2e_steps,
           "ms_per_step": e2e_ms / e2e_steps,
           "how": "pinned host buffers; H2D, kernel and D2H pipelined over chunks of the independent axis, steps back to back, "
                  "one join before the closing event"}

    cpu = None
    if rank == 0 and world == 1:
        fn, work, sample = wl.cpu_sample(oracle)
        fn()  # untimed: starts the oracle's worker threads and pages the sample in
        passes, t0 = 0, time.perf_counter()
        while passes < 2 or time.perf_counter() - t0 < args.cpu_seconds:
            fn()
            passes += 1
        dt = time.perf_counter() - t0
        cpu = {"value": work * passes / dt / scale, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
               "sample": f"{sample}, {passes} passes", "seconds": dt}

    name, shape, dtype, unit, metric = wl.name, wl.shape, wl.dtype, wl.unit, wl.metric
    del wl
    torch.cuda.empty_cache()

    others = []
    if not args.no_others:
        for oname, cls in WORKLOADS.items():
            if oname == name:
                continue
            ow = cls()
            try:
                ow.make(dev, seed=99 + rank)
                ow.step()
                torch.cuda.synchronize()
                ow.check(oracle)
                o_ms, o_val, o_roof = measure(ow, max(3, min(args.steps, 10)), 3, world, dev, peaks, peak_src)
                others.append({"workload": oname, "value": o_val, "unit": ow.unit, "dtype": ow.dtype,
                               "roofline": o_roof})
            except Exception as exc:  # a workload this build cannot run yet is reported, not hidden
                others.append({"workload": oname, "error": f"{type(exc).__name__}: {exc}"[:300]})
            del ow
            torch.cuda.empty_cache()

    if world > 1:
        torch.distributed.destroy_process_group()
    return {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype, "data": "synthetic (seeded torch.Generator per rank)",
        "config": {"workload": name, "shape": shape, "per_gpu_batch": "the full configuration on every rank",
                   "parallelism": f"rows sharded over {world} GPU(s), no collective",
                   "l2": "working set larger than the 126 MB L2; no flush between steps"},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
        "clocks": clocks, "other_workloads": others,
    }


def run_reference(args) -> dict | None:
    """The reference's CPU path (the oracle port) on the host cores; rank 0 only."""
    rank, _, world = dist_env()
    if rank != 0:
        return None
    from oracle import binding as oracle
    cls = SELECTABLE[args.workload]
    scale = 1e9 if cls.bound == "hbm" else 1e12
    rng = np.random.default_rng(1234)
    if issubclass(cls, SoftmaxRows):
        rows = cls.rows
        x = (4 * rng.standard_normal((rows, cls.cols), dtype=np.float32))
        fn, work = (lambda: oracle.softmax_rows(x)), 2.0 * rows * cls.cols * 4
        sample = f"all {rows} rows per step"
    elif cls is LayernormRows:
        rows = 2048
        x = oracle.f32_to_bf16(rng.standard_normal((rows, cls.cols), dtype=np.float32))
        g = oracle.f32_to_bf16(np.ones(cls.cols, np.float32))
        b = oracle.f32_to_bf16(np.zeros(cls.cols, np.float32))
        fn, work = (lambda: oracle.layernorm_rows_bf16(x, g, b, 1e-5)), 2.0 * rows * cls.cols * 2
        sample = f"{rows} of {cls.rows} rows per step"
    elif cls is ReduceOuter:
        nb = 8
        t = rng.uniform(-100, 100, (nb, cls.nk, cls.nc)).astype(np.float32)
        fn, work = (lambda: oracle.reduce_outer(t)), nb * cls.nk * cls.nc * 4.0 + 3.0 * nb * cls.nc * 4
        sample = f"{nb} of {cls.nb} batches per step"
    elif cls is MapRowsum:
        x = rng.uniform(-1, 1, (cls.rows, cls.cols)).astype(np.float32)
        fn, work = (lambda: oracle.map_rowsum_affine_sq(x)), cls.rows * cls.cols * 4.0 + cls.rows * 4
        sample = "the full [4096, 1024] input per step"
    else:
        rows = 16
        sc = 1.0 / np.sqrt(cls.k)
        a = oracle.f32_to_bf16((rng.standard_normal((rows, cls.k), dtype=np.float32) * sc))
        b = oracle.f32_to_bf16((rng.standard_normal((cls.k, cls.n), dtype=np.float32) * sc))
        bias = (rng.standard_normal(cls.n, dtype=np.float32) * 0.02)
        fn, work = (lambda: oracle.gemm_bias_act_bf16(a, b, bias, "relu")), 2.0 * rows * cls.n * cls.k
        sample = f"{rows} of {cls.m} rows of a (all of b) per step"
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    value = work * args.steps / dt / scale
    cpu = {"value": value, "unit": cls.unit, "cores": oracle.num_threads(), "kind": "port", "sample": sample}
    return {
        "impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cls.dtype,
        "data": "synthetic (seeded numpy Generator)",
        "config": {"workload": cls.name, "shape": cls.shape,
                   "note": "CPU restatement of the reference's naive fp32 loops; the reference is Go and "
                           "cannot be built in this image"},
        "cpu_baseline": cpu,
        "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(SELECTABLE), default=DEFAULT)
    ap.add_argument("--no-others", action="store_true", help="skip the kernel-only lines of the other workloads")
    ap.add_argument("--cpu-seconds", type=float, default=10.0,
                    help="how long the CPU baseline leg repeats its sample (at least two passes)")
    ap.add_argument("--preload-ms", type=float, default=300.0,
                    help="untimed load before the timed region so that the clocks settle (0 for profiler runs)")
    args = ap.parse_args(argv)
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3  # timing hygiene: at least three untimed steps
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.gpus != world and world > 1:
        print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}; using the launcher's world", file=sys.stderr)
    if args.gpus > 1 and world == 1:
        raise SystemExit("bench.py: launch multi-GPU runs with python -m torch.distributed.run "
                         "--nproc-per-node N bench.py --gpus N ...")
    line = run_reference(args) if args.impl == "reference" else run_ours(args)
    if line is not None and int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
