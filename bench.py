#!/usr/bin/env python
"""Benchmark of the B200 map / reduce / contraction path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line. A step is one pass of the hot path over one batch of
seeded synthetic input. The default workload is the row-softmax chain
(fp32 [16384, 4096]); the other configurations are measured in the same run
and reported under "other_workloads", each with its own roofline, end-to-end
figure, CPU baseline and parity counts; any of them can be made the headline
with --workload.

Per workload:
  value / roofline   kernel-only, inputs resident in HBM, CUDA events, max over ranks;
  e2e                the same operator through the library's host-buffer pipeline
                     (tcab_pipeline_*: pinned host memory in, pinned host memory out,
                     upload | kernel | download of successive chunks overlapped);
  cpu_baseline       the CPU oracle (a restatement of the reference's naive fp32 loops)
                     on the host cores, a bounded sample, rank 0 at N = 1 only;
  parity             how many output elements were compared with the oracle before
                     timing and how many of them passed only through the oracle's own
                     distance to the fp64 value (oracle/checks.py).

Multi-GPU (launched by torchrun, one rank per GPU): every workload shards along
its independent axis with no data-path collective. The headline value is weak
scaling (every rank runs the full configuration on its own data); "strong"
reports the SAME global configuration cut N ways with tcacomp_b200.shard.block,
"copy_ceiling" the bare pinned-memory copy rate of all ranks at once, and
"sharded_axis_check" one reduction along a sharded axis (the only place NCCL is
on a data path) checked against the oracle outside the timed region.

--impl reference times the CPU oracle (the reference itself is Go and cannot be
built in this image) on the host cores, rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SUSTAINED_SECONDS = 2.0   # a timed region at least this long is compared with the sustained tensor peak


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


_UNIT = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}


def ncu_traffic(profile: str | None, units_here: int):
    """DRAM bytes per launch from the committed ncu summary of the workload's kernel (profiles/<profile>):
    mean over the captured launches of dram__bytes_read.sum + dram__bytes_write.sum, scaled by the units of the
    independent axis when the capture ran on a reduced case (the summary then carries a line
    `units captured: N`). None when there is no summary."""
    if not profile:
        return None
    path = os.path.join(ROOT, "profiles", profile)
    if not os.path.exists(path):
        return None
    text = open(path).read()
    rd = re.findall(r"\| dram__bytes_read\.sum \| ([\d.,]+) \| (\w+) \|", text)
    wr = re.findall(r"\| dram__bytes_write\.sum \| ([\d.,]+) \| (\w+) \|", text)
    if not rd or len(rd) != len(wr):
        return None
    tot = [float(a.replace(",", "")) * _UNIT[ua] + float(b.replace(",", "")) * _UNIT[ub] for (a, ua), (b, ub) in zip(rd, wr)]
    per_launch = sum(tot) / len(tot)
    m = re.search(r"units captured: (\d+)", text)
    scale = units_here / int(m.group(1)) if m else 1.0
    return {"bytes": per_launch * scale, "source": f"profiles/{profile}",
            "scaled_from_units": int(m.group(1)) if m else None}


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------
class Workload:
    """One benchmark configuration: seeded inputs, the C-ABI call, its algorithmic work.

    `units` is the extent of the independent axis on this GPU (rows / batches / rows of a); the strong-scaling
    leg and reduced profiler captures build the same workload with fewer units."""
    name = ""
    dtype = ""
    bound = "hbm"          # roofline that bounds the kernel
    unit = "GB/s"
    metric = "hbm_gbs"
    shape = ""
    full_units = 0
    launches_per_step = 1
    profile = None         # the ncu summary of this workload's kernel under profiles/
    chunks = 8             # chunks of the independent axis the host-buffer pipeline cuts one step into

    def __init__(self, units: int | None = None):
        self.units = self.full_units if units is None else units

    def work(self) -> float:           # algorithmic bytes (or flops) of one step on one GPU
        raise NotImplementedError

    def e2e_work(self) -> float:       # algorithmic work of one end-to-end step (defaults to a full step)
        return self.work()

    def make(self, dev, seed):         # device-resident inputs and outputs
        raise NotImplementedError

    def step(self):                    # one pass of the hot path (asynchronous)
        raise NotImplementedError

    def pipeline_spec(self, chunk_units):   # tcacomp_b200.pipeline.PipelineSpec of the end-to-end leg
        raise NotImplementedError

    def host_buffers(self):            # -> (pinned inputs, pinned outputs) of one step
        raise NotImplementedError

    def host_setup(self):
        from tcacomp_b200.pipeline import Pipeline
        self.h_in, self.h_out = self.host_buffers()
        self.h2d = sum(t.numel() * t.element_size() for t in self.h_in)
        self.d2h = sum(t.numel() * t.element_size() for t in self.h_out)
        self.pipe = Pipeline(self.pipeline_spec(max(1, self.units // self.chunks)))

    def e2e_step(self):                # upload of the inputs, the call, download of the result: one library call
        self.pipe.run(self.h_in, self.h_out, self.units)

    def e2e_join(self):                # the current stream waits for every chunk the end-to-end steps queued
        self.pipe.join()

    def close(self):
        pipe = getattr(self, "pipe", None)
        if pipe is not None:
            pipe.close()

    def cpu_sample(self, oracle):      # -> (one pass as a callable, work per pass, description)
        raise NotImplementedError

    def check(self, oracle, full: bool) -> dict:   # parity against the oracle (raises on mismatch) -> counts
        return {}


class SoftmaxRows(Workload):
    name = "softmax_rows_f32_16384x4096"
    dtype = "f32"
    full_units, cols = 16384, 4096
    shape = "x fp32 [16384, 4096] ~ 4*N(0,1) -> y fp32 [16384, 4096]"
    profile = "softmax_rows_softmax_rows_f32_16384x4096.md"

    def work(self):
        return 2.0 * self.units * self.cols * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = 4 * torch.randn((self.units, self.cols), generator=g, device=dev)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.softmax_rows(self.x, out=self.y)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("softmax_rows", self.x.device, chunk_units, (self.cols,), torch.float32)

    def host_buffers(self):
        hx = self.x.cpu().pin_memory()
        return [hx], [torch.empty_like(hx).pin_memory()]

    def cpu_sample(self, oracle):
        x = self.x.cpu().numpy()
        return (lambda: oracle.softmax_rows(x)), self.work(), f"all {self.units} rows per pass"

    def check(self, oracle, full):
        from oracle import checks
        if full:   # every output element: the CPU port does the whole tensor in tens of milliseconds
            rep = checks.softmax_report_fast(self.y.cpu().numpy(), self.x.cpu().numpy())
        else:
            idx = torch.linspace(0, self.units - 1, min(self.units, 64), device=self.x.device).long()
            rep = checks.softmax_report_fast(self.y[idx].cpu().numpy(), self.x[idx].cpu().numpy())
        assert rep.ok, f"softmax parity check failed: {rep}"
        return rep.as_dict()


class SoftmaxLongRows(SoftmaxRows):
    """Rows too long for a CTA's registers (the shared-memory row kernel); selectable, not part of the default line."""
    name = "softmax_rows_f32_8192x16384"
    full_units, cols = 8192, 16384
    shape = "x fp32 [8192, 16384] ~ 4*N(0,1) -> y fp32 [8192, 16384]"
    profile = "softmax_rows_smem_softmax_rows_f32_8192x16384.md"


class SoftmaxVocabRows(SoftmaxRows):
    """Rows as long as a vocabulary (the streaming clusters: two passes, the second from L2); selectable only."""
    name = "softmax_rows_f32_2048x65536"
    full_units, cols = 2048, 65536
    shape = "x fp32 [2048, 65536] ~ 4*N(0,1) -> y fp32 [2048, 65536]"
    profile = "softmax_rows_cluster_stream_softmax_rows_f32_2048x65536.md"


class LayernormHeadRows(Workload):
    """Rows of one attention head (the per-head normalisation of queries and keys); selectable only."""
    name = "layernorm_rows_bf16_1048576x128"
    dtype = "bf16"
    full_units, cols = 1048576, 128
    shape = "x bf16 [1048576, 128] ~ N(0,1), gamma/beta bf16 [128] -> y bf16 [1048576, 128]"
    profile = "layernorm_rows_reg_layernorm_rows_bf16_1048576x128.md"

    def work(self):
        return 2.0 * self.units * self.cols * 2 + 2 * self.cols * 2

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.randn((self.units, self.cols), generator=g, device=dev).to(torch.bfloat16)
        self.gamma = (1 + 0.1 * torch.randn((self.cols,), generator=g, device=dev)).to(torch.bfloat16)
        self.beta = (0.1 * torch.randn((self.cols,), generator=g, device=dev)).to(torch.bfloat16)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.layernorm_rows(self.x, self.gamma, self.beta, 1e-5, out=self.y)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("layernorm_rows", self.x.device, chunk_units, (self.cols,), torch.bfloat16, eps=1e-5,
                            resident=(self.gamma, self.beta))

    def host_buffers(self):
        hx = self.x.cpu().pin_memory()
        return [hx], [torch.empty_like(hx).pin_memory()]

    def cpu_sample(self, oracle):
        rows = min(65536, self.units)
        x, g, b = bits16(self.x[:rows]), bits16(self.gamma), bits16(self.beta)
        return (lambda: oracle.layernorm_rows_bf16(x, g, b, 1e-5)), 2.0 * rows * self.cols * 2, f"first {rows} of {self.units} rows per pass"

    def check(self, oracle, full):
        from oracle import checks
        idx = torch.arange(0, self.units, max(1, self.units // (65536 if full else 256)), device=self.x.device)
        rep = checks.layernorm_bf16_report_fast(bits16(self.y[idx]), bits16(self.x[idx]), bits16(self.gamma), bits16(self.beta), 1e-5)
        assert rep.ok, f"layer-norm parity check failed: {rep}"
        return rep.as_dict()


class LayernormRows(Workload):
    name = "layernorm_rows_bf16_65536x8192"
    dtype = "bf16"
    full_units, cols = 65536, 8192
    shape = "x bf16 [65536, 8192] ~ N(0,1), gamma/beta bf16 [8192] -> y bf16 [65536, 8192]"
    profile = "layernorm_rows_layernorm_rows_bf16_65536x8192.md"

    def work(self):
        return 2.0 * self.units * self.cols * 2 + 2 * self.cols * 2

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.empty((self.units, self.cols), device=dev, dtype=torch.bfloat16)
        for lo in range(0, self.units, 8192):  # generate in slabs: no 2 GB fp32 temporary
            n = min(8192, self.units - lo)
            self.x[lo:lo + n] = torch.randn((n, self.cols), generator=g, device=dev).to(torch.bfloat16)
        self.gamma = (1 + 0.1 * torch.randn(self.cols, generator=g, device=dev)).to(torch.bfloat16)
        self.beta = (0.1 * torch.randn(self.cols, generator=g, device=dev)).to(torch.bfloat16)
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.layernorm_rows(self.x, self.gamma, self.beta, 1e-5, out=self.y)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("layernorm_rows", self.x.device, chunk_units, (self.cols,), torch.bfloat16, eps=1e-5,
                            resident=(self.gamma, self.beta))

    def host_buffers(self):
        hx = self.x.cpu().pin_memory()
        return [hx], [torch.empty_like(hx).pin_memory()]

    def cpu_sample(self, oracle):
        rows = min(2048, self.units)
        x, g, b = bits16(self.x[:rows]), bits16(self.gamma), bits16(self.beta)
        return ((lambda: oracle.layernorm_rows_bf16(x, g, b, 1e-5)), 2.0 * rows * self.cols * 2,
                f"first {rows} of {self.units} rows per pass")

    def check(self, oracle, full):
        from oracle import checks
        rows = self.units if full else min(self.units, 1024)
        idx = slice(0, rows) if full else torch.linspace(0, self.units - 1, rows, device=self.x.device).long()
        rep = checks.layernorm_bf16_report_fast(bits16(self.y[idx]), bits16(self.x[idx]), bits16(self.gamma), bits16(self.beta))
        assert rep.ok, f"layernorm parity check failed: {rep}"
        return rep.as_dict()


class ReduceOuter(Workload):
    name = "reduce_outer_f32_256x1024x1024"
    dtype = "f32"
    full_units, nk, nc = 256, 1024, 1024
    shape = "t fp32 [256, 1024, 1024] ~ U(-100,100) -> sum f32, max f32, argmax i32 [256, 1024] in one pass"
    profile = "reduce_outer_kernel_reduce_outer_f32_256x1024x1024.md"

    def work(self):
        return self.units * self.nk * self.nc * 4.0 + 3.0 * self.units * self.nc * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.t = torch.rand((self.units, self.nk, self.nc), generator=g, device=dev) * 200 - 100
        self.out = {"sum": torch.empty((self.units, self.nc), device=dev),
                    "max": torch.empty((self.units, self.nc), device=dev),
                    "argmax": torch.empty((self.units, self.nc), device=dev, dtype=torch.int32)}

    def step(self):
        self.T.reduce_outer(self.t, out=self.out)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("reduce_outer", self.t.device, chunk_units, (self.nk, self.nc), torch.float32)

    def host_buffers(self):
        ht = self.t.cpu().pin_memory()
        return [ht], [torch.empty_like(self.out[k], device="cpu").pin_memory() for k in ("sum", "max", "argmax")]

    def cpu_sample(self, oracle):
        nb = min(16, self.units)
        t = self.t[:nb].cpu().numpy()
        return ((lambda: oracle.reduce_outer(t)), nb * self.nk * self.nc * 4.0 + 3.0 * nb * self.nc * 4,
                f"first {nb} of {self.units} batches per pass")

    def check(self, oracle, full):
        from oracle import checks
        rep = checks.Report()
        batches = range(0, self.units, 16) if full else range(0, min(self.units, 16), 16)
        for lo in batches:
            sl = self.t[lo:lo + 16].cpu().numpy()
            s, m, a = oracle.reduce_outer(sl)
            assert np.array_equal(self.out["argmax"][lo:lo + 16].cpu().numpy(), a), "argmax parity check failed"
            assert np.array_equal(self.out["max"][lo:lo + 16].cpu().numpy(), m), "max parity check failed"
            rep.merge(checks.outer_sum_report(self.out["sum"][lo:lo + 16].cpu().numpy(), s, sl))
        assert rep.ok, f"sum parity check failed: {rep}"
        d = rep.as_dict()
        d["max_and_argmax"] = "bit-exact on the same elements"
        return d


class ReduceOuterNarrow(ReduceOuter):
    """Narrow rows (16 columns): a warp per (b, column tile) instead of a CTA; selectable only."""
    name = "reduce_outer_f32_65536x256x16"
    full_units, nk, nc = 65536, 256, 16
    shape = "t fp32 [65536, 256, 16] ~ U(-100,100) -> sum f32, max f32, argmax i32 [65536, 16] in one pass"
    profile = "reduce_outer_flat_reduce_outer_f32_65536x256x16.md"


class ReduceOuterColumnStats(ReduceOuter):
    """Column statistics of a tall narrow matrix: one batch, 2^23 rows of 16 columns. CTAs of the warp-per-tile
    kernel share the reduced axis and a second launch folds their partial states; selectable only (one unit: it
    does not shard)."""
    name = "reduce_outer_f32_1x8388608x16"
    full_units, nk, nc = 1, 8388608, 16
    launches_per_step = 2
    shape = "t fp32 [1, 8388608, 16] ~ U(-100,100) -> sum f32, max f32, argmax i32 [1, 16] in one pass over t"
    profile = "reduce_outer_flat_reduce_outer_f32_1x8388608x16.md"


class MapRowsum(Workload):
    name = "map_rowsum_f32_4096x1024"
    dtype = "f32"
    full_units, cols = 4096, 1024
    copies = 16  # distinct input buffers per step: 256 MiB in total, larger than L2
    launches_per_step = 1
    chunks = 1   # end to end, a 16 MiB step is one upload, one launch, one 16 KiB download; successive steps overlap
    shape = ("x fp32 [4096, 1024] ~ U(-1,1) -> y[i] = sum_j (0.5*x+0.25)^2 fp32 [4096]; one step = 16 such problems "
             "on 16 distinct inputs handed over as ONE batched launch (a lone 16 MB launch is bounded by launch latency "
             "and the wait for its predecessor, and L2-resident when repeated; see roofline.one_launch_each and "
             "roofline.as_specified)")
    EXPR = "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)"
    profile = "chain_inner_batched_map_rowsum_f32_4096x1024.md"

    def work(self):
        return self.copies * (self.units * self.cols * 4.0 + self.units * 4)

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.xs = [torch.rand((self.units, self.cols), generator=g, device=dev) * 2 - 1 for _ in range(self.copies)]
        self.ys = [torch.empty((self.units,), device=dev) for _ in range(self.copies)]
        self.y = self.ys[0]
        self.bound_call = T.BoundChainReduce([self.xs[0]], self.EXPR, out=self.ys[0])
        self._launch_all()              # first calls outside capture (occupancy queries are cached)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._launch_all()
        self._launch_batched()
        torch.cuda.synchronize()
        self.graph_batched = torch.cuda.CUDAGraph()   # one kernel node: replaying it skips the Python binding's
        with torch.cuda.graph(self.graph_batched):    # per-call work (16 tensor views), not anything on the GPU
            self._launch_batched()

    def _launch_batched(self):
        self.T.chain_reduce_batched([[x] for x in self.xs], self.EXPR, outs=self.ys)

    def _launch_all(self):
        for x, y in zip(self.xs, self.ys):
            self.T.chain_reduce([x], self.EXPR, out=y)

    def step(self):
        """16 problems, one launch (tcab_chain_reduce_batched), replayed from a one-node CUDA graph."""
        self.graph_batched.replay()

    def step_one_launch_each(self):
        """The same 16 problems as 16 launches that follow each other on one stream, replayed from a CUDA graph
        (no host launch path): every launch waits for its predecessor, as stream order demands."""
        self.graph.replay()

    def step_as_specified(self):
        """The configuration exactly as stated: ONE [4096, 1024] buffer, one ordinary launch per step, no graph.
        16.8 MB stay resident in the 126 MB L2 between steps, and every step pays the host's launch path: one
        tcab_chain_reduce call over descriptors built once, as a host of the reference keeps its tca::Tensor views."""
        self.bound_call()

    def e2e_work(self):
        return self.work() / self.copies   # the end-to-end step moves and reduces ONE [4096, 1024] input

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("chain_reduce", self.xs[0].device, chunk_units, (self.cols,), torch.float32, map_expr=self.EXPR)

    def host_buffers(self):
        return [self.xs[0].cpu().pin_memory()], [torch.empty((self.units,)).pin_memory()]

    def cpu_sample(self, oracle):
        x = self.xs[0].cpu().numpy()
        return (lambda: oracle.map_rowsum_affine_sq(x)), self.work() / self.copies, f"the full [{self.units}, 1024] input per pass"

    def check(self, oracle, full):
        from oracle import checks
        rep = checks.Report()
        for x, y in zip(self.xs, self.ys) if full else [(self.xs[0], self.ys[0])]:   # every output of every buffer
            rep.merge(checks.rowsum_report(y.cpu().numpy(), x.cpu().numpy()))
        assert rep.ok, f"rowsum parity check failed: {rep}"
        return rep.as_dict()


class GemmBiasRelu(Workload):
    name = "gemm_bias_relu_bf16_8192"
    dtype = "bf16"
    bound = "tensor"
    unit = "TFLOP/s"
    metric = "bf16_tflops"
    full_units = n = k = 8192
    shape = "a, b bf16 [8192, 8192] ~ N(0,1)/sqrt(8192), bias fp32 [8192] -> c = relu(a@b+bias) bf16, fp32 accumulate"
    profile = "gemm_bias_act_gemm_bias_relu_bf16_8192.md"

    def work(self):
        return 2.0 * self.units * self.n * self.k

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        sc = 1.0 / np.sqrt(self.k)
        self.a = (torch.randn((self.units, self.k), generator=g, device=dev) * sc).to(torch.bfloat16)
        self.b = (torch.randn((self.k, self.n), generator=g, device=dev) * sc).to(torch.bfloat16)
        self.bias = torch.randn((self.n,), generator=g, device=dev) * 0.02
        self.c = torch.empty((self.units, self.n), device=dev, dtype=torch.bfloat16)

    def step(self):
        self.T.gemm_bias_act(self.a, self.b, self.bias, "relu", out=self.c)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec   # a is the per-step input; b and bias are weights resident in HBM
        return PipelineSpec("gemm_bias_act", self.a.device, chunk_units, (self.k,), torch.bfloat16, act="relu",
                            resident=(self.b, self.bias))

    def host_buffers(self):
        return [self.a.cpu().pin_memory()], [torch.empty_like(self.c, device="cpu").pin_memory()]

    def cpu_sample(self, oracle):
        rows = min(16, self.units)
        a, b, bias = bits16(self.a[:rows]), bits16(self.b), self.bias.cpu().numpy()
        return ((lambda: oracle.gemm_bias_act_bf16(a, b, bias, "relu")), 2.0 * rows * self.n * self.k,
                f"first {rows} of {self.units} rows of a (all of b) per pass")

    def check(self, oracle, full):
        # two rows per band of 128 rows (one per 64-row half) and the last row when full, else eight rows
        if full:
            bands = (self.units + 127) // 128
            picks = sorted({min(self.units - 1, b * 128 + (b * 37) % 64) for b in range(bands)} |
                           {min(self.units - 1, b * 128 + 64 + (b * 11) % 64) for b in range(bands)} | {self.units - 1})
        else:
            picks = sorted({0, 1, self.units // 2, self.units - 1})
        rows = torch.tensor(picks, device=self.a.device)
        want = oracle.bf16_to_f32(oracle.gemm_bias_act_bf16(bits16(self.a[rows]), bits16(self.b), self.bias.cpu().numpy(), "relu"))
        got = self.c[rows].float().cpu().numpy()
        err = float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
        assert err <= 1e-3, f"gemm parity check failed: relative Frobenius error {err}"
        return {"checked": int(got.size), "rows": len(picks), "failed": 0, "rel_frobenius": err}


class MapOnly(Workload):
    name = "map_affine_sq_f32_16384x4096"
    dtype = "f32"
    full_units, cols = 16384, 4096
    shape = "x fp32 [16384, 4096] ~ U(-1,1) -> y = (0.5*x+0.25)^2 fp32 [16384, 4096] (the map lambda of the first configuration, stored)"
    EXPR = MapRowsum.EXPR
    profile = "chain_map_map_affine_sq_f32_16384x4096.md"

    def work(self):
        return 2.0 * self.units * self.cols * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.rand((self.units, self.cols), generator=g, device=dev) * 2 - 1
        self.y = torch.empty_like(self.x)

    def step(self):
        self.T.map([self.x], self.EXPR, out=self.y)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("map", self.x.device, chunk_units, (self.cols,), torch.float32, map_expr=self.EXPR)

    def host_buffers(self):
        hx = self.x.cpu().pin_memory()
        return [hx], [torch.empty_like(hx).pin_memory()]

    def cpu_sample(self, oracle):
        from oracle import lambda_eval
        x = self.x[:min(4096, self.units)].cpu().numpy()
        return ((lambda: lambda_eval.evaluate(self.EXPR, [x])), 2.0 * x.size * 4,
                f"first {x.shape[0]} of {self.units} rows per pass, one thread (the lambda compiled by the host compiler)")

    def check(self, oracle, full):
        from oracle import lambda_eval
        rows = self.units if full else min(self.units, 256)
        x = self.x[:rows].cpu().numpy()
        want = lambda_eval.evaluate(self.EXPR, [x])
        got = self.y[:rows].cpu().numpy()
        key = lambda a: np.where(a.view(np.int32) < 0, -(a.view(np.int32) & 0x7fffffff).astype(np.int64), a.view(np.int32).astype(np.int64))  # noqa: E731
        d = np.abs(key(got) - key(want))
        assert d.max() <= 2, f"map parity check failed: {int(d.max())} ulp"   # fp32 maps: within 2 ulp
        return {"checked": int(got.size), "failed": 0, "max_ulp": int(d.max()), "via_fp64_term": 0}


class ShortRowsum(Workload):
    """Rows of 64 columns (16 vectors): a thread per row in ascending order over a coalesced copy; selectable only."""
    name = "map_rowsum_f32_4194304x64"
    dtype = "f32"
    full_units, cols = 4194304, 64
    shape = "x fp32 [4194304, 64] ~ U(-1,1) -> y[i] = sum_j (0.5*x+0.25)^2 fp32 [4194304]"
    EXPR = MapRowsum.EXPR
    profile = "chain_inner_rows32_map_rowsum_f32_4194304x64.md"

    def work(self):
        return self.units * self.cols * 4.0 + self.units * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = torch.rand((self.units, self.cols), generator=g, device=dev) * 2 - 1
        self.y = torch.empty((self.units,), device=dev)

    def step(self):
        self.T.chain_reduce([self.x], self.EXPR, axis=1, out=self.y)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("chain_reduce", self.x.device, chunk_units, (self.cols,), torch.float32, map_expr=self.EXPR)

    def host_buffers(self):
        hx = self.x.cpu().pin_memory()
        return [hx], [torch.empty((self.units,), dtype=torch.float32).pin_memory()]

    def cpu_sample(self, oracle):
        x = self.x[:min(1 << 20, self.units)].cpu().numpy()
        return (lambda: oracle.map_rowsum_affine_sq(x, 0.5, 0.25)), x.size * 4.0 + x.shape[0] * 4, f"first {x.shape[0]} of {self.units} rows per pass"

    def check(self, oracle, full):
        from oracle import checks
        rows = self.units if full else min(self.units, 65536)
        rep = checks.rowsum_report(self.y[:rows].cpu().numpy(), self.x[:rows].cpu().numpy())
        assert rep.ok, f"row-sum parity check failed: {rep}"
        return rep.as_dict()


class RowsumBf16(ShortRowsum):
    """The C1 chain over a bf16 operand (run-time compiled: the ahead-of-time table is fp32): rows read as 16-byte
    vectors of eight, fp32 arithmetic and output; selectable only."""
    name = "map_rowsum_bf16_65536x4096"
    dtype = "f32"
    full_units, cols = 65536, 4096
    shape = "x bf16 [65536, 4096] ~ U(-1,1) -> y[i] = sum_j (0.5*f32(x)+0.25)^2 fp32 [65536]"
    EXPR = "(0.5f*f32(p0) + 0.25f) * (0.5f*f32(p0) + 0.25f)"
    profile = "chain_inner_map_rowsum_bf16_65536x4096.md"

    def work(self):
        return self.units * self.cols * 2.0 + self.units * 4

    def make(self, dev, seed):
        import tcacomp_b200 as T
        self.T = T
        g = torch.Generator(device=dev).manual_seed(seed)
        self.x = (torch.rand((self.units, self.cols), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
        self.y = torch.empty((self.units,), device=dev)

    def pipeline_spec(self, chunk_units):
        from tcacomp_b200.pipeline import PipelineSpec
        return PipelineSpec("chain_reduce", self.x.device, chunk_units, (self.cols,), torch.bfloat16, map_expr=self.EXPR,
                            out_dtype=torch.float32)

    def cpu_sample(self, oracle):
        x = self.x[:min(16384, self.units)].float().cpu().numpy()      # widening bf16 is exact
        return (lambda: oracle.map_rowsum_affine_sq(x, 0.5, 0.25)), x.size * 2.0 + x.shape[0] * 4, f"first {x.shape[0]} of {self.units} rows per pass"

    def check(self, oracle, full):
        from oracle import checks
        rows = self.units if full else min(self.units, 16384)
        rep = checks.rowsum_report(self.y[:rows].cpu().numpy(), self.x[:rows].float().cpu().numpy())
        assert rep.ok, f"row-sum parity check failed: {rep}"
        return rep.as_dict()


WORKLOADS = {w.name: w for w in (SoftmaxRows, LayernormRows, ReduceOuter, MapRowsum, GemmBiasRelu, MapOnly)}
SELECTABLE = dict(WORKLOADS, **{SoftmaxLongRows.name: SoftmaxLongRows, SoftmaxVocabRows.name: SoftmaxVocabRows,
                                LayernormHeadRows.name: LayernormHeadRows, ReduceOuterNarrow.name: ReduceOuterNarrow,
                                ReduceOuterColumnStats.name: ReduceOuterColumnStats, ShortRowsum.name: ShortRowsum,
                                RowsumBf16.name: RowsumBf16})
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


def scale_of(wl) -> float:
    return 1e9 if wl.bound == "hbm" else 1e12


def measure(wl, steps, warmup, world, dev, peaks, peak_src):
    """Kernel-only throughput of one workload with inputs resident in HBM."""
    ms = timed(wl.step, steps, warmup, world, dev)
    per_gpu = wl.work() * steps / (ms * 1e-3)               # bytes/s or flop/s of one GPU
    scale = scale_of(wl)
    roofline = {"bound": wl.bound, "achieved": per_gpu / scale, "unit": wl.unit,
                "algorithmic_per_launch": wl.work() / wl.launches_per_step,
                "avg_launch_ms": ms / (steps * wl.launches_per_step), "timed_region_ms": ms}
    if wl.bound == "hbm":
        peak, key = peaks["hbm_gbs"], "hbm_gbs"
    else:
        # A timed region of milliseconds is a burst measurement: the clocks have not yet settled under the power
        # cap, so it is compared with the burst peak; a region of seconds with the sustained peak. Both
        # fractions are given, `frac` is the one that belongs to this region.
        burst, sustained = peaks["bf16_tflops"], peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
        long_region = ms * 1e-3 >= SUSTAINED_SECONDS
        peak, key = (sustained, "bf16_tflops_sustained") if long_region else (burst, "bf16_tflops")
        roofline["frac_of_burst_peak"] = per_gpu / scale / burst
        roofline["frac_of_sustained_peak"] = per_gpu / scale / sustained
        roofline["region"] = "sustained (seconds)" if long_region else "burst (milliseconds)"
    roofline["peak"] = peak
    roofline["frac"] = per_gpu / scale / peak
    roofline["peak_source"] = f"{peak_src}:{key}"
    if roofline["frac"] > 1.0:
        roofline["note"] = ("above 1.0: the peak is a plain copy (HBM) or a cuBLAS GEMM (tensor) measured on this pool, "
                            "which a read-mostly kernel or a fused epilogue can exceed")
    t = ncu_traffic(wl.profile, wl.units)
    roofline["traffic"] = t["bytes"] if t else None
    roofline["traffic_source"] = t["source"] if t else None
    return ms, per_gpu * world / scale, roofline


def sustained_tensor(wl, peaks, world, dev) -> dict:
    """The contraction back to back for SUSTAINED_SECONDS, against the sustained tensor peak."""
    one = timed(wl.step, 3, 1, world, dev) / 3
    n = max(10, int(SUSTAINED_SECONDS * 1.1 * 1e3 / one))
    ms = timed(wl.step, n, 0, world, dev)
    ach = wl.work() * n / (ms * 1e-3) / 1e12
    sustained = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]
    return {"launches": n, "seconds": ms * 1e-3, "achieved": ach, "unit": "TFLOP/s", "peak": sustained,
            "frac": ach / sustained, "peak_key": "bf16_tflops_sustained"}


def measure_e2e(wl, steps, world, dev) -> dict:
    """The same operator with pinned HOST buffers through the library's pipeline: every step uploads its inputs
    and downloads its result inside the timed region; steps follow each other without a join, one join before
    the closing event."""
    wl.host_setup()
    # a small problem (C1 moves 16 MiB per step) gets as many steps as move 1 GiB: ten of them are a 3 ms region that
    # mostly measures how the copy engines start up
    steps = max(steps, min(200, -(-(1 << 30) // max(1, wl.h2d + wl.d2h))))
    # untimed: 0.1 s of the same steps. The phases before this one leave the GPU idle for seconds (parity checks and
    # the CPU baseline run on the host) and the first copies after that run well below the link's rate.
    t0 = time.perf_counter()
    while time.perf_counter() - t0 < 0.1:
        wl.e2e_step()
        wl.e2e_join()
        torch.cuda.synchronize()
    ms = timed(wl.e2e_step, steps, 3, world, dev, after=wl.e2e_join)
    return {"value": wl.e2e_work() * steps * world / (ms * 1e-3) / scale_of(wl), "unit": wl.unit,
            "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "steps": steps, "ms_per_step": ms / steps,
            "copy_gbs": (wl.h2d + wl.d2h) * steps * world / (ms * 1e-3) / 1e9,
            "how": "tcab_pipeline_run (C ABI): pinned host buffers; upload, kernel and download pipelined over "
                   f"{wl.chunks} chunks of the independent axis on three streams, steps back to back, one join before "
                   "the closing event"}


def measure_cpu(wl, oracle, seconds: float) -> dict:
    fn, work, sample = wl.cpu_sample(oracle)
    fn()  # untimed: starts the oracle's worker threads and pages the sample in
    passes, t0 = 0, time.perf_counter()
    while passes < 2 or time.perf_counter() - t0 < seconds:
        fn()
        passes += 1
    dt = time.perf_counter() - t0
    cores = 1 if "one thread" in sample else oracle.num_threads()
    return {"value": work * passes / dt / scale_of(wl), "unit": wl.unit, "cores": cores, "kind": "port",
            "sample": f"{sample}, {passes} passes", "seconds": dt}


def copy_ceiling(world: int, dev, mib: int = 256, reps: int = 6) -> dict:
    """Bare copies between pinned host memory and the device on every rank at once: one cudaMemcpyAsync per
    direction and repetition, a stream per direction. `value` is both directions together (what a workload
    with as much output as input can reach at most), `h2d_only` the upload direction alone (the ceiling of a
    reduction, whose output is small). The host-buffer path cannot beat these."""
    n = mib << 20
    h_up = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_dn = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_up = torch.empty(n, dtype=torch.uint8, device=dev)
    d_dn = torch.empty(n, dtype=torch.uint8, device=dev)
    s_up, s_dn = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def run(down: bool) -> float:
        def once():
            with torch.cuda.stream(s_up):
                d_up.copy_(h_up, non_blocking=True)
            if down:
                with torch.cuda.stream(s_dn):
                    h_dn.copy_(d_dn, non_blocking=True)

        def join():
            cur = torch.cuda.current_stream(dev)
            cur.wait_stream(s_up)
            cur.wait_stream(s_dn)

        t0 = time.perf_counter()   # untimed: 0.1 s of the same copies (measure_e2e warms up the same way)
        while time.perf_counter() - t0 < 0.1:
            once()
            join()
            torch.cuda.synchronize()
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        cur = torch.cuda.current_stream(dev)
        s_up.wait_stream(cur)
        s_dn.wait_stream(cur)
        for _ in range(reps):
            once()
        join()
        e1.record()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world, dev)

    both, up = run(True), run(False)
    return {"value": 2.0 * n * reps * world / (both * 1e-3) / 1e9, "unit": "GB/s (both directions, all ranks)",
            "h2d_only": 1.0 * n * reps * world / (up * 1e-3) / 1e9, "mib_per_direction": mib, "reps": reps}


def frac_of_ceiling(e2e: dict, ceiling: dict):
    """An end-to-end rate against the copy ceiling that applies to it: both directions when the step downloads at
    least a quarter of what it uploads, the upload direction alone otherwise."""
    up, dn = e2e["h2d_bytes_per_step"], e2e["d2h_bytes_per_step"]
    key = "value" if dn * 4 >= up else "h2d_only"
    c = ceiling.get(key)
    return {"frac_of_copy_ceiling": e2e["copy_gbs"] / c if c else None,
            "copy_ceiling_used": "both directions" if key == "value" else "upload only"}


def sharded_axis_check(rank: int, world: int, dev, oracle) -> str:
    """One reduction ALONG a sharded axis (each rank holds a block of k; three small NCCL collectives combine the
    partial sum / max / argmax), against the oracle. Outside every timed region."""
    from tcacomp_b200.shard import block
    from tcacomp_b200.sharded import reduce_outer_sharded_k
    rng = np.random.default_rng(77)                       # the same tensor on every rank
    t = rng.uniform(-100, 100, (8, 600, 260)).astype(np.float32)
    t[0, 10, :] = 500.0
    t[0, 590, :] = 500.0                                   # a tie between the first and the last shard
    lo, hi = block(t.shape[1], world, rank)
    res = reduce_outer_sharded_k(torch.from_numpy(np.ascontiguousarray(t[:, lo:hi])).to(dev), lo)
    torch.cuda.synchronize()
    s, m, a = oracle.reduce_outer(t)
    ok = (np.array_equal(res["argmax"].cpu().numpy(), a) and np.array_equal(res["max"].cpu().numpy(), m)
          and bool((np.abs(res["sum"].cpu().numpy() - s) <= 1e-5 * np.abs(t).sum(1)).all()))
    flag = torch.tensor([1 if ok else 0], device=dev)
    torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
    return "ok" if int(flag.item()) == 1 else "MISMATCH"


def run_workload(cls, args, rank, world, dev, peaks, peak_src, oracle, headline: bool, sampler=None) -> dict:
    """Everything one workload reports. The headline workload is timed for args.steps with clocks sampled; the
    others for fewer steps."""
    import tcacomp_b200 as T
    units = args.units if (args.units and headline) else None
    wl = cls(units)
    wl.make(dev, seed=(1234 if headline else 99) + rank)
    wl.step()
    torch.cuda.synchronize()
    # correctness of what is about to be timed: every output element on a single GPU; with several ranks on one
    # host the check is sampled (eight full checks at once would only measure the host)
    parity = wl.check(oracle, full=not args.quick_check and world == 1)
    steps = args.steps if headline else max(3, min(args.steps, 10))
    out = {"workload": wl.name, "unit": wl.unit, "dtype": wl.dtype, "metric": wl.metric, "shape": wl.shape}
    t_load0 = time.perf_counter()
    if headline:
        for _ in range(args.warmup):
            wl.step()
        # keep the GPU under the same load for a moment before timing, so that the clocks have settled
        # and the sampler sees them under load even when the timed region lasts a few milliseconds
        while time.perf_counter() - t_load0 < args.preload_ms * 1e-3:
            for _ in range(8):
                wl.step()
            torch.cuda.synchronize()
    n0 = T.launch_count()
    ms, value, roofline = measure(wl, steps, 0 if headline else 3, world, dev, peaks, peak_src)
    launches = T.launch_count() - n0
    if hasattr(wl, "graph_batched"):  # launches replayed from a CUDA graph do not pass through the library's counter
        launches = steps * wl.launches_per_step
    roofline["step_ms"] = per_step_ms(wl.step, max(20, steps) if headline else steps)
    if sampler is not None:
        out["clocks"] = sampler.stop(t_load0, time.perf_counter())
    if wl.bound == "tensor" and not args.no_sustained:
        roofline["sustained"] = sustained_tensor(wl, peaks, world, dev)
    if hasattr(wl, "step_one_launch_each"):
        n = max(steps, 20)
        g_ms = timed(wl.step_one_launch_each, n, 3, world, dev)
        per = wl.work() / wl.copies
        roofline["one_launch_each"] = {
            "what": "the same 16 problems as 16 dependent launches on one stream, replayed from a CUDA graph (programmatic "
                    "dependent launch, L2 prefetch before the dependency wait, 1024-thread CTAs)",
            "us_per_launch": g_ms * 1e3 / (n * wl.copies), "achieved": wl.work() * n / (g_ms * 1e-3) / 1e9, "unit": "GB/s",
            "frac": wl.work() * n / (g_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "hbm_time_us": per / (peaks["hbm_gbs"] * 1e9) * 1e6,
            "floor": "an EMPTY grid costs 0.8 us per dependent launch in such a graph with 148 CTAs of 1024 threads and 1.7 us "
                     "with 1024 CTAs of 128 (measured on this pool); the same kernel without the dependency wait runs "
                     "2.5-2.8 us per launch (0.94-1.04)"}
    if hasattr(wl, "step_as_specified"):
        # single ordinary launches on one L2-resident buffer: what the configuration says, beside the graph figure
        a_ms = timed(wl.step_as_specified, max(steps, 50), 5, world, dev)
        n = max(steps, 50)
        per = wl.work() / wl.copies
        roofline["as_specified"] = {
            "what": "one [4096, 1024] buffer (L2-resident after the first step), one ordinary launch per step (one "
                    "tcab_chain_reduce call over descriptors built once), no CUDA graph",
            "ms_per_launch": a_ms / n, "achieved": per * n / (a_ms * 1e-3) / 1e9, "unit": "GB/s (L2-resident: not an HBM figure)",
            "frac_of_hbm_peak": per * n / (a_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    out.update({"value": value, "ms_per_step": ms / steps, "steps": steps, "roofline": roofline, "parity": parity,
                "gpu_launches": int(launches)})
    e2e_steps = max(2, min(steps, 10))
    out["e2e"] = measure_e2e(wl, e2e_steps, world, dev)
    if rank == 0 and world == 1 and args.cpu_seconds > 0:
        out["cpu_baseline"] = measure_cpu(wl, oracle, args.cpu_seconds if headline else min(args.cpu_seconds, 1.5))
    else:
        out["cpu_baseline"] = None
    wl.close()
    del wl
    torch.cuda.empty_cache()
    return out


def run_strong(cls, args, rank, world, dev, oracle, weak_value: float) -> dict:
    """The SAME global configuration cut over the ranks: rank r takes shard.block(units, world, r) of the
    independent axis (replicated operands copied to every GPU before timing); no collective."""
    from tcacomp_b200.shard import block
    lo, hi = block(cls.full_units, world, rank)
    wl = cls(hi - lo)
    wl.make(dev, seed=4321 + rank)
    wl.step()
    torch.cuda.synchronize()
    wl.check(oracle, full=False)
    steps = max(3, min(args.steps, 10))
    ms = timed(wl.step, steps, 3, world, dev)
    total = cls(cls.full_units).work()                      # the whole configuration, done once per step by all ranks
    value = total * steps / (ms * 1e-3) / scale_of(wl)
    barrier(world)
    e2e = measure_e2e(wl, max(2, min(steps, 10)), 1, dev)   # timed per rank; the slowest rank counts, the work is the global one
    e2e_ms = max_over_ranks(e2e["ms_per_step"], world, dev)
    e2e_value = cls(cls.full_units).e2e_work() / (e2e_ms * 1e-3) / scale_of(wl)
    wl.close()
    del wl
    torch.cuda.empty_cache()
    return {"workload": cls.name, "units_per_gpu": hi - lo, "value": value, "unit": cls.unit, "ms_per_step": ms / steps,
            "e2e": e2e_value, "e2e_ms_per_step": e2e_ms,
            "efficiency": value / weak_value if weak_value else None,
            "efficiency_is": "strong value / weak value of this run: 1.0 when a GPU is as fast on 1/N of the problem as on all of it"}


def run_ours(args) -> dict:
    rank, local_rank, world = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path (use --impl reference)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NVLS off: the only collectives here are barriers, scalar reductions and the sharded-axis check
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.distributed.init_process_group("nccl", device_id=dev)
    from oracle import binding as oracle  # checker and CPU baseline only

    peaks, peak_src = load_peaks()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    head = run_workload(SELECTABLE[args.workload], args, rank, world, dev, peaks, peak_src, oracle, True,
                        sampler if rank == 0 else None)

    others = []
    if not args.no_others:
        for oname, cls in WORKLOADS.items():
            if oname == head["workload"]:
                continue
            try:
                others.append(run_workload(cls, args, rank, world, dev, peaks, peak_src, oracle, False))
            except Exception as exc:  # a workload this build cannot run is reported, not hidden
                others.append({"workload": oname, "error": f"{type(exc).__name__}: {exc}"[:300]})
            torch.cuda.empty_cache()

    extra = {}
    if not args.no_others:
        extra["copy_ceiling"] = copy_ceiling(world, dev)
        head["e2e"].update(frac_of_ceiling(head["e2e"], extra["copy_ceiling"]))
        for o in others:
            if "e2e" in o:
                o["e2e"].update(frac_of_ceiling(o["e2e"], extra["copy_ceiling"]))
    if world > 1:
        extra["sharded_axis_check"] = sharded_axis_check(rank, world, dev, oracle)
        strong = []
        weak = {head["workload"]: head["value"], **{o["workload"]: o.get("value") for o in others}}
        for name, cls in ([(head["workload"], SELECTABLE[head["workload"]])] +
                          ([] if args.no_others else [(n, c) for n, c in WORKLOADS.items() if n != head["workload"]])):
            try:
                strong.append(run_strong(cls, args, rank, world, dev, oracle, weak.get(name)))
            except Exception as exc:
                strong.append({"workload": name, "error": f"{type(exc).__name__}: {exc}"[:300]})
        extra["strong"] = strong[0]
        extra["strong_others"] = strong[1:]
        extra["strong"]["limiter"] = ("kernel-only: the per-GPU share of the problem shrinks with N, so launch latency and the "
                                      "kernel's ramp and tail weigh more; end to end: the host's memory and PCIe root shared by "
                                      "all ranks (see copy_ceiling)")
    if world > 1:
        torch.distributed.destroy_process_group()
    line = {
        "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic (seeded torch.Generator per rank)",
        "config": {"workload": head["workload"], "shape": head["shape"],
                   "per_gpu_batch": "the full configuration on every rank" if not args.units else f"{args.units} units (reduced)",
                   "parallelism": f"rows sharded over {world} GPU(s), no collective",
                   "l2": "working set larger than the 126 MB L2; no flush between steps"},
        "roofline": head["roofline"], "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"],
        "gpu_launches": head["gpu_launches"], "parity": head["parity"], "clocks": head.get("clocks"),
        "other_workloads": others,
    }
    line.update(extra)
    return line


def run_reference(args) -> dict | None:
    """The reference's CPU path (the oracle port) on the host cores; rank 0 only."""
    rank, _, world = dist_env()
    if rank != 0:
        return None
    from oracle import binding as oracle
    cls = SELECTABLE[args.workload]
    scale = 1e9 if cls.bound == "hbm" else 1e12
    rng = np.random.default_rng(1234)
    cores = oracle.num_threads()
    if issubclass(cls, SoftmaxRows):
        rows = cls.full_units
        x = (4 * rng.standard_normal((rows, cls.cols), dtype=np.float32))
        fn, work = (lambda: oracle.softmax_rows(x)), 2.0 * rows * cls.cols * 4
        sample = f"all {rows} rows per step"
    elif cls is LayernormRows:
        rows = 2048
        x = oracle.f32_to_bf16(rng.standard_normal((rows, cls.cols), dtype=np.float32))
        g = oracle.f32_to_bf16(np.ones(cls.cols, np.float32))
        b = oracle.f32_to_bf16(np.zeros(cls.cols, np.float32))
        fn, work = (lambda: oracle.layernorm_rows_bf16(x, g, b, 1e-5)), 2.0 * rows * cls.cols * 2
        sample = f"{rows} of {cls.full_units} rows per step"
    elif cls is ReduceOuter:
        nb = 8
        t = rng.uniform(-100, 100, (nb, cls.nk, cls.nc)).astype(np.float32)
        fn, work = (lambda: oracle.reduce_outer(t)), nb * cls.nk * cls.nc * 4.0 + 3.0 * nb * cls.nc * 4
        sample = f"{nb} of {cls.full_units} batches per step"
    elif cls is MapRowsum:
        x = rng.uniform(-1, 1, (cls.full_units, cls.cols)).astype(np.float32)
        fn, work = (lambda: oracle.map_rowsum_affine_sq(x)), cls.full_units * cls.cols * 4.0 + cls.full_units * 4
        sample = "the full [4096, 1024] input per step"
    elif cls is MapOnly:
        from oracle import lambda_eval
        x = rng.uniform(-1, 1, (4096, cls.cols)).astype(np.float32)
        fn, work = (lambda: lambda_eval.evaluate(cls.EXPR, [x])), 2.0 * x.size * 4
        sample, cores = f"4096 of {cls.full_units} rows per step, one thread", 1
    else:
        rows = 16
        sc = 1.0 / np.sqrt(cls.k)
        a = oracle.f32_to_bf16((rng.standard_normal((rows, cls.k), dtype=np.float32) * sc))
        b = oracle.f32_to_bf16((rng.standard_normal((cls.k, cls.n), dtype=np.float32) * sc))
        bias = (rng.standard_normal(cls.n, dtype=np.float32) * 0.02)
        fn, work = (lambda: oracle.gemm_bias_act_bf16(a, b, bias, "relu")), 2.0 * rows * cls.n * cls.k
        sample = f"{rows} of {cls.full_units} rows of a (all of b) per step"
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = time.perf_counter() - t0
    value = work * args.steps / dt / scale
    cpu = {"value": value, "unit": cls.unit, "cores": cores, "kind": "port", "sample": sample}
    return {
        "impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cls.dtype,
        "data": "synthetic (seeded numpy Generator)",
        "config": {"workload": cls.name, "shape": cls.shape,
                   "per_gpu_batch": "CPU restatement of the reference's naive fp32 loops (the reference is Go and cannot "
                                    "be built in this image); a bounded sample per step, see cpu_baseline.sample",
                   "parallelism": f"{cores} host thread(s), rank 0 only",
                   "l2": "not applicable (host)"},
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
    ap.add_argument("--no-others", action="store_true",
                    help="only the headline workload: no other workloads, no copy ceiling, no strong-scaling legs of the others")
    ap.add_argument("--cpu-seconds", type=float, default=10.0,
                    help="how long the headline's CPU baseline leg repeats its sample (the others: at most 1.5 s)")
    ap.add_argument("--preload-ms", type=float, default=300.0,
                    help="untimed load before the timed region so that the clocks settle (0 for profiler runs)")
    ap.add_argument("--units", type=int, default=0,
                    help="profiler runs: build the headline workload with this many units of its independent axis")
    ap.add_argument("--quick-check", action="store_true", help="profiler runs: sampled instead of full pre-timing parity")
    ap.add_argument("--no-sustained", action="store_true", help="profiler runs: skip the seconds-long contraction loop")
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
