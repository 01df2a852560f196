#!/usr/bin/env python
"""Benchmark of the RMSNorm hot path (and, as side results, the SwiGLU MLP) on B200.

    python bench.py --gpus N --steps K --warmup W            # this library (default N=1)
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path, host cores
    torchrun --nproc-per-node N ... bench.py --gpus N ...    # N > 1: one rank per GPU

A step is one RMSNorm forward + backward over one batch: bf16, 65536 rows x hidden 8192 IN TOTAL
(x ~ N(0,2), w = 1 + 0.1 N(0,1), dy ~ N(0,1), eps 1e-6, seeded). With N > 1 the rows are split into N
contiguous blocks, one per rank (strong scaling: the job is fixed), and the fp32 dW partial is all-reduced
over NCCL each step, then rounded once. The metric is algorithmic bytes per second: every rank's
5*R*H*s + 3*H*s + 8*R bytes, summed over the ranks, divided by the slowest rank's time.

Rank 0 prints ONE JSON line. `value` is timed with inputs resident in HBM; `e2e` goes through the
library's host-tensor entry with pinned host buffers and host<->device copies inside the timed region.
The same line carries, as compact keys, the other half of the metric -- `block`: the bf16 pre-norm block
RMSNorm(8192) -> SwiGLU(d_ff 28672) over 16384 tokens, tensor-parallel over the N ranks (TFLOP/s); `mlp`
(N = 1): the fp16 SwiGLU MLP of d_model 4096 -- and, for N > 1, `parity_n`: sharded results checked
against the one-rank result on the spot, `weak`: the 65536-rows-per-GPU figure, and `allreduce`: what the
latency-bound dW collective costs on the compute stream and beside the next forward.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch

METRIC = "RMSNorm fwd+bwd GB/s"
UNIT = "GB/s"
TOTAL_ROWS = 65536       # the benchmark's batch; split over the ranks
ROWS_PER_GPU = 65536     # the weak-scaling side figure keeps this many rows on every GPU
HIDDEN = 8192
EPS = 1e-6
SEED = 1234
CPU_SAMPLE_ROWS = 4096
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per algorithmic byte of one backward launch,
# from the ncu capture summarised in profiles/rmsnorm_bf16_h8192_reg_kernels.txt: 16384 rows x 8192 bf16,
# 537.0 MB read + 235.7 MB written against 805.4 MB algorithmic. Traffic grows in proportion to the rows,
# so the full-size figure is this ratio times the full launch's algorithmic bytes.
def _traffic_per_algorithmic_byte():
    """Read from the committed ncu summary (the figures of the capture, not a copy of them); None when it is not there."""
    import re
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles", "rmsnorm_bf16_h8192_reg_kernels.txt")
    try:
        text = open(path).read()
        block = text.split("kernel: rms_bwd_reg<__nv_bfloat16, 256, 4, 0>")[1].split("kernel:")[0]
        rd = float(re.search(r"dram__bytes_read\.sum\s+([0-9.]+) Mbyte", block).group(1))
        wr = float(re.search(r"dram__bytes_write\.sum\s+([0-9.]+) Mbyte", block).group(1))
        rows = int(re.search(r"one launch each, (\d+) rows x 8192 bf16", text).group(1))
    except (OSError, IndexError, AttributeError, ValueError):
        return None
    algorithmic = 3 * rows * 8192 * 2 + 2 * 8192 * 2 + 4 * rows
    return (rd + wr) * 1e6 / algorithmic


TRAFFIC_PER_ALGO_BYTE = _traffic_per_algorithmic_byte()


def rms_bytes(rows: int, cols: int, s: int) -> dict:
    fwd = 2 * rows * cols * s + cols * s + 4 * rows
    bwd = 3 * rows * cols * s + 2 * cols * s + 4 * rows
    return {"fwd": fwd, "bwd": bwd, "total": fwd + bwd}


def measured_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------------------------------
# clocks during the timed region (read-only NVML queries)
# ---------------------------------------------------------------------------------------------------

class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, device_index: int, period_s: float = 0.005):
        self.period = period_s
        self.samples: list[tuple[float, int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            h = None
            try:
                uuid = str(torch.cuda.get_device_properties(device_index).uuid)
                if not uuid.startswith("GPU-"):
                    uuid = "GPU-" + uuid
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                h = None
            if h is None:
                vis = os.environ.get("CUDA_VISIBLE_DEVICES")
                idx = device_index
                if vis:
                    ent = vis.split(",")[device_index].strip()
                    idx = int(ent) if ent.isdigit() else device_index
                h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self._h = h
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _reasons(self) -> int:
        nv = self._nv
        for name in ("nvmlDeviceGetCurrentClocksEventReasons", "nvmlDeviceGetCurrentClocksThrottleReasons"):
            fn = getattr(nv, name, None)
            if fn is not None:
                try:
                    return int(fn(self._h))
                except Exception:
                    continue
        return 0

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.samples.append((time.perf_counter(), mhz, self._reasons()))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, t0: float, t1: float) -> dict:
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0,
                    "note": "no NVML sample fell inside the timed region"}
        bits = 0
        for s in inside:
            bits |= s[2]
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        return {"sm_mhz": int(statistics.median(s[1] for s in inside)), "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(inside)}


# ---------------------------------------------------------------------------------------------------
# the reference's CPU path (torch formula on the host cores), used by both arms
# ---------------------------------------------------------------------------------------------------

def cpu_sample_inputs(rows: int, cols: int):
    g = torch.Generator().manual_seed(SEED)
    x = (2.0 ** 0.5 * torch.randn(rows, cols, generator=g)).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(torch.bfloat16)
    dy = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
    return x, w, dy


def cpu_step(x, w, dy):
    """One forward+backward of the reference formula on bf16 host tensors: fp32 math (the reference's
    kernels accumulate in fp32), results rounded back to bf16."""
    from oracle import oracle

    y, dx, dw = oracle.rmsnorm_formula_torch(x.float(), w.float(), EPS, dy.float())
    return y.to(torch.bfloat16), dx.to(torch.bfloat16), dw.to(torch.bfloat16)


def time_cpu(steps: int, warmup: int, budget_s: float | None = None) -> dict:
    x, w, dy = cpu_sample_inputs(CPU_SAMPLE_ROWS, HIDDEN)
    for _ in range(warmup):
        cpu_step(x, w, dy)
    times = []
    t_begin = time.perf_counter()
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_step(x, w, dy)
        times.append(time.perf_counter() - t0)
        if budget_s is not None and time.perf_counter() - t_begin > budget_s:
            break
    per_step = sum(times) / len(times)
    nbytes = rms_bytes(CPU_SAMPLE_ROWS, HIDDEN, 2)["total"]
    return {"value": nbytes / per_step / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"torch formula fwd+bwd (fp32 math on bf16 tensors) on {CPU_SAMPLE_ROWS} of the {TOTAL_ROWS} rows x {HIDDEN} per step "
                      f"(1/{TOTAL_ROWS // CPU_SAMPLE_ROWS} of the workload), {len(times)} steps, bytes counted as for the GPU arm (2 B/element)",
            "ms_per_step": per_step * 1e3, "steps": len(times), "os_cpu_count": os.cpu_count()}


def reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # torchrun exports OMP_NUM_THREADS=1 to every rank; the CPU arm is meant to use all the host cores
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    res = time_cpu(args.steps, max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": res["steps"], "warmup": max(args.warmup, 1), "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(args.gpus), cpu_sample_rows_per_step=CPU_SAMPLE_ROWS,
                       cpu_sample=f"each CPU step covers {CPU_SAMPLE_ROWS} of the {TOTAL_ROWS} rows; one host process, whatever --gpus says"),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(n_gpus: int, rows: int = TOTAL_ROWS) -> dict:
    per = -(-rows // n_gpus)
    return {"workload": f"RMSNorm bf16 forward+backward, {rows} rows x hidden {HIDDEN} in total, eps 1e-6 "
                        "(x~N(0,2), w=1+0.1N(0,1), dy~N(0,1))" + ("" if rows == TOTAL_ROWS else " [REDUCED CASE, not the benchmark]"),
            "rows_total": rows, "rows_per_gpu": per, "hidden": HIDDEN,
            "sharding": (f"contiguous row blocks over {n_gpus} ranks, fp32 dW summed across the ranks every step, "
                         "one rounding after it") if n_gpus > 1 else "none",
            "l2": f"inputs larger than L2 ({per * HIDDEN * 2 >> 20} MiB per tensor and GPU, four tensors per step, 126 MB L2)", "seed": SEED}


# ---------------------------------------------------------------------------------------------------
# this library
# ---------------------------------------------------------------------------------------------------

def make_inputs(rows: int, cols: int, dtype, device, seed: int, x_scale: float):
    g = torch.Generator(device=device).manual_seed(seed)
    x = (x_scale * torch.randn(rows, cols, generator=g, device=device)).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g, device=device)).to(dtype)
    dy = torch.randn(rows, cols, generator=g, device=device).to(dtype)
    return x, w, dy


class RmsBuffers:
    """Pre-allocated device tensors for one problem; launches go straight to the C ABI."""

    def __init__(self, L, rows, cols, dtype, device, seed, x_scale=1.0):
        from mgrrmsnorm_b200 import rmsnorm_cuda_ops as ops

        self.L, self.rows, self.cols = L, rows, cols
        self.code = ops._DTYPES[dtype]
        self.x, self.w, self.dy = make_inputs(rows, cols, dtype, device, seed, x_scale)
        self.y = torch.empty_like(self.x)
        self.dx = torch.empty_like(self.x)
        self.inv = torch.empty(rows, dtype=torch.float32, device=device)
        self.dw = torch.empty_like(self.w)
        self.dw32 = torch.empty(cols, dtype=torch.float32, device=device)
        nws = int(L.mgr_rmsnorm_bwd_workspace_bytes(rows, cols, self.code))
        self.ws = torch.empty(max(nws, 16), dtype=torch.uint8, device=device)
        self._fwd_args = self._bwd_args = None
        self.dw_pairs = [(self.dw32, self.dw)]

    def second_dw_pair(self):
        """A second (dw_f32, dw) output pair, used alternately with the first when the cross-rank sum of dW runs off
        the compute stream: the backward of step i+1 then writes other buffers than the ones step i's all-reduce
        still reads, as the backward passes of two different layers (or micro-batches) do in a training loop."""
        if len(self.dw_pairs) == 1:
            self.dw_pairs.append((torch.empty_like(self.dw32), torch.empty_like(self.dw)))
            self._fwd_args = None

    def _pointers(self):
        # device addresses looked up once per buffer set (they are re-read if a tensor is swapped): a 10 us kernel
        # does not wait for seven data_ptr() calls per launch
        key = tuple(t.data_ptr() for t in (self.y, self.inv, self.x, self.w, self.dx, self.dw, self.dw32, self.dy, self.ws))
        if self._fwd_args is None or self._key != key:
            y, inv, x, w, dx, dw, dw32, dy, ws = key
            self._key = key
            self._fwd_args = (y, inv, x, w, self.rows, self.cols, EPS, self.code)
            self._bwd_args = (dx, dw, dw32, dy, x, w, inv, self.rows, self.cols, self.code, ws, self.ws.numel())
            self._bwd_args_alt = None
            if len(self.dw_pairs) > 1:
                d32, d = self.dw_pairs[1]
                self._bwd_args_alt = (dx, d.data_ptr(), d32.data_ptr(), dy, x, w, inv, self.rows, self.cols, self.code, ws, self.ws.numel())

    def freeze(self):
        """Fixes the argument lists (call after any tensor of the set has been replaced)."""
        self._fwd_args = None
        self._pointers()

    def fwd(self, stream):
        if self._fwd_args is None:
            self._pointers()
        st = self.L.mgr_rmsnorm_fwd(*self._fwd_args, stream)
        if st:
            raise RuntimeError(f"mgr_rmsnorm_fwd status {st}")

    def bwd(self, stream, pair=0):
        if self._bwd_args is None or self._fwd_args is None:
            self._pointers()
        st = self.L.mgr_rmsnorm_bwd(*(self._bwd_args if pair == 0 else self._bwd_args_alt), stream)
        if st:
            raise RuntimeError(f"mgr_rmsnorm_bwd status {st}")


def time_device_resident(bufsets, steps, warmup, world, sampler=None, reduce="side", per_kernel_events=True, peer=None):
    """K steps over `bufsets` (rotated), CUDA events on the launching stream. Returns total ms, mean
    fwd-call ms, mean bwd-call ms and the wall-clock window of the timed region."""
    import torch.distributed as dist

    stream = torch.cuda.current_stream()
    sp = stream.cuda_stream
    # N > 1, reduce="side": the all-reduce of the fp32 dW partial (32 KB, latency-bound) and the one rounding after
    # it run on a side stream, beside the NEXT step's forward, as in a training loop where dW is not needed before
    # the optimizer step. The next backward that overwrites the same dW buffer waits for it, and so does the end of
    # the timed region, so every step's collective completes inside the region it is timed in.
    # (mgrrmsnorm_b200.sharding.AsyncDwReduce is the library's helper for exactly this.)
    # reduce="inline": the same all-reduce and rounding on the compute stream, right after the backward
    # (sharding.allreduce_dw), so its whole latency is exposed.
    # reduce="peer": the sum as ONE kernel per rank over NVLink peer memory (sharding.PeerDwAllReduce,
    # mgr_peer_allreduce_f32) on the compute stream right after the backward: a few microseconds where the NCCL
    # collective takes 18 (2-4 GPUs) to 55 (8 GPUs).
    # reduce="peer_side": that kernel on the (high-priority) side stream, beside the next forward.
    red = None
    inline = world > 1 and reduce == "inline"
    use_peer = world > 1 and reduce == "peer" and peer is not None
    if world > 1 and reduce in ("side", "peer_side"):
        from mgrrmsnorm_b200.sharding import AsyncDwReduce

        red = AsyncDwReduce(torch.cuda.current_device(), peer=peer if reduce == "peer_side" else None)
        for b in bufsets:
            b.second_dw_pair()
    turn = [0]

    def step(b, evs=None):
        if evs:
            evs[0].record(stream)
        b.fwd(sp)
        if evs:
            evs[1].record(stream)
        pair = 0
        if red is not None:
            # two output pairs used alternately: this backward only waits for the all-reduce of TWO steps ago (the
            # persistent forward kernel fills every SM, so the collective of the previous step may still be queued
            # behind it; waiting for it here would put its latency back between forward and backward)
            pair = turn[0] & 1
            turn[0] += 1
            red.wait_for(b.dw_pairs[pair][0])
        b.bwd(sp, pair)
        if evs:
            evs[2].record(stream)
        if red is not None:
            red.start(*b.dw_pairs[pair])
        elif use_peer:
            peer(b.dw32, b.dw)                       # fp32 sum over the ranks in rank order, one rounding
        elif inline:
            dist.all_reduce(b.dw32, op=dist.ReduceOp.SUM)
            b.dw.copy_(b.dw32)                       # the single rounding

    def drain():
        if red is not None:
            red.drain()

    for i in range(warmup):
        step(bufsets[i % len(bufsets)])
    drain()
    # Per-kernel events on every step when a step is long (one GPU: 0.8 ms), on every 8th when the rows are split over
    # several ranks: three event records cost a few microseconds, which is 5 % of a 125 us step at 8 ranks and would
    # be charged to the headline. The forward / backward means are then taken over the sampled steps.
    every = 1 if world == 1 else 8
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] if per_kernel_events and i % every == 0 else None for i in range(steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(stream)
    for i in range(steps):
        step(bufsets[i % len(bufsets)], evs[i])
    drain()
    e1.record(stream)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if world > 1:
        dist.barrier()
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    timed = [e for e in evs if e is not None]
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in timed) / len(timed) if timed else None
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in timed) / len(timed) if timed else None
    return {"total_ms": total_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "window": (t0, t1)}


def time_e2e(rows, cols, device, steps, warmup, world, src, pipelined=True):
    """Through the public API with pinned host buffers: every step copies x and dy host->device, runs
    forward and backward, and copies y, dx and dW back. pipelined=True uses the library's host-tensor
    entry (HostRMSNormPipeline: row chunks over three streams, inbound and outbound copies overlapped);
    pipelined=False is the plain module call between two whole-tensor copies."""
    import torch.distributed as dist

    from mgrrmsnorm_b200 import RMSNorm
    from mgrrmsnorm_b200.hostpipe import HostRMSNormPipeline

    dt = torch.bfloat16
    hx = torch.empty((rows, cols), dtype=dt).pin_memory()
    hdy = torch.empty((rows, cols), dtype=dt).pin_memory()
    hy = torch.empty((rows, cols), dtype=dt).pin_memory()
    hdx = torch.empty((rows, cols), dtype=dt).pin_memory()
    hdw = torch.empty((cols,), dtype=dt).pin_memory()
    hx.copy_(src.x)
    hdy.copy_(src.dy)
    from mgrrmsnorm_b200.sharding import RowShardedRMSNorm

    norm = (RowShardedRMSNorm(cols, epsilon=EPS) if world > 1 else RMSNorm(cols, epsilon=EPS)).to(device).to(dt)
    with torch.no_grad():
        norm.weight.copy_(src.w)
    stream = torch.cuda.current_stream()
    pipe = HostRMSNormPipeline(rows, cols, dt, device) if pipelined else None

    from mgrrmsnorm_b200 import sharding

    def step_pipelined():
        # every rank's fp32 column sum is added across the ranks first and rounded once, as on the resident path
        dw32 = pipe.run(hx, hdy, norm.weight.detach(), EPS, hy, hdx, return_f32=True)
        dw = sharding.allreduce_dw(dw32, dt) if world > 1 else dw32.to(dt)
        hdw.copy_(dw, non_blocking=True)

    def step():
        if pipelined:
            return step_pipelined()
        x = hx.to(device, non_blocking=True).requires_grad_(True)
        dy = hdy.to(device, non_blocking=True)
        norm.weight.grad = None
        y = norm(x)                 # RowShardedRMSNorm when world > 1: its backward all-reduces the fp32 dW, then rounds
        y.backward(dy)
        dw = norm.weight.grad
        hy.copy_(y.detach(), non_blocking=True)
        hdx.copy_(x.grad, non_blocking=True)
        hdw.copy_(dw, non_blocking=True)

    for _ in range(warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    es = 2
    return {"ms_per_step": ms / steps, "steps": steps, "h2d": 2 * rows * cols * es, "d2h": 2 * rows * cols * es + cols * es}


def graph_timed(sets, nb, peak_gbs, l2_note) -> dict:
    """Forward, backward and forward+backward over the rotating buffer `sets`, replayed from CUDA graphs:
    no host launch gaps, device time only (microseconds per call)."""
    stream = torch.cuda.current_stream()

    def graph_of(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            sp = torch.cuda.current_stream().cuda_stream
            for b in sets:
                fn(b, sp)
        return g

    def replay_us(g, n=50):
        for _ in range(5):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(n):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (n * len(sets))

    try:
        sp0 = stream.cuda_stream
        for b in sets:     # every first-call set-up (attributes, occupancy queries) happens before capture
            b.fwd(sp0)
            b.bwd(sp0)
        torch.cuda.synchronize()
        gf = graph_of(lambda b, sp: b.fwd(sp))
        gb = graph_of(lambda b, sp: b.bwd(sp))
        gfb = graph_of(lambda b, sp: (b.fwd(sp), b.bwd(sp)))
        # the same bytes as one forward (read x, write y) moved by a plain device copy, same protocol: what a kernel
        # of this size can reach at all (launch ramp and first-touch latency weigh more the smaller the tensor)
        gc = graph_of(lambda b, sp: b.y.copy_(b.x))
        f_us, b_us, fb_us, c_us = replay_us(gf), replay_us(gb), replay_us(gfb), replay_us(gc)
        return {"l2": l2_note, "fwd_us": f_us, "bwd_us": b_us, "us_per_step": fb_us, "copy_of_x_to_y_us": c_us,
                "fwd_time_over_copy_time": f_us / c_us,
                "GBps": nb["total"] / (fb_us * 1e-6) / 1e9,
                "fwd_frac_of_peak": nb["fwd"] / (f_us * 1e-6) / 1e9 / peak_gbs,
                "bwd_frac_of_peak": nb["bwd"] / (b_us * 1e-6) / 1e9 / peak_gbs}
    except Exception as e:   # a capture problem must not take the headline line down with it
        return {"error": str(e)[:200]}


def side_results(L, device, peak_gbs) -> dict:
    """Other configurations, N=1 only: the fp16 [4096,4096] shape the reference publishes (L2-cold by
    rotating 8 buffer sets = 1.25 GiB) and the bf16 hidden sweep at 2^29 elements."""
    out = {}
    sets = [RmsBuffers(L, 4096, 4096, torch.float16, device, SEED + i) for i in range(8)]
    r = time_device_resident(sets, 400, 40, 1)
    plain = time_device_resident(sets, 400, 40, 1, per_kernel_events=False)
    nb = rms_bytes(4096, 4096, 2)
    out["rmsnorm_fp16_4096x4096"] = {
        "l2": "cold: 8 rotating buffer sets (1.25 GiB)", "us_per_step": plain["total_ms"] * 1e3 / 400,
        "GBps": nb["total"] / (plain["total_ms"] / 400 * 1e-3) / 1e9,
        "with_an_event_between_the_kernels": {"us_per_step": r["total_ms"] * 1e3 / 400, "fwd_us": r["fwd_ms"] * 1e3, "bwd_us": r["bwd_ms"] * 1e3,
                                              "fwd_frac_of_peak": nb["fwd"] / (r["fwd_ms"] * 1e-3) / 1e9 / peak_gbs,
                                              "bwd_frac_of_peak": nb["bwd"] / (r["bwd_ms"] * 1e-3) / 1e9 / peak_gbs},
        "launch": "one C-ABI call per kernel from Python, no CUDA graph; us_per_step is timed with two events around all 400 steps "
                  "(a timing event recorded between two 10-25 us kernels costs a few microseconds of its own)"}
    out["rmsnorm_fp16_4096x4096_cuda_graph"] = graph_timed(sets, nb, peak_gbs, "cold: 8 rotating buffer sets (1.25 GiB)")
    del sets
    torch.cuda.empty_cache()
    sweep = {}
    for h in (1024, 4096, 8192, 16384):
        rows = (1 << 29) // h
        b = RmsBuffers(L, rows, h, torch.bfloat16, device, SEED, x_scale=2.0 ** 0.5)
        r = time_device_resident([b], 30, 5, 1)
        nb = rms_bytes(rows, h, 2)
        sweep[str(h)] = {"rows": rows, "ms_per_step": r["total_ms"] / 30,
                         "GBps": nb["total"] / (r["total_ms"] / 30 * 1e-3) / 1e9,
                         "fwd_frac_of_peak": nb["fwd"] / (r["fwd_ms"] * 1e-3) / 1e9 / peak_gbs,
                         "bwd_frac_of_peak": nb["bwd"] / (r["bwd_ms"] * 1e-3) / 1e9 / peak_gbs}
        del b
        torch.cuda.empty_cache()
    out["rmsnorm_bf16_hidden_sweep_2^29_elements"] = sweep
    # config 1's shape (fp32 [4096, 4096], the CPU-runnable case) on the GPU, L2-cold, graph-timed
    sets = [RmsBuffers(L, 4096, 4096, torch.float32, device, SEED + i) for i in range(4)]
    out["rmsnorm_fp32_4096x4096_cuda_graph"] = graph_timed(sets, rms_bytes(4096, 4096, 4), peak_gbs, "cold: 4 rotating buffer sets (1.25 GiB)")
    del sets
    torch.cuda.empty_cache()
    # the sweep's latency regime: ONE row block of 2^20 elements per call (rows = 2^20 / hidden), L2-cold
    lat = {}
    for h in (1024, 4096, 8192, 16384):
        rows = (1 << 20) // h
        sets = [RmsBuffers(L, rows, h, torch.bfloat16, device, SEED + i, x_scale=2.0 ** 0.5) for i in range(24)]
        r = graph_timed(sets, rms_bytes(rows, h, 2), peak_gbs, "cold: 24 rotating buffer sets (200 MB)")
        r["rows"] = rows
        lat[str(h)] = r
        del sets
        torch.cuda.empty_cache()
    out["rmsnorm_bf16_hidden_sweep_2^20_elements_latency"] = lat
    out["add_rmsnorm_bf16_65536x8192"] = add_rmsnorm_side_result(device, peak_gbs)
    out["swiglu_mlp_fp16_M4096_D4096_F6912"] = mlp_side_result(device)
    return out


def add_rmsnorm_side_result(device, peak_gbs) -> dict:
    """Residual add fused into the norm, bf16 [65536, 8192] (tensors of 1 GiB, far beyond L2): forward reads
    x, residual and writes h, y (4*R*H*s bytes); backward reads dy, dres, h and writes dh (4*R*H*s).
    Beside it the same work done the unfused way: torch add + norm forward (5 passes), norm backward +
    torch add of the two gradients (6 passes)."""
    import rmsnorm_cuda_ops as ops

    rows, cols = 65536, 8192
    g = torch.Generator(device=device).manual_seed(SEED)
    x, res, dy, dres = (torch.randn(rows, cols, device=device, generator=g).to(torch.bfloat16) for _ in range(4))
    w = (1 + 0.1 * torch.randn(cols, device=device, generator=g)).to(torch.bfloat16)
    _, h, inv = ops.add_rmsnorm_forward(x, res, w, 1e-6)
    pass_bytes = rows * cols * 2

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    def unfused_fwd():
        ops.rmsnorm_forward(x + res, w, 1e-6)

    def unfused_bwd():
        dx, _ = ops.rmsnorm_backward(dy, h, w, inv)
        dx.add_(dres)

    f_ms = timed(lambda: ops.add_rmsnorm_forward(x, res, w, 1e-6))
    b_ms = timed(lambda: ops.add_rmsnorm_backward(dy, dres, h, w, inv))
    uf_ms, ub_ms = timed(unfused_fwd), timed(unfused_bwd)
    return {"fwd_ms": f_ms, "bwd_ms": b_ms,
            "fwd_frac_of_peak": 4 * pass_bytes / (f_ms * 1e-3) / 1e9 / peak_gbs,
            "bwd_frac_of_peak": 4 * pass_bytes / (b_ms * 1e-3) / 1e9 / peak_gbs,
            "unfused_fwd_ms": uf_ms, "unfused_bwd_ms": ub_ms,
            "speedup_fwd_bwd": (uf_ms + ub_ms) / (f_ms + b_ms)}


def mlp_side_result(device) -> dict:
    """SwiGLU MLP forward+backward, fp16, x [32,128,4096], hidden 6912 (the module's default), through the
    public module on the tensor-core kernels. 18*M*D*F algorithmic flops per step (the projection that
    backward recomputes is not counted). Weights (162 MiB) and activations exceed L2 together."""
    from mgrrmsnorm_b200 import MegaGemmTriton

    peaks, _ = measured_peaks()
    torch.manual_seed(SEED)
    mlp = MegaGemmTriton(4096).to(device).half()
    g = torch.Generator(device=device).manual_seed(SEED)
    x = torch.randn(32, 128, 4096, device=device, generator=g).half().requires_grad_(True)
    dy = torch.randn(32, 128, 4096, device=device, generator=g).half()
    m, d, f = 4096, 4096, mlp.hidden

    def step():
        x.grad = None
        mlp.w12.weight.grad = None
        mlp.w3.weight.grad = None
        mlp(x).backward(dy)

    def fwd_only():
        with torch.no_grad():
            mlp(x)

    res = {}
    for name, fn, flops in (("fwd_bwd", step, 18 * m * d * f), ("fwd", fwd_only, 6 * m * d * f)):
        for _ in range(5):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 20
        res[name] = {"ms": ms, "TFLOPs": flops / ms / 1e9, "frac_of_bf16_burst_peak": flops / ms / 1e9 / float(peaks["bf16_tflops"])}
    res["hidden"] = f
    return res


MLP_TOKENS = 4096
MLP_D = 4096


def mlp_line(args, device, warmup, peaks, peak_kind, sm_count, steps=None, no_e2e=None, no_cpu=None) -> dict:
    """SwiGLU MLP forward+backward (config 4: fp16, x [32,128,4096], hidden = the module's default 6912,
    nn.Linear default init from a seed) through the public module. Returns the JSON line; the roofline entry
    is the fused projection kernel (tensor-bound), timed in its own loop of launches in the same run."""
    steps = args.steps if steps is None else steps
    no_e2e = args.no_e2e if no_e2e is None else no_e2e
    no_cpu = args.no_cpu if no_cpu is None else no_cpu
    from mgrrmsnorm_b200 import MegaGemmTriton
    from mgrrmsnorm_b200 import rmsnorm_cuda_ops as ops

    m, d = args.tokens, MLP_D
    torch.manual_seed(SEED)
    mlp = MegaGemmTriton(d).to(device).half()
    f = mlp.hidden
    g = torch.Generator(device=device).manual_seed(SEED)
    x = torch.randn(m, d, device=device, generator=g).half().requires_grad_(True)
    dy = torch.randn(m, d, device=device, generator=g).half()
    stream = torch.cuda.current_stream()

    def step():
        x.grad = None
        mlp.w12.weight.grad = None
        mlp.w3.weight.grad = None
        y = mlp(x)
        y.backward(dy)
        return y

    def timed(fn, n, w):
        for _ in range(w):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n, (t0, time.perf_counter())

    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms, window = timed(step, steps, warmup)
    sampler.stop()
    flops = 18 * m * d * f
    xd = x.detach()
    w12 = mlp.w12.weight.detach()
    k_ms, _ = timed(lambda: ops.swiglu_fused_forward(xd, w12, f), max(min(steps, 50), 20), warmup)
    k_flops = 4 * m * d * f
    peak_tf = float(peaks["bf16_tflops"])

    e2e = None
    if not no_e2e:
        hx, hdy = xd.cpu().pin_memory(), dy.cpu().pin_memory()
        hy, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()

        def e2e_step():
            xx = hx.to(device, non_blocking=True).requires_grad_(True)
            dd = hdy.to(device, non_blocking=True)
            mlp.w12.weight.grad = None
            mlp.w3.weight.grad = None
            y = mlp(xx)
            y.backward(dd)
            hy.copy_(y.detach(), non_blocking=True)
            hdx.copy_(xx.grad, non_blocking=True)

        e_ms, _ = timed(e2e_step, max(args.e2e_steps, 3), 2)
        e2e = {"value": flops / e_ms / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * m * d * 2, "d2h_bytes_per_step": 2 * m * d * 2,
               "ms_per_step": e_ms, "path": "pinned host x, dy -> MegaGemmTriton fwd+bwd -> pinned host y, dx (weight grads stay on the device)"}
    cpu = None
    if not no_cpu:
        cpu = time_cpu_mlp(mlp, f)
    reduced = m != MLP_TOKENS
    line = {
        "metric": "SwiGLU MLP TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
        "config": {"workload": f"SwiGLU MLP fp16 forward+backward, {m} tokens, d_model {d}, hidden {f} (MegaGemmTriton default), "
                               "fused SiLU(gate)*value epilogue" + (" [REDUCED CASE, not the benchmark]" if reduced else ""),
                   "tokens": m, "d_model": d, "hidden": f, "flops_per_step": flops,
                   "l2": "weights 162 MiB + activations exceed the 126 MB L2", "seed": SEED},
        "frac_of_bf16_peak": flops / ms / 1e9 / peak_tf,
        "roofline": {"bound": "tensor", "kernel": "gemm_kernel<swiglu epilogue> (mgr_swiglu_fused_fwd: x w12^T -> silu(gate)*value)",
                     "achieved": k_flops / k_ms / 1e9, "peak": peak_tf, "unit": "TFLOP/s", "frac": k_flops / k_ms / 1e9 / peak_tf,
                     "peak_source": f"of {peak_kind} (cuBLAS bf16 burst)", "algorithmic_flops_per_launch": k_flops, "avg_launch_ms": k_ms,
                     "timed": "own loop of launches in this run", "traffic": None},
        "frac_of_bf16_sustained_peak": flops / ms / 1e9 / float(peaks["bf16_tflops_sustained"]),
        "e2e": e2e, "gpu_launches": 6 * steps,
        "clocks": sampler.summary(*window), "sm_count": sm_count,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    return line


def run_mlp(args, L, device, warmup, peaks, peak_kind, sm_count) -> int:
    print(json.dumps(mlp_line(args, device, warmup, peaks, peak_kind, sm_count)), flush=True)
    return 0


BLOCK_TOKENS = 16384
BLOCK_D = 8192
BLOCK_F = 28672


def block_line(args, device, warmup, peaks, peak_kind, world, rank, steps=None):
    """Config 5: bf16 pre-norm MLP block, y = SwiGLU(RMSNorm(x)), d = 8192, d_ff = 28672, 16384 tokens.
    Tensor-parallel over the ranks: w12 split by hidden units (gate and value rows of each rank), w3 by
    columns, x and the norm replicated, one NCCL all-reduce of y in forward and one of dx in backward.
    Strong scaling: the block is fixed, each GPU does 1/P of the GEMM work. Value = 18*M*D*F / time.
    Returns the JSON line on rank 0 and None on the other ranks."""
    import torch.distributed as dist

    steps = args.steps if steps is None else steps
    from mgrrmsnorm_b200 import MegaGemmTriton, RMSNorm, sharding

    m, d, f = (args.tokens if args.tokens != MLP_TOKENS else BLOCK_TOKENS), BLOCK_D, BLOCK_F
    dt = torch.bfloat16
    f0, f1 = sharding.tp_hidden_slice(f, world, rank)
    if world == 1:
        mlp = MegaGemmTriton(d, hidden_multiple=3.5)
        assert mlp.hidden == f
        mlp = mlp.to(device).to(dt)
        local = mlp
    else:
        # MGR_TP_MODE=sp: rows sharded outside the MLP (norm on 1/P of the rows, all-gather / reduce-scatter per
        # row slab); default: replicated rows, all-reduces overlapped with GEMMs (MGR_TP_OVERLAP=0: not overlapped)
        seq_parallel = os.environ.get("MGR_TP_MODE", "ar") == "sp"
        cls = sharding.SequenceParallelSwiGLU if seq_parallel else sharding.TensorParallelSwiGLU
        mlp = cls(d, f, world, rank).to(device).to(dt)
        mlp.overlap = os.environ.get("MGR_TP_OVERLAP", "1") != "0"
        mlp.slabs = int(os.environ.get("MGR_TP_SLABS", mlp.slabs))
        local = mlp.local
    # nn.Linear's default init, U(-1/sqrt(fan_in), 1/sqrt(fan_in)), drawn on the device; fan_in of w3 is the FULL d_ff
    g = torch.Generator(device=device).manual_seed(SEED + 17 * rank)
    with torch.no_grad():
        local.w12.weight.copy_((torch.rand(local.w12.weight.shape, device=device, generator=g) * 2 - 1) / d ** 0.5)
        local.w3.weight.copy_((torch.rand(local.w3.weight.shape, device=device, generator=g) * 2 - 1) / f ** 0.5)
    seq_parallel = world > 1 and os.environ.get("MGR_TP_MODE", "ar") == "sp"
    norm =(sharding.RowShardedRMSNorm(d, epsilon=EPS) if seq_parallel else RMSNorm(d, epsilon=EPS)).to(device).to(dt)
    gx = torch.Generator(device=device).manual_seed(SEED)            # replicated input: same seed on every rank
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(d, device=device, generator=gx)).to(dt))
    x = torch.randn(m, d, device=device, generator=gx).to(dt)
    dy = torch.randn(m, d, device=device, generator=gx).to(dt)
    if seq_parallel:                                                  # this rank's row block of the same tensors
        r0, r1 = sharding.row_shard(m, world, rank)
        x, dy = x[r0:r1].clone(), dy[r0:r1].clone()
    x.requires_grad_(True)
    stream = torch.cuda.current_stream()

    def step():
        x.grad = None
        for p in list(mlp.parameters()) + [norm.weight]:
            p.grad = None
        mlp(norm(x)).backward(dy)

    for _ in range(warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(device.index or 0) if rank == 0 else None
    if sampler:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if world > 1:
        dist.barrier()
    if sampler:
        sampler.stop()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= steps
    flops = 18 * m * d * f
    line = None
    if rank == 0:
        peak_tf = float(peaks["bf16_tflops_sustained"])
        line = {
            "metric": "Pre-norm MLP block TFLOP/s", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": f"bf16 pre-norm block RMSNorm({d}) -> SwiGLU(d_ff {f}) over {m} tokens, forward+backward, "
                                   f"tensor-parallel x{world}" + (", rows sharded outside the MLP (sequence-parallel)" if seq_parallel else "")
                                   + (" [REDUCED CASE]" if m != BLOCK_TOKENS else ""),
                       "tokens": m, "d_model": d, "d_ff": f, "d_ff_per_gpu": f1 - f0, "flops_per_step": flops,
                       "allreduce_bytes_per_step": 0 if world == 1 else 2 * m * d * 2, "seed": SEED},
            "tflops_per_gpu": flops / ms / 1e9 / world,
            "frac_of_bf16_sustained_peak_per_gpu": flops / ms / 1e9 / world / peak_tf, "peak_source": f"of {peak_kind} (cuBLAS bf16 sustained)",
            "gpu_launches": 8 * steps, "clocks": sampler.summary(t0, t1) if sampler else None,
        }
    return line


def run_block(args, device, warmup, peaks, peak_kind, world, rank) -> int:
    import torch.distributed as dist

    line = block_line(args, device, warmup, peaks, peak_kind, world, rank)
    if line is not None:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_decode(args, device, warmup, peaks, peak_kind) -> int:
    """Inference-sized MLP forward: fp16, d_model 4096, hidden 6912, --tokens rows (default 16), no autograd.
    Two kernels (fused projection, w3 GEMM) whose cost is reading the 162 MB of weights once, so the bound is
    HBM: achieved = weight bytes / time. Timed from a CUDA graph of the two launches (a decoding loop replays
    graphs; host launch gaps would otherwise dominate a 40 us step); the weights exceed L2, and each replay
    streams all of them again. Beside it: torch's library GEMMs + elementwise activation on the same tensors."""
    import torch.nn.functional as F

    from mgrrmsnorm_b200 import MegaGemmTriton
    from mgrrmsnorm_b200 import rmsnorm_cuda_ops as ops

    m = args.tokens if args.tokens != MLP_TOKENS else 16
    torch.manual_seed(SEED)
    mlp = MegaGemmTriton(MLP_D).to(device).half()
    f = mlp.hidden
    w12, w3 = mlp.w12.weight.detach(), mlp.w3.weight.detach()
    g = torch.Generator(device=device).manual_seed(SEED)
    x = torch.randn(m, MLP_D, device=device, generator=g).half()
    h0 = ops.swiglu_fused_forward(x, w12, f)

    def ours():
        return ops.linear_tn(ops.swiglu_fused_forward(x, w12, f), w3)

    def library():
        gv = F.linear(x, w12)
        return F.linear(F.silu(gv[:, :f]) * gv[:, f:], w3)

    per_graph = 4

    def graph_us(fn, replays):
        fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(per_graph):
                fn()
        for _ in range(warmup):
            gr.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(replays):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (replays * per_graph) * 1e3

    replays = max(1, args.steps // per_graph)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    t0 = time.perf_counter()
    us = graph_us(ours, replays)
    t1 = time.perf_counter()
    sampler.stop()
    us_proj = graph_us(lambda: ops.swiglu_fused_forward(x, w12, f), replays)
    us_w3 = graph_us(lambda: ops.linear_tn(h0, w3), replays)
    us_lib = graph_us(library, replays)
    wbytes = (w12.numel() + w3.numel()) * 2
    peak = float(peaks["hbm_gbs"])
    line = {
        "metric": "SwiGLU MLP forward (decode) weight GB/s", "value": wbytes / us / 1e3, "unit": "GB/s", "n_gpus": 1,
        "steps": replays * per_graph, "warmup": warmup * per_graph, "ms_per_step": us / 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"fp16 SwiGLU MLP forward, {m} tokens, d_model {MLP_D}, hidden {f}; CUDA graph of the two kernels; "
                               "weights (162 MB) larger than L2, streamed again by every step", "tokens": m, "seed": SEED},
        "roofline": {"bound": "hbm", "achieved": wbytes / us / 1e3, "peak": peak, "unit": "GB/s", "frac": wbytes / us / 1e3 / peak,
                     "traffic": None, "peak_source": f"of {peak_kind} (copy bandwidth)"},
        "us": {"step": us, "fused_projection_alone": us_proj, "w3_gemm_alone": us_w3, "weights_at_peak": wbytes / peak / 1e3,
               "library_gemms_plus_activation": us_lib},
        "gpu_launches": 2 * replays * per_graph, "clocks": sampler.summary(t0, t1),
    }
    print(json.dumps(line), flush=True)
    return 0


def time_cpu_mlp(mlp, f) -> dict:
    """The reference's CPU path for the MLP: the PyTorchSwiGLU formula (benchmark_swiglu.py:40-58) in fp32
    on the host cores, forward+backward, on a 128-token sample of the batch."""
    from oracle import oracle

    m = 128
    g = torch.Generator().manual_seed(SEED)
    x = torch.randn(m, MLP_D, generator=g)
    dy = torch.randn(m, MLP_D, generator=g)
    w12 = mlp.w12.weight.detach().float().cpu()
    w3 = mlp.w3.weight.detach().float().cpu()
    oracle.swiglu_formula_torch(x, w12, w3, dy)
    times = []
    t_begin = time.perf_counter()
    while len(times) < 10 and time.perf_counter() - t_begin < 15.0:
        t0 = time.perf_counter()
        oracle.swiglu_formula_torch(x, w12, w3, dy)
        times.append(time.perf_counter() - t0)
    per = sum(times) / len(times)
    return {"value": 18 * m * MLP_D * f / per / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"PyTorchSwiGLU formula fwd+bwd in fp32 on {m} of the {MLP_TOKENS} tokens, {len(times)} steps"}



# ---------------------------------------------------------------------------------------------------
# compact side records of the default run
# ---------------------------------------------------------------------------------------------------

def allreduce_cost(buf, steps, warmup, world, job_bytes, side_run, peer=None, peer_run=None) -> dict:
    """What the latency-bound dW collective costs: the same resident loop with the fp32 NCCL all-reduce and the
    rounding on the COMPUTE stream (fully exposed), on a side stream beside the next forward, and -- the default
    where peer memory is available -- as the library's own peer-memory kernel on the compute stream; and each
    collective alone, back to back on one stream."""
    import torch.distributed as dist

    inline = time_device_resident([buf], steps, warmup, world, reduce="inline")
    if peer is not None and side_run is None:
        side_run = time_device_resident([buf], steps, warmup, world, reduce="side")
    t = torch.zeros(HIDDEN, dtype=torch.float32, device=buf.x.device)
    for _ in range(10):
        dist.all_reduce(t)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 200
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        dist.all_reduce(t)
    e1.record()
    torch.cuda.synchronize()
    alone_us = e0.elapsed_time(e1) * 1e3 / n
    ms_inline = inline["total_ms"] / steps
    ms_side = side_run["total_ms"] / steps
    out = {"bytes": HIDDEN * 4, "nccl_alone_us": alone_us,
           "nccl_on_compute_stream": {"ms_per_step": ms_inline, "value": job_bytes / ms_inline / 1e6},
           "nccl_beside_next_forward": {"ms_per_step": ms_side, "value": job_bytes / ms_side / 1e6},
           "note": "32 KB fp32 all-reduce per step: far below any bandwidth regime, so NCCL runs it as a low-latency (LL protocol) "
                   "exchange and its cost is launch + NVLink round trips, not bytes; the peer-memory kernel is one launch per rank "
                   "(stores to every peer, a bounded wait on flags, a local sum in rank order)"}
    if peer is not None and peer_run is not None:
        out_t = torch.empty(HIDDEN, dtype=torch.bfloat16, device=buf.x.device)
        for _ in range(10):
            peer(t, out_t)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            peer(t, out_t)
        e1.record()
        torch.cuda.synchronize()
        ms_peer = peer_run["total_ms"] / steps
        out["peer_kernel_alone_us"] = e0.elapsed_time(e1) * 1e3 / n
        out["peer_kernel_beside_next_forward"] = {"ms_per_step": ms_peer, "value": job_bytes / ms_peer / 1e6, "default": True}
        ms_pi = time_device_resident([buf], steps, warmup, world, reduce="peer", peer=peer)["total_ms"] / steps
        out["peer_kernel_on_compute_stream"] = {"ms_per_step": ms_pi, "value": job_bytes / ms_pi / 1e6}
    return out


def weak_scaling_figure(L, device, rank, world, warmup, peer=None) -> dict:
    """The same loop with 65536 rows on EVERY GPU (per-GPU work fixed as N grows)."""
    buf = RmsBuffers(L, ROWS_PER_GPU, HIDDEN, torch.bfloat16, device, SEED + rank, x_scale=2.0 ** 0.5)
    steps = 40
    r = time_device_resident([buf], steps, warmup, world, reduce="peer_side" if peer is not None else "side", peer=peer)
    ms = r["total_ms"] / steps
    out = {"scaling": "weak", "rows_per_gpu": ROWS_PER_GPU, "steps": steps, "ms_per_step": ms,
           "value": world * rms_bytes(ROWS_PER_GPU, HIDDEN, 2)["total"] / ms / 1e6, "unit": UNIT}
    del buf
    torch.cuda.empty_cache()
    return out


def mlp_compact(args, device, peaks, peak_kind, sm_count) -> dict:
    """Config 4 (fp16 SwiGLU MLP, 1 GPU) in two regimes: a 100-step run, long enough for the 1 kW power cap to
    set the clock, and a 20-step burst near the maximum clock; each with its own clock sample."""
    out = {}
    for name, steps in (("sustained_100_steps", 100), ("burst_20_steps", 20)):
        ln = mlp_line(args, device, 5, peaks, peak_kind, sm_count, steps=steps, no_e2e=True, no_cpu=True)
        out[name] = {"ms_per_step": ln["ms_per_step"], "TFLOPs": ln["value"], "frac_of_bf16_burst_peak": ln["frac_of_bf16_peak"],
                     "frac_of_bf16_sustained_peak": ln["frac_of_bf16_sustained_peak"], "clocks": ln["clocks"],
                     "fused_projection_kernel": {"TFLOPs": ln["roofline"]["achieved"], "frac_of_burst_peak": ln["roofline"]["frac"]}}
        torch.cuda.empty_cache()
    out["config"] = ln["config"]["workload"]
    out["peak_source"] = f"of {peak_kind} (cuBLAS bf16: burst {peaks['bf16_tflops']}, sustained {peaks['bf16_tflops_sustained']} TFLOP/s)"
    return out


def block_compact(args, device, peaks, peak_kind, world, rank):
    """Config 5 (bf16 pre-norm block, tensor-parallel over the ranks of this run): 3 warm-up + 8 timed steps."""
    ln = block_line(args, device, 3, peaks, peak_kind, world, rank, steps=8)
    torch.cuda.empty_cache()
    if ln is None:
        return None
    return {"metric": ln["metric"], "value": ln["value"], "unit": ln["unit"], "ms_per_step": ln["ms_per_step"], "steps": ln["steps"],
            "scaling": "strong", "tflops_per_gpu": ln["tflops_per_gpu"],
            "frac_of_bf16_sustained_peak_per_gpu": ln["frac_of_bf16_sustained_peak_per_gpu"], "peak_source": ln["peak_source"],
            "allreduce_bytes_per_step": ln["config"]["allreduce_bytes_per_step"], "d_ff_per_gpu": ln["config"]["d_ff_per_gpu"],
            "workload": ln["config"]["workload"], "clocks": ln["clocks"]}


def prenorm_inference_compact(device) -> dict:
    """Config 5's block, forward only and without autograd, on one GPU: the two modules (the norm writes the
    normalised [M, D] tensor, the projection reads it back) against PreNormSwiGLU (norm weight folded into w12,
    row scales from a read-only pass over x, applied in the projection's epilogue)."""
    from mgrrmsnorm_b200 import MegaGemmTriton, PreNormSwiGLU, RMSNorm

    m, d, dt = BLOCK_TOKENS, BLOCK_D, torch.bfloat16
    torch.manual_seed(SEED)
    mlp = MegaGemmTriton(d, hidden_multiple=3.5).to(device).to(dt)
    norm = RMSNorm(d, epsilon=EPS).to(device).to(dt)
    g = torch.Generator(device=device).manual_seed(SEED)
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(d, device=device, generator=g)).to(dt))
    x = torch.randn(m, d, device=device, generator=g).to(dt)
    block = PreNormSwiGLU(norm, mlp)

    def timed(fn, n=10):
        with torch.no_grad():
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(n):
                fn()
            e1.record()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    two = timed(lambda: mlp(norm(x)))
    fused = timed(lambda: block(x))
    with torch.no_grad():
        diff = float((block(x).float() - mlp(norm(x)).float()).abs().max())
    flops = 6 * m * d * mlp.hidden
    return {"workload": f"bf16 RMSNorm({d}) -> SwiGLU(d_ff {mlp.hidden}) forward, {m} tokens, no autograd", "two_modules_ms": two,
            "norm_folded_into_projection_ms": fused, "TFLOPs_folded": flops / fused / 1e9, "max_abs_diff_between_the_two": diff,
            "hbm_bytes_not_moved": 2 * m * d * 2}


def parity_check(device, world, rank, peer=None) -> dict:
    """Sharded results against the one-rank result of the same library on the same seeded inputs, computed on the
    spot on every rank: row-sharded RMSNorm (y, dx bit-equal; dW = fp32 sum across ranks, one rounding, within one
    bf16 ulp of the one-rank dW), the side-stream all-reduce against the synchronous one (same bits), and the
    tensor-parallel MLP against the full MLP. Reduced to booleans and worst errors; `ok` is the AND over all ranks."""
    import torch.distributed as dist

    from mgrrmsnorm_b200 import MegaGemmTriton, RMSNorm, sharding
    from mgrrmsnorm_b200 import rmsnorm_cuda_ops as ops

    dt = torch.bfloat16
    g = torch.Generator().manual_seed(SEED)
    rows, cols = 4096, HIDDEN
    x = (2 ** 0.5 * torch.randn(rows, cols, generator=g)).to(dt).to(device)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dt).to(device)
    dy = torch.randn(rows, cols, generator=g).to(dt).to(device)
    full = RMSNorm(cols, epsilon=EPS).to(device).to(dt)
    shard = sharding.RowShardedRMSNorm(cols, epsilon=EPS).to(device).to(dt)
    with torch.no_grad():
        full.weight.copy_(w)
        shard.weight.copy_(w)
    xf = x.clone().requires_grad_(True)
    yf = full(xf)
    yf.backward(dy)
    r0, r1 = sharding.row_shard(rows, world, rank)
    xs = x[r0:r1].clone().requires_grad_(True)
    ys = shard(xs)
    ys.backward(dy[r0:r1])
    rows_equal = bool(torch.equal(ys, yf[r0:r1]) and torch.equal(xs.grad, xf.grad[r0:r1]))
    dws, dwf = shard.weight.grad.float(), full.weight.grad.float()
    ulp = torch.maximum(dws.abs(), dwf.abs()) * 2.0 ** -7 + 1e-4     # one bf16 ulp (+ a floor for columns that cancel)
    dw_ulps = float(((dws - dwf).abs() / ulp).max())
    dw_differ = float((dws != dwf).float().mean())
    _, inv = ops.rmsnorm_forward(xs.detach(), shard.weight.detach(), EPS)
    red = sharding.AsyncDwReduce(device)
    _, _, dw32 = ops.rmsnorm_backward_full(dy[r0:r1].contiguous(), xs.detach(), shard.weight.detach(), inv, True)
    dw_async = torch.empty_like(shard.weight)
    red.start(dw32, dw_async)
    red.drain()
    torch.cuda.synchronize()
    async_equal = bool(torch.equal(dw_async, shard.weight.grad))
    # the peer-memory kernel: the partials added in rank order, the same bits on every rank, one rounding
    peer_equal = None
    if peer is not None:
        _, _, part = ops.rmsnorm_backward_full(dy[r0:r1].contiguous(), xs.detach(), shard.weight.detach(), inv, True)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        ordered = parts[0].clone()
        for q in range(1, world):
            ordered += parts[q]
        dw_peer, dw_peer32 = torch.empty_like(shard.weight), torch.empty_like(part)
        peer(part, dw_peer, dw_peer32)
        torch.cuda.synchronize()
        peer_equal = bool(torch.equal(dw_peer32, ordered) and torch.equal(dw_peer, ordered.to(dt)))

    torch.manual_seed(SEED)
    mlp = MegaGemmTriton(1024, multiple_of=256, hidden_multiple=2.0).to(device).to(dt)     # hidden 2048: divides by 2, 4, 8
    for p_ in mlp.parameters():
        dist.broadcast(p_.data, src=0)
    tp = sharding.TensorParallelSwiGLU.from_full(mlp, world, rank)
    xm = torch.randn(512, 1024, generator=g).to(dt).to(device)
    dym = torch.randn(512, 1024, generator=g).to(dt).to(device)
    a = xm.clone().requires_grad_(True)
    ya = mlp(a)
    ya.backward(dym)
    b = xm.clone().requires_grad_(True)
    yb = tp(b)
    yb.backward(dym)
    f0, f1 = sharding.tp_hidden_slice(mlp.hidden, world, rank)
    gw12 = torch.cat([mlp.w12.weight.grad[f0:f1], mlp.w12.weight.grad[mlp.hidden + f0:mlp.hidden + f1]])

    def rel(got, want):
        got, want = got.detach().float(), want.detach().float()
        return float((got - want).abs().max()) / max(float(want.abs().max()), 1e-6)

    errs = {"y": rel(yb, ya), "dx": rel(b.grad, a.grad), "dw12": rel(tp.local.w12.weight.grad, gw12),
            "dw3": rel(tp.local.w3.weight.grad, mlp.w3.weight.grad[:, f0:f1])}
    torch.cuda.synchronize()
    status = int(_capi_status())
    ok = rows_equal and async_equal and peer_equal is not False and dw_ulps <= 1.0 and dw_differ < 0.05 and max(errs.values()) < 2e-2 and status == 0
    flag = torch.tensor([1.0 if ok else 0.0, dw_ulps, max(errs.values())], device=device)
    lo = flag.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return {"ok": bool(lo[0].item() == 1.0), "ranks": world,
            "rmsnorm": {"rows": rows, "hidden": cols, "y_dx_bit_equal_to_one_rank": rows_equal, "dw_max_bf16_ulps_from_one_rank": float(flag[1].item()),
                        "dw_columns_differing": dw_differ, "async_allreduce_bit_equal_to_sync": async_equal,
                        "peer_memory_sum_bit_equal_to_rank_ordered_sum": peer_equal},
            "tp_mlp": {"tokens": 512, "d_model": 1024, "hidden": mlp.hidden, "max_rel_err_over_ranks": float(flag[2].item()),
                       "rank0_rel_err": errs, "tolerance": 2e-2},
            "device_status": status}


def _capi_status() -> int:
    from mgrrmsnorm_b200 import _capi

    return _capi.lib().mgr_device_status(1)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-side", action="store_true", help="skip the other configurations (N=1 extras)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--rows", type=int, default=TOTAL_ROWS,
                    help="rows in total (split over the ranks); anything but the default is a reduced case for profiler captures, not a bench value")
    ap.add_argument("--workload", choices=["rmsnorm", "mlp", "block", "decode"], default="rmsnorm",
                    help="rmsnorm (default, the headline); mlp: SwiGLU MLP fp16 d_model 4096 hidden 6912 forward+backward, 1 GPU; "
                         "block: bf16 pre-norm block RMSNorm(8192) -> SwiGLU(d_ff 28672) over 16384 tokens, tensor-parallel over --gpus; "
                         "decode: the fp16 MLP forward alone at --tokens rows (default 16), bound by streaming the weights")
    ap.add_argument("--tokens", type=int, default=MLP_TOKENS,
                    help="tokens for --workload mlp; anything but the default is a reduced case for profiler captures")
    args = ap.parse_args(argv)
    if args.impl == "reference":
        return reference_arm(args)

    import torch.distributed as dist

    from mgrrmsnorm_b200 import _capi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        print(f"bench.py --gpus {args.gpus} must be launched with one rank per GPU (torchrun --nproc-per-node {args.gpus})",
              file=sys.stderr)
        return 2
    if not torch.cuda.is_available():
        print("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)", file=sys.stderr)
        return 2
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    L = _capi.lib()   # raises when the kernel library is missing
    sms = ctypes.c_int(0)
    _capi.check("mgr_device_check", L.mgr_device_check(ctypes.byref(sms)))
    warmup = max(args.warmup, 3)
    peaks, peak_kind = measured_peaks()
    peak_gbs = float(peaks["hbm_gbs"])
    if args.workload == "mlp":
        if world != 1:
            print("--workload mlp runs on one GPU", file=sys.stderr)
            return 2
        return run_mlp(args, L, device, warmup, peaks, peak_kind, sms.value)
    if args.workload == "block":
        return run_block(args, device, warmup, peaks, peak_kind, world, rank)
    if args.workload == "decode":
        if world != 1:
            print("--workload decode runs on one GPU", file=sys.stderr)
            return 2
        return run_decode(args, device, warmup, peaks, peak_kind)

    from mgrrmsnorm_b200 import sharding

    r0, r1 = sharding.row_shard(args.rows, world, rank)
    local_rows = r1 - r0
    main_buf = RmsBuffers(L, local_rows, HIDDEN, torch.bfloat16, device, SEED + rank, x_scale=2.0 ** 0.5)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    # dW across the ranks: the library's peer-memory kernel where symmetric memory can be had (every rank takes the
    # same branch: the constructor is collective and its outcome is agreed on below), else NCCL on a side stream
    peer = None
    if world > 1:
        import torch.distributed as dist

        try:
            peer = sharding.PeerDwAllReduce(HIDDEN, device)
            have = 1
        except Exception as e:  # noqa: BLE001
            peer_error = f"{type(e).__name__}: {str(e)[:200]}"
            have = 0
        flag = torch.tensor([have], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            peer = None
    r = time_device_resident([main_buf], args.steps, warmup, world, reduce="peer_side" if peer is not None else "side", peer=peer)
    if sampler:
        sampler.stop()
    nb = rms_bytes(local_rows, HIDDEN, 2)                 # this rank (rank 0 holds a largest block)
    job_bytes = sum(rms_bytes(b - a, HIDDEN, 2)["total"] for a, b in (sharding.row_shard(args.rows, world, i) for i in range(world)))
    ms_per_step = r["total_ms"] / args.steps
    value = job_bytes / (ms_per_step * 1e-3) / 1e9

    extras = {}

    def guarded(name, fn):
        """Side measurements must not take the headline down: an exception becomes a recorded error string.
        (Every rank takes the same path, so a failure on all ranks leaves the collectives in step.)"""
        try:
            out = fn()
            if out is not None:
                extras[name] = out
        except Exception as e:  # noqa: BLE001
            extras[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}

    if world > 1:
        guarded("allreduce", lambda: allreduce_cost(main_buf, args.steps, warmup, world, job_bytes, None if peer is not None else r,
                                                    peer=peer, peer_run=r if peer is not None else None))

    e2e = None
    if not args.no_e2e:
        from mgrrmsnorm_b200.hostpipe import place_near_gpu

        placement = place_near_gpu(device)      # before the pinned buffers are allocated
        e2e = time_e2e(local_rows, HIDDEN, device, args.e2e_steps, 1, world, main_buf, pipelined=True)
        e2e_value = job_bytes / (e2e["ms_per_step"] * 1e-3) / 1e9
        e2e_plain = time_e2e(local_rows, HIDDEN, device, args.e2e_steps, 1, world, main_buf, pipelined=False)
        e2e["unpipelined_value"] = job_bytes / (e2e_plain["ms_per_step"] * 1e-3) / 1e9

    del main_buf
    torch.cuda.empty_cache()
    if world > 1 and not args.no_side:
        guarded("weak", lambda: weak_scaling_figure(L, device, rank, world, warmup, peer))
        guarded("parity_n", lambda: parity_check(device, world, rank, peer))
    side = {}
    if world == 1 and not args.no_side:
        side = side_results(L, device, peak_gbs)
        guarded("mlp", lambda: mlp_compact(args, device, peaks, peak_kind, sms.value))
        guarded("prenorm_inference", lambda: prenorm_inference_compact(device))
    if not args.no_side:
        guarded("block", lambda: block_compact(args, device, peaks, peak_kind, world, rank))
    cpu = None
    if world == 1 and rank == 0 and not args.no_cpu:
        cpu = time_cpu(steps=40, warmup=1, budget_s=15.0)
    status = L.mgr_device_status(1)       # the host is idle here: did any kernel give up a bounded wait?

    if rank == 0:
        bwd_gbs = nb["bwd"] / (r["bwd_ms"] * 1e-3) / 1e9
        fwd_gbs = nb["fwd"] / (r["fwd_ms"] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(world, args.rows),
            "dw_reduction": (None if world == 1 else
                             "the library's peer-memory kernel (stores to every rank over NVLink, sum in rank order) on a high-priority side stream, beside the next step's forward" if peer is not None
                             else "NCCL all-reduce on a side stream, beside the next step's forward"),
            "frac_of_hbm_peak": value / world / peak_gbs,
            "roofline": {"bound": "hbm", "kernel": "rms_bwd_reg + rms_dw_reduce4 (one mgr_rmsnorm_bwd call: dx and per-CTA partial rows of dW, then their fixed-order column sum)",
                         "achieved": bwd_gbs, "peak": peak_gbs, "unit": "GB/s", "frac": bwd_gbs / peak_gbs,
                         "peak_source": f"of {peak_kind}",
                         "algorithmic_bytes_per_launch": nb["bwd"], "avg_launch_ms": r["bwd_ms"],
                         "traffic": (TRAFFIC_PER_ALGO_BYTE * nb["bwd"]) if TRAFFIC_PER_ALGO_BYTE else None},
            "roofline_fwd": {"bound": "hbm", "kernel": "rms_fwd_reg", "achieved": fwd_gbs, "peak": peak_gbs, "unit": "GB/s",
                             "frac": fwd_gbs / peak_gbs, "algorithmic_bytes_per_launch": nb["fwd"], "avg_launch_ms": r["fwd_ms"]},
            "e2e": None if e2e is None else {
                "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": e2e["h2d"] * world, "d2h_bytes_per_step": e2e["d2h"] * world,
                "ms_per_step": e2e["ms_per_step"], "steps": e2e["steps"],
                "host_placement_rank0": placement,
                "per_gpu": {"h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                            "h2d_GBps": e2e["h2d"] / e2e["ms_per_step"] / 1e6, "d2h_GBps": e2e["d2h"] / e2e["ms_per_step"] / 1e6},
                "bound": "the host side: every step moves each rank's x, dy in and y, dx out over its PCIe link, both directions at once; "
                         "the kernels need under 2 % of the step. With several ranks on one host the links share the host's memory "
                         "and root-complex bandwidth (all pinned buffers of this process tree come from the same host DRAM), so the "
                         "per-GPU rate falls as ranks are added; no collective is involved beyond the 32 KB dW all-reduce",
                "path": "pinned host x, dy -> HostRMSNormPipeline (32 MiB row chunks, copy-in / compute / copy-out streams) -> pinned host y, dx; "
                        "dW: fp32 sum all-reduced across ranks, rounded once, copied to pinned host memory",
                "unpipelined_value": e2e["unpipelined_value"],
                "unpipelined_path": "pinned host -> whole-tensor copies around the RMSNorm module fwd+bwd -> pinned host"},
            "gpu_launches": (4 if peer is not None else 3) * args.steps,
            "launches_per_step": dict({"rms_fwd_reg": 1, "rms_bwd_reg": 1, "rms_dw_reduce4": 1}, **({"peer_allreduce_f32": 1} if peer is not None else {})),
            "clocks": sampler.summary(*r["window"]) if sampler else None,
            "sm_count": sms.value, "device_status": status,
        }
        if cpu:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if side:
            line["also"] = side
        line.update(extras)           # compact keys last: block, mlp (N = 1), weak / allreduce / parity_n (N > 1)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
