#!/usr/bin/env python
"""Benchmark of the quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference] [--selftest]

Prints ONE JSON line.  The headline workload is the INT8 per-channel quantize + dequantize of a bf16
8192 x 8192 weight (the configuration the GB/s metric is quoted on); a *step* is one quantize plus one
dequantize of that tensor.  ``value`` is algorithmic GB/s with inputs resident in HBM, ``e2e`` the same
through the public API from pinned host buffers, ``roofline`` the dominant kernel against the measured HBM
peak, ``cpu_baseline`` the PyTorch CPU formulation on this host's cores.

Beside the headline the line carries
  ``configs``   the other benchmark configurations measured the same way: per-tensor FP8 (4096 x 4096),
                per-group INT8 (16384 x 8192, groups of 128, bf16 and fp16 dequantize), the W8A16 linear
                (N = 14336, K = 4096) per M with its end-to-end figure, and its LLM.int8 variant;
  ``next_rows`` the rows next to the path: fused RMSNorm -> INT8, per-column and non-last-axis per-group INT8 in place,
                the W8A8 and W4A16 layers, the generic tcgen05 GEMM wrapper (device time only);
  ``sharded``   the multi-GPU forms of the path over the N ranks of this launch (N = 1 is the baseline of
                the scaling curve): one bf16 tensor of 2^33 elements quantized per tensor to FP8 with its rows
                split over the ranks (strong scaling; local amax, ONE NCCL max-allreduce of a float32, cast;
                every phase timed on its own), the W8A16 linear at M = 2048 with its output features split
                over the ranks, and ``quantize_model`` on a Llama-3-8B-shaped decoder with every Linear's rows
                split over the ranks;
  ``selftest``  bit-equality checks of those sharded forms (the same scale on every rank, checksums of codes
                that do not depend on N, a layer's codes against the CPU oracle); ``--selftest`` makes a failed
                check the exit code.

With N > 1 (one process per GPU under torch.distributed.run) every rank runs the headline workload on its own
rows (weak scaling, no data-path collective) and the time is the max over ranks.  ``--impl reference`` times
the CPU formulation instead; ``--impl reference_gpu`` times the reference's own CUDA extensions when they are
built under ``oracle/_ref`` (context only).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
MIN_REGION_S = 0.2  # a timed region is repeated until it lasts at least this long
# DRAM bytes (read + write) per launch of each workload's kernels, from one ncu capture of that workload
# (dram__bytes_read.sum + dram__bytes_write.sum, caches flushed before each captured launch); None where no capture
# was taken.  Stores that were still dirty in the 126 MB L2 when a captured launch ended are not in its count.
# "quantize" of the per-tensor workload is its two launches (amax: 33.57 MB, cast: 33.57 MB under ncu -- live, the
# cast finds part of x in L2).
NCU_TRAFFIC_BYTES = {
    "int8_channel": {"quantize": 164_258_409, "dequantize": 140_661_321},
    "fp8_tensor": {"quantize": 67_135_317, "dequantize": 16_789_163},
    "int8_group": {"quantize": 362_416_971, "dequantize": 346_577_701},
    "int8_group_axis0": {"quantize": 167_694_528, "dequantize": 143_982_496},
}


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------
# clocks sampler (NVML, read-only)
# --------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.samples, self.seen, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.seen.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.seen), "samples": len(self.samples)}


# --------------------------------------------------------------------------------------
# quantize + dequantize workloads
# --------------------------------------------------------------------------------------
class Int8ChannelWorkload:
    """INT8 symmetric per-channel (axis 0) quantize + dequantize of a bf16 [rows, cols] weight."""

    name = "int8_channel"
    dtype = "int8"
    dominant = "quant_segments_kernel (one-pass per-channel INT8 quantize)"

    def __init__(self, device, rows=8192, cols=8192, sets=3):
        from cublade_b200 import workloads as W

        self.rows, self.cols, self.sets = rows, cols, sets
        x_host = W.int8_channel_case(rows, cols)
        self._host_buffers(x_host, device, sets)
        self.n = rows * cols
        self.q_bytes = self.n * 3 + rows * 4  # 2 B read + 1 B write per element, 4 B scale per row
        self.dq_bytes = self.n * 3 + rows * 4
        self.bytes_per_step = self.q_bytes + self.dq_bytes
        self.device = device
        self.qt = [None] * sets
        self.launches_per_step = 2

    def _host_buffers(self, x_host, device, sets):
        # device=None builds the host input only (CPU reference arm).  Rotating buffer sets: the
        # footprint (sets * 5 B/elem) exceeds 2 x L2, so no launch finds its input in L2.
        if device is None:
            self.x_host, self.y_host, self.x = x_host, None, []
            return
        self.x_host = x_host.pin_memory()
        self.y_host = torch.empty_like(x_host).pin_memory()
        self.x = [x_host.to(device) for _ in range(sets)]

    def config(self):
        """Identical in the GPU and the reference arm: the workload, its bytes and its seed."""
        return {"workload": f"int8_per_channel_axis0_quant+dequant bf16 {self.rows}x{self.cols}",
                "bytes_per_step": self.bytes_per_step, "seed": 1}

    def l2_policy(self):
        return (f"rotating {self.sets} buffer sets ({self.sets * self.n * 5 / 1e6:.0f} MB footprint > 2x L2); "
                "dequantize reads codes written at least one step earlier")

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.int8, mode="channel", ch_axis=0)

    def dequantize(self, qt):
        import cublade_b200 as cb

        return cb.dequantize_tensor(qt)

    def extra_kernels(self):
        return {}

    def prime(self):
        for i in range(self.sets):
            self.qt[i] = self.quantize(self.x[i])
        torch.cuda.synchronize()

    def step(self, i):
        a, b = i % self.sets, (i + 1) % self.sets
        self.qt[a] = self.quantize(self.x[a])
        return self.dequantize(self.qt[b])

    def step_e2e(self, i):
        x = self.x_host.to(self.device, non_blocking=True)
        y = self.dequantize(self.quantize(x))
        self.y_host.copy_(y, non_blocking=True)
        return y

    e2e_h2d = property(lambda self: self.n * 2)
    e2e_d2h = property(lambda self: self.n * 2)

    # CPU formulation of the same step (oracle = checker / baseline only)
    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s = O.int8_quantize_channel(x_cpu)
        return O.int8_dequantize_rows(q, s, torch.bfloat16)

    def cpu_input(self):
        return self.x_host


class Fp8TensorWorkload(Int8ChannelWorkload):
    """Per-tensor FP8 E4M3 quantize + dequantize of a bf16 [rows, cols] tensor with 16 outliers."""

    name = "fp8_tensor"
    dtype = "e4m3"
    dominant = "amax_tensor_kernel + cast_tensor_kernel (per-tensor FP8 quantize, two dependent launches)"

    def __init__(self, device, rows=4096, cols=4096, sets=12):
        from cublade_b200 import workloads as W

        self.rows, self.cols, self.sets = rows, cols, sets
        x_host = W.fp8_tensor_case(rows, cols)
        self._host_buffers(x_host, device, sets)
        self.n = rows * cols
        self.q_bytes = self.n * 3 + 4  # the tensor fits in L2: the second read of x is not HBM traffic
        self.dq_bytes = self.n * 3 + 4
        self.bytes_per_step = self.q_bytes + self.dq_bytes
        self.device = device
        self.qt = [None] * sets
        self.launches_per_step = 3

    def config(self):
        return {"workload": f"fp8_e4m3_per_tensor_quant+dequant bf16 {self.rows}x{self.cols} (16 outliers of 300)",
                "bytes_per_step": self.bytes_per_step, "seed": 0}

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.float8_e4m3fn, mode="tensor")

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s = O.fp8_quantize(x_cpu)
        return O.fp8_dequantize(q, s, torch.bfloat16)


class Int8GroupWorkload(Int8ChannelWorkload):
    """INT8 per-group (128 along the last axis) quantize + dequantize of bf16 Student-t activations."""

    name = "int8_group"
    dominant = "quant_segments_kernel (one-pass per-group INT8 quantize)"

    def __init__(self, device, rows=16384, cols=8192, sets=2, group=128):
        from cublade_b200 import workloads as W

        self.rows, self.cols, self.sets, self.group = rows, cols, sets, group
        x_host = W.int8_group_case(rows, cols)
        self._host_buffers(x_host, device, sets)
        self.n = rows * cols
        self.q_bytes = self.n * 3 + (self.n // group) * 4
        self.dq_bytes = self.q_bytes
        self.bytes_per_step = self.q_bytes + self.dq_bytes
        self.device = device
        self.qt = [None] * sets
        self.launches_per_step = 2

    def config(self):
        return {"workload": f"int8_per_group_{self.group}_quant+dequant bf16 {self.rows}x{self.cols} (Student-t nu=3 x0.5)",
                "bytes_per_step": self.bytes_per_step, "seed": 2}

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=self.group, ch_axis=-1)

    def extra_kernels(self):
        """The float16 dequantize of the same codes (the reference's legacy output type for this configuration)."""
        import copy

        import cublade_b200 as cb

        def dq16(i):
            qt = copy.copy(self.qt[i % self.sets])
            qt.original_dtype = torch.float16
            return cb.dequantize_tensor(qt)

        return {"dequantize_fp16": (dq16, self.dq_bytes)}

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s = O.int8_quantize_group(x_cpu.view(-1, self.group), self.group)
        return O.int8_dequantize_rows(q, s, torch.bfloat16)


class Int8GroupAxis0Workload(Int8GroupWorkload):
    """INT8 per-group quantize + dequantize with the groups of 128 running DOWN the rows of a bf16 [rows, cols]
    matrix (ch_axis = 0), in place: the reference makes two transposing copies around its row kernel for this."""

    name = "int8_group_axis0"
    dominant = "quant_group_axis_kernel (one-pass per-group INT8 quantize, groups along a non-last axis)"

    def __init__(self, device, rows=8192, cols=8192, sets=3, group=128):
        super().__init__(device, rows, cols, sets, group)

    def config(self):
        return {"workload": (f"int8_per_group_{self.group}_along_axis0_quant+dequant bf16 {self.rows}x{self.cols} "
                             f"(Student-t nu=3 x0.5)"),
                "bytes_per_step": self.bytes_per_step, "seed": 2}

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=self.group, ch_axis=0)

    def extra_kernels(self):
        return {}

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        xt = x_cpu.t().contiguous()
        q, s = O.int8_quantize_group(xt.view(-1, self.group), self.group)
        return O.int8_dequantize_rows(q, s, torch.bfloat16).view(self.cols, self.rows).t().contiguous()


class RmsnormInt8Workload(Int8ChannelWorkload):
    """Fused RMSNorm -> per-token INT8 quantize of bf16 activations [tokens, hidden], then dequantize."""

    name = "rmsnorm_int8"
    dominant = "rmsnorm_quant_rows_kernel (one-pass RMSNorm + per-token INT8 quantize)"

    def __init__(self, device, rows=16384, cols=8192, sets=2):
        from cublade_b200 import workloads as W

        self.rows, self.cols, self.sets = rows, cols, sets
        x_host = W.int8_group_case(rows, cols)  # Student-t activations, the same generator as the per-group config
        self._host_buffers(x_host, device, sets)
        g = torch.Generator().manual_seed(4)
        self.gain_host = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(torch.bfloat16)
        self.gain = self.gain_host.to(device) if device is not None else None
        self.n = rows * cols
        self.q_bytes = self.n * 3 + rows * 4 + cols * 2  # x once in, codes once out, one scale per token, the gain
        self.dq_bytes = self.n * 3 + rows * 4
        self.bytes_per_step = self.q_bytes + self.dq_bytes
        self.device = device
        self.qt = [None] * sets
        self.launches_per_step = 2

    def config(self):
        return {"workload": (f"rmsnorm+int8_per_token_quant (fused, 3 B/elem instead of 7 unfused) + dequant bf16 "
                             f"{self.rows}x{self.cols} (Student-t nu=3 x0.5)"),
                "bytes_per_step": self.bytes_per_step, "seed": 2}

    def quantize(self, x):
        from cublade_b200.quantization import rmsnorm_quantize_tensor

        return rmsnorm_quantize_tensor(x, self.gain)

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s, _, _ = O.rmsnorm_quantize(x_cpu, self.gain_host)
        return O.int8_dequantize_rows(q, s, torch.bfloat16)


WORKLOADS = {"int8_channel": Int8ChannelWorkload, "fp8_tensor": Fp8TensorWorkload, "int8_group": Int8GroupWorkload,
             "int8_group_axis0": Int8GroupAxis0Workload, "rmsnorm_int8": RmsnormInt8Workload}
LINEAR_WORKLOADS = ("w8a16", "w8a8", "w4a16")


# --------------------------------------------------------------------------------------
# timing helpers
# --------------------------------------------------------------------------------------
class Runtime:
    """Device, ranks and the barrier shared by every measurement of one launch."""

    def __init__(self, device, dist, rank, world, local_rank):
        self.device, self.dist, self.rank, self.world, self.local_rank = device, dist, rank, world, local_rank
        self.side = torch.cuda.Stream()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *values):
        if self.dist is None:
            return values if len(values) > 1 else values[0]
        t = torch.tensor(values, device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        out = tuple(float(v) for v in t.tolist())
        return out if len(out) > 1 else out[0]

    def capture(self, fn):
        """fn() recorded into a CUDA graph on the side stream."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.side):
            with torch.cuda.graph(g, stream=self.side):
                keep = fn()
        torch.cuda.synchronize()
        g._keep = keep  # outputs stay allocated while the graph lives
        return g

    def time_graphs(self, graphs, units, min_s=MIN_REGION_S, collective=True):
        """Replays the list of graphs (``units`` steps / launches in total) between two CUDA events, repeating the
        list until the region lasts at least ``min_s``.  Returns (ms per unit, repeats).  Device time; with
        ``collective`` the repeat count is agreed over the ranks and barriers bracket the region."""
        for g in graphs:
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for g in graphs:
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        once = max(e0.elapsed_time(e1) * 1e-3, 1e-6)
        reps = max(1, math.ceil(1.1 * min_s / once))  # the probe replay can be slower than the steady state
        if collective:
            reps = int(self.max_over_ranks(float(reps)))
            self.barrier()
        e0.record()
        for _ in range(reps):
            for g in graphs:
                g.replay()
        e1.record()
        if collective:
            self.barrier()
        else:
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (reps * units), reps


def measure_quant(rt: Runtime, wl, K: int, warmup: int, *, collective=True, min_s=MIN_REGION_S, e2e=True):
    """Device-resident and end-to-end timing of one quantize + dequantize workload.

    The K steps are consecutive nodes of CUDA graphs (at most 200 steps per graph): step i quantizes x[i % sets]
    and dequantizes the codes of set i + 1, written earlier (not in L2 any more); outputs of the last `sets` steps
    stay allocated, so the written buffers rotate like the inputs.  The K-step region is repeated until it lasts
    MIN_REGION_S.  Per-kernel times come from graphs holding only that kernel, K times."""
    from cublade_b200 import _native as N

    wl.prime()
    for i in range(warmup):
        wl.step(i)
    torch.cuda.synchronize()
    kChain = 200
    static_qt = list(wl.qt)
    extras = wl.extra_kernels()

    def chain(kind, n):
        def body():
            ring = [None] * wl.sets
            for i in range(n):
                out = []
                if kind in ("step", "q"):
                    out.append(wl.quantize(wl.x[i % wl.sets]))
                if kind in ("step", "dq"):
                    out.append(wl.dequantize(static_qt[(i + 1) % wl.sets]))
                if kind in extras:
                    out.append(extras[kind][0](i + 1))
                ring[i % wl.sets] = out
            return ring

        return rt.capture(body)

    def graphs_for(kind):
        full, rest = divmod(K, kChain)
        gs = [chain(kind, kChain)] * full if full else []
        if rest:
            gs.append(chain(kind, rest))
        return gs

    kinds = ["step", "q", "dq"] + list(extras)
    graphs = {k: graphs_for(k) for k in kinds}  # capture everything before the sampler and the timed regions start
    launches0 = N.launch_count()
    with ClockSampler(rt.local_rank) as clocks:
        ms_step, reps = rt.time_graphs(graphs["step"], K, min_s, collective)
        per_kernel = {k: rt.time_graphs(graphs[k], K, min_s / 4, collective)[0] for k in kinds[1:]}
    replay_launches = N.launch_count() - launches0  # 0: graph replays do not pass through the library's host code
    if collective:
        ms_step = rt.max_over_ranks(ms_step)
    rec = {"ms_per_step": ms_step, "repeats": reps, "timed_region_s": ms_step * K * reps * 1e-3,
           "clocks": clocks.summary(), "host_launch_calls_in_replays": int(replay_launches),
           "q_ms": per_kernel["q"], "dq_ms": per_kernel["dq"],
           "extra_ms": {k: per_kernel[k] for k in extras}}
    del graphs

    # eager (no graph) pacing of the same step through the Python API, for information
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_eager = min(K, 100)
    e0.record()
    for i in range(n_eager):
        wl.step(i)
    e1.record()
    torch.cuda.synchronize()
    rec["eager_ms_per_step"] = e0.elapsed_time(e1) / n_eager
    if not e2e:
        return rec

    # ---- end to end through the public API from pinned host memory ------------------------------
    # Every step copies its input host -> device, runs quantize_tensor + dequantize_tensor, and copies the
    # result device -> host.  Steps alternate between two CUDA streams (two pinned output buffers), so the upload
    # of one step overlaps the download of the previous one on the full-duplex PCIe link -- the ordinary way a
    # caller pipelines this API.  The same loop without the two kernels gives the copy floor.
    e2e_steps = max(4, min(K, 20))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    y_hosts = [wl.y_host, torch.empty_like(wl.y_host).pin_memory()]
    y_dev = [torch.empty_like(wl.x[0]) for _ in range(2)]

    def e2e_pass(n, compute=True):
        for i in range(n):
            st = streams[i & 1]
            with torch.cuda.stream(st):
                if compute:
                    wl.y_host = y_hosts[i & 1]
                    wl.step_e2e(i)
                else:
                    x = wl.x_host.to(rt.device, non_blocking=True)
                    y_hosts[i & 1].copy_(y_dev[i & 1], non_blocking=True)
                    del x
        for st in streams:
            st.synchronize()

    def wall(compute):
        e2e_pass(4, compute)
        rt.barrier() if collective else torch.cuda.synchronize()
        t0 = time.perf_counter()
        e2e_pass(e2e_steps, compute)
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t0) * 1e3 / e2e_steps  # host clock around fully synchronised passes
        rt.barrier() if collective else torch.cuda.synchronize()
        return rt.max_over_ranks(dt) if collective else dt

    rec["e2e_ms"], rec["e2e_steps"] = wall(True), e2e_steps
    rec["copy_floor_ms"] = wall(False)
    return rec


def quant_record(wl, rec, peaks, world):
    """The JSON sub-record of one measured quantize + dequantize workload."""
    q_ms, dq_ms = rec["q_ms"], rec["dq_ms"]
    achieved = wl.q_bytes / (q_ms * 1e-3) / 1e9
    traffic = NCU_TRAFFIC_BYTES.get(wl.name, {})
    out = {
        "workload": wl.config()["workload"], "value": world * wl.bytes_per_step / (rec["ms_per_step"] * 1e-3) / 1e9,
        "unit": "GB/s", "ms_per_step": rec["ms_per_step"], "repeats": rec["repeats"],
        "timed_region_s": rec["timed_region_s"], "eager_ms_per_step": rec["eager_ms_per_step"],
        "l2_policy": wl.l2_policy(),
        "roofline": {"bound": "hbm", "kernel": wl.dominant, "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "traffic": traffic.get("quantize"), "algorithmic_bytes_per_launch": wl.q_bytes,
                     "avg_launch_us": q_ms * 1e3, "frac_of_nominal_8000": achieved / 8000.0},
        "kernels": {"quantize": {"avg_us": q_ms * 1e3, "gbs": achieved, "frac": achieved / peaks["hbm_gbs"]},
                    "dequantize": {"avg_us": dq_ms * 1e3, "gbs": wl.dq_bytes / (dq_ms * 1e-3) / 1e9,
                                   "frac": wl.dq_bytes / (dq_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                   "traffic": traffic.get("dequantize")}},
    }
    for name, ms in rec["extra_ms"].items():
        nbytes = wl.extra_kernels()[name][1]
        out["kernels"][name] = {"avg_us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9,
                                "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    if "e2e_ms" in rec:
        e2e_bytes = world * wl.bytes_per_step
        out["e2e"] = {"value": e2e_bytes / (rec["e2e_ms"] * 1e-3) / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": wl.e2e_h2d, "d2h_bytes_per_step": wl.e2e_d2h,
                      "ms_per_step": rec["e2e_ms"], "steps": rec["e2e_steps"],
                      "copy_floor_ms_per_step": rec["copy_floor_ms"],
                      "frac_of_copy_floor": rec["copy_floor_ms"] / rec["e2e_ms"],
                      "copy_floor_note": "the same two-stream loop with only the host->device and device->host copies; "
                                         "what is left of a step is the host link, not the kernels"}
    return out


# --------------------------------------------------------------------------------------
# W8A16 linear: the per-M table (N = 14336, K = 4096), plain and LLM.int8
# --------------------------------------------------------------------------------------
def w8a16_table(rt: Runtime, peaks, ms=(1, 16, 128, 2048), outliers=False):
    """Per M: device time with the weights streamed from HBM (a CUDA graph that walks over copies of the layer
    larger than 2 x L2), TFLOP/s, the roofline that bounds the shape (HBM for the weight stream, tensor for
    M = 2048), and the end-to-end figure (activations from pinned host memory, result back to the host)."""
    import cublade_b200 as cb
    from tests.golden import cases

    device = rt.device
    N_, K_ = cases.W8A16_N, cases.W8A16_K
    w, cols, bias = cases.w8a16_weight(outliers)
    sets = -(-2 * L2_BYTES // (N_ * K_)) + 1
    layers = []
    for _ in range(sets):
        layer = cb.cuBladeW8A16LinearLayer(K_, N_, bias=bias is not None, dtype=torch.bfloat16, handle_outliers=outliers)
        layer.quantize(w.to(device))
        if bias is not None:
            layer.bias = torch.nn.Parameter(bias.clone())
        layers.append(layer.to(device))
    out = {}
    for M in ms:
        x_host = cases.w8a16_activations(M, cols).pin_memory()
        y_host = torch.empty(M, N_, dtype=torch.bfloat16).pin_memory()
        x = x_host.to(device)
        for lay in layers:
            lay(x)
        g = rt.capture(lambda: [lay(x) for _ in range(2) for lay in layers])  # no copy twice in a row
        t_ms, _ = rt.time_graphs([g], 2 * sets, min_s=0.05, collective=False)
        g = rt.capture(lambda: [layers[0](x) for _ in range(10)])
        warm_ms, _ = rt.time_graphs([g], 10, min_s=0.02, collective=False)
        del g
        # end to end: one forward per step, alternating two streams
        streams = [torch.cuda.Stream(), torch.cuda.Stream()]
        y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]

        def e2e_pass(n):
            for i in range(n):
                with torch.cuda.stream(streams[i & 1]):
                    y = layers[i % sets](x_host.to(device, non_blocking=True))
                    y_hosts[i & 1].copy_(y, non_blocking=True)
            for st in streams:
                st.synchronize()

        e2e_pass(4)
        torch.cuda.synchronize()
        n_e2e = 20
        t0 = time.perf_counter()
        e2e_pass(n_e2e)
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
        t = t_ms * 1e-3
        flops = 2.0 * M * N_ * K_
        kn = K_ - len(cols)
        bytes_ = N_ * kn + 2 * N_ + 2 * M * K_ + 2 * M * N_ + 2 * N_ * len(cols)
        tf, gbs = flops / t / 1e12, bytes_ / t / 1e9
        bound = "tensor" if M >= 1024 else "hbm"
        frac = tf / peaks["bf16_tflops"] if bound == "tensor" else gbs / peaks["hbm_gbs"]
        out[f"M={M}"] = {
            "us": t * 1e6, "tflops": tf, "gbs": gbs,
            "roofline": {"bound": bound, "achieved": tf if bound == "tensor" else gbs,
                         "peak": peaks["bf16_tflops"] if bound == "tensor" else peaks["hbm_gbs"],
                         "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": frac,
                         "frac_of_sustained_peak": tf / peaks["bf16_tflops_sustained"] if bound == "tensor" else None,
                         "kernel": ("w8a16_tc_kernel (tcgen05 / TMEM / TMA)" if M >= 17 else "w8a16_stream_fast_kernel")
                                   + (" after two gather_cols_kernel launches" if outliers else ""),
                         "algorithmic_bytes_per_launch": bytes_, "flops_per_launch": flops, "traffic": None},
            "us_l2_warm": warm_ms * 1e3,
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": M * K_ * 2, "d2h_bytes_per_step": M * N_ * 2, "steps": n_e2e},
        }
    return {"shape": f"N={N_} K={K_} bf16 activations, int8 per-output-channel weights"
                     + (f", {len(cols)} outlier columns kept in bf16 (K - {len(cols)} int8 columns), bias" if outliers else ""),
            "method": f"CUDA graph over {sets} copies of the layer ({sets * N_ * K_ / 1e6:.0f} MB of weights > 2x L2)",
            "per_m": out}


# --------------------------------------------------------------------------------------
# the rows next to the path (fused RMSNorm -> quantize, other axes, W8A8 / W4A16, the dense GEMM)
# --------------------------------------------------------------------------------------
def next_rows(rt: Runtime, peaks, K, warmup):
    import cublade_b200 as cb
    from cublade_b200.bindings.triton import matmul
    from tests.golden import cases

    device = rt.device
    out = {}
    wl = RmsnormInt8Workload(device)
    out["rmsnorm_int8_fused_16384x8192"] = quant_record(
        wl, measure_quant(rt, wl, min(K, 50), warmup, collective=False, min_s=0.05, e2e=False), peaks, 1)
    del wl
    torch.cuda.empty_cache()

    def us(fn, n):
        g = rt.capture(lambda: [fn(i) for i in range(n)])
        ms, _ = rt.time_graphs([g], n, min_s=0.03, collective=False)
        return ms * 1e3

    gen = torch.Generator(device=device).manual_seed(9)
    xs = [(torch.randn(8192, 8192, generator=gen, device=device) * 0.5).to(torch.bfloat16) for _ in range(3)]
    n = 8192 * 8192
    for key, kw in (("int8_per_column_8192x8192_in_place", dict(mode="channel", ch_axis=1)),
                    ("int8_groups_of_128_down_the_rows_8192x8192_in_place", dict(mode="group", group_size=128, ch_axis=0))):
        qts = [cb.quantize_tensor(x, dtype=torch.int8, **kw) for x in xs]
        tq = us(lambda i: cb.quantize_tensor(xs[i % 3], dtype=torch.int8, **kw), 6)
        td = us(lambda i: cb.dequantize_tensor(qts[(i + 1) % 3]), 6)
        out[key] = {"quantize_us": tq, "dequantize_us": td, "quantize_gbs_at_3B_per_element": n * 3 / tq / 1e3,
                    "dequantize_gbs_at_3B_per_element": n * 3 / td / 1e3,
                    "note": "the reference: NotImplementedError (channel) / two transposing copies around the row kernel (group)"}
        del qts
    del xs
    torch.cuda.empty_cache()
    w, _, _ = cases.w8a16_weight(False)
    N_, K_ = cases.W8A16_N, cases.W8A16_K
    for name, cls, M in (("w8a8_linear_M2048", cb.quantization.cuBladeW8A8LinearLayer, 2048),
                         ("w4a16_linear_M1", cb.quantization.cuBladeW4A16LinearLayer, 1)):
        sets = 1 if M >= 1024 else 6
        layers = []
        for _ in range(sets):
            lay = cls(K_, N_, bias=False, dtype=torch.bfloat16)
            lay.quantize(w.to(device))
            layers.append(lay.to(device))
        x = cases.w8a16_activations(M).to(device)
        for lay in layers:
            lay(x)
        t = us(lambda i: layers[i % sets](x), 2 * sets if sets > 1 else 6)
        out[name] = {"us": t, "tera_ops": 2.0 * M * N_ * K_ / t / 1e6,
                     "shape": f"M={M} N={N_} K={K_}" + (", per-token activation quantization inside the step" if "w8a8" in name else "")}
        del layers
    torch.cuda.empty_cache()
    a = torch.randn(4096, 4096, generator=gen, device=device).to(torch.bfloat16)
    b = torch.randn(4096, 4096, generator=gen, device=device).to(torch.bfloat16)
    matmul(a, b)
    t = us(lambda i: matmul(a, b), 4)
    out["matmul_bf16_4096x4096x4096"] = {"us": t, "tflops": 2.0 * 4096 ** 3 / t / 1e6,
                                         "note": "generic GEMM wrapper on tcgen05 (transpose of B included)"}
    return out


# --------------------------------------------------------------------------------------
# sharded forms of the path (all ranks take part)
# --------------------------------------------------------------------------------------
def sharded_fp8(rt: Runtime, checks, total=1 << 33, chunk=1 << 27, steps=5):
    """ONE bf16 tensor of `total` elements, N(0, 1), chunk c generated on its owning device from a seed that depends
    only on c (the content does not depend on the number of GPUs), rows split contiguously over the ranks.  A step is
    local amax -> ONE exchange of a float32 maximum -> cast of the local shard -> dequantize of the local shard;
    every phase is timed with CUDA events on the launching stream, the step is the max over ranks."""
    import cublade_b200 as cb
    from cublade_b200 import workloads as W
    from cublade_b200.bindings.cuda.split_phase import amax_abs, cast_per_tensor
    from cublade_b200.quantization.tensor import QuantizedTensor
    from cublade_b200.sharding import quantize_tensor_sharded, shard_range

    dist, device = rt.dist, rt.device
    nchunks = total // chunk
    c0, c1 = shard_range(nchunks, rt.rank, rt.world)
    n_local = (c1 - c0) * chunk
    x = torch.empty(n_local, dtype=torch.bfloat16, device=device)
    for i, c in enumerate(range(c0, c1)):
        x[i * chunk:(i + 1) * chunk] = W.sharded_fp8_chunk(c, chunk, device=device)
    x = x.view(-1, 8192)
    zp = torch.zeros((), dtype=torch.float32, device=device)

    def phases(record, exchange):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        amax = amax_abs(x)
        ev[1].record()
        if exchange is not None:
            amax = exchange.exchange(amax)
        elif dist is not None:
            dist.all_reduce(amax, op=dist.ReduceOp.MAX)
        ev[2].record()
        q, scale = cast_per_tensor(x, amax, torch.float8_e4m3fn, 1e-12)
        ev[3].record()
        y = cb.dequantize_tensor(QuantizedTensor(q, scale, zp, "tensor", 0, 32, torch.float8_e4m3fn, x.dtype))
        ev[4].record()
        if record is not None:
            record.append(ev)
        return amax, q, scale, y

    def timed(exchange):
        for _ in range(2):
            out = phases(None, exchange)
        del out
        rt.barrier()
        rec = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            res = phases(rec, exchange)
        e1.record()
        rt.barrier()
        ms = rt.max_over_ranks(e0.elapsed_time(e1) / steps)
        mine = [statistics.median(ev[i].elapsed_time(ev[i + 1]) for ev in rec) for i in range(4)]
        return ms, rt.max_over_ranks(*mine), res

    # The exchange between the phases: NCCL's all_reduce(MAX) of one float, and -- where torch's symmetric memory maps
    # the ranks' buffers into one another -- the library's own peer-memory exchange (a 64-bit store per peer over
    # NVLink and a bounded wait, one small kernel per rank).  Both are timed; every rank must agree on which ran.
    peer, peer_why = None, "one rank"
    if dist is not None:
        from cublade_b200.sharding import PeerAmaxExchange

        try:
            peer = PeerAmaxExchange()
            built = 1.0
        except Exception as e:  # no symmetric memory on this system: the collective stays
            peer, built, peer_why = None, 0.0, f"{type(e).__name__}: {str(e)[:160]}"
        if -rt.max_over_ranks(-built) < 1.0:
            peer = None
    names = ("amax", "exchange", "cast", "dequantize")
    nccl_ms = nccl_worst = None
    if peer is not None:
        nccl_ms, nccl_worst, res = timed(None)
        nccl_scale_bits = int(res[2].view(torch.int32).item())
        del res
        torch.cuda.empty_cache()
    step_ms, worst, (amax, q, scale, y) = timed(peer)
    if peer is not None:
        checks.append(("fp8_sharded: the peer-memory exchange gives the scale the NCCL all-reduce gives",
                       bool(nccl_scale_bits == int(scale.view(torch.int32).item()))))
    # ---- checks: the same scale everywhere; checksums that do not depend on the number of ranks ----
    local_amax = amax_abs(x)
    sums = torch.stack([q.view(torch.uint8).sum(dtype=torch.int64),
                        (q.view(torch.uint8).to(torch.int32) ** 2).sum(dtype=torch.int64) if n_local <= (1 << 28)
                        else sum((q.view(torch.uint8).view(-1)[i:i + (1 << 28)].to(torch.int32) ** 2).sum(dtype=torch.int64)
                                 for i in range(0, n_local, 1 << 28)),
                        y.view(torch.int16).to(torch.int32).sum(dtype=torch.int64) if n_local <= (1 << 28)
                        else sum(y.view(torch.int16).view(-1)[i:i + (1 << 28)].to(torch.int32).sum(dtype=torch.int64)
                                 for i in range(0, n_local, 1 << 28))])
    scale_bits = scale.view(torch.int32).reshape(1).to(torch.int64)
    gathered_amax = local_amax.reshape(1).clone()
    if dist is not None:
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        lo, hi = scale_bits.clone(), scale_bits.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dist.all_reduce(gathered_amax, op=dist.ReduceOp.MAX)
        checks.append(("fp8_sharded: scale bits identical on every rank", bool(lo.item() == hi.item())))
    checks.append(("fp8_sharded: reduced amax equals the max of the ranks' local amax",
                   bool(gathered_amax.item() == amax.item())))
    # the one-call public form on the whole local shard must give the same scale and codes
    qt = quantize_tensor_sharded(x, dtype=torch.float8_e4m3fn)
    checks.append(("fp8_sharded: quantize_tensor_sharded scale equals the phased run's",
                   bool(qt.scale.view(torch.int32).item() == scale.view(torch.int32).item())))
    checks.append(("fp8_sharded: quantize_tensor_sharded codes equal the phased run's on the local shard",
                   bool(torch.equal(qt.data.view(torch.uint8), q.view(torch.uint8)))))
    del qt
    a = float(amax.item())
    want_scale = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(448.0, dtype=torch.float32).div(
        torch.tensor(max(a, 1e-12), dtype=torch.float32))
    checks.append(("fp8_sharded: scale = 1 / (448 / amax) in float32", bool(want_scale.item() == scale.item())))
    total_bytes = total * 8  # quantize 5 B/elem (two compulsory passes over x: the shard cannot stay on chip) + dequantize 3
    rec_out = {
        "workload": f"fp8_e4m3_per_tensor_sharded_quant+dequant bf16 2^{total.bit_length() - 1} elements N(0,1) over "
                    f"{rt.world} GPU(s), one max-exchange of the fp32 amax per step",
        "scaling": "strong", "elements": total, "elements_per_rank": n_local, "steps": steps,
        "ms_per_step": step_ms, "value": total_bytes / (step_ms * 1e-3) / 1e9, "unit": "GB/s",
        "per_gpu_gbs": total_bytes / (step_ms * 1e-3) / 1e9 / rt.world,
        "exchange": ("peer memory: cb_amax_peer_exchange, one 64-bit store per peer over NVLink + a bounded wait"
                     if peer is not None else "none (one rank)" if dist is None
                     else f"NCCL all_reduce(MAX) of one float32 (peer-memory form not used: {peer_why})"),
        "phase_ms_max_over_ranks": dict(zip(names, worst)),
        "with_nccl_all_reduce": (None if nccl_ms is None else
                                 {"ms_per_step": nccl_ms, "phase_ms_max_over_ranks": dict(zip(names, nccl_worst))}),
        "phase_gbs_per_gpu": {"amax": n_local * 2 / (worst[0] * 1e-3) / 1e9, "cast": n_local * 3 / (worst[2] * 1e-3) / 1e9,
                              "dequantize": n_local * 3 / (worst[3] * 1e-3) / 1e9},
        "amax": a, "scale_bits": int(scale_bits.item()),
        "checksums": {"sum_codes": int(sums[0].item()), "sum_codes_squared": int(sums[1].item()),
                      "sum_dequantized_bits": int(sums[2].item()),
                      "note": "summed over all ranks; equal values at N = 1, 2, 4, 8 mean identical codes and outputs"},
    }
    del x, q, y
    torch.cuda.empty_cache()
    return rec_out


def sharded_w8a16(rt: Runtime, peaks, checks, M=2048):
    """W8A16 linear at M = 2048 with the output features split over the ranks (activations replicated, no
    collective inside the op).  Device time of the local GEMM per rank, max over ranks."""
    import cublade_b200 as cb
    from cublade_b200.sharding import shard_range, shard_w8a16_layer
    from tests.golden import cases

    device = rt.device
    N_, K_ = cases.W8A16_N, cases.W8A16_K
    w, _, _ = cases.w8a16_weight(False)
    full = cb.cuBladeW8A16LinearLayer(K_, N_, bias=False, dtype=torch.bfloat16)
    full.quantize(w.to(device))
    full = full.to(device)
    n0, n1 = shard_range(N_, rt.rank, rt.world)
    import copy

    mine = shard_w8a16_layer(copy.deepcopy(full), rt.rank, rt.world).to(device)
    x = cases.w8a16_activations(M).to(device)
    y_full, y_mine = full(x), mine(x)
    checks.append((f"w8a16 sharded over output features: rank {rt.rank}'s slice equals the unsharded layer's columns",
                   bool(torch.equal(y_mine, y_full[:, n0:n1]))))
    g = rt.capture(lambda: [mine(x) for _ in range(10)])
    ms, _ = rt.time_graphs([g], 10, min_s=0.1, collective=True)
    ms = rt.max_over_ranks(ms)
    flops = 2.0 * M * N_ * K_
    tf = flops / (ms * 1e-3) / 1e12
    return {"workload": f"w8a16_linear M={M} N={N_} K={K_}, output features over {rt.world} rank(s), activations replicated",
            "scaling": "strong", "ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "per_gpu_tflops": tf / rt.world,
            "frac_of_burst_peak_per_gpu": tf / rt.world / peaks["bf16_tflops"], "collective": "none inside the op"}


def sharded_quantize_model(rt: Runtime, checks):
    """``quantize_model`` ("w8a16", lm_head excluded) on a random-init Llama-3-8B-shaped decoder (32 layers of
    q 4096x4096, k/v 1024x4096, o 4096x4096, gate/up 14336x4096, down 4096x14336, bf16, on the GPU), every Linear's
    output rows split over the ranks.  Wall time of the call (synchronised), weight traffic per rank, and one
    layer's codes and scales against the CPU oracle."""
    import torch.nn as nn

    from cublade_b200.sharding import quantize_model_sharded, shard_range
    from oracle import oracle as O

    device = rt.device
    H, I, KV, L = 4096, 14336, 1024, 32
    shapes = {"q_proj": (H, H), "k_proj": (KV, H), "v_proj": (KV, H), "o_proj": (H, H), "gate_proj": (I, H),
              "up_proj": (I, H), "down_proj": (H, I)}
    source = "plain nn.Module tree with the decoder's 224 Linear shapes"
    model = None
    try:  # the real architecture when transformers is importable (random init, no checkpoint involved)
        from transformers import LlamaConfig, LlamaForCausalLM

        cfg = LlamaConfig(hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=32,
                          num_key_value_heads=8, vocab_size=128256, tie_word_embeddings=False, torch_dtype=torch.bfloat16)
        with torch.device("meta"):
            model = LlamaForCausalLM(cfg).to(torch.bfloat16)
        model = model.to_empty(device=device)
        source = "transformers LlamaForCausalLM(LlamaConfig Llama-3-8B sizes), random init"
    except Exception as exc:  # pragma: no cover - depends on the installed transformers
        source += f" (transformers model not used: {type(exc).__name__})"
        layers = nn.ModuleList()
        with torch.device(device):
            for _ in range(L):
                blk = nn.Module()
                for name, (o, i) in shapes.items():
                    setattr(blk, name, nn.Linear(i, o, bias=False, dtype=torch.bfloat16))
                layers.append(blk)
        model = nn.Module()
        model.layers = layers
    gen = torch.Generator(device=device).manual_seed(5)
    linears = [(n, m) for n, m in model.named_modules() if isinstance(m, nn.Linear) and "lm_head" not in n]
    with torch.no_grad():
        for _, m in linears:
            m.weight.copy_(torch.randn(m.weight.shape, generator=gen, device=device, dtype=torch.float32) * 0.02)
    probe_name, probe = linears[0]
    a, b = shard_range(probe.out_features, rt.rank, rt.world)
    probe_rows = probe.weight.detach()[a:b].cpu()
    elems = sum(m.weight.numel() for _, m in linears)
    local = sum((lambda r: (r[1] - r[0]) * m.in_features)(shard_range(m.out_features, rt.rank, rt.world)) for _, m in linears)
    rt.barrier()
    t0 = time.perf_counter()
    quantize_model_sharded(model, rt.rank, rt.world, "w8a16", exclude_modules=["lm_head"])
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    rt.barrier()
    dt = rt.max_over_ranks(dt)
    mod = dict(model.named_modules())[probe_name]
    q_ref, s_ref = O.int8_quantize_channel(probe_rows)
    checks.append((f"quantize_model sharded: rank {rt.rank}'s rows of {probe_name} equal the CPU oracle's codes",
                   bool(torch.equal(mod.int8_weights.cpu(), q_ref))))
    checks.append((f"quantize_model sharded: rank {rt.rank}'s scales of {probe_name} equal the CPU oracle's",
                   bool(torch.equal(mod.scales.cpu().view(torch.int16), s_ref.to(torch.bfloat16).view(torch.int16)))))
    n_layers = sum(1 for m in model.modules() if type(m).__name__ == "cuBladeW8A16LinearLayer")
    rec = {"workload": f"quantize_model w8a16 on a Llama-3-8B-shaped decoder ({len(linears)} Linear layers, {elems / 1e9:.2f} G "
                       f"weights, bf16), output rows of every Linear over {rt.world} rank(s)",
           "model": source, "scaling": "strong", "layers_replaced": n_layers, "seconds": dt,
           "weight_elements_per_rank": int(local), "gbs_per_rank": local * 3 / dt / 1e9,
           "value": elems * 3 / dt / 1e9, "unit": "GB/s of algorithmic weight traffic (3 B/element), whole job",
           "note": "wall time of the Python call, one Linear after the other; the quantize kernels themselves account for "
                   f"{local * 3 / 6.0e12 * 1e3:.1f} ms of it at 6 TB/s"}
    del model
    torch.cuda.empty_cache()
    return rec


# --------------------------------------------------------------------------------------
# reference arms
# --------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """CPU formulation of the same step on this host's cores (rank 0 only; other ranks do nothing)."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)  # launchers such as torchrun pin OMP_NUM_THREADS=1
    if args.workload in LINEAR_WORKLOADS:
        from cublade_b200 import workloads as W
        from oracle import oracle as O

        a8 = args.workload == "w8a8"
        forward = O.w8a8_forward if a8 else O.w8a16_forward
        M = min(args.m, 64)
        w, x, _ = W.w8a16_case(M)
        lay = O.w4a16_quantize(w, torch.bfloat16) if args.workload == "w4a16" else O.w8a16_quantize(w, torch.bfloat16)
        forward(x, lay)
        steps = max(1, min(args.steps, 5))
        t0 = time.perf_counter()
        for _ in range(steps):
            forward(x, lay)
        dt = (time.perf_counter() - t0) / steps
        v = 2.0 * M * 14336 * 4096 / dt / 1e12
        sample = f"first {M} of {args.m} activation rows per step (reference CPU branch of the layer), {steps} steps"
        print(json.dumps({"impl": "reference", "metric": linear_metric(args.workload), "value": v, "unit": "TFLOP/s",
                          "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                          "dtype": "int8" if a8 else "bf16", "data": "synthetic",
                          "config": linear_config(args.workload, args.m),
                          "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                           "sample": sample},
                          "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    wl = WORKLOADS[args.workload](None)
    x = wl.cpu_input()
    cores = torch.get_num_threads()
    for _ in range(max(1, min(args.warmup, 2))):
        wl.cpu_step(x)
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        wl.cpu_step(x)
    dt = (time.perf_counter() - t0) / steps
    value = wl.bytes_per_step / dt / 1e9
    sample = f"full tensor {tuple(x.shape)}, mean of {steps} steps (steps capped at 20), PyTorch CPU formulation"
    print(json.dumps({
        "impl": "reference", "metric": "quant/dequant GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
        "l2_policy": "n/a (CPU)", "launch": "n/a (CPU)",
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


_REF_GPU_STAGE = r"""
import json, sys, torch
sys.path.insert(0, {root!r})
from oracle.build_ref import load_ref
from cublade_b200 import workloads as W
stage, name = {stage!r}, {name!r}
def timed(fn, n=50):
    for _ in range(5): fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(n): fn()
    b.record(); torch.cuda.synchronize()
    return a.elapsed_time(b) / n * 1e3
if name == "fp8_tensor":
    xs = [W.fp8_tensor_case().cuda() for _ in range(12)]
elif name == "int8_channel":
    xs = [W.int8_channel_case().cuda() for _ in range(3)]
else:
    x0 = W.int8_group_case().view(-1, 128)
    xs = [x0.cuda() for _ in range(2)]
i = [0]
def nxt(seq):
    i[0] += 1
    return seq[i[0] % len(seq)]
out = {{}}
if stage == "quant":
    m = load_ref("cublade_quantize_per_tensor_fp8" if name == "fp8_tensor" else "cublade_quantize_int8")
    fn = {{"fp8_tensor": lambda: m.quantize_per_tensor_fp8(nxt(xs), 1e-12),
          "int8_channel": lambda: m.quantize_per_channel_int8(nxt(xs), 1e-12),
          "int8_group": lambda: m.quantize_per_group_int8(nxt(xs), 128, 1e-12)}}[name]
    out["quantize_us"] = timed(fn)
else:
    import cublade_b200 as cb
    if name == "fp8_tensor":
        qs = [cb.quantize_tensor(x, dtype=torch.float8_e4m3fn, mode="tensor") for x in xs]
    elif name == "int8_channel":
        qs = [cb.quantize_tensor(x, dtype=torch.int8, mode="channel") for x in xs]
    else:
        qs = [cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=128, ch_axis=-1) for x in xs]
    m = load_ref("cublade_dequantize_per_tensor_fp8" if name == "fp8_tensor" else "cublade_dequantize_int8")
    def dq():
        q = nxt(qs)
        if name == "fp8_tensor": return m.dequantize_per_tensor_fp8(q.data, q.scale, torch.bfloat16)
        if name == "int8_channel": return m.dequantize_per_channel_int8(q.data, q.scale, torch.bfloat16)
        return m.dequantize_per_group_int8(q.data, q.scale, 128, torch.bfloat16)
    out["dequantize_us"] = timed(dq)
print("REFGPU " + json.dumps(out))
"""


def run_reference_gpu(args, rank):
    """The reference's own CUDA extensions (built unmodified into oracle/_ref by oracle/build_ref.py) timed on this GPU
    with CUDA events over rotating buffers, eager launches as its Python API issues them.  Each extension runs in a
    process of its own.  Context for the kernel-vs-kernel comparison; not the arm the speed-up is quoted against."""
    if rank != 0:
        return
    name = args.workload
    built = (ROOT / "oracle" / "_ref" / "cublade_quantize_int8" / "cublade_quantize_int8.so").exists()
    if name not in WORKLOADS or name == "rmsnorm_int8" or not built or not torch.cuda.is_available():
        why = ("no reference kernel for this workload" if name not in ("int8_channel", "fp8_tensor", "int8_group")
               else "oracle/_ref is not built (run oracle/build_ref.py where the reference checkout exists)" if not built
               else "no CUDA device")
        print(json.dumps({"impl": "reference_gpu", "unavailable": why}))
        return
    res = {}
    for stage in ("quant", "dequant"):
        code = _REF_GPU_STAGE.format(root=str(ROOT), stage=stage, name=name)
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=900)
        line = [ln for ln in r.stdout.splitlines() if ln.startswith("REFGPU ")]
        if r.returncode != 0 or not line:
            print(json.dumps({"impl": "reference_gpu", "unavailable": f"stage {stage} failed: {r.stderr[-300:]}"}))
            return
        res.update(json.loads(line[0][7:]))
    wl = WORKLOADS[name](None)
    ms = (res["quantize_us"] + res["dequantize_us"]) * 1e-3
    print(json.dumps({"impl": "reference_gpu", "metric": "quant/dequant GB/s", "value": wl.bytes_per_step / (ms * 1e-3) / 1e9,
                      "unit": "GB/s", "n_gpus": 1, "ms_per_step": ms, "higher_is_better": True, "dtype": wl.dtype,
                      "data": "synthetic", "config": wl.config(), "kernels_us": res,
                      "launch": "eager launches through the reference's extension functions (it allocates its outputs "
                                "and zero-fills its scratch inside every call)"}))


def linear_metric(kind):
    return ("W8A8 TOPS (2*M*N*K per step, activation quantization included)" if kind == "w8a8" else
            "W4A16 TFLOPS" if kind == "w4a16" else "W8A16 TFLOPS")


def linear_config(kind, M):
    return {"workload": f"{kind}_linear M={M} N=14336 K=4096 {'int4' if kind == 'w4a16' else 'int8'} per-output-channel "
                        "weights, bf16 activations" + (" quantized per token to int8 in the step" if kind == "w8a8" else ""),
            "seed": 3}


def run_linear(args, rt: Runtime):
    """--workload w8a16 | w8a8 | w4a16: the linear layer of the benchmark configuration (N=14336, K=4096, weights
    quantized per output channel from N(0, 0.02), bf16 activations N(0,1)), M = --rows.  A step is one forward.
    With N > 1 ranks the output features are sharded (strong scaling, no collective)."""
    import cublade_b200 as cb
    from cublade_b200 import workloads as W
    from cublade_b200.sharding import shard_range

    peaks = _peaks()
    device, rank, world = rt.device, rt.rank, rt.world
    M, N_, K_ = args.m, 14336, 4096
    w, x_host, _ = W.w8a16_case(M)
    n0, n1 = shard_range(N_, rank, world)
    a8, a4 = args.workload == "w8a8", args.workload == "w4a16"
    layer_cls = (cb.quantization.cuBladeW8A8LinearLayer if a8 else
                 cb.quantization.cuBladeW4A16LinearLayer if a4 else cb.cuBladeW8A16LinearLayer)
    tensor_bound = M >= 1024
    w_bytes = (n1 - n0) * K_ // (2 if a4 else 1)
    # HBM-bound shapes (M < 1024): the weights would stay in the 126 MB L2 between replays, so the timed graph walks
    # over `sets` copies of the layer (> 2x L2 in total) and every forward streams its weights from HBM
    sets = 1 if tensor_bound else max(2, -(-2 * L2_BYTES // w_bytes) + 1)
    layers = []
    for _ in range(sets):
        lay = layer_cls(K_, n1 - n0, bias=False, dtype=torch.bfloat16)
        lay.quantize(w[n0:n1].to(device))
        layers.append(lay.to(device))
    layer = layers[0]
    x_pinned = x_host.pin_memory()
    y_pinned = torch.empty(M, n1 - n0, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    warmup, K = max(args.warmup, 3), args.steps
    for _ in range(warmup):
        for lay in layers:
            lay(x)
    g = rt.capture(lambda: [lay(x) for lay in layers])
    K = -(-K // sets) * sets  # whole walks over the weight sets
    with ClockSampler(rt.local_rank) as clocks:
        ms, reps = rt.time_graphs([g] * (K // sets), K, MIN_REGION_S, True)
    ms = rt.max_over_ranks(ms)
    for _ in range(3):
        layer(x_pinned.to(device, non_blocking=True))
    rt.barrier()
    steps_e2e = max(3, min(K, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps_e2e):
        y = layer(x_pinned.to(device, non_blocking=True))
        y_pinned.copy_(y, non_blocking=True)
    e1.record()
    rt.barrier()
    e2e_ms = rt.max_over_ranks(e0.elapsed_time(e1) / steps_e2e)
    if rank != 0:
        return
    flops = 2.0 * M * N_ * K_
    tf = flops / (ms * 1e-3) / 1e12
    local_tf = tf / world
    bytes_local = w_bytes + 2 * (n1 - n0) + 2 * M * K_ + 2 * M * (n1 - n0)
    roof = ({"bound": "tensor", "achieved": local_tf, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
             "frac": local_tf / peaks["bf16_tflops_sustained"], "frac_of_burst_peak": local_tf / peaks["bf16_tflops"],
             "peak_note": "sustained cuBLAS bf16 figure: the kernel is timed back to back inside a long loop"}
            if tensor_bound else
            {"bound": "hbm", "achieved": bytes_local / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
             "frac": bytes_local / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})
    roof.update({"kernel": "w8a16_tc_kernel (tcgen05/TMEM)" if M >= 17 else "w8a16_stream_kernel", "traffic": None,
                 "peak_source": peaks["source"], "avg_launch_us": ms * 1e3})
    per_step = 2 if a8 else 1
    if a4:
        per_step = 1 if M <= 16 else 2
        roof["kernel"] = "w4a16_stream_kernel" if M <= 16 else "w4_unpack_kernel + " + roof["kernel"]
    if a8:
        roof["kernel"] = "w8a8_tc_kernel (tcgen05 kind::i8) + per-token quantize_segments_kernel"
        roof["peak_note"] = ("measured cuBLAS bf16 figure; no int8 peak was measured on this pool, the integer path's "
                             "nominal rate is twice the bf16 one")
    out = {"metric": linear_metric(args.workload), "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": K,
           "repeats": reps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
           "vs_baseline": None, "dtype": "int8" if a8 else "bf16", "data": "synthetic",
           "config": linear_config(args.workload, M),
           "l2_policy": ("back-to-back replays; weights (58.7 MB) + activations stay L2-resident, the shape is tensor-bound"
                         if tensor_bound else
                         f"each step streams its weights from HBM: the graph walks over {sets} copies of the layer "
                         f"({sets * w_bytes / 1e6:.0f} MB of quantized weights, L2 is 126 MB)"),
           "launch": "one CUDA graph per step" if sets == 1 else f"one CUDA graph per {sets} steps",
           "sharding": f"output features over {world} rank(s)",
           "clocks": clocks.summary(),
           "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K_ * 2,
                   "d2h_bytes_per_step": M * (n1 - n0) * 2, "ms_per_step": e2e_ms, "steps": steps_e2e},
           "gpu_launches": K * reps * per_step,
           "gpu_launches_note": f"{per_step} kernel(s) of libcublade_b200.so per step, replayed from a CUDA graph",
           "roofline": roof}
    if not args.no_cpu_baseline:
        from oracle import oracle as O

        torch.set_num_threads(os.cpu_count() or 1)
        ms_cpu = min(M, 64)
        lay = O.w8a16_quantize(w, torch.bfloat16)
        fwd = O.w8a8_forward if a8 else O.w8a16_forward
        fwd(x_host[:ms_cpu], lay)
        t0 = time.perf_counter()
        fwd(x_host[:ms_cpu], lay)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": 2.0 * ms_cpu * N_ * K_ / dt / 1e12, "unit": "TFLOP/s",
                               "cores": torch.get_num_threads(), "kind": "port",
                               "sample": f"first {ms_cpu} activation rows, one forward after one warm-up "
                                         "(reference CPU branch of the layer)"}
    print(json.dumps(out))


def cpu_baseline(wl, budget_s=12.0):
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    x = wl.cpu_input()
    wl.cpu_step(x)  # warm-up
    best, reps, t_all = None, 0, time.perf_counter()
    while reps < 3 or (time.perf_counter() - t_all < budget_s and reps < 10):
        t0 = time.perf_counter()
        wl.cpu_step(x)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        reps += 1
    return {"value": wl.bytes_per_step / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"tensor of {tuple(x.shape)} ({x.numel()} elements), best of {reps} "
                      "(PyTorch CPU formulation of the reference ops)"}


def single_gpu_extras(rt: Runtime, peaks, K, warmup):
    """The other configurations and the rows next to the path, one GPU: `configs`, `next_rows`, `w8a16`."""
    device = rt.device
    cfgs = {}
    for key, cls in (("1_fp8_per_tensor_4096x4096", Fp8TensorWorkload),
                     ("3_int8_per_group128_16384x8192", Int8GroupWorkload)):
        w2 = cls(device)
        r2 = measure_quant(rt, w2, min(K, 100), warmup, collective=False, min_s=0.1)
        cfgs[key] = quant_record(w2, r2, peaks, 1)
        del w2, r2
        torch.cuda.empty_cache()
    cfgs["4_w8a16_linear"] = w8a16_table(rt, peaks)
    cfgs["4p_w8a16_linear_llm_int8"] = w8a16_table(rt, peaks, outliers=True)
    return {"configs": cfgs, "next_rows": next_rows(rt, peaks, K, warmup),
            "w8a16": {k: {"us": v["us"], "tflops": v["tflops"], "gbs": v["gbs"], "bound": v["roofline"]["bound"],
                          "frac": v["roofline"]["frac"]} for k, v in cfgs["4_w8a16_linear"]["per_m"].items()}}


def single_gpu_extras_in_child(K, warmup, local_rank):
    """Runs single_gpu_extras() in a process of its own on the same GPU and returns its three keys.  These are some
    hundred thousand launches of a dozen kernels beside the headline measurement; a CUDA error in any of them is
    sticky for the process that met it, and it must not cost the line the headline (already measured by the caller) and
    the sharded forms.  A child that fails is reported under the same keys."""
    env = {k: v for k, v in os.environ.items()
           if k not in ("RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "MASTER_ADDR", "MASTER_PORT")
           and not k.startswith("TORCHELASTIC")}
    env["LOCAL_RANK"] = str(local_rank)
    cmd = [sys.executable, str(Path(__file__).resolve()), "--section", "single_gpu_extras", "--steps", str(K),
           "--warmup", str(warmup)]
    try:
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if r.returncode == 0 and lines:
            return json.loads(lines[-1])
        why = f"exit status {r.returncode}: {r.stderr.strip().splitlines()[-1][:300] if r.stderr.strip() else 'no output'}"
    except subprocess.TimeoutExpired:
        why = "no result within 1200 s"
    return {k: {"error": why} for k in ("configs", "next_rows", "w8a16")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="int8_channel", choices=sorted(WORKLOADS) + list(LINEAR_WORKLOADS))
    ap.add_argument("--m", "--rows", dest="m", type=int, default=2048,
                    help="activation rows for the linear workloads (spell it --rows under torchrun, whose own parser "
                         "rejects --m as an ambiguous abbreviation)")
    ap.add_argument("--impl", default="cublade_b200", choices=["cublade_b200", "reference", "reference_gpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only: no `configs`, no `sharded`")
    ap.add_argument("--selftest", action="store_true", help="exit with status 1 when a sharded-form check fails")
    ap.add_argument("--sharded-elements-log2", type=int, default=33,
                    help="size of the sharded per-tensor FP8 tensor (default 2^33 elements; tests use less)")
    ap.add_argument("--section", default="", help=argparse.SUPPRESS)  # internal: see single_gpu_extras_in_child
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        return run_reference(args, rank, world)
    if args.impl == "reference_gpu":
        return run_reference_gpu(args, rank)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    from cublade_b200 import _native as N

    N.lib()  # fail loudly if the extension is missing
    rt = Runtime(device, dist, rank, world, local_rank)
    try:
        if args.workload in LINEAR_WORKLOADS:
            run_linear(args, rt)
            return 0
        if args.section == "single_gpu_extras":
            print(json.dumps(single_gpu_extras(rt, _peaks(), args.steps, max(args.warmup, 3))))
            return 0
        warmup = max(args.warmup, 3)
        K = args.steps
        peaks = _peaks()
        wl = WORKLOADS[args.workload](device)
        rec = measure_quant(rt, wl, K, warmup, collective=True)
        out = None
        if rank == 0:
            sub = quant_record(wl, rec, peaks, world)
            out = {
                "metric": "quant/dequant GB/s", "value": sub["value"], "unit": "GB/s", "n_gpus": world, "steps": K,
                "repeats": rec["repeats"], "timed_region_s": rec["timed_region_s"],
                "warmup": warmup, "ms_per_step": rec["ms_per_step"], "eager_ms_per_step": rec["eager_ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
                "config": wl.config(), "l2_policy": wl.l2_policy(),
                "launch": "the K steps are consecutive nodes of CUDA graphs (at most 200 steps per graph); the K-step "
                          f"region is replayed `repeats` times so that it lasts at least {MIN_REGION_S} s",
                "clocks": rec["clocks"], "e2e": sub["e2e"],
                "gpu_launches": int(K * rec["repeats"] * wl.launches_per_step),
                "gpu_launches_note": f"{wl.launches_per_step} kernels of libcublade_b200.so per step, replayed from CUDA graphs",
                "roofline": sub["roofline"], "kernels": sub["kernels"],
            }
        del wl
        torch.cuda.empty_cache()
        checks = []
        if not args.no_extras:
            # ---- the other configurations, one GPU each: rank 0 measures, the others wait at the barrier ----
            if rank == 0:
                out.update(single_gpu_extras_in_child(K, warmup, local_rank))
            rt.barrier()
            # ---- the sharded forms, all ranks ----
            sh = {"fp8_per_tensor_2p%d" % args.sharded_elements_log2:
                  sharded_fp8(rt, checks, total=1 << args.sharded_elements_log2,
                              chunk=min(1 << 27, 1 << args.sharded_elements_log2))}
            sh["w8a16_m2048_output_features"] = sharded_w8a16(rt, peaks, checks)
            sh["quantize_model_llama3_8b_shape"] = sharded_quantize_model(rt, checks)
            # every rank's verdicts, gathered
            ok_local = all(ok for _, ok in checks)
            ok_all = ok_local
            if dist is not None:
                t = torch.tensor([1.0 if ok_local else 0.0], device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                ok_all = bool(t.item() == 1.0)
            if rank == 0:
                out["sharded"] = sh
                out["selftest"] = {"passed": ok_all, "ranks": world,
                                   "checks_rank0": [{"check": c, "ok": ok} for c, ok in checks]}
            if args.selftest and not ok_all:
                if rank == 0:
                    print(json.dumps(out))
                return 1
        if rank == 0:
            if not args.no_cpu_baseline:
                out["cpu_baseline"] = cpu_baseline(WORKLOADS[args.workload](None))
            print(json.dumps(out))
        return 0
    finally:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main() or 0)
