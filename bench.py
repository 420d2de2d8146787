#!/usr/bin/env python
"""Benchmark of the quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  The default workload is the INT8 per-channel quantize + dequantize of a
bf16 8192 x 8192 weight (the configuration the GB/s metric is quoted on); a *step* is one
quantize plus one dequantize of that tensor.  ``value`` is algorithmic GB/s with inputs resident
in HBM, ``e2e`` the same through the public API from pinned host buffers, ``roofline`` the
dominant kernel against the measured HBM peak, ``cpu_baseline`` the PyTorch CPU formulation on
this host's cores.  With N > 1 (one process per GPU under torch.distributed.run) every rank
runs the same per-GPU workload on its own rows (weak scaling, no data-path collective) and the
time is the max over ranks.  ``--impl reference`` times the CPU formulation instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
# dram bytes (read + write) of one launch of the dominant kernel from an ncu capture of this
# workload (profiles/quant_segments_int8_channel_8192x8192.md: 134.2 MB read + 29.0 MB written; the
# rest of the 67 MB of codes was still dirty in the 126 MB L2 when the captured launch ended).
NCU_TRAFFIC_BYTES = {"int8_channel": 163_215_616, "fp8_tensor": None, "int8_group": None}


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
# workloads: each returns an object with .step(i), .step_e2e(i), algorithmic bytes, etc.
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
        self.kernel_ms = []  # (quant_ms, dequant_ms) per timed step

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
        return {"workload": f"int8_per_channel_axis0_quant+dequant bf16 {self.rows}x{self.cols}",
                "bytes_per_step": self.bytes_per_step,
                "l2_policy": f"rotating {self.sets} buffer sets ({self.sets * self.n * 5 / 1e6:.0f} MB footprint > 2x L2); "
                             "dequantize reads codes written two steps earlier",
                "seed": 1}

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.int8, mode="channel", ch_axis=0)

    def dequantize(self, qt):
        import cublade_b200 as cb

        return cb.dequantize_tensor(qt)

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
    dominant = "cast_tensor_kernel (per-tensor FP8 cast, second pass)"

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
        self.kernel_ms = []

    def config(self):
        c = super().config()
        c["workload"] = f"fp8_e4m3_per_tensor_quant+dequant bf16 {self.rows}x{self.cols} (16 outliers of 300)"
        c["seed"] = 0
        return c

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
        self.kernel_ms = []

    def config(self):
        c = super().config()
        c["workload"] = f"int8_per_group_{self.group}_quant+dequant bf16 {self.rows}x{self.cols} (Student-t nu=3 x0.5)"
        c["seed"] = 2
        return c

    def quantize(self, x):
        import cublade_b200 as cb

        return cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=self.group, ch_axis=-1)

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s = O.int8_quantize_group(x_cpu.view(-1, self.group), self.group)
        return O.int8_dequantize_rows(q, s, torch.bfloat16)


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
        self.kernel_ms = []

    def config(self):
        c = super().config()
        c["workload"] = (f"rmsnorm+int8_per_token_quant (fused, 3 B/elem instead of 7 unfused) + dequant bf16 "
                         f"{self.rows}x{self.cols} (Student-t nu=3 x0.5)")
        c["seed"] = 2
        return c

    def quantize(self, x):
        from cublade_b200.quantization import rmsnorm_quantize_tensor

        return rmsnorm_quantize_tensor(x, self.gain)

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s, _, _ = O.rmsnorm_quantize(x_cpu, self.gain_host)
        return O.int8_dequantize_rows(q, s, torch.bfloat16)


class Fp8ShardedWorkload(Int8ChannelWorkload):
    """Per-tensor FP8 E4M3 quantize + dequantize of ONE bf16 tensor of 2^33 elements, N(0,1), rows
    split contiguously over the ranks (strong scaling): local amax, one NCCL max-allreduce of a
    float32, cast; dequantize is local.  Two HBM passes over x are compulsory (5 B/elem) because a
    2 GiB..16 GiB shard cannot stay on chip between the amax and the cast."""

    name = "fp8_sharded"
    dtype = "e4m3"
    dominant = "cast_tensor_kernel (per-tensor FP8 cast over the local shard)"
    use_graphs = False
    scaling = "strong"
    TOTAL = 1 << 33
    CHUNK = 1 << 27

    def __init__(self, device, world=1, rank=0, total=None):
        from cublade_b200 import workloads as W
        from cublade_b200.sharding import shard_range

        self.total = total or self.TOTAL
        self.rows, self.cols = self.total // 8192, 8192
        self.world, self.rank, self.sets = world, rank, 1
        nchunks = self.total // self.CHUNK
        c0, c1 = shard_range(nchunks, rank, world)
        self.n = (c1 - c0) * self.CHUNK
        self.device = device
        if device is None:
            self.x_host = W.sharded_fp8_chunk(0, self.CHUNK, device="cpu")
            self.x, self.y_host = [], None
        else:
            x = torch.empty(self.n, dtype=torch.bfloat16, device=device)
            for i, c in enumerate(range(c0, c1)):
                x[i * self.CHUNK:(i + 1) * self.CHUNK] = W.sharded_fp8_chunk(c, self.CHUNK, device=device)
            self.x = [x.view(-1, 8192)]
            self.x_host = torch.empty(self.CHUNK, dtype=torch.bfloat16).pin_memory()
            self.x_host.copy_(x[: self.CHUNK])
            self.y_host = torch.empty(self.CHUNK, dtype=torch.bfloat16).pin_memory()
        # algorithmic bytes of the WHOLE tensor per step: quant 5 B/elem, dequant 3 B/elem
        self.q_bytes_total = self.total * 5
        self.dq_bytes_total = self.total * 3
        self.bytes_per_step_total = self.q_bytes_total + self.dq_bytes_total
        self.q_bytes = self.n * 3  # the cast kernel alone on the local shard (x read + q write)
        self.dq_bytes = self.n * 3
        self.bytes_per_step = self.n * 8
        self.qt = [None]
        self.launches_per_step = 3

    def config(self):
        return {"workload": f"fp8_e4m3_per_tensor_sharded_quant+dequant bf16 2^{self.total.bit_length() - 1} elements "
                            f"N(0,1) over {self.world} GPU(s), NCCL max-allreduce of the fp32 amax",
                "bytes_per_step": self.bytes_per_step_total,
                "l2_policy": "inputs larger than L2 (local shard >= 2 GiB)", "seed": 4}

    def quantize(self, x):
        from cublade_b200.sharding import quantize_tensor_sharded

        return quantize_tensor_sharded(x, dtype=torch.float8_e4m3fn)

    def step_e2e(self, i):
        # one 2^27-element chunk per step from pinned host memory and back (the full shard would
        # only time PCIe); the amax exchange still runs
        x = self.x_host.to(self.device, non_blocking=True)
        y = self.dequantize(self.quantize(x))
        self.y_host.copy_(y, non_blocking=True)
        return y

    e2e_h2d = property(lambda self: self.CHUNK * 2)
    e2e_d2h = property(lambda self: self.CHUNK * 2)
    e2e_bytes = property(lambda self: self.CHUNK * 8)

    def cpu_step(self, x_cpu):
        from oracle import oracle as O

        q, s = O.fp8_quantize(x_cpu)
        return O.fp8_dequantize(q, s, torch.bfloat16)


WORKLOADS = {"int8_channel": Int8ChannelWorkload, "fp8_tensor": Fp8TensorWorkload, "int8_group": Int8GroupWorkload,
             "rmsnorm_int8": RmsnormInt8Workload,
             "fp8_sharded": Fp8ShardedWorkload}


def w8a16_extras(device, peaks, ms=(1, 16, 128, 2048)):
    """W8A16 linear (N=14336, K=4096, per-output-channel int8 weights, bf16 activations) timed per M:
    TFLOP/s and the roofline that bounds each shape (HBM for the weight stream, tensor for M=2048)."""
    from cublade_b200 import workloads as W
    import cublade_b200 as cb

    out = {}
    w, _, _ = W.w8a16_case(1)
    N_, K_ = 14336, 4096
    # HBM-bound shapes stream their weights: the timed graph walks over copies of the layer larger than 2x L2
    sets = -(-2 * L2_BYTES // (N_ * K_)) + 1
    layers = []
    for _ in range(sets):
        layer = cb.cuBladeW8A16LinearLayer(K_, N_, bias=False, dtype=torch.bfloat16)
        layer.quantize(w.to(device))
        layers.append(layer.to(device))
    side = torch.cuda.Stream()

    def graph_ms(fn, launches):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                fn()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / 2)
        return sorted(ts)[len(ts) // 2] / launches

    for M in ms:
        x = torch.randn(M, K_, device=device, dtype=torch.float32).to(torch.bfloat16)
        for lay in layers:
            lay(x)
        t = graph_ms(lambda: [lay(x) for lay in layers for _ in range(2)], 2 * sets) * 1e-3
        warm = graph_ms(lambda: [layers[0](x) for _ in range(10)], 10) * 1e-3
        flops = 2.0 * M * N_ * K_
        bytes_ = N_ * K_ + 2 * N_ + 2 * M * K_ + 2 * M * N_
        tf, gbs = flops / t / 1e12, bytes_ / t / 1e9
        bound = "tensor" if M >= 1024 else "hbm"
        frac = tf / peaks["bf16_tflops"] if bound == "tensor" else gbs / peaks["hbm_gbs"]
        out[f"M={M}"] = {"us": t * 1e6, "tflops": tf, "gbs": gbs, "bound": bound, "frac": frac,
                         "us_l2_warm": warm * 1e6, "tflops_l2_warm": flops / warm / 1e12,
                         "method": f"CUDA graph over {sets} copies of the layer ({sets * N_ * K_ / 1e6:.0f} MB of weights)"}
    return out


# --------------------------------------------------------------------------------------
def run_reference(args, rank, world):
    """CPU formulation of the same step on this host's cores (rank 0 only; other ranks do nothing)."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)  # launchers such as torchrun pin OMP_NUM_THREADS=1
    if args.workload in ("w8a16", "w8a8", "w4a16"):
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
        metric = ("W8A8 TOPS (2*M*N*K per step, activation quantization included)" if a8 else
                  "W4A16 TFLOPS" if args.workload == "w4a16" else "W8A16 TFLOPS")
        print(json.dumps({"impl": "reference", "metric": metric, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
                          "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "int8" if a8 else "bf16", "data": "synthetic",
                          "config": {"workload": f"{args.workload}_linear M={args.m} N=14336 K=4096"},
                          "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                           "sample": sample},
                          "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return
    wl = WORKLOADS[args.workload](None)
    if args.workload == "fp8_sharded":  # bounded sample: one 2^27-element chunk, scaled to the metric's unit
        wl.bytes_per_step = wl.CHUNK * 8
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
    cfg = wl.config()
    cfg["l2_policy"] = "n/a (CPU)"
    print(json.dumps({
        "impl": "reference", "metric": "quant/dequant GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_w8a16(args, rank, world, local_rank, device, dist):
    """--workload w8a16: the W8A16 linear of the benchmark configuration (N=14336, K=4096, int8 weights
    quantized per output channel from N(0, 0.02), bf16 activations N(0,1)), M = --m rows.  A step is
    one forward.  With N > 1 ranks the output features are sharded (strong scaling, no collective)."""
    import cublade_b200 as cb
    from cublade_b200 import _native as N
    from cublade_b200 import workloads as W
    from cublade_b200.sharding import shard_range

    peaks = _peaks()
    M, N_, K_ = args.m, 14336, 4096
    w, x_host, _ = W.w8a16_case(M)
    n0, n1 = shard_range(N_, rank, world)
    a8 = args.workload == "w8a8"  # int8 activations (quantized per token inside the step) on the integer tensor cores
    a4 = args.workload == "w4a16"  # 4-bit weights: half the weight bytes; M > 16 unpacks to int8 and runs the W8A16 path
    layer_cls = (cb.quantization.cuBladeW8A8LinearLayer if a8 else
                 cb.quantization.cuBladeW4A16LinearLayer if a4 else cb.cuBladeW8A16LinearLayer)
    layer = layer_cls(K_, n1 - n0, bias=False, dtype=torch.bfloat16)
    layer.quantize(w[n0:n1].to(device))
    layer = layer.to(device)
    # HBM-bound shapes (M < 1024): the 58.7 MB of weights would stay in the 126 MB L2 between replays, so the
    # timed graph walks over `sets` copies of the layer (> 2x L2 in total) and every forward streams from HBM.
    tensor_bound = M >= 1024
    w_bytes = (n1 - n0) * K_ // (2 if a4 else 1)
    sets = 1 if tensor_bound else max(2, -(-2 * 126_000_000 // w_bytes) + 1)
    layers = [layer]
    for _ in range(sets - 1):
        extra = layer_cls(K_, n1 - n0, bias=False, dtype=torch.bfloat16)
        extra.quantize(w[n0:n1].to(device))
        layers.append(extra.to(device))
    x_pinned = x_host.pin_memory()
    y_pinned = torch.empty(M, n1 - n0, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    warmup, K = max(args.warmup, 3), args.steps

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        for lay in layers:
            lay(x)
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for lay in layers:
                y_static = lay(x)
    for _ in range(warmup):
        g.replay()
    K = -(-K // sets) * sets  # whole walks over the weight sets
    replays = K // sets
    barrier()
    launches0 = N.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        barrier()
    ms = e0.elapsed_time(e1) / K
    # end to end: activations from pinned host memory, result back to the host
    for _ in range(3):
        layer(x_pinned.to(device, non_blocking=True))
    barrier()
    steps_e2e = max(3, min(K, 20))
    e0.record()
    for _ in range(steps_e2e):
        y = layer(x_pinned.to(device, non_blocking=True))
        y_pinned.copy_(y, non_blocking=True)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / steps_e2e
    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0].item()), float(t[1].item())
    if rank != 0:
        return
    flops = 2.0 * M * N_ * K_
    tf = flops / (ms * 1e-3) / 1e12
    local_tf = tf / world
    bytes_local = (n1 - n0) * K_ // (2 if a4 else 1) + 2 * (n1 - n0) + 2 * M * K_ + 2 * M * (n1 - n0)
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
    out = {"metric": ("W8A8 TOPS (2*M*N*K per step, activation quantization included)" if a8 else
                      "W4A16 TFLOPS" if a4 else "W8A16 TFLOPS"), "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": warmup,
           "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "int8" if a8 else "bf16", "data": "synthetic",
           "config": {"workload": f"{args.workload}_linear M={M} N={N_} K={K_} {'int4' if a4 else 'int8'} per-output-channel weights, bf16 activations"
                                  + (" quantized per token to int8 in the step" if a8 else ""),
                      "l2_policy": "back-to-back replays; weights (58.7 MB) + activations stay L2-resident, the shape is "
                                   "tensor-bound" if tensor_bound else
                                   f"each step streams its weights from HBM: the graph walks over {sets} copies of the layer "
                                   f"({sets * w_bytes / 1e6:.0f} MB of quantized weights, L2 is 126 MB)",
                      "launch": "one CUDA graph per step" if sets == 1 else f"one CUDA graph per {sets} steps", "seed": 3, "sharding": f"output features over {world} rank(s)"},
           "clocks": clocks.summary(),
           "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": M * K_ * 2,
                   "d2h_bytes_per_step": M * (n1 - n0) * 2, "ms_per_step": e2e_ms, "steps": steps_e2e},
           "gpu_launches": K * per_step,
           "gpu_launches_note": f"{per_step} kernel(s) of libcublade_b200.so per step, replayed from a CUDA graph",
           "roofline": roof}
    if not args.no_cpu_baseline and a8:
        from oracle import oracle as O

        torch.set_num_threads(os.cpu_count() or 1)
        ms_cpu = min(M, 64)
        lay = O.w8a16_quantize(w, torch.bfloat16)
        O.w8a8_forward(x_host[:ms_cpu], lay)
        t0 = time.perf_counter()
        O.w8a8_forward(x_host[:ms_cpu], lay)
        dt = time.perf_counter() - t0
        out["cpu_baseline"] = {"value": 2.0 * ms_cpu * N_ * K_ / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                               "kind": "port", "sample": f"first {ms_cpu} activation rows, one forward after one warm-up"}
    elif not args.no_cpu_baseline:
        # the reference's own CPU branch of the layer (x @ W.t() in the activation dtype), bounded sample
        from oracle import oracle as O

        torch.set_num_threads(os.cpu_count() or 1)
        ms_cpu = min(M, 64)
        lay = O.w8a16_quantize(w, torch.bfloat16)
        xs = x_host[:ms_cpu]
        O.w8a16_forward(xs, lay)
        t0 = time.perf_counter()
        O.w8a16_forward(xs, lay)
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
    nbytes = x.numel() * (8 if getattr(wl, "scaling", "weak") == "strong" else 6) + 0
    if getattr(wl, "scaling", "weak") != "strong":
        nbytes = wl.bytes_per_step
    return {"value": nbytes / best / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"tensor of {tuple(x.shape)} ({x.numel()} elements), best of {reps} "
                      "(PyTorch CPU formulation of the reference ops)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--workload", default="int8_channel", choices=sorted(WORKLOADS) + ["w8a16", "w8a8", "w4a16"])
    ap.add_argument("--m", "--rows", dest="m", type=int, default=2048,
                    help="activation rows for the linear workloads (spell it --rows under torchrun, whose own parser "
                         "rejects --m as an ambiguous abbreviation)")
    ap.add_argument("--impl", default="cublade_b200", choices=["cublade_b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-w8a16", action="store_true", help="skip the W8A16 TFLOP/s table")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

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
    if args.workload in ("w8a16", "w8a8", "w4a16"):
        run_w8a16(args, rank, world, local_rank, device, dist)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return
    warmup = max(args.warmup, 3)
    if args.workload == "fp8_sharded":
        wl = Fp8ShardedWorkload(device, world=world, rank=rank)
    else:
        wl = WORKLOADS[args.workload](device)
    wl.prime()
    use_graphs = getattr(wl, "use_graphs", True)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: the K-step loop is captured into CUDA graphs ------------------
    # Step i quantizes x[i % sets] and dequantizes the codes of set i+1, which were written
    # before the timed region (not in L2 any more).  Consecutive steps are nodes of ONE graph (up to
    # kChain steps per graph), so the loop pays one graph launch, not one per step; outputs of the
    # last `sets` steps stay allocated, so the written buffers rotate like the inputs do.
    for i in range(warmup):
        wl.step(i)
    torch.cuda.synchronize()
    K = args.steps
    kChain = 200
    side = torch.cuda.Stream()
    static_qt = list(wl.qt)
    chains = {}

    class Eager:  # same interface as a CUDA graph, launches through the Python API every time
        def __init__(self, fn, n):
            self.fn, self.n = fn, n

        def replay(self):
            for _ in range(self.n):
                self.fn()

    def chain(kind, n):
        """One CUDA graph holding n consecutive steps ("step"), quantize calls ("q") or dequantize calls ("dq")."""
        if (kind, n) in chains:
            return chains[(kind, n)]
        g = torch.cuda.CUDAGraph()
        ring = [None] * wl.sets
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for i in range(n):
                    out = []
                    if kind in ("step", "q"):
                        out.append(wl.quantize(wl.x[i % wl.sets]))
                    if kind in ("step", "dq"):
                        out.append(wl.dequantize(static_qt[(i + 1) % wl.sets]))
                    ring[i % wl.sets] = out
                del ring, out
        torch.cuda.synchronize()
        chains[(kind, n)] = g
        return g

    if not use_graphs:
        from cublade_b200.bindings.cuda.split_phase import amax_abs, cast_per_tensor

        # the dominant kernel alone: the cast over the local shard with a precomputed global amax
        amax_static = amax_abs(wl.x[0])
        eager_fns = {"step": lambda: wl.step(0),
                     "q": lambda: cast_per_tensor(wl.x[0], amax_static, torch.float8_e4m3fn),
                     "dq": lambda: wl.dequantize(static_qt[0])}

        def chain(kind, n):  # noqa: F811
            return Eager(eager_fns[kind], n)

    def timed(kind, n):
        parts = [chain(kind, kChain)] * (n // kChain) + ([chain(kind, n % kChain)] if n % kChain else [])
        chain(kind, warmup).replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for g in parts:
            g.replay()
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / n

    for kind in ("step", "q", "dq"):  # capture everything before the clock sampler and the timed regions start
        timed(kind, K)

    launches0 = N.launch_count()
    with ClockSampler(local_rank) as clocks:
        ms_per_step = timed("step", K)
        q_avg = timed("q", K)
        dq_avg = timed("dq", K)
    launches_per_step = wl.launches_per_step
    launches = K * launches_per_step
    captured = N.launch_count() - launches0  # 0: replays do not go through the library's host code
    if dist is not None:
        t = torch.tensor([ms_per_step], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item())
    strong = getattr(wl, "scaling", "weak") == "strong"
    step_bytes = wl.bytes_per_step_total if strong else world * wl.bytes_per_step
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # eager (no graph) pacing of the same step through the Python API, for information
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(min(K, 100)):
        wl.step(i)
    e1.record()
    barrier()
    eager_ms = e0.elapsed_time(e1) / min(K, 100)

    # ---- end to end through the public API from pinned host memory -----------------------------
    # Every step copies its input host -> device, runs quantize_tensor + dequantize_tensor, and
    # copies the result device -> host.  Steps alternate between two CUDA streams (two pinned
    # output buffers), so the upload of one step overlaps the download of the previous one on the
    # full-duplex PCIe link -- the ordinary way a caller pipelines this API.
    e2e_steps = max(4, min(K, 20))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    y_hosts = [wl.y_host, torch.empty_like(wl.y_host).pin_memory()]

    def e2e_pass(n):
        for i in range(n):
            st = streams[i & 1]
            with torch.cuda.stream(st):
                wl.y_host = y_hosts[i & 1]
                wl.step_e2e(i)
        for st in streams:
            st.synchronize()

    e2e_pass(4)
    barrier()
    t0 = time.perf_counter()
    e2e_pass(e2e_steps)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps  # host clock around fully synchronised passes
    barrier()
    if dist is not None:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * getattr(wl, "e2e_bytes", wl.bytes_per_step) / (e2e_ms * 1e-3) / 1e9

    if rank == 0:
        peaks = _peaks()
        achieved = wl.q_bytes / (q_avg * 1e-3) / 1e9
        out = {
            "metric": "quant/dequant GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": warmup, "ms_per_step": ms_per_step, "eager_ms_per_step": eager_ms, "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(), launch=f"the K steps are consecutive nodes of one CUDA graph (at most {kChain} steps per graph)" if use_graphs
                           else "eager launches through the Python API"),
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": wl.e2e_h2d, "d2h_bytes_per_step": wl.e2e_d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": int(launches), "gpu_launches_note": f"{launches_per_step} kernels of libcublade_b200.so per step, replayed from a CUDA graph",
            "roofline": {"bound": "hbm", "kernel": wl.dominant, "achieved": achieved, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "traffic": NCU_TRAFFIC_BYTES.get(wl.name), "algorithmic_bytes_per_launch": wl.q_bytes,
                         "avg_launch_us": q_avg * 1e3, "frac_of_nominal_8000": achieved / 8000.0},
            "kernels": {"quantize": {"avg_us": q_avg * 1e3, "gbs": achieved},
                        "dequantize": {"avg_us": dq_avg * 1e3, "gbs": wl.dq_bytes / (dq_avg * 1e-3) / 1e9,
                                       "frac": wl.dq_bytes / (dq_avg * 1e-3) / 1e9 / peaks["hbm_gbs"]}},
        }
        if not args.no_w8a16:
            out["w8a16"] = w8a16_extras(device, peaks)
        if not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(out))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
