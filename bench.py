#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload int8_8192 | int8_512 | int8_8192_presummed | int8_decode |
                                int4_w4a16 | int4_w4a16_decode | int4_w4a8 | int4_w4a8_decode |
                                int8_swiglu | dequant | rmsnorm_quant | layer_sweep] [--no-extras] [--no-cpu-baseline]

One "step" is one `solve` call over one batch of synthetic input.  The default workload is
the INT8 quantized matmul M=N=K=8192 (uniform int8 inputs, per-tensor scales and non-zero
zero points drawn from a fixed seed).

With N > 1 GPUs (launched under torchrun, one rank per GPU) the FIXED problem is sharded by
weight columns (strong scaling): rank r owns columns [r*N/g, (r+1)*N/g) of B as its own
contiguous slab, multiplies the replicated A by it, and the all-gather of C is fused into the
matmul's epilogue (every finished row segment is stored into every GPU's copy of C over
NVLink - through the NVSwitch multicast mapping where there is one - so after one
symmetric-memory barrier every rank holds the whole row-major C).  `value` = 2*M*N*K over the
max-over-ranks step time of that fused call.  The same JSON line also carries the matmul
without any gather (`gemm_only_ms`), with an NCCL all-gather + permute after it
(`nccl_gather_ms`), a `layers` object (the four projections of a transformer layer at
M = 8192, column-sharded the same way) and a `parity` object: outside the timed region every
rank checks sampled rows of its slab against the CPU oracle and that its fused-gather copy of
C equals the NCCL-gathered one byte for byte.

With N = 1 the line carries a `configs` object (the other shapes of the hot path: the small
512x512x1024 case, the 16-row decode shape, W4A16 at four group sizes, W4A8, dequantization)
each with its time, roofline fraction and - `reference_gpu` - the time of the reference's own
kernel recompiled for sm_100a on the same GPU in the same process (a baseline leg: it runs
after, never inside, the timed regions of this library).

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (CUDA events, max
over ranks); `sustained` repeats it over at least two seconds with its own clock record;
`e2e` is the same call with host buffers (pinned upload of A and B, download of C inside the
timed region); `roofline` describes the dominant kernel, timed with CUDA events;
`cpu_baseline` is the CPU oracle on a bounded sample of rows.

`--impl reference` times the reference's CPU path (the oracle port, all host threads) on a
bounded sample of rows of the same workload and prints the same line shape.
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

import numpy as np  # noqa: E402

METRIC = "quantized_matmul_throughput"
UNIT = "TOPS"
SEED = 2024

# NVIDIA's published dense figures for one B200 (context next to the measured denominators).
SPEC_INT8_TOPS = 4500.0
SPEC_F16_TFLOPS = 2250.0
SPEC_HBM_GBS = 8000.0

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of each workload's
# dominant kernel, from one ncu capture of that launch (bytes; absent where none was taken).
# Writes still sitting in L2 when the kernel ends are not in it.
NCU_TRAFFIC = {
    "int8_8192": 366.2e6,
    "int8_8192_presummed": 395.0e6,
    "int8_decode": 239.0e6,
    "int4_w4a16": 328.5e6,
    "int4_w4a8": 119.9e6,
    "dequant": 482.8e6,
    "rmsnorm_quant": 826.5e6,
}
TRAFFIC_NOTE = "ncu, one launch of the dominant kernel: dram__bytes_read.sum + dram__bytes_write.sum"

LAYERS = [("qkv", 8192, 10240), ("o_proj", 8192, 8192), ("gate_up", 8192, 57344), ("down", 28672, 8192)]


# ----------------------------------------------------------------------------- workloads
def workload_spec(name: str):
    if name == "int8_8192":
        return dict(op="mm_int8", M=8192, N=8192, K=8192, dtype="int8",
                    desc="INT8 zero-point/scale matmul M=N=K=8192, uniform int8 operands, "
                         "non-zero zero points (both sums needed)")
    if name == "int8_512":
        return dict(op="mm_int8", M=512, N=512, K=1024, dtype="int8",
                    desc="INT8 matmul M=512 K=1024 N=512 (the reference's CPU-runnable case); "
                         "launch-bound: 1.3 MB of operands stay in L2")
    if name == "int8_8192_presummed":
        return dict(op="mm_int8", M=8192, N=8192, K=8192, dtype="int8", presummed=True,
                    desc="INT8 matmul M=N=K=8192 as an inference engine would issue it: colsum(B) "
                         "cached with the weight handle, rowsum(A) delivered by the activation "
                         "producer - the tensor kernel alone, no pre-pass")
    if name == "int8_decode":
        return dict(op="mm_int8", M=16, N=28672, K=8192, dtype="int8",
                    desc="INT8 decode-shaped matmul M=16 K=8192 N=28672 (MLP up-projection, "
                         "activations round(N(0,20)))")
    if name == "int4_w4a16":
        return dict(op="mm_int4", M=4096, N=8192, K=8192, G=128, dtype="f16",
                    desc="W4A16 matmul M=4096 K=8192 N=8192 G=128 (packed INT4 weights, FP16 "
                         "activations: the reference's mm_int4 operator)")
    if name == "int4_w4a8":
        return dict(op="mm_int4a8", M=4096, N=8192, K=8192, dtype="int8",
                    desc="W4A8 matmul M=4096 K=8192 N=8192: packed INT4 weights, INT8 activations, "
                         "per-tensor scales and zero points")
    if name == "int4_w4a16_decode":
        return dict(op="mm_int4", M=16, N=28672, K=8192, G=128, dtype="f16",
                    desc="W4A16 decode-shaped matmul M=16 K=8192 N=28672 G=128 (HBM-bound: the packed "
                         "weights are read once)")
    if name == "int4_w4a8_decode":
        return dict(op="mm_int4a8", M=16, N=28672, K=8192, dtype="int8",
                    desc="W4A8 decode-shaped matmul M=16 K=8192 N=28672 (HBM-bound: the packed weights "
                         "are read once)")
    if name == "dequant":
        return dict(op="dequantization", M=8192, N=8192, T=128, dtype="f32",
                    desc="tile-scale dequantization 8192x8192 T=128")
    if name == "int8_swiglu":
        return dict(op="mm_int8_swiglu", M=8192, N=3584, K=8192, dtype="int8",
                    desc="INT8 gate/up projection with fused SwiGLU + requantisation: M=8192 K=8192, "
                         "2x3584 interleaved weight columns -> H [8192, 3584] (one GPU's eighth of a "
                         "57344-column gate/up layer)")
    if name == "rmsnorm_quant":
        return dict(op="rms_norm_quant", M=8192, N=8192, dtype="f32",
                    desc="RMSNorm(x + residual) * weight quantised to int8 (+ residual stream out), "
                         "8192 rows x 8192 features: the producer of the INT8 matmul's activations")
    raise SystemExit(f"unknown workload {name}")


def quant_params():
    rng = np.random.default_rng(SEED)
    sa, sb = (float(np.float32(v)) for v in rng.uniform(0.005, 0.05, 2))
    sc = float(np.float32(rng.uniform(0.5, 2.0)))
    za, zb, zc = (int(v) for v in rng.integers(-8, 9, 3))
    return (sa, sb, sc, za or 3, zb or -5, zc)


def swiglu_scales(spec):
    """Weight scales that put gate and up values at a few units, and the output scale."""
    q = quant_params()
    spread = q[0] * 128 * 74 * np.sqrt(spec["K"])
    return float(np.float32(1.5 / spread)), float(np.float32(2.0 / spread)), float(np.float32(0.03))


def algorithmic_work(spec):
    """(ops per step, minimum bytes per step) of the whole problem."""
    if spec["op"] == "mm_int8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        return 2.0 * M * N * K, float(M * K + K * N + M * N)
    if spec["op"] == "mm_int4":
        M, N, K, G = spec["M"], spec["N"], spec["K"], spec["G"]
        return 2.0 * M * N * K, float(2 * M * K + N * K // 2 + 2 * N * (K // G) + 2 * M * N)
    if spec["op"] == "mm_int4a8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        return 2.0 * M * N * K, float(M * K + N * K // 2 + M * N)
    if spec["op"] == "mm_int8_swiglu":
        M, F, K = spec["M"], spec["N"], spec["K"]  # N holds F, the number of output columns
        return 2.0 * M * 2 * F * K, float(M * K + K * 2 * F + M * F)
    if spec["op"] == "rms_norm_quant":
        M, N = spec["M"], spec["N"]  # rows x features; reads x, residual (+weight), writes q and z
        return float(M * N), float(13 * M * N + 4 * N)
    M, N, T = spec["M"], spec["N"], spec["T"]
    return float(M * N), float(8 * M * N + 4 * (-(-M // T)) * (-(-N // T)))


def hbm_bound(spec) -> bool:
    return spec["op"] in ("dequantization", "rms_norm_quant") or (
        spec["op"] in ("mm_int8", "mm_int4", "mm_int4a8") and spec["M"] <= 32)


# ------------------------------------------------------------------------- clock sampling
class ClockSampler:
    """SM clock and clock-event reasons of one GPU, read in-process through NVML every couple of
    milliseconds (nothing is ever set).  `window(t0, t1)` summarises the samples whose
    time.perf_counter() stamp falls inside a timed region; a region shorter than NVML's own
    refresh interval may hold none, in which case the nearest samples on either side are
    reported and `samples` says 0."""

    REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x40, "hw_thermal_slowdown"), (0x80, "hw_power_brake_slowdown"))

    def __init__(self, device_index: int, uuid: str | None = None, period_s: float = 0.002):
        self.period = period_s
        self.samples = []  # (t, sm_mhz, reasons_mask)
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None
        self._smi = None
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = None
            if uuid:
                try:
                    handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
                except Exception:
                    handle = None
            if handle is None:
                handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self._nvml, self._handle = pynvml, handle
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
        self.index = device_index

    def _read_nvml(self):
        nv, h = self._nvml, self._handle
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = int(get_reasons(h))
                self.samples.append((time.perf_counter(), mhz, mask))
            except Exception:
                pass
            self._stop.wait(self.period)

    def _read_smi(self):
        for line in self._smi.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz = float(parts[0])
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            mask = 0
            for bit, flag in zip((0x8, 0x40, 0x20, 0x4), parts[2:6]):
                if flag.lower().startswith("active"):
                    mask |= bit
            self.samples.append((time.perf_counter(), mhz, mask))

    def start(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._read_nvml, daemon=True)
            self._thread.start()
            return
        fields = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.sw_power_cap")
        try:
            self._smi = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={fields}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._read_smi, daemon=True)
            self._thread.start()
        except OSError:
            self._smi = None

    def stop(self):
        self._stop.set()
        if self._smi is not None:
            self._smi.terminate()  # the exact process started above
            try:
                self._smi.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._smi.kill()
        if self._thread:
            self._thread.join(timeout=2)

    def window(self, t0: float, t1: float):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no clock samples"], "samples": 0}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        used = inside
        if not used:
            before = [s for s in self.samples if s[0] < t0][-1:]
            after = [s for s in self.samples if s[0] > t1][:1]
            used = before + after
        mask = 0
        for s in used:
            mask |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in used) if used else None,
                "sm_max_mhz": self.max_mhz,
                "reasons": sorted(name for bit, name in self.REASONS if mask & bit),
                "samples": len(inside),
                "source": "NVML in-process, %.0f ms cadence" % (self.period * 1e3) if self._nvml
                          else "nvidia-smi -lms 20",
                "region_ms": (t1 - t0) * 1e3}


# ------------------------------------------------------------------------------ CPU arm
def load_oracle():
    from tests import harness  # the oracle is test infrastructure; used here as the CPU baseline

    return harness.load_oracle(), harness


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def cpu_inputs(spec, harness):
    """Host copies of the synthetic inputs for the CPU arm (same value distributions as the GPU
    arm's, deterministic in the seed)."""
    rng = np.random.default_rng(SEED)
    if spec["op"] == "mm_int8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        if M == 16:
            A = np.clip(np.rint(rng.normal(0, 20, (M, K))), -128, 127).astype(np.int8)
        else:
            A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        B = rng.integers(-128, 128, (K, N), dtype=np.int8)
        return A, B
    if spec["op"] == "mm_int4a8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        return (rng.integers(-128, 128, (M, K), dtype=np.int8),
                rng.integers(0, 256, (N, K // 2), dtype=np.uint8))
    if spec["op"] == "mm_int8_swiglu":
        M, F, K = spec["M"], spec["N"], spec["K"]
        return (rng.integers(-128, 128, (M, K), dtype=np.int8),
                rng.integers(-128, 128, (K, 2 * F), dtype=np.int8))
    if spec["op"] == "mm_int4":
        M, N, K, G = spec["M"], spec["N"], spec["K"], spec["G"]
        x = harness.float_to_half_bits(rng.normal(0, 1, (M, K)))
        w = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
        s = harness.float_to_half_bits(rng.uniform(0.01, 0.11, (N, K // G)))
        return x, w, s
    if spec["op"] == "rms_norm_quant":
        M, N = spec["M"], spec["N"]
        return (rng.normal(0, 1.5, (M, N)).astype(np.float32), rng.normal(0, 0.7, (M, N)).astype(np.float32),
                rng.uniform(0.5, 1.5, N).astype(np.float32))
    M, N, T = spec["M"], spec["N"], spec["T"]
    X = rng.uniform(-8, 8, (M, N)).astype(np.float32)
    S = rng.uniform(0.5, 2.0, (-(-M // T), -(-N // T))).astype(np.float32)
    return X, S


def cpu_run_rows(oracle, spec, inputs, q, r0, r1):
    if spec["op"] == "mm_int8":
        A, B = inputs
        oracle.mm_int8(A, B, spec["M"], spec["N"], spec["K"], q, mode=1, rows=(r0, r1))
    elif spec["op"] == "mm_int4a8":
        A, w = inputs
        oracle.mm_int4a8(A, w, spec["M"], spec["N"], spec["K"], q, rows=(r0, r1))
    elif spec["op"] == "mm_int8_swiglu":
        A, B = inputs
        sg, su, sh = swiglu_scales(spec)
        oracle.mm_int8_swiglu(A, B, spec["M"], spec["N"], spec["K"], q[0], sg, su, sh, q[3], q[4], -q[4],
                              rows=(r0, r1))
    elif spec["op"] == "mm_int4":
        x, w, s = inputs
        oracle.mm_int4(x, w, s, spec["M"], spec["N"], spec["K"], spec["G"], rows=(r0, r1))
    elif spec["op"] == "rms_norm_quant":
        x, r, w = inputs
        y, _ = oracle.rms_norm_w_residual(x[r0:r1], r[r0:r1], w, 1e-5)
        np.clip(np.rint(y / 0.03) + 3, -128, 127).astype(np.int8)
    else:
        X, S = inputs
        oracle.dequantization(X, S, spec["M"], spec["N"], spec["T"])


def cpu_rate(spec, seconds_per_step: float, steps: int, warmup: int):
    """Times the CPU oracle on row samples; returns (units/s, rows per step, seconds list, threads).
    The OpenMP thread count is set here to every host core this process may run on (launchers
    such as torchrun export OMP_NUM_THREADS=1)."""
    oracle, harness = load_oracle()
    threads = oracle.set_threads(host_threads())
    inputs = cpu_inputs(spec, harness)
    q = quant_params()
    M = spec["M"]
    ops, _ = algorithmic_work(spec)
    if spec["op"] == "dequantization":
        rows = M
    else:
        probe = min(M, max(2, threads))
        t0 = time.perf_counter()
        cpu_run_rows(oracle, spec, inputs, q, 0, probe)
        per_row = max((time.perf_counter() - t0) / probe, 1e-6)
        rows = int(max(1, min(M, seconds_per_step / per_row)))
        if rows >= threads:
            rows -= rows % threads  # whole rounds of the row-parallel loop
    times = []
    for i in range(warmup + steps):
        r0 = (i * rows) % max(1, M - rows + 1)
        t0 = time.perf_counter()
        cpu_run_rows(oracle, spec, inputs, q, r0, r0 + rows)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    total = sum(times)
    rate = ops * (rows / M) * len(times) / total
    return rate, rows, times, threads


def run_reference_arm(args, spec, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU reference runs once, on rank 0
    budget = 120.0  # seconds for the whole run
    per_step = max(0.2, budget / (args.steps + args.warmup))
    rate, rows, times, threads = cpu_rate(spec, per_step, args.steps, args.warmup)
    value = rate / 1e12
    sample = f"{rows} of {spec['M']} output rows per step (all columns, full K)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * sum(times) / len(times), "higher_is_better": True,
        "scaling": "strong" if (args.gpus > 1 and spec["op"] == "mm_int8") else "weak",
        "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
        "config": {"workload": workload, "description": spec["desc"],
                   "reference_path": "CPU loop of the reference harness restated in C "
                                     "(int64 dot, double scaling), OpenMP over rows",
                   "omp_threads": threads, "host_cores_available": host_threads(),
                   "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS")},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm
class Ctx:
    """Process-wide handles of the GPU arm."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        from texo_b200 import _lib

        self.torch, self.dist = torch, dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.lib = _lib.load()
        self.q = quant_params()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        t = self.torch.tensor([ms], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, flag: bool) -> bool:
        if self.world == 1:
            return bool(flag)
        t = self.torch.tensor([1 if flag else 0], device=self.dev, dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def timed(self, fn, steps: int, warmup: int) -> float:
        """ms per step: CUDA events on the launching stream around `steps` calls of fn(i), a
        barrier + device synchronisation on both sides, max over ranks."""
        torch = self.torch
        for i in range(warmup):
            fn(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def build_workload(ctx: Ctx, spec, with_e2e: bool = True, strong: bool = False):
    """Device-resident inputs and the step functions of one workload.

    Returns a dict: step(i), e2e_step(i) (None without with_e2e), h2d / d2h (bytes per step of
    the whole job), note (how L2 reuse between steps is prevented), ops_job / ops_gpu /
    bytes_gpu (algorithmic work), ref (reference-kernel step or None), parity (callable or
    None), extras (dict)."""
    torch, dev, lib, q = ctx.torch, ctx.dev, ctx.lib, ctx.q
    from texo_b200 import ops, sharded

    world, rank = ctx.world, ctx.rank
    ops_total, bytes_total = algorithmic_work(spec)
    g_a = torch.Generator(device=dev).manual_seed(SEED)
    g_b = torch.Generator(device=dev).manual_seed(SEED + 1 + (0 if strong else rank))
    wl = dict(e2e_step=None, h2d=0, d2h=0, ref=None, parity=None, extras={}, ops_job=ops_total * (1 if strong else world),
              ops_gpu=ops_total / (world if strong else 1), bytes_gpu=bytes_total, keep=[])

    if spec["op"] == "mm_int8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        if M == 16:
            A = torch.clamp(torch.round(torch.randn((M, K), generator=g_a, device=dev) * 20),
                            -128, 127).to(torch.int8)
        else:
            A = torch.randint(-128, 128, (M, K), generator=g_a, device=dev, dtype=torch.int8)
        if strong:
            return build_strong_int8(ctx, spec, wl, A, g_b, with_e2e)
        # Rotate over enough weight/output sets that a step never finds its inputs in L2.
        small = (M * K + K * N + M * N) < 32e6
        nsets = 2 if small else max(2, int(np.ceil(3 * 126e6 / (K * N))) if M * K < 64e6 else 2)
        Bs = [torch.randint(-128, 128, (K, N), generator=g_b, device=dev, dtype=torch.int8)
              for _ in range(nsets)]
        Cs = [torch.empty((M, N), device=dev, dtype=torch.int8) for _ in range(nsets)]

        if spec.get("presummed"):
            handles = [lib.texo_mm_int8_prepare_weights(b.data_ptr(), K, N) for b in Bs]
            row_sums = A.to(torch.int32).sum(dim=1, dtype=torch.int32).contiguous()
            torch.cuda.synchronize()

            def step(i):
                j = i % nsets
                lib.texo_mm_int8_solve_presummed(A.data_ptr(), row_sums.data_ptr(), handles[j],
                                                 Cs[j].data_ptr(), M, *q)
        else:
            def step(i):
                j = i % nsets
                lib.texo_mm_int8_solve(A.data_ptr(), Bs[j].data_ptr(), Cs[j].data_ptr(), M, N, K, *q)

        if with_e2e:
            host_in = [torch.empty((M, K), dtype=torch.int8).pin_memory(),
                       torch.empty((K, N), dtype=torch.int8).pin_memory()]
            host_in[0].copy_(A)
            host_in[1].copy_(Bs[0])
            host_out = torch.empty((M, N), dtype=torch.int8).pin_memory()

            def e2e_step(i):
                ops.mm_int8_host(host_in[0], host_in[1], host_out, *q)

            wl["e2e_step"] = e2e_step
            wl["e2e_api"] = "texo_mm_int8_solve_host (pipelined upload / solve / download)"
        wl["h2d"], wl["d2h"] = (M * K + K * N) * world, M * N * world
        wl["note"] = ("operands smaller than L2 by nature (launch-bound case): they stay resident"
                      if small else
                      f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + K * N + M * N) / 2**20:.0f} MiB exceeds the 126 MB L2")
        wl["step"] = step

        ref = load_reference_kernel("mm_int8")
        if ref is not None:
            C_ref = torch.empty((M, N), device=dev, dtype=torch.int8)

            def ref_step(i):
                ref.solve(A.data_ptr(), Bs[i % nsets].data_ptr(), C_ref.data_ptr(), M, N, K, *q)

            wl["ref"] = ref_step

        def parity():
            oracle, _ = load_oracle()
            step(0)
            torch.cuda.synchronize()
            A_h, B_h = A.cpu().numpy(), Bs[0].cpu().numpy()
            rows = sorted(set(np.linspace(0, M - 1, 4).astype(int).tolist()))
            ok = True
            for r in rows:
                want = oracle.mm_int8(A_h, B_h, M, N, K, q, rows=(r, r + 1))
                ok = ok and bool(np.array_equal(Cs[0][r].cpu().numpy(), want[0]))
            return {"rows_vs_oracle": ok, "rows_checked": len(rows),
                    "c_checksum": int(Cs[0].to(torch.int64).sum().item())}

        wl["parity"] = parity
        wl["keep"] += [A, Bs, Cs]
    elif spec["op"] == "mm_int8_swiglu":
        M, F, K = spec["M"], spec["N"], spec["K"]
        sg, su, sh = swiglu_scales(spec)
        A = torch.randint(-128, 128, (M, K), generator=g_a, device=dev, dtype=torch.int8)
        nsets = 3
        Bs = [torch.randint(-128, 128, (K, 2 * F), generator=g_b, device=dev, dtype=torch.int8)
              for _ in range(nsets)]
        Hs = [torch.empty((M, F), device=dev, dtype=torch.int8) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_mm_int8_swiglu_solve(A.data_ptr(), Bs[j].data_ptr(), Hs[j].data_ptr(), M, F, K,
                                          q[0], sg, su, sh, q[3], q[4], -q[4], q[5])

        if with_e2e:
            hA, hB = A.cpu().pin_memory(), Bs[0].cpu().pin_memory()
            hH = torch.empty((M, F), dtype=torch.int8).pin_memory()
            dA, dB, dH = torch.empty_like(A), torch.empty_like(Bs[0]), torch.empty_like(Hs[0])

            def e2e_step(i):
                dA.copy_(hA, non_blocking=True)
                dB.copy_(hB, non_blocking=True)
                ops.mm_int8_swiglu(dA, dB, q[0], sg, su, sh, q[3], q[4], -q[4], q[5], out=dH)
                hH.copy_(dH, non_blocking=True)

            wl["e2e_step"] = e2e_step
        wl["h2d"], wl["d2h"] = (M * K + K * 2 * F) * world, M * F * world
        wl["note"] = (f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + K * 2 * F + M * F) / 2**20:.0f} MiB")
        wl["step"] = step
    elif spec["op"] == "mm_int4a8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        A = torch.randint(-128, 128, (M, K), generator=g_a, device=dev, dtype=torch.int8)
        nsets = max(3, int(np.ceil(3 * 126e6 / (N * K // 2))))
        Ws = [torch.randint(0, 256, (N, K // 2), generator=g_b, device=dev, dtype=torch.uint8)
              for _ in range(nsets)]
        Cs = [torch.empty((M, N), device=dev, dtype=torch.int8) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_mm_int4a8_solve(A.data_ptr(), Ws[j].data_ptr(), Cs[j].data_ptr(), M, N, K, *q)

        if with_e2e:
            hA, hW = A.cpu().pin_memory(), Ws[0].cpu().pin_memory()
            hC = torch.empty((M, N), dtype=torch.int8).pin_memory()
            dA, dW, dC = torch.empty_like(A), torch.empty_like(Ws[0]), torch.empty_like(Cs[0])

            def e2e_step(i):
                dA.copy_(hA, non_blocking=True)
                dW.copy_(hW, non_blocking=True)
                ops.mm_int4a8(dA, dW, *q, out=dC)
                hC.copy_(dC, non_blocking=True)

            wl["e2e_step"] = e2e_step
        wl["h2d"], wl["d2h"] = (M * K + N * K // 2) * world, M * N * world
        wl["note"] = (f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + N * K // 2 + M * N) / 2**20:.0f} MiB (A stays in L2, weights and "
                      f"outputs do not)")
        wl["step"] = step
    elif spec["op"] == "mm_int4":
        M, N, K, G = spec["M"], spec["N"], spec["K"], spec["G"]
        x = torch.randn((M, K), generator=g_a, device=dev).to(torch.float16)
        nsets = 2 if M > 32 else max(3, int(np.ceil(3 * 126e6 / (N * K // 2))))
        Ws = [torch.randint(0, 256, (N, K // 2), generator=g_b, device=dev, dtype=torch.uint8)
              for _ in range(nsets)]
        Ss = [(torch.rand((N, K // G), generator=g_b, device=dev) * 0.1 + 0.01).to(torch.float16)
              for _ in range(nsets)]
        Ys = [torch.empty((M, N), device=dev, dtype=torch.float16) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_mm_int4_solve(x.data_ptr(), Ws[j].data_ptr(), Ss[j].data_ptr(),
                                   Ys[j].data_ptr(), M, N, K, G)

        if with_e2e:
            hx, hw, hs = (t.cpu().pin_memory() for t in (x, Ws[0], Ss[0]))
            hy = torch.empty((M, N), dtype=torch.float16).pin_memory()
            dx, dw, ds, dy = (torch.empty_like(t) for t in (x, Ws[0], Ss[0], Ys[0]))

            def e2e_step(i):
                dx.copy_(hx, non_blocking=True)
                dw.copy_(hw, non_blocking=True)
                ds.copy_(hs, non_blocking=True)
                ops.mm_int4(dx, dw, ds, G, out=dy)
                hy.copy_(dy, non_blocking=True)

            wl["e2e_step"] = e2e_step
        wl["h2d"] = (2 * M * K + N * K // 2 + 2 * N * (K // G)) * world
        wl["d2h"] = 2 * M * N * world
        wl["note"] = f"{nsets} weight/output sets rotated; working set per step exceeds L2"
        wl["step"] = step
        ref = load_reference_kernel("mm_int4")
        if ref is not None:
            y_ref = torch.empty((M, N), device=dev, dtype=torch.float16)

            def ref_step(i):
                j = i % nsets
                ref.solve(x.data_ptr(), Ws[j].data_ptr(), Ss[j].data_ptr(), y_ref.data_ptr(), M, N, K, G)

            wl["ref"] = ref_step
        wl["keep"] += [x, Ws, Ss, Ys]
    elif spec["op"] == "rms_norm_quant":
        M, N = spec["M"], spec["N"]
        nsets = 2
        Xs = [torch.randn((M, N), generator=g_b, device=dev) * 1.5 for _ in range(nsets)]
        Rs = [torch.randn((M, N), generator=g_b, device=dev) * 0.7 for _ in range(nsets)]
        Wt = torch.rand((N,), generator=g_a, device=dev) + 0.5
        Qs = [torch.empty((M, N), device=dev, dtype=torch.int8) for _ in range(nsets)]
        Zs = [torch.empty((M, N), device=dev) for _ in range(nsets)]
        RS = torch.empty((M,), device=dev, dtype=torch.int32)

        def step(i):
            j = i % nsets
            lib.texo_rms_norm_quant_solve(Xs[j].data_ptr(), Rs[j].data_ptr(), Wt.data_ptr(),
                                          Qs[j].data_ptr(), Zs[j].data_ptr(), RS.data_ptr(), M, N, 1e-5,
                                          0.03, 3)

        if with_e2e:
            hX, hR = Xs[0].cpu().pin_memory(), Rs[0].cpu().pin_memory()
            hQ = torch.empty((M, N), dtype=torch.int8).pin_memory()
            hZ = torch.empty((M, N)).pin_memory()
            dX, dR = torch.empty_like(Xs[0]), torch.empty_like(Rs[0])
            dQ, dZ = torch.empty_like(Qs[0]), torch.empty_like(Zs[0])

            def e2e_step(i):
                dX.copy_(hX, non_blocking=True)
                dR.copy_(hR, non_blocking=True)
                ops.rms_norm_quant(dX, dR, Wt, 1e-5, 0.03, 3, out=dQ, z_out=dZ)
                hQ.copy_(dQ, non_blocking=True)
                hZ.copy_(dZ, non_blocking=True)

            wl["e2e_step"] = e2e_step
        wl["h2d"], wl["d2h"] = 8 * M * N * world, 5 * M * N * world
        wl["note"] = f"{nsets} input/output sets rotated; 832 MiB per step exceeds L2"
        wl["step"] = step
    else:
        M, N, T = spec["M"], spec["N"], spec["T"]
        nsets = 2
        Xs = [torch.rand((M, N), generator=g_b, device=dev) * 16 - 8 for _ in range(nsets)]
        S = torch.rand((-(-M // T), -(-N // T)), generator=g_a, device=dev) * 1.5 + 0.5
        Ys = [torch.empty((M, N), device=dev) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_dequantization_solve(Xs[j].data_ptr(), S.data_ptr(), Ys[j].data_ptr(), M, N, T)

        if with_e2e:
            hX, hS = Xs[0].cpu().pin_memory(), S.cpu().pin_memory()
            hY = torch.empty((M, N)).pin_memory()
            dX, dS, dY = torch.empty_like(Xs[0]), torch.empty_like(S), torch.empty_like(Ys[0])

            def e2e_step(i):
                dX.copy_(hX, non_blocking=True)
                dS.copy_(hS, non_blocking=True)
                ops.dequantization(dX, dS, T, out=dY)
                hY.copy_(dY, non_blocking=True)

            wl["e2e_step"] = e2e_step
        wl["h2d"], wl["d2h"] = (4 * M * N + 4 * S.numel()) * world, 4 * M * N * world
        wl["note"] = f"{nsets} input/output sets rotated; 512 MiB per step exceeds L2"
        wl["step"] = step
        ref = load_reference_kernel("dequantization")
        if ref is not None:
            Y_ref = torch.empty((M, N), device=dev)

            def ref_step(i):
                ref.solve(Xs[i % nsets].data_ptr(), S.data_ptr(), Y_ref.data_ptr(), M, N, T)

            wl["ref"] = ref_step
        wl["keep"] += [Xs, S, Ys]
    return wl


def build_strong_int8(ctx: Ctx, spec, wl, A0, g_b, with_e2e: bool):
    """The fixed [M,K] x [K,N] INT8 problem column-sharded over the ranks, the all-gather of C
    fused into the matmul (see the module docstring).  Everything a step touches is rotated
    between two sets (activations included), so a step never finds operands in L2 although one
    rank's slab alone would fit."""
    torch, dev, lib, q, dist = ctx.torch, ctx.dev, ctx.lib, ctx.q, ctx.dist
    from texo_b200 import ops, sharded

    world, rank = ctx.world, ctx.rank
    M, N, K = spec["M"], spec["N"], spec["K"]
    n0, n1 = sharded.column_slab(N, world, rank)
    w = n1 - n0
    nsets = 2
    # every rank draws the same logical B (same seed) and keeps its own columns
    As, B_slabs = [A0, A0.clone()], []
    for _ in range(nsets):
        B_full = torch.randint(-128, 128, (K, N), generator=g_b, device=dev, dtype=torch.int8)
        B_slabs.append(B_full[:, n0:n1].contiguous())
        del B_full
    outs = [sharded.GatheredOutput(M, N, dev) for _ in range(nsets)]
    C_slabs = [torch.empty((M, w), device=dev, dtype=torch.int8) for _ in range(nsets)]

    def step(i):
        j = i % nsets
        sharded.mm_int8_allgather(As[j], B_slabs[j], outs[j], *q)
        outs[j].wait()

    def gemm_only(i):
        j = i % nsets
        lib.texo_mm_int8_solve(As[j].data_ptr(), B_slabs[j].data_ptr(), C_slabs[j].data_ptr(), M, w, K, *q)

    def gemm_nccl(i):
        gemm_only(i)
        sharded.all_gather_columns(C_slabs[i % nsets], N)

    outs_uni = []

    def fused_unicast(i):
        j = i % nsets
        sharded.mm_int8_allgather(As[j], B_slabs[j], outs_uni[j], *q)
        outs_uni[j].wait()

    def variants(steps, warmup):
        """Per-variant ms/step (max over ranks) of the same sharded problem."""
        res = {"gemm_only_ms": ctx.timed(gemm_only, steps, warmup),
               "nccl_gather_ms": ctx.timed(gemm_nccl, steps, warmup)}
        if outs[0].multicast_ptr:
            outs_uni.extend(sharded.GatheredOutput(M, N, dev, multicast=False) for _ in range(nsets))
            res["fused_gather_unicast_ms"] = ctx.timed(fused_unicast, steps, warmup)
            outs_uni.clear()
        return res

    if with_e2e:
        hA = A0.cpu().pin_memory()
        hB = B_slabs[0].cpu().pin_memory()
        hC = torch.empty((M, w), dtype=torch.int8).pin_memory()
        dA, dB, dC = torch.empty_like(A0), torch.empty_like(B_slabs[0]), torch.empty_like(C_slabs[0])

        def e2e_step(i):
            sharded.upload_replicated_rows(hA, dA)
            dB.copy_(hB, non_blocking=True)
            ops.mm_int8(dA, dB, *q, out=dC)
            hC.copy_(dC, non_blocking=True)

        wl["e2e_step"] = e2e_step
        wl["e2e_api"] = ("sharded.upload_replicated_rows (each rank uploads M/g rows of A over its own "
                         "PCIe link, NCCL all-gather over NVLink completes them) + ops.mm_int8 on the "
                         "rank's weight slab + download of the rank's slab of C")
    wl["h2d"], wl["d2h"] = M * K + K * N, M * N  # whole job: each rank 1/world of it
    wl["note"] = (f"{nsets} sets of activations, weight slabs and gathered outputs rotated: "
                  f"{nsets} x {(M * K + K * w + M * N) / 2**20:.0f} MiB per GPU exceeds the 126 MB L2")
    wl["step"] = step
    wl["variants"] = variants
    wl["multicast"] = bool(outs[0].multicast_ptr)

    def parity():
        oracle, _ = load_oracle()
        outs[0].tensor.fill_(77)
        outs[0].wait()
        step(0)
        gemm_only(0)
        gathered = sharded.all_gather_columns(C_slabs[0], N)
        torch.cuda.synchronize()
        fused_equals_nccl = bool(torch.equal(outs[0].tensor, gathered))
        A_h, B_h = As[0].cpu().numpy(), B_slabs[0].cpu().numpy()
        rows = sorted(set(np.linspace(0, M - 1, 4).astype(int).tolist()))
        rows_ok = True
        for r in rows:
            want = oracle.mm_int8(A_h, B_h, M, w, K, q, rows=(r, r + 1))
            rows_ok = rows_ok and bool(np.array_equal(outs[0].tensor[r, n0:n1].cpu().numpy(), want[0]))
        return {"rows_vs_oracle": ctx.all_true(rows_ok), "rows_checked": len(rows) * world,
                "fused_equals_nccl": ctx.all_true(fused_equals_nccl),
                "c_checksum": int(outs[0].tensor.to(torch.int64).sum().item())}

    wl["parity"] = parity
    wl["keep"] += [As, B_slabs, outs, C_slabs]
    return wl


def load_reference_kernel(op: str):
    """The reference's own kernel for `op`, recompiled for sm_100a from the reference checkout
    at build time (a baseline leg of the benchmark, never part of this library's path).  None
    when it was not built."""
    path = os.path.join(ROOT, "oracle", "_ref", f"libref_{op}.so")
    if not os.path.exists(path):
        return None
    try:
        ref = ctypes.CDLL(path)
    except OSError:
        return None
    ref.solve.restype = None
    if op == "mm_int8":
        ref.solve.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3 + [ctypes.c_float] * 3 + [ctypes.c_int] * 3
    elif op == "mm_int4":
        ref.solve.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 4
    else:
        ref.solve.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 3
    return ref


def time_reference_kernel(ctx: Ctx, ref_step, est_ms: float):
    """The reference's timing method (its tests/gemm.cu:111-134): 5 warm-ups, then the median of
    5 CUDA-event batches of R back-to-back calls."""
    torch = ctx.torch
    for i in range(5):
        ref_step(i)
    torch.cuda.synchronize()
    reps = int(max(2, min(50, 30.0 / max(est_ms, 0.01))))
    batches = []
    for b in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            ref_step(b * reps + i)
        e1.record()
        torch.cuda.synchronize()
        batches.append(e0.elapsed_time(e1) / reps)
    return statistics.median(batches), reps


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def roofline_for(spec, kernel_ms: float, ops_gpu: float, bytes_gpu: float, long_run: bool, ceilings):
    """Roofline object of the dominant kernel: algorithmic work / its average launch duration
    against the measured peak (copy bandwidth or cuBLAS bf16 from the pool's peak file; the
    stated fallback when that file is absent), with the other denominators beside it."""
    peaks = measured_peaks()
    if hbm_bound(spec):
        peak = peaks.get("hbm_gbs", 6650.0)
        achieved = bytes_gpu / (kernel_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": None,
                "peak_source": "measured copy bandwidth" if peaks else "fallback 6650 GB/s",
                "denominators": {"measured_copy_gbs": peak, "spec_hbm_gbs": SPEC_HBM_GBS},
                "frac_of_spec": achieved / SPEC_HBM_GBS}
    # No INT8 figure is measured on this pool; kind::i8 issues at twice the bf16 rate, so the
    # denominator is 2x the measured cuBLAS bf16 throughput (W4A16 runs kind::f16: 1x).
    int8 = spec["op"] in ("mm_int8", "mm_int4a8", "mm_int8_swiglu")
    factor = 2.0 if int8 else 1.0
    key = "bf16_tflops_sustained" if long_run else "bf16_tflops"
    base = peaks.get(key, 1400.0 if long_run else 1590.0)
    peak = factor * base
    achieved = ops_gpu / (kernel_ms * 1e-3) / 1e12
    spec_peak = SPEC_INT8_TOPS if int8 else SPEC_F16_TFLOPS
    out = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
           "frac": achieved / peak, "traffic": None,
           "peak_source": f"{factor:g} x {'measured' if peaks else 'fallback'} bf16 "
                          f"{'sustained' if long_run else 'burst'} ({base:.0f} TFLOP/s)",
           "denominators": {"bf16_measured_x%g" % factor: peak, "spec_dense": spec_peak},
           "frac_of_spec": achieved / spec_peak}
    ceiling = (ceilings or {}).get("int8" if int8 else "f16")
    if ceiling and ceiling > 0:
        out["denominators"]["issue_ceiling_measured_in_this_run"] = ceiling
        out["frac_of_issue_ceiling"] = achieved / ceiling
    return out


def issue_ceilings(ctx: Ctx):
    """Box-measured tensor-pipe ceilings, taken in this run: CTA-pair MMAs issued back to back
    on shared-memory-resident operands (no loads, no epilogue), about 10 ms each."""
    out = {}
    try:
        ctx.lib.texo_int8_issue_ceiling_tops(1, 200)  # warm-up
        out["int8"] = float(ctx.lib.texo_int8_issue_ceiling_tops(1, 2000))
        out["f16"] = float(ctx.lib.texo_f16_issue_rate_tflops(1, 2000, 64))
    except Exception:
        pass
    return {k: v for k, v in out.items() if v > 0}


def kernel_bracket(ctx: Ctx, step, n: int):
    """Average duration of the dominant kernel over n steps, from the library's CUDA-event
    bracket around it (records between the kernels of a call defeat their programmatic
    dependent launch overlap, so this never runs inside a region that `value` times)."""
    lib = ctx.lib
    lib.texo_profile_enable(1)
    for i in range(n):
        step(i)
    ctx.torch.cuda.synchronize()
    kernel_ms, kernel_n = ctypes.c_float(0), ctypes.c_int(0)
    lib.texo_profile_read(ctypes.byref(kernel_ms), ctypes.byref(kernel_n))
    lib.texo_profile_enable(0)
    return kernel_ms.value / max(1, kernel_n.value), kernel_n.value


def quick_config(ctx: Ctx, name: str, steps: int, warmup: int, ceilings, spec=None):
    """One entry of the `configs` object: device-resident time of a secondary workload, its
    roofline fraction and the reference kernel's time on the same GPU."""
    torch = ctx.torch
    spec = spec or workload_spec(name)
    wl = build_workload(ctx, spec, with_e2e=False)
    launches0 = ctx.lib.texo_kernel_launches()
    ms = ctx.timed(wl["step"], steps, warmup)
    launches = (ctx.lib.texo_kernel_launches() - launches0) // (steps + warmup)
    kernel_ms, _ = kernel_bracket(ctx, wl["step"], max(3, min(steps, 50)))
    k_ms = ms if launches == 1 else kernel_ms
    ops_gpu, bytes_gpu = wl["ops_gpu"], wl["bytes_gpu"]
    entry = {"description": spec["desc"], "ms": ms, "launches_per_step": int(launches), "kernel_ms": k_ms,
             "kernel_ms_isolated": kernel_ms,
             "roofline": roofline_for(spec, k_ms, ops_gpu, bytes_gpu, False, ceilings)}
    if hbm_bound(spec):
        entry["gbs"] = bytes_gpu / (ms * 1e-3) / 1e9
    else:
        entry["tops"] = ops_gpu / (ms * 1e-3) / 1e12
    if name in NCU_TRAFFIC:
        entry["roofline"]["traffic"] = NCU_TRAFFIC[name]
    if wl["ref"] is not None:
        ref_ms, reps = time_reference_kernel(ctx, wl["ref"], ms * 4)
        entry["reference_gpu"] = {"ms": ref_ms, "speedup": ref_ms / ms,
                                  "what": "the reference's kernel recompiled for sm_100a, same GPU, same "
                                          "inputs; 5 warm-ups, median of 5 event batches of %d calls" % reps}
    del wl
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return entry


def measure_layers(ctx: Ctx, steps: int, warmup: int):
    """The four INT8 projections of a transformer layer at M = 8192, weight columns sharded
    over the ranks (strong scaling: the layer is fixed, each GPU owns N/g columns): the matmul
    alone, with an NCCL all-gather + permute after it, and with the gather fused into the
    matmul's epilogue.  ms per call, max over ranks."""
    torch, dev, lib, q = ctx.torch, ctx.dev, ctx.lib, ctx.q
    from texo_b200 import sharded

    world, rank = ctx.world, ctx.rank
    M = 8192
    g = torch.Generator(device=dev).manual_seed(SEED + 100 + rank)
    results = []
    for name, K, N in LAYERS:
        n0, n1 = sharded.column_slab(N, world, rank)
        w = n1 - n0
        A = torch.randint(-128, 128, (M, K), generator=torch.Generator(device=dev).manual_seed(SEED),
                          device=dev, dtype=torch.int8)
        B = torch.randint(-128, 128, (K, w), generator=g, device=dev, dtype=torch.int8)
        C = torch.empty((M, w), device=dev, dtype=torch.int8)

        def gemm(i):
            lib.texo_mm_int8_solve(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, w, K, *q)

        def gemm_gather(i):
            gemm(i)
            sharded.all_gather_columns(C, N)

        ms = ctx.timed(gemm, steps, warmup)
        entry = {"layer": name, "K": K, "N": N, "slab": w, "gemm_ms": ms,
                 "tops": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
        if world > 1:
            entry["gemm_plus_nccl_gather_ms"] = ctx.timed(gemm_gather, steps, warmup)
            out = sharded.GatheredOutput(M, N, dev)

            def fused(i):
                sharded.mm_int8_allgather(A, B, out, *q)
                out.wait()

            entry["gemm_fused_gather_ms"] = ctx.timed(fused, steps, warmup)
            entry["fused_over_gemm"] = entry["gemm_fused_gather_ms"] / ms
            entry["multicast"] = bool(out.multicast_ptr)
            # bytes each GPU must send (its slab to the others once with multicast, g-1 times without)
            entry["gather_bytes_out_per_gpu"] = M * w * (1 if out.multicast_ptr else world - 1)
            del out
        results.append(entry)
        del A, B, C
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    return results


def run_ours(args, spec, workload):
    ctx = Ctx()
    torch, lib = ctx.torch, ctx.lib
    world, rank = ctx.world, ctx.rank
    strong = world > 1 and spec["op"] == "mm_int8" and not spec.get("presummed")
    wl = build_workload(ctx, spec, with_e2e=True, strong=strong)
    step = wl["step"]
    props = torch.cuda.get_device_properties(ctx.dev)
    uuid = str(getattr(props, "uuid", "") or "") or None

    # ---- device-resident timed region
    for i in range(args.warmup):
        step(i)
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank, uuid)
    if rank == 0:
        sampler.start()
        time.sleep(0.05)
    launches0 = lib.texo_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx.barrier()
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    ctx.barrier()
    t1 = time.perf_counter()
    total_ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    launches = lib.texo_kernel_launches() - launches0
    clocks = sampler.window(t0, t1) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    # Dominant-kernel duration for the roofline: the same steps again, directly after and still
    # under load, this time with the library's CUDA-event bracket around the kernel.
    n_prof = max(3, min(args.steps, 500))
    bracketed_ms, bracketed_n = kernel_bracket(ctx, step, n_prof)
    status = lib.texo_mm_int8_status()

    # ---- sustained: at least two seconds of back-to-back steps, with its own clock record
    sustained = None
    if not args.no_sustained:
        n_sus = int(min(200000, max(args.steps, np.ceil(2000.0 / max(ms_per_step, 1e-3)))))
        ctx.barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts0 = time.perf_counter()
        s0.record()
        for i in range(n_sus):
            step(i)
        s1.record()
        ctx.barrier()
        ts1 = time.perf_counter()
        sus_ms = ctx.max_over_ranks(s0.elapsed_time(s1)) / n_sus
        sustained = {"value": wl["ops_job"] / (sus_ms * 1e-3) / 1e12, "unit": UNIT, "steps": n_sus,
                     "ms_per_step": sus_ms, "seconds": sus_ms * n_sus / 1e3,
                     "clocks": sampler.window(ts0, ts1) if rank == 0 else None}
    if rank == 0:
        sampler.stop()

    # ---- end to end through the public API with host buffers
    e2e_step = wl["e2e_step"]
    n_e2e = max(3, min(args.steps, 20))
    e2e_ms = ctx.timed(e2e_step, n_e2e, min(2, args.warmup))

    # ---- the same sharded problem without / with the other forms of the gather; layer sweep
    extras = {}
    if strong and not args.no_extras:
        extras.update(wl["variants"](max(5, min(args.steps, 20)), 3))
        extras["fused_gather_ms"] = ms_per_step
        extras["collective"] = ("all-gather of C fused into the matmul epilogue: "
                                + ("multimem.st through the NVSwitch multicast mapping"
                                   if wl["multicast"] else "per-peer st.global over NVLink")
                                + " + one symmetric-memory barrier per step")
    if spec["op"] == "mm_int8" and workload == "int8_8192" and not args.no_extras:
        extras["layers"] = measure_layers(ctx, 10, 3)
    parity = None
    if wl["parity"] is not None and not args.no_extras:
        parity = wl["parity"]()

    if rank != 0:
        ctx.close()
        return

    ceilings = issue_ceilings(ctx) if not args.no_extras else {}
    value = wl["ops_job"] / (ms_per_step * 1e-3) / 1e12
    # One launch per step: the timed region's own events give the average launch duration
    # (events around K back-to-back launches / K), which is what the roofline wants.  With
    # several kernels per step the dominant one is taken from the bracketed second pass.
    single_launch_steps = launches == args.steps and not strong
    kernel_avg_ms = ms_per_step if single_launch_steps else bracketed_ms
    long_run = total_ms > 300.0  # long enough for the power cap to pull the clocks down
    roofline = roofline_for(spec, kernel_avg_ms, wl["ops_gpu"],
                            wl["bytes_gpu"] if not strong else
                            float(spec["M"] * spec["K"] + spec["K"] * spec["N"] // world + spec["M"] * spec["N"] // world),
                            long_run, ceilings)
    if workload in NCU_TRAFFIC and not strong:
        roofline["traffic"], roofline["traffic_source"] = NCU_TRAFFIC[workload], TRAFFIC_NOTE
    roofline["kernel_ms"] = kernel_avg_ms
    if single_launch_steps:
        roofline["kernel_launches_timed"] = int(launches)
        roofline["kernel_timing"] = ("one launch per step: CUDA events around the timed region / "
                                     "launches (back to back, as a caller issues them)")
        roofline["kernel_ms_isolated"] = bracketed_ms
    else:
        roofline["kernel_launches_timed"] = int(bracketed_n)
        roofline["kernel_timing"] = ("CUDA events around the dominant kernel over the %d steps "
                                     "that directly follow the timed region" % n_prof)
    if clocks and clocks.get("sm_mhz"):
        roofline["sm_mhz_during_timed_region"] = clocks["sm_mhz"]

    configs = None
    reference_gpu = None
    if world == 1 and workload == "int8_8192" and not args.no_extras:
        configs = {}
        for name in ("int8_512", "int8_decode", "int4_w4a16", "int4_w4a16_decode", "int4_w4a8",
                     "int4_w4a8_decode", "dequant"):
            configs[name] = quick_config(ctx, name, 20, 5, ceilings)
        for G in (64, 32, 16):
            s = dict(workload_spec("int4_w4a16"), G=G)
            s["desc"] = f"W4A16 matmul M=4096 K=8192 N=8192 G={G}"
            configs[f"int4_w4a16_g{G}"] = quick_config(ctx, f"int4_w4a16_g{G}", 10, 3, ceilings, spec=s)
    if world == 1 and wl["ref"] is not None and not args.no_extras:
        ref_ms, reps = time_reference_kernel(ctx, wl["ref"], ms_per_step * 5)
        reference_gpu = {"ms": ref_ms, "tops": wl["ops_gpu"] / (ref_ms * 1e-3) / 1e12,
                         "speedup": ref_ms / ms_per_step,
                         "what": "the reference's kernel recompiled for sm_100a, same GPU, same inputs, "
                                 "outside this library's timed regions; 5 warm-ups, median of 5 event "
                                 "batches of %d calls" % reps}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rate, rows, times, threads = cpu_rate(spec, 6.0, 2, 0)
        cpu = {"value": rate / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{rows} of {spec['M']} output rows x 2 runs (all columns, full K), "
                         f"{sum(times):.1f} s of CPU work"}

    N = spec["N"]
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": spec["dtype"],
        "data": "synthetic",
        "config": {"workload": workload, "description": spec["desc"],
                   "sharding": (f"fixed problem, {world} column slabs of {N // world} of {N} output columns, "
                                f"one per GPU, all-gather of C fused into the matmul" if strong else
                                f"{world} independent replica(s) of the problem, one per GPU"),
                   "l2": wl["note"], "quant": ctx.q, "status_word": status},
        "clocks": clocks,
        "sustained": sustained,
        "e2e": {"value": wl["ops_job"] / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": wl["h2d"], "d2h_bytes_per_step": wl["d2h"], "ms_per_step": e2e_ms,
                "api": wl.get("e2e_api", "texo_b200.ops on device tensors, pinned host copies around it")},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    line.update(extras)
    if parity is not None:
        line["parity"] = parity
    if configs is not None:
        line["configs"] = configs
    if reference_gpu is not None:
        line["reference_gpu"] = reference_gpu
    print(json.dumps(line), flush=True)
    ctx.close()


def run_layer_sweep(args):
    """The layer sweep on its own (the default workload's line carries the same object)."""
    ctx = Ctx()
    steps = args.steps or 20
    layers = measure_layers(ctx, steps, max(3, args.warmup))
    if ctx.rank == 0:
        total_ops = sum(2.0 * 8192 * e["N"] * e["K"] for e in layers)
        total_ms = sum(e["gemm_ms"] for e in layers)
        print(json.dumps({
            "metric": METRIC, "value": total_ops / (total_ms * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": ctx.world, "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": total_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": "layer_sweep",
                       "description": "INT8 QKV / O / gate-up / down projections at M=8192, N sharded",
                       "quant": ctx.q},
            "layers": layers}), flush=True)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="int8_8192")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline measurement (no configs / layers / parity / reference kernel)")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--group-size", type=int, default=None,
                    help="scale group size for the int4_w4a16 workload (16, 32, 64 or 128; default 128)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.workload == "layer_sweep":
        run_layer_sweep(args)
        return
    spec = workload_spec(args.workload)
    if args.group_size and spec["op"] == "mm_int4" and spec["M"] > 32:
        spec["G"] = args.group_size
        spec["desc"] = spec["desc"].replace("G=128", f"G={args.group_size}")
    if args.steps is None:
        # about a second of GPU work, so that clocks under load are actually sampled
        args.steps = {"int8_8192": 2000, "int8_8192_presummed": 2000, "int8_decode": 10000,
                      "int4_w4a16": 1500, "int4_w4a8": 3000, "dequant": 5000, "rmsnorm_quant": 4000,
                      "int8_swiglu": 2500, "int8_512": 20000, "int4_w4a16_decode": 10000,
                      "int4_w4a8_decode": 10000}[args.workload]
        if args.impl == "reference":
            args.steps = 5
    if args.impl == "reference":
        run_reference_arm(args, spec, args.workload)
    else:
        run_ours(args, spec, args.workload)


if __name__ == "__main__":
    main()
