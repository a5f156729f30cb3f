#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload int8_8192 | int8_8192_presummed | int8_decode | int4_w4a16 |
                                int4_w4a8 | int8_swiglu | dequant | rmsnorm_quant | layer_sweep]

One "step" is one `solve` call over one batch of synthetic input.  The default workload is
the INT8 quantized matmul M=N=K=8192 (uniform int8 inputs, per-tensor scales and non-zero
zero points drawn from a fixed seed).  With N > 1 GPUs (launched under torchrun, one rank
per GPU) the weight columns are sharded: every rank owns its own [K, 8192] slab and writes
its own slab of C, with no data-path collective (weak scaling: per-GPU work is fixed).

Prints ONE JSON line on rank 0.  `value` is device-resident throughput (CUDA events, max
over ranks); `e2e` is the same call with host buffers (pinned upload of A and B, download of
C inside the timed region); `roofline` describes the dominant kernel, timed with CUDA events
inside the timed region; `cpu_baseline` is the CPU oracle on a bounded sample of rows.

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


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of each workload's
# dominant kernel, from the ncu captures summarised under profiles/ (bytes; null where no
# capture has been taken).  Writes still sitting in L2 when the kernel ends are not in it.
NCU_TRAFFIC = {
    "int8_8192": (395.0e6, "profiles/int8_8192_umma_pair_kernel.md"),
    "int8_8192_presummed": (395.0e6, "profiles/int8_8192_umma_pair_kernel.md"),
    "int8_decode": (239.0e6, "profiles/int8_decode_skinny_kernel.md"),
    "int4_w4a16": (324.4e6, "profiles/int4_w4a16_tensor_kernel.md"),
    "int4_w4a8": (106.9e6, "profiles/int4_w4a8_pair_kernel.md"),
    "dequant": (482.8e6, "profiles/dequant_rows_vec4_kernel.md"),
    "rmsnorm_quant": (826.5e6, "profiles/rmsnorm_quant_row_kernel.md"),
}

# ----------------------------------------------------------------------------- workloads
def workload_spec(name: str):
    if name == "int8_8192":
        return dict(op="mm_int8", M=8192, N=8192, K=8192, dtype="int8",
                    desc="INT8 zero-point/scale matmul M=N=K=8192 (BASELINE config 2)")
    if name == "int8_8192_presummed":
        return dict(op="mm_int8", M=8192, N=8192, K=8192, dtype="int8", presummed=True,
                    desc="INT8 matmul M=N=K=8192 as an inference engine would issue it: colsum(B) "
                         "cached with the weight handle, rowsum(A) delivered by the activation "
                         "producer - the tensor kernel alone, no pre-pass")
    if name == "int8_decode":
        return dict(op="mm_int8", M=16, N=28672, K=8192, dtype="int8",
                    desc="INT8 decode-shaped matmul M=16 K=8192 N=28672 (BASELINE config 3)")
    if name == "int4_w4a16":
        return dict(op="mm_int4", M=4096, N=8192, K=8192, G=128, dtype="f16",
                    desc="W4A16 matmul M=4096 K=8192 N=8192 G=128 (BASELINE config 4)")
    if name == "int4_w4a8":
        return dict(op="mm_int4a8", M=4096, N=8192, K=8192, dtype="int8",
                    desc="W4A8 matmul M=4096 K=8192 N=8192: packed INT4 weights, INT8 activations, "
                         "per-tensor scales and zero points (BASELINE config 4, literal reading)")
    if name == "dequant":
        return dict(op="dequantization", M=8192, N=8192, T=128, dtype="f32",
                    desc="tile-scale dequantization 8192x8192 T=128")
    if name == "int8_swiglu":
        return dict(op="mm_int8_swiglu", M=8192, N=3584, K=8192, dtype="int8",
                    desc="INT8 gate/up projection with fused SwiGLU + requantisation: M=8192 K=8192, "
                         "2x3584 interleaved weight columns -> H [8192, 3584] (one GPU's share of the "
                         "BASELINE config 5 gate/up layer)")
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
    """(ops per step, minimum bytes per step)."""
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


# ------------------------------------------------------------------------- clock sampling
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.thread:
            self.thread.join(timeout=2)
        mhz, max_mhz, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                max_mhz = float(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max_mhz,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------ CPU arm
def load_oracle():
    from tests import harness  # the oracle is test infrastructure; used here as the CPU baseline

    return harness.load_oracle(), harness


def cpu_inputs(spec, harness):
    """Host copies of the synthetic inputs for the CPU arm (same generators as the GPU arm
    uses for parity, deterministic in the seed)."""
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
    """Times the CPU oracle on row samples; returns (units/s, rows per step, seconds list, threads)."""
    oracle, harness = load_oracle()
    inputs = cpu_inputs(spec, harness)
    q = quant_params()
    M = spec["M"]
    ops, _ = algorithmic_work(spec)
    if spec["op"] == "dequantization":
        rows = M
    else:
        probe = min(M, 2)
        t0 = time.perf_counter()
        cpu_run_rows(oracle, spec, inputs, q, 0, probe)
        per_row = max((time.perf_counter() - t0) / probe, 1e-6)
        rows = int(max(1, min(M, seconds_per_step / per_row)))
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
    return rate, rows, times, oracle.threads


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
        "scaling": "weak", "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
        "config": {"workload": workload, "description": spec["desc"],
                   "reference_path": "CPU loop of the reference harness restated in C "
                                     "(int64 dot, double scaling), OpenMP over rows"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------ GPU arm
def run_ours(args, spec, workload):
    import torch
    import torch.distributed as dist

    from texo_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    q = quant_params()
    ops_per_step, bytes_per_step = algorithmic_work(spec)

    # ---- inputs: resident in HBM before the timed region.  Each rank owns its own slab of
    # the weights (seeded by rank), activations are replicated (same seed everywhere).
    g_a = torch.Generator(device=dev).manual_seed(SEED)
    g_b = torch.Generator(device=dev).manual_seed(SEED + 1 + rank)
    if spec["op"] == "mm_int8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        if M == 16:
            A = torch.clamp(torch.round(torch.randn((M, K), generator=g_a, device=dev) * 20),
                            -128, 127).to(torch.int8)
        else:
            A = torch.randint(-128, 128, (M, K), generator=g_a, device=dev, dtype=torch.int8)
        # Rotate over enough weight/output sets that a step never finds its inputs in L2.
        nsets = max(2, int(np.ceil(3 * 126e6 / (K * N))) if M * K < 64e6 else 2)
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

        host_in = [torch.empty((M, K), dtype=torch.int8).pin_memory(),
                   torch.empty((K, N), dtype=torch.int8).pin_memory()]
        host_in[0].copy_(A)
        host_in[1].copy_(Bs[0])
        host_out = torch.empty((M, N), dtype=torch.int8).pin_memory()

        def e2e_step(i):
            ops.mm_int8_host(host_in[0], host_in[1], host_out, *q)

        h2d, d2h = M * K + K * N, M * N
        flush_note = (f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + K * N + M * N) / 2**20:.0f} MiB exceeds the 126 MB L2")
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

        hA, hB = A.cpu().pin_memory(), Bs[0].cpu().pin_memory()
        hH = torch.empty((M, F), dtype=torch.int8).pin_memory()
        dA, dB, dH = torch.empty_like(A), torch.empty_like(Bs[0]), torch.empty_like(Hs[0])

        def e2e_step(i):
            dA.copy_(hA, non_blocking=True)
            dB.copy_(hB, non_blocking=True)
            ops.mm_int8_swiglu(dA, dB, q[0], sg, su, sh, q[3], q[4], -q[4], q[5], out=dH)
            hH.copy_(dH, non_blocking=True)

        h2d, d2h = M * K + K * 2 * F, M * F
        flush_note = (f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + K * 2 * F + M * F) / 2**20:.0f} MiB")
    elif spec["op"] == "mm_int4a8":
        M, N, K = spec["M"], spec["N"], spec["K"]
        A = torch.randint(-128, 128, (M, K), generator=g_a, device=dev, dtype=torch.int8)
        nsets = 3
        Ws = [torch.randint(0, 256, (N, K // 2), generator=g_b, device=dev, dtype=torch.uint8)
              for _ in range(nsets)]
        Cs = [torch.empty((M, N), device=dev, dtype=torch.int8) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_mm_int4a8_solve(A.data_ptr(), Ws[j].data_ptr(), Cs[j].data_ptr(), M, N, K, *q)

        hA, hW = A.cpu().pin_memory(), Ws[0].cpu().pin_memory()
        hC = torch.empty((M, N), dtype=torch.int8).pin_memory()
        dA, dW, dC = torch.empty_like(A), torch.empty_like(Ws[0]), torch.empty_like(Cs[0])

        def e2e_step(i):
            dA.copy_(hA, non_blocking=True)
            dW.copy_(hW, non_blocking=True)
            ops.mm_int4a8(dA, dW, *q, out=dC)
            hC.copy_(dC, non_blocking=True)

        h2d, d2h = M * K + N * K // 2, M * N
        flush_note = (f"{nsets} weight/output sets rotated; working set per step "
                      f"{(M * K + N * K // 2 + M * N) / 2**20:.0f} MiB (A stays in L2, weights and "
                      f"outputs do not)")
    elif spec["op"] == "mm_int4":
        M, N, K, G = spec["M"], spec["N"], spec["K"], spec["G"]
        x = torch.randn((M, K), generator=g_a, device=dev).to(torch.float16)
        nsets = 2
        Ws = [torch.randint(0, 256, (N, K // 2), generator=g_b, device=dev, dtype=torch.uint8)
              for _ in range(nsets)]
        Ss = [(torch.rand((N, K // G), generator=g_b, device=dev) * 0.1 + 0.01).to(torch.float16)
              for _ in range(nsets)]
        Ys = [torch.empty((M, N), device=dev, dtype=torch.float16) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_mm_int4_solve(x.data_ptr(), Ws[j].data_ptr(), Ss[j].data_ptr(),
                                   Ys[j].data_ptr(), M, N, K, G)

        hx, hw, hs = (t.cpu().pin_memory() for t in (x, Ws[0], Ss[0]))
        hy = torch.empty((M, N), dtype=torch.float16).pin_memory()
        dx, dw, ds, dy = (torch.empty_like(t) for t in (x, Ws[0], Ss[0], Ys[0]))

        def e2e_step(i):
            dx.copy_(hx, non_blocking=True)
            dw.copy_(hw, non_blocking=True)
            ds.copy_(hs, non_blocking=True)
            ops.mm_int4(dx, dw, ds, G, out=dy)
            hy.copy_(dy, non_blocking=True)

        h2d = 2 * M * K + N * K // 2 + 2 * N * (K // G)
        d2h = 2 * M * N
        flush_note = f"{nsets} weight/output sets rotated; working set per step exceeds L2"
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

        h2d, d2h = 8 * M * N, 5 * M * N
        flush_note = f"{nsets} input/output sets rotated; 832 MiB per step exceeds L2"
    else:
        M, N, T = spec["M"], spec["N"], spec["T"]
        nsets = 2
        Xs = [torch.rand((M, N), generator=g_b, device=dev) * 16 - 8 for _ in range(nsets)]
        S = torch.rand((-(-M // T), -(-N // T)), generator=g_a, device=dev) * 1.5 + 0.5
        Ys = [torch.empty((M, N), device=dev) for _ in range(nsets)]

        def step(i):
            j = i % nsets
            lib.texo_dequantization_solve(Xs[j].data_ptr(), S.data_ptr(), Ys[j].data_ptr(), M, N, T)

        hX, hS = Xs[0].cpu().pin_memory(), S.cpu().pin_memory()
        hY = torch.empty((M, N)).pin_memory()
        dX, dS, dY = torch.empty_like(Xs[0]), torch.empty_like(S), torch.empty_like(Ys[0])

        def e2e_step(i):
            dX.copy_(hX, non_blocking=True)
            dS.copy_(hS, non_blocking=True)
            ops.dequantization(dX, dS, T, out=dY)
            hY.copy_(dY, non_blocking=True)

        h2d, d2h = 4 * M * N + 4 * S.numel(), 4 * M * N
        flush_note = f"{nsets} input/output sets rotated; 512 MiB per step exceeds L2"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timed region
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    launches0 = lib.texo_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    launches = lib.texo_kernel_launches() - launches0
    # Dominant-kernel duration for the roofline: the same steps again, immediately after and
    # still under load, this time with the library's CUDA-event bracket around the kernel.
    # (The bracket puts event records between the kernels of a call, which defeats the
    # programmatic-dependent-launch overlap, so it is kept out of the region `value` times.)
    n_prof = max(3, min(args.steps, 500))
    lib.texo_profile_enable(1)
    for i in range(n_prof):
        step(i)
    torch.cuda.synchronize()
    kernel_ms, kernel_n = ctypes.c_float(0), ctypes.c_int(0)
    lib.texo_profile_read(ctypes.byref(kernel_ms), ctypes.byref(kernel_n))
    lib.texo_profile_enable(0)
    clocks = sampler.stop() if rank == 0 else None
    status = lib.texo_mm_int8_status()

    # ---- end to end through the public API with host buffers
    for i in range(min(2, args.warmup)):
        e2e_step(i)
    barrier()
    n_e2e = max(3, min(args.steps, 20))
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(n_e2e):
        e2e_step(i)
    f1.record()
    barrier()
    e2e_ms = max_over_ranks(f0.elapsed_time(f1)) / n_e2e

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    ms_per_step = total_ms / args.steps
    value = ops_per_step * world / (ms_per_step * 1e-3) / 1e12
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    bracketed_ms = kernel_ms.value / max(1, kernel_n.value)
    # One launch per step: the timed region's own events give the average launch duration
    # (events around K back-to-back launches / K), which is what the roofline wants.  With
    # several kernels per step the dominant one is taken from the bracketed second pass.
    single_launch_steps = launches == args.steps
    kernel_avg_ms = ms_per_step if single_launch_steps else bracketed_ms
    long_run = total_ms > 300.0  # long enough for the power cap to pull the clocks down
    if spec["op"] in ("dequantization", "rms_norm_quant") or (spec["op"] == "mm_int8" and spec["M"] <= 32):
        peak = peaks.get("hbm_gbs", 6650.0)
        achieved = bytes_per_step / (kernel_avg_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": None,
                    "peak_source": "measured copy bandwidth" if peaks else "fallback 6650 GB/s"}
    else:
        # No INT8 figure is measured on this pool; kind::i8 issues at twice the bf16 rate, so
        # the denominator is 2x the measured cuBLAS bf16 throughput (W4A16 runs kind::f16: 1x).
        factor = 2.0 if spec["op"] in ("mm_int8", "mm_int4a8", "mm_int8_swiglu") else 1.0
        key = "bf16_tflops_sustained" if long_run else "bf16_tflops"
        base = peaks.get(key, 1400.0 if long_run else 1590.0)
        peak = factor * base
        achieved = ops_per_step / (kernel_avg_ms * 1e-3) / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
                    "frac": achieved / peak, "traffic": None,
                    "peak_source": f"{factor:g} x {'measured' if peaks else 'fallback'} bf16 "
                                   f"{'sustained' if long_run else 'burst'} ({base:.0f} TFLOP/s)"}
    if workload in NCU_TRAFFIC:
        roofline["traffic"], roofline["traffic_source"] = NCU_TRAFFIC[workload]
    roofline["kernel_ms"] = kernel_avg_ms
    if single_launch_steps:
        roofline["kernel_launches_timed"] = launches
        roofline["kernel_timing"] = ("one launch per step: CUDA events around the timed region / "
                                     "launches (back to back, as a caller issues them)")
        roofline["kernel_ms_isolated"] = bracketed_ms
    else:
        roofline["kernel_launches_timed"] = kernel_n.value
        roofline["kernel_timing"] = ("CUDA events around the dominant kernel over the %d steps "
                                     "that directly follow the timed region" % n_prof)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rate, rows, times, threads = cpu_rate(spec, 6.0, 2, 0)
        cpu = {"value": rate / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{rows} of {spec['M']} output rows x 2 runs (all columns, full K), "
                         f"{sum(times):.1f} s of CPU work"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
        "config": {"workload": workload, "description": spec["desc"],
                   "sharding": f"{world} column slab(s) of {spec['N']} output columns, one per GPU",
                   "l2": flush_note, "quant": q, "status_word": status},
        "clocks": clocks,
        "e2e": {"value": ops_per_step * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_layer_sweep(args):
    """BASELINE config 5: the four INT8 projections of a transformer layer at M = 8192, weight
    columns sharded over the ranks (strong scaling: the layer is fixed, each GPU owns N/g
    columns), without the all-gather of C, with an NCCL all-gather after the matmul, and with
    the gather fused into the matmul's epilogue (peer stores).  Prints one JSON line with one
    entry per projection; `value` is the aggregate TOPS of the four GEMMs without the gather."""
    import torch
    import torch.distributed as dist

    from texo_b200 import _lib, sharded

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    q = quant_params()
    M = 8192
    layers = [("qkv", 8192, 10240), ("o_proj", 8192, 8192), ("gate_up", 8192, 57344),
              ("down", 28672, 8192)]
    steps = args.steps or 50
    g = torch.Generator(device=dev).manual_seed(SEED + rank)
    results, total_ops, total_ms = [], 0.0, 0.0

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for name, K, N in layers:
        n0, n1 = sharded.column_slab(N, world, rank)
        A = torch.randint(-128, 128, (M, K), generator=torch.Generator(device=dev).manual_seed(SEED),
                          device=dev, dtype=torch.int8)
        B = torch.randint(-128, 128, (K, n1 - n0), generator=g, device=dev, dtype=torch.int8)
        C = torch.empty((M, n1 - n0), device=dev, dtype=torch.int8)

        def gemm():
            lib.texo_mm_int8_solve(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, n1 - n0, K, *q)

        def gemm_gather():
            gemm()
            if world > 1:
                sharded.all_gather_columns(C, N)

        ms = timed(gemm)
        ms_g = timed(gemm_gather) if world > 1 else ms
        # the gather fused into the matmul's epilogue: every rank stores its slab into all
        # ranks' copies of C (symmetric memory); one barrier per call makes the result usable
        ms_f = ms
        if world > 1:
            out = sharded.GatheredOutput(M, N, dev)

            def gemm_fused_gather():
                sharded.mm_int8_allgather(A, B, out, *q)
                out.wait()

            ms_f = timed(gemm_fused_gather)
            del out
        ops = 2.0 * M * N * K
        results.append({"layer": name, "K": K, "N": N, "slab": n1 - n0, "gemm_ms": ms,
                        "gemm_plus_gather_ms": ms_g, "gemm_fused_gather_ms": ms_f,
                        "tops": ops / (ms * 1e-3) / 1e12})
        total_ops += ops
        total_ms += ms
        del A, B, C
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": total_ops / (total_ms * 1e-3) / 1e12, "unit": UNIT,
            "n_gpus": world, "steps": steps, "warmup": max(3, args.warmup), "ms_per_step": total_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic",
            "config": {"workload": "layer_sweep",
                       "description": "INT8 QKV / O / gate-up / down projections at M=8192, N sharded",
                       "quant": q},
            "layers": results}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="int8_8192")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.workload == "layer_sweep":
        run_layer_sweep(args)
        return
    spec = workload_spec(args.workload)
    if args.steps is None:
        # about a second of GPU work, so that clocks under load are actually sampled
        args.steps = {"int8_8192": 2000, "int8_8192_presummed": 2000, "int8_decode": 10000,
                      "int4_w4a16": 1500, "int4_w4a8": 3000, "dequant": 5000, "rmsnorm_quant": 4000,
                      "int8_swiglu": 2500}[args.workload]
        if args.impl == "reference":
            args.steps = 5
    if args.impl == "reference":
        run_reference_arm(args, spec, args.workload)
    else:
        run_ours(args, spec, args.workload)


if __name__ == "__main__":
    main()
