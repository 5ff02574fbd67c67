#!/usr/bin/env python
"""Headline benchmark: FP32-I/O GEMM TFLOP/s on 8192^3, N-column sharded over 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision tf32|3xtf32]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path: C = A.B with A [8192,8192], B [8192,8192] (this rank's column block of a
[8192, 8192*N] matrix), FP32 in and out, synthetic uniform(-1,1) inputs.  Every rank holds all of A and its own
columns of B and produces its own columns of C; nothing is exchanged while computing (weak scaling: the per-GPU
work stays 8192^3 as N grows).  FLOPs are counted as 2*M*N*K in both precision modes, the reference's
convention (src/benchmarks/matmul_benchmark.cpp:73-76).

Prints ONE JSON line: the device-resident throughput (`value`), the same metric through the host-buffer entry
point with the PCIe copies inside the timed region (`e2e`), the roofline of the GEMM kernel against the measured
tensor peak, the reference's CPU matmul timed on this box's host cores (`cpu_baseline`), and the clocks seen.

`--impl reference` times the reference's own CPU implementation (oracle/_ref, compiled from its sources) on a
bounded sample of the same workload and prints the same line shape with "impl": "reference".
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N_PER_GPU = K = 8192
METRIC = "gemm_fp32_io_tflops"
UNIT = "TFLOP/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed region runs (read-only query)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0, t1):
        sm, smax, power, reasons = [], [], [], set()
        for ts, line in self.rows:
            if ts < t0 or ts > t1:
                continue
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(smax), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_gemm(size, repeats=1):
    """Times Tensor::matmul of the reference's CPU path (single-threaded by construction) on size^3.
    Returns (TFLOP/s, kind, cores, seconds)."""
    import numpy as np
    from oracle import binding
    rng = binding.SeededRng(42)
    a, b = rng.uniform((size, size)), rng.uniform((size, size))
    if binding.Reference.available():
        ref = binding.Reference()
        va, vb = binding.ref_view(a.shape), binding.ref_view(b.shape)
        run = lambda: ref.matmul(a, va, b, vb, out_shape=(size, size))
        kind = "reference"
    else:
        orc = binding.Oracle()
        run = lambda: orc.matmul(a, b)
        kind = "port"
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        run()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return 2.0 * size ** 3 / best / 1e12, kind, 1, best


def run_reference_arm(args, rank, world):
    """The reference's own CPU matmul, timed on the host cores; rank 0 only."""
    if rank != 0:
        return
    size = 1024      # one step = one 1024^3 product: 1/512 of the flops of an 8192^3 step, ~1 s of CPU work
    for _ in range(min(args.warmup, 1)):
        cpu_reference_gemm(size)
    t0 = time.perf_counter()
    kind = "reference"
    for _ in range(args.steps):
        _, kind, _, _ = cpu_reference_gemm(size)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = 2.0 * size ** 3 / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind,
                         "sample": "Tensor::matmul %d^3 per step (1/%d of the flops of one 8192^3 step); the reference CPU "
                                   "matmul is single-threaded, so 1 of %d host cores" % (size, (8192 // size) ** 3, os.cpu_count() or 1)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    if getattr(args, "scaling", "weak") == "strong":
        return {"workload": "gemm_fp32_8192x8192x8192_total", "M": M, "N_total": N_PER_GPU, "K": K,
                "layout": "row-major A . row-major B", "precision_mode": args.precision,
                "sharding": "N column blocks of 8192/world, no collective in the timed region", "world": world,
                "l2": "operands larger than the 126 MB L2"}
    return {"workload": "gemm_fp32_8192x8192x8192_per_gpu", "M": M, "N_per_gpu": N_PER_GPU, "K": K,
            "layout": "row-major A . row-major B", "precision_mode": args.precision,
            "sharding": "N column blocks, one block per GPU, no collective in the timed region", "world": world,
            "l2": "operands (268 MB each) larger than the 126 MB L2"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak (default): every GPU multiplies its own 8192-column block; strong: one 8192^3 product "
                         "split into N column blocks of 8192/N")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from torch_engine_b200 import lib as L
    from torch_engine_b200 import ops, sharding

    assert torch.cuda.is_available(), "bench.py needs a GPU; the backend has no CPU path"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    be = ops.Backend(local_rank, workspace_bytes=(3 << 30) if args.precision == "3xtf32" else (64 << 20))

    # This rank's column block of the [K, 8192*world] right-hand matrix, already local and contiguous.
    if args.scaling == "weak":
        n0, ncols = sharding.column_shard(N_PER_GPU * world, world, rank, N_PER_GPU)
        assert ncols == N_PER_GPU
    else:
        n0, ncols = sharding.column_shard(N_PER_GPU, world, rank, sharding.COLUMN_ALIGN)
    gen = torch.Generator(device="cuda").manual_seed(42 + rank)
    a = torch.rand(M, K, device="cuda", generator=gen) * 2 - 1
    b = torch.rand(K, ncols, device="cuda", generator=gen) * 2 - 1
    c = torch.empty(M, ncols, device="cuda")
    d = L.GemmDesc()
    d.M, d.N, d.K = M, ncols, K
    d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    d.lda, d.ldb, d.ldc = K, ncols, ncols
    d.batch_outer = d.batch_inner = 1
    d.alpha = 1.0
    d.precision = L.TE_PREC_TF32 if args.precision == "tf32" else L.TE_PREC_3XTF32

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        be.gemm(d)
    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    launches0 = be.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record()
    for _ in range(args.steps):
        be.gemm(d)
    e1.record()
    barrier()
    t_wall1 = time.time()
    launches = be.launches - launches0
    ms_total = e0.elapsed_time(e1)
    # keep the same kernel running (untimed) until the sampler has a second of readings under load
    t_keep = time.time()
    while time.time() - t_keep < 1.0:
        for _ in range(20):
            be.gemm(d)
        torch.cuda.synchronize()
    t_wall2 = time.time()
    sampler.stop()
    be.check_device_status()

    t = torch.tensor([ms_total], device="cuda", dtype=torch.float64)
    ln = torch.tensor([launches], device="cuda", dtype=torch.int64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(ln, op=dist.ReduceOp.SUM)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    flops_step = 2.0 * M * K * (N_PER_GPU * world if args.scaling == "weak" else N_PER_GPU)
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- end to end: host buffers in pinned memory, H2D of A and B and D2H of C inside the timed region ----
    ha = torch.empty(M, K, dtype=torch.float32).pin_memory()
    hb = torch.empty(K, ncols, dtype=torch.float32).pin_memory()
    hc = torch.empty(M, ncols, dtype=torch.float32).pin_memory()
    ha.copy_(a)
    hb.copy_(b)
    hd = L.GemmDesc()
    hd.M, hd.N, hd.K = M, ncols, K
    hd.a, hd.b, hd.c = ha.data_ptr(), hb.data_ptr(), hc.data_ptr()
    hd.lda, hd.ldb, hd.ldc = K, ncols, ncols
    hd.batch_outer = hd.batch_inner = 1
    hd.alpha = 1.0
    hd.precision = d.precision
    be.gemm_host(hd)      # warm-up (allocates the staging buffers)
    be.gemm_host(hd)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        be.gemm_host(hd)  # synchronises internally: the result is in host memory when it returns
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    te = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = flops_step / float(te.item()) / 1e12
    checksum_ok = bool(torch.isfinite(hc[::997, ::991]).all().item())

    if rank == 0:
        peaks = measured_peaks()
        tf32_peak = peaks["bf16_burst"] / 2.0
        per_gpu_tflops = value / world
        clocks = sampler.summary(t_wall0, t_wall2)
        clocks["window"] = "timed region plus %.1f s of the same kernel untimed" % (t_wall2 - t_wall1)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "tf32" if args.precision == "tf32" else "3xtf32", "data": "synthetic",
            "config": workload_config(args, world),
            "gpu_launches": int(ln.item()),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * (M * K + K * ncols),
                    "d2h_bytes_per_step": 4 * M * ncols, "finite": checksum_ok},
            "roofline": {"bound": "tensor", "achieved": per_gpu_tflops, "peak": tf32_peak, "unit": "TFLOP/s",
                         "frac": per_gpu_tflops / tf32_peak,
                         "peak_source": "%s bf16 burst %.1f TFLOP/s / 2 (tf32 runs at half the bf16 rate)" % (peaks["source"], peaks["bf16_burst"]),
                         "frac_of_nominal_1125": per_gpu_tflops / 1125.0,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one 8192x8192x8192 launch, single-pass ncu
                         # capture of this kernel (profiles/gemm_tf32_pair_8192_bench_launch_list.md)
                         "traffic": 2412997888 if (ncols == N_PER_GPU and args.precision == "tf32") else None,
                         "algorithmic_bytes": 4 * (M * K + K * ncols + M * ncols)},
            "clocks": clocks,
        }
        if not args.no_cpu_baseline:
            v, kind, cores, secs = cpu_reference_gemm(2048)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                                    "sample": "one Tensor::matmul 2048^3 (%.1f s; 1/64 of the flops of an 8192^3 step), "
                                              "single-threaded as the reference is: 1 of %d host cores" % (secs, os.cpu_count() or 1)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()


if __name__ == "__main__":
    main()
