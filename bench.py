#!/usr/bin/env python
"""Headline benchmark: FP32-I/O GEMM TFLOP/s on 8192^3, N-column sharded over 1/2/4/8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision tf32|3xtf32]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is one pass of the hot path over ONE product C = A.B with A [8192,8192], B [8192,8192], FP32 in and out,
synthetic uniform(-1,1) inputs.  With N GPUs the product is split into N column blocks of 8192/N (strong scaling, the
default): every rank holds all of A and its own columns of B in its own HBM and produces its own columns of C; nothing is
exchanged while computing.  `--scaling weak` instead gives every rank a whole 8192-column block of an [8192, 8192*N]
right-hand side.  FLOPs are counted as 2*M*N*K in both precision modes, the reference's convention
(src/benchmarks/matmul_benchmark.cpp:73-76).

Prints ONE JSON line:
  value            device-resident throughput of the timed steps (CUDA events, max over ranks)
  value_sustained  the same over a loop of at least two seconds (the power-capped clock), with the clocks seen
  with_all_gather  the step followed by the all-gather that reassembles C on every rank (library's NCCL driver + one
                   re-tile kernel), N > 1 only: time, throughput, NVLink bytes received per rank
  e2e              the same product through the host-buffer entry points with pinned HOST operands, PCIe copies inside
                   the timed region: te_b200_gemm_f32_host at N = 1, te_b200_gemm_f32_host_sharded at N > 1 (each rank
                   uploads 1/N of A and its columns of B, the ranks replicate A over NVLink)
  check            relative error of 16 sampled rows of C against a float64 product (the run fails above the tolerance)
  modes            the other precision mode on the same operands: value, roofline against peak/3, error
  roofline         achieved / measured tensor peak of the GEMM kernel
  comparators      the reference's own CUDA FP32 matmul (cublasSgemm path and `custom` kernel, built for sm_100a) and
                   cuBLAS with TF32 math, timed in this process on rank 0 (N = 1 only)
  cpu_baseline     the reference's CPU Tensor::matmul on this box's host cores (N = 1 only)

`--impl reference` times the reference's own CPU implementation (oracle/_ref, compiled from its sources) on a bounded
sample of the same workload and prints the same line shape with "impl": "reference".
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

M = N_FULL = K = 8192
METRIC = "gemm_fp32_io_tflops"
UNIT = "TFLOP/s"
TOL = {"tf32": 2e-3, "3xtf32": 1e-5}
REFERENCE_SAMPLE = 1024      # the reference arm times Tensor::matmul on REFERENCE_SAMPLE^3 per step


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "hbm_gbs": p["hbm_gbs"],
                "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU while the timed regions run (read-only query)."""
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
                                          "--format=csv,noheader,nounits", "-lms", "20"],
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
        """Only the samples taken between t0 and t1."""
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
    size = REFERENCE_SAMPLE   # 1/512 of the flops of an 8192^3 step, ~0.6 s of CPU work per step
    for _ in range(min(args.warmup, 1)):
        cpu_reference_gemm(size)
    t0 = time.perf_counter()
    kind = "reference"
    for _ in range(args.steps):
        _, kind, _, _ = cpu_reference_gemm(size)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = 2.0 * size ** 3 / dt / 1e12
    cfg = workload_config(args, world)     # the GPU arm's config, unchanged; what is actually timed is stated beside it
    sample = ("each timed step is Tensor::matmul on %d^3 (1/%d of the flops of the 8192^3 step the GPU arm times); "
              "TFLOP/s is a rate and the CPU rate does not depend on the size" % (size, (8192 // size) ** 3))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": cfg, "timed_sample": sample,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind,
                         "sample": "Tensor::matmul %d^3 per step (1/%d of the flops of one 8192^3 step); the reference CPU "
                                   "matmul is single-threaded, so 1 of %d host cores" % (size, (8192 // size) ** 3, os.cpu_count() or 1)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    if args.scaling == "strong":
        return {"workload": "gemm_fp32_8192x8192x8192", "M": M, "N": N_FULL, "K": K,
                "layout": "row-major A . row-major B", "precision_mode": args.precision,
                "sharding": "one product split into %d column block(s) of %d; no collective inside the product" % (world, N_FULL // max(world, 1)),
                "world": world, "l2": "A (268 MB) is larger than the 126 MB L2"}
    return {"workload": "gemm_fp32_8192x8192x8192_per_gpu", "M": M, "N_per_gpu": N_FULL, "K": K,
            "layout": "row-major A . row-major B", "precision_mode": args.precision,
            "sharding": "N column blocks, one 8192-column block per GPU, no collective inside the product", "world": world,
            "l2": "operands (268 MB each) larger than the 126 MB L2"}


def comparators(torch, a, b, c_ours, steps):
    """The reference's own CUDA FP32 matmul on this GPU (its cublasSgemm path and its `custom` cp.async kernel, built
    from its sources for sm_100a with the b200 binding applied) and cuBLAS with TF32 math, in this process.  The
    reference's numbers are measured through its Tensor::matmul on mt19937(42) operands, including its per-call
    cudaMalloc of the result."""
    out = {}
    flops = 2.0 * M * K * N_FULL
    try:
        from oracle import binding
        if not binding.ReferenceCuda.available():
            raise RuntimeError("oracle/_ref_cuda/libref_cuda.so was not built (needs the reference sources at build time)")
        ref = binding.ReferenceCuda(backend=None)
        ref.cublas_tf32(False)
        ms, _ = ref.time_matmul(M, K, N_FULL, warmup=2, iters=5)
        out["reference_cublas_sgemm_fp32"] = {"ms": ms, "tflops": flops / ms / 1e9}
        ref.configure("custom")
        ms, _ = ref.time_matmul(M, K, N_FULL, warmup=1, iters=3)
        out["reference_custom_kernel_fp32"] = {"ms": ms, "tflops": flops / ms / 1e9}
        ref.configure("b200", "tf32")
        ms, _ = ref.time_matmul(M, K, N_FULL, warmup=2, iters=5)
        out["reference_with_b200_backend_tf32"] = {"ms": ms, "tflops": flops / ms / 1e9,
                                                   "note": "the reference's Tensor::matmul with TENSOR_GEMM_BACKEND=b200"}
        ref.configure(None)
        ref.cublas_tf32(True)
        ms, _ = ref.time_matmul(M, K, N_FULL, warmup=2, iters=5)
        out["reference_cublas_with_tf32_math"] = {"ms": ms, "tflops": flops / ms / 1e9,
                                                  "note": "a mode the reference never enables; comparator only"}
        ref.cublas_tf32(False)
    except Exception as e:   # the comparators are reported, never required
        out["reference_cuda"] = {"unavailable": str(e)[:200]}
    try:
        torch.backends.cuda.matmul.allow_tf32 = True
        for _ in range(3):
            torch.matmul(a, b)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            torch.matmul(a, b)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out["cublas_tf32_via_torch"] = {"ms": ms, "tflops": flops / ms / 1e9}
    except Exception as e:
        out["cublas_tf32_via_torch"] = {"unavailable": str(e)[:200]}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): one 8192^3 product split into N column blocks of 8192/N; weak: every GPU "
                         "multiplies its own 8192-column block")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-comparators", action="store_true")
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
    be = ops.Backend(local_rank, workspace_bytes=(3 << 30))
    comm = sharding.Communicator(be, world, rank) if world > 1 else None

    # This rank's column block of the right-hand matrix, already local and contiguous.
    if args.scaling == "weak":
        n_total = N_FULL * world
        n0, ncols = sharding.column_shard(n_total, world, rank, N_FULL)
        assert ncols == N_FULL
    else:
        n_total = N_FULL
        n0, ncols = sharding.column_shard(n_total, world, rank, sharding.COLUMN_ALIGN)
    gen = torch.Generator(device="cuda").manual_seed(42)
    a = torch.rand(M, K, device="cuda", generator=gen) * 2 - 1                    # the same A on every rank
    gen.manual_seed(1000 + rank)
    b = torch.rand(K, ncols, device="cuda", generator=gen) * 2 - 1
    c = torch.empty(M, ncols, device="cuda")

    def desc_for(precision, aa=a, bb=b, cc=c):
        d = L.GemmDesc()
        d.M, d.N, d.K = M, ncols, K
        d.a, d.b, d.c = aa.data_ptr(), bb.data_ptr(), cc.data_ptr()
        d.lda, d.ldb, d.ldc = K, ncols, ncols
        d.batch_outer = d.batch_inner = 1
        d.alpha = 1.0
        d.precision = L.TE_PREC_TF32 if precision == "tf32" else L.TE_PREC_3XTF32
        return d

    d = desc_for(args.precision)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps):
        """ms per step of `steps` back-to-back calls, CUDA events on the launching stream, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps, t0, time.time()

    flops_step = 2.0 * M * K * n_total
    warm = max(args.warmup, 3)
    for _ in range(warm):
        be.gemm(d)
    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- the timed steps ---------------------------------------------------------------------------------------
    launches0 = be.launches
    ms_step, tb0, tb1 = timed(lambda: be.gemm(d), args.steps)
    launches = be.launches - launches0
    value = flops_step / (ms_step * 1e-3) / 1e12

    # ---- sustained: the same step for at least --sustained-seconds ------------------------------------------------
    n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / ms_step) + 1)
    ms_sus, ts0, ts1 = timed(lambda: be.gemm(d), n_sus)
    value_sustained = flops_step / (ms_sus * 1e-3) / 1e12
    be.check_device_status()

    # ---- correctness of what was timed: 16 sampled rows against a float64 product -----------------------------------
    rows = torch.linspace(0, M - 1, 16, device="cuda").long()
    ref_rows = a[rows].double() @ b.double()
    err = float((c[rows].double() - ref_rows).abs().max() / ref_rows.abs().max())
    err = max_over_ranks(err)

    # ---- the step followed by the all-gather of C (N > 1) -----------------------------------------------------------
    gather = None
    if comm is not None and args.scaling == "strong":
        c_full = torch.empty(M, n_total, device="cuda")
        staging = torch.empty(M * n_total, device="cuda")

        def step_and_gather():
            be.gemm(d)
            comm.all_gather_columns(c, n_total, out=c_full, staging=staging)

        for _ in range(3):
            step_and_gather()
        ms_g, _, _ = timed(step_and_gather, args.steps)
        ms_ag, _, _ = timed(lambda: comm.all_gather_columns(c, n_total, out=c_full, staging=staging), args.steps)
        be.check_device_status()
        ok = bool(torch.equal(c_full[:, n0:n0 + ncols], c))
        rows_g = a[rows].double() @ b.double()
        gather = {"ms_per_step": ms_g, "value": flops_step / (ms_g * 1e-3) / 1e12, "unit": UNIT,
                  "all_gather_ms": ms_ag, "nvlink_bytes_received_per_rank": 4 * M * (n_total - ncols),
                  "nvlink_gbs_per_rank": 4 * M * (n_total - ncols) / (ms_ag * 1e-3) / 1e9,
                  "own_block_intact": ok,
                  "how": "te_b200_all_gather_columns: one NCCL all-gather of the [M, N/world] blocks + one re-tile kernel; C [M,N] on every rank"}
        del c_full, staging, rows_g

    # ---- the other precision mode on the same operands ------------------------------------------------------------
    other = "3xtf32" if args.precision == "tf32" else "tf32"
    c2 = torch.empty_like(c)
    d2 = desc_for(other, cc=c2)
    for _ in range(2):
        be.gemm(d2)
    n_other = max(5, args.steps // 4)
    ms_other, _, _ = timed(lambda: be.gemm(d2), n_other)
    be.check_device_status()
    err_other = max_over_ranks(float((c2[rows].double() - ref_rows).abs().max() / ref_rows.abs().max()))
    del c2

    # ---- end to end: pinned host operands, PCIe copies inside the timed region --------------------------------------
    sharded_e2e = comm is not None and args.scaling == "strong"
    if not sharded_e2e:
        ha = torch.empty(M, K, dtype=torch.float32).pin_memory()
        hb = torch.empty(K, ncols, dtype=torch.float32).pin_memory()
        hc = torch.empty(M, ncols, dtype=torch.float32).pin_memory()
        ha.copy_(a)
        hb.copy_(b)
        hd = desc_for(args.precision, ha, hb, hc)
        run_e2e = lambda: be.gemm_host(hd)
        h2d, d2h = 4 * (M * K + K * ncols), 4 * M * ncols
        e2e_how = "te_b200_gemm_f32_host: row-block pipelined H2D / product / D2H on three streams"
        hc_block, hb_cols = hc, hb
    else:
        # every rank holds the whole host operands (of ITS view of the problem: all of A, the full-width B) and gets its
        # columns of C back; over PCIe it moves 1/world of A, its columns of B and its columns of C
        hb_full = torch.empty(K, n_total, dtype=torch.float32).pin_memory()
        gen_cpu = torch.Generator().manual_seed(7)
        hb_full.uniform_(-1, 1, generator=gen_cpu)
        ha = torch.empty(M, K, dtype=torch.float32).pin_memory()
        ha.copy_(a)
        hc = torch.zeros(M, n_total, dtype=torch.float32).pin_memory()
        hd = L.GemmDesc()
        hd.M, hd.N, hd.K = M, n_total, K
        hd.a, hd.b, hd.c = ha.data_ptr(), hb_full.data_ptr(), hc.data_ptr()
        hd.lda, hd.ldb, hd.ldc = K, n_total, n_total
        hd.batch_outer = hd.batch_inner = 1
        hd.alpha = 1.0
        hd.precision = d.precision
        run_e2e = lambda: comm.gemm_host_sharded(hd, sharding.COLUMN_ALIGN)
        hc_block, hb_cols = hc[:, n0:n0 + ncols], hb_full[:, n0:n0 + ncols]
        h2d, d2h = 4 * (M * K // world + K * ncols), 4 * M * ncols
        e2e_how = ("te_b200_gemm_f32_host_sharded: each rank uploads M/world rows of A and its columns of B, NCCL all-gather of A "
                   "over NVLink (%d bytes received per rank), product, D2H of its columns of C" % (4 * (M - M // world) * K))
    run_e2e()      # warm-up (allocates the staging buffers)
    run_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        run_e2e()  # synchronises internally: the result is in host memory when it returns
    barrier()
    e2e_s = max_over_ranks((time.perf_counter() - t0) / args.e2e_steps)
    e2e_value = flops_step / e2e_s / 1e12
    hrow = hc_block[M // 2].double()
    href = ha[M // 2].double() @ hb_cols.double()
    e2e_err = max_over_ranks(float((hrow - href).abs().max() / href.abs().max()))
    sampler.stop()

    ln = torch.tensor([launches], device="cuda", dtype=torch.int64)
    if world > 1:
        dist.all_reduce(ln, op=dist.ReduceOp.SUM)

    if rank == 0:
        peaks = measured_peaks()
        tf32_peak, tf32_sustained = peaks["bf16_burst"] / 2.0, peaks["bf16_sustained"] / 2.0
        denom = {"tf32": 1.0, "3xtf32": 3.0}
        per_gpu = value / world
        clocks = sampler.summary(ts0, ts1)
        clocks["window"] = "the sustained timed loop (%.2f s, %d steps)" % (ts1 - ts0, n_sus)
        clocks["timed_steps_window"] = dict(sampler.summary(tb0, tb1), seconds=tb1 - tb0)
        if clocks["sm_mhz"]:
            clocks["ms_times_sm_mhz_sustained"] = ms_sus * clocks["sm_mhz"]
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": args.precision, "data": "synthetic",
            "config": workload_config(args, world),
            "gpu_launches": int(ln.item()),
            "value_sustained": {"value": value_sustained, "unit": UNIT, "ms_per_step": ms_sus, "steps": n_sus,
                                "frac_of_sustained_peak": value_sustained / world / (tf32_sustained / denom[args.precision]),
                                "peak": tf32_sustained / denom[args.precision],
                                "peak_source": "%s bf16 sustained %.1f TFLOP/s / 2%s" % (peaks["source"], peaks["bf16_sustained"], " / 3 (three MMAs per product term)" if args.precision == "3xtf32" else "")},
            "check": {"rows": 16, "rel_err_vs_fp64": err, "tolerance": TOL[args.precision], "e2e_rel_err_vs_fp64": e2e_err},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "how": e2e_how},
            "modes": {other: {"value": flops_step / (ms_other * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_other, "steps": n_other,
                              "rel_err_vs_fp64": err_other, "tolerance": TOL[other],
                              "roofline_frac": flops_step / (ms_other * 1e-3) / 1e12 / world / (tf32_peak / denom[other]),
                              "roofline_peak": tf32_peak / denom[other],
                              "note": "credited 2*M*N*K; the 3xTF32 mode issues three MMAs per term, so its ceiling is a third of the TF32 peak"}},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": tf32_peak / denom[args.precision], "unit": "TFLOP/s",
                         "frac": per_gpu / (tf32_peak / denom[args.precision]),
                         "peak_source": "%s bf16 burst %.1f TFLOP/s / 2 (tf32 runs at half the bf16 rate)" % (peaks["source"], peaks["bf16_burst"]),
                         "frac_of_nominal_1125": per_gpu / 1125.0,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one 8192x8192x8192 launch, single-pass ncu
                         # capture of this kernel (profiles/gemm_tf32_pair_8192_bench_launch_list.md)
                         "traffic": 2412997888 if (ncols == N_FULL and args.precision == "tf32") else None,
                         "algorithmic_bytes": 4 * (M * K + K * ncols + M * ncols)},
            "clocks": clocks,
        }
        if gather is not None:
            line["with_all_gather"] = gather
        if world == 1 and not args.no_comparators:
            line["comparators"] = comparators(torch, a, b, c, max(5, args.steps // 2))
        if world == 1 and not args.no_cpu_baseline:
            v, kind, cores, secs = cpu_reference_gemm(2048)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                                    "sample": "one Tensor::matmul 2048^3 (%.1f s; 1/64 of the flops of an 8192^3 step), "
                                              "single-threaded as the reference is: 1 of %d host cores" % (secs, os.cpu_count() or 1)}
        print(json.dumps(line), flush=True)
    failed = err > TOL[args.precision] or err_other > TOL[other] or e2e_err > TOL[args.precision]
    if failed and rank == 0:
        print("bench.py: a sampled row of C is outside the tolerance (%.3e, %.3e, %.3e)" % (err, err_other, e2e_err), file=sys.stderr)
    if comm is not None:
        comm.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    be.close()
    if failed:
        sys.exit(1)


if __name__ == "__main__":
    main()
