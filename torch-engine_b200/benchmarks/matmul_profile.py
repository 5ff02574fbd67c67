"""Profiling harness: one warm-up launch and a few profiled launches of the GEMM kernel on one shape, the
role src/benchmarks/matmul_profile.cpp (:47-50, :149-187) plays for the reference's kernels under
src/benchmarks/run_ncu_sweep.sh.  Meant to be run under `ncu -k regex:gemm_tf32`.

    python torch-engine_b200/benchmarks/matmul_profile.py --m 4096 --n 4096 --k 4096 --precision tf32 --layout nn
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from torch_engine_b200 import ops  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32"])
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tn"],
                    help="nn: row-major A and B; nt: column-major B (Linear weight); tn: column-major A, row-major B (weight gradient dY^T . X)")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--epilogue", default="none", choices=["none", "bias", "bias_gelu"],
                    help="with --layout nt: run the product as Linear::forward with the bias (and GELU) in the GEMM epilogue")
    args = ap.parse_args()
    be = ops.Backend(0, workspace_bytes=2 << 30)
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.rand(args.m, args.k, device="cuda", generator=g) * 2 - 1
    if args.layout == "tn":
        a = (torch.rand(args.k, args.m, device="cuda", generator=g) * 2 - 1).t()
    if args.layout in ("nn", "tn"):
        b = torch.rand(args.k, args.n, device="cuda", generator=g) * 2 - 1
    else:
        b = (torch.rand(args.n, args.k, device="cuda", generator=g) * 2 - 1).t()
    if args.epilogue != "none":
        assert args.layout == "nt", "--epilogue runs Linear::forward, whose weight is the nt layout"
        w, bias = b.t(), torch.rand(args.n, device="cuda", generator=g)
        run = lambda: be.linear_forward(a, w, bias, gelu=args.epilogue == "bias_gelu", precision=args.precision)
    else:
        run = lambda: be.matmul(a, b, precision=args.precision)
    run()          # warm-up
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.launches):
        c = run()
    e1.record()
    torch.cuda.synchronize()
    be.check_device_status()
    ms = e0.elapsed_time(e1) / args.launches
    print("%dx%dx%d %s %s: %.3f ms/launch, %.1f TFLOP/s, checksum %.6e" %
          (args.m, args.n, args.k, args.precision, args.layout, ms, 2.0 * args.m * args.n * args.k / ms / 1e9,
           float(c[::97, ::89].double().sum())))


if __name__ == "__main__":
    main()
