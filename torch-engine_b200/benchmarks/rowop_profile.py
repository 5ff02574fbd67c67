"""Profiling harness for the streaming kernels around the matmuls: two warm-up calls and a few timed calls of one of
them on a [rows, cols] activation, meant to be run under `ncu -k regex:<kernel>`.

    python torch-engine_b200/benchmarks/rowop_profile.py --op gelu_backward --rows 16384 --cols 3072

Ops: gelu, gelu_backward, colsum, layernorm, layernorm_backward, layernorm_backward_residual (with the gradient of a
bypassing branch added and the column sums of the result), softmax, softmax_backward.  The printed GB/s uses the
algorithmic bytes (every input read once, every output written once).
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
    ap.add_argument("--op", default="gelu_backward")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=3072)
    ap.add_argument("--calls", type=int, default=3)
    args = ap.parse_args()
    be = ops.Backend(0, workspace_bytes=64 << 20)
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn(args.rows, args.cols, device="cuda", generator=g)
    dy = torch.randn(args.rows, args.cols, device="cuda", generator=g)
    gamma = torch.rand(args.cols, device="cuda", generator=g) + 0.5
    beta = torch.randn(args.cols, device="cuda", generator=g)
    beta_rows = torch.randn(args.rows, args.cols, device="cuda", generator=g) if args.op == "layernorm_backward_residual" else None
    n = 4.0 * x.numel()
    calls = {
        "gelu": (lambda: be.gelu(x), 2 * n),
        "gelu_backward": (lambda: be.gelu_backward(x, dy), 3 * n),
        "colsum": (lambda: be.colsum(dy), n),
        "layernorm": (lambda: be.layernorm(x, gamma, beta), 2 * n),
        "layernorm_backward": (lambda: be.layernorm_backward(x, gamma, dy)[0], 3 * n),
        "layernorm_backward_residual": (lambda: be.layernorm_backward(x, gamma, dy, dx_residual=beta_rows, want_dx_colsum=True)[0], 4 * n),
        "softmax": (lambda: be.softmax(x), 2 * n),
        "softmax_backward": (lambda: be.softmax_backward(x, dy), 3 * n),
    }
    if args.op not in calls:
        raise SystemExit("unknown --op %r (one of %s)" % (args.op, ", ".join(sorted(calls))))
    fn, byts = calls[args.op]
    keep = [fn() for _ in range(2)]          # warm-up; fills torch's allocator cache
    del keep
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.calls):
        out = fn()
    e1.record()
    torch.cuda.synchronize()
    be.check_device_status()
    ms = e0.elapsed_time(e1) / args.calls
    print("%s [%d, %d]: %.3f ms/call, %.1f GB/s of %.1f MB algorithmic, checksum %.6e" %
          (args.op, args.rows, args.cols, ms, byts / ms / 1e6, byts / 1e6, float(out.reshape(-1)[::97].double().sum())))


if __name__ == "__main__":
    main()
