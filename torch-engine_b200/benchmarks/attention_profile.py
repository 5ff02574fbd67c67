"""Profiling harness for the fused attention kernels: one warm-up call and a few profiled calls of
ScaledDot::forward (or, with --backward, of its backward) on [B, 12, 256, 64] operands, meant to be run under
`ncu -k regex:attention`.

    python torch-engine_b200/benchmarks/attention_profile.py --batch 32 [--backward]
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
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--seq", type=int, default=256)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--calls", type=int, default=3)
    ap.add_argument("--backward", action="store_true", help="profile the fused backward instead of the forward")
    args = ap.parse_args()
    be = ops.Backend(0, workspace_bytes=64 << 20)
    g = torch.Generator(device="cuda").manual_seed(42)
    shape = (args.batch, args.heads, args.seq, args.head_dim)
    q, k, v = (torch.randn(shape, device="cuda", generator=g) for _ in range(3))
    o, p = be.scaled_dot(q, k, v)
    if args.backward:
        d_o = torch.randn(shape, device="cuda", generator=g)
        keep = [be.scaled_dot_backward(q, k, v, p, d_o, o=o) for _ in range(2)]   # fills torch's allocator cache
        del keep
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.calls):
            dq, dk, dv = be.scaled_dot_backward(q, k, v, p, d_o, o=o)
        e1.record()
        torch.cuda.synchronize()
        be.check_device_status()
        ms = e0.elapsed_time(e1) / args.calls
        byts = 4.0 * (8 * q.numel() + p.numel())      # Q, K, V, O, dO read, dQ, dK, dV written, P read
        print("attention backward %s: %.3f ms/call, %.1f GB/s of %.1f MB algorithmic, checksum %.6e" %
              (shape, ms, byts / ms / 1e6, byts / 1e6, float((dq + dk + dv)[::3, ::5, ::7].double().sum())))
        return
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.calls):
        o, p = be.scaled_dot(q, k, v)
    e1.record()
    torch.cuda.synchronize()
    be.check_device_status()
    ms = e0.elapsed_time(e1) / args.calls
    byts = 4.0 * (3 * q.numel() + o.numel() + p.numel())
    print("attention %s: %.3f ms/call, %.1f GB/s of %.1f MB algorithmic, checksum %.6e" %
          (shape, ms, byts / ms / 1e6, byts / 1e6, float(o[::3, ::5, ::7].double().sum())))


if __name__ == "__main__":
    main()
