"""Shape sweep of the matmul path, the counterpart of src/benchmarks/matmul_benchmark.cpp of the reference.

Writes a JSON list with the reference's fields (kernel_name, dtype, M, K, N, time_ms, tflops, bandwidth_gb_s,
pct_of_cublas, gpu_name; src/benchmarks/matmul_benchmark.cpp:342-362) plus mode, pct_of_tensor_peak,
pct_of_hbm_peak, gpus, cpu_time_ms, cpu_cores.  Timing follows :53-94 there: CUDA events around `iters` launches
after max(3, iters/5) warm-up launches, iters by problem size (raised to >= 20 for the large shapes), best and
median of 7 trials.  FLOPs = 2*M*K*N, bytes = 4*(M*K + K*N + M*N) (:73-82).  Inputs: seed 42, uniform(-1, 1).

    python torch-engine_b200/benchmarks/matmul_benchmark.py [out.json] [--cpu] [--quick]

Cases: the square sweep 1024..16384 and the skinny shapes of the GEMM sweep configuration, the attention pair of
batched products (B=16, H=12, T=256, d=64) with the softmax between them and its backward, and the MLP Linear forward (+GELU) and
backward (X [4096,768], W [3072,768]).  `pct_of_cublas` compares with torch.matmul in TF32 mode (a cuBLAS call) as a
comparator only.  With --cpu the reference's own CPU Tensor::matmul (single-threaded) is timed beside the small
shapes and extrapolated, labelled as such, for the large ones.
"""
import argparse
import json
import os
import statistics
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import ctypes as C  # noqa: E402

from torch_engine_b200 import lib as L, ops  # noqa: E402


def plan(M, K, N, mode, sm_count=148, scratch=4 << 30):
    """(tile width, CTA pair?, K splits) the backend's cost model picks for a dense row-major product."""
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a = d.b = d.c = 0x1000
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.alpha = 1.0
    d.precision = L.TE_PREC_3XTF32 if mode == "3xtf32" else L.TE_PREC_TF32
    bn, pair, sp = C.c_int(), C.c_int(), C.c_int()
    if L.load().te_b200_gemm_plan(C.byref(d), sm_count, scratch, C.byref(bn), C.byref(pair), C.byref(sp)) != L.TE_OK:
        return None
    return {"tile_n": bn.value, "cta_pair": bool(pair.value), "k_splits": sp.value}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["bf16_tflops"] / 2.0, p["hbm_gbs"], "measured"
    return 1590.0 / 2.0, 6650.0, "fallback"


def iters_for(flops):
    if flops < 2 * 512 ** 3:
        return 100
    if flops < 2 * 2048 ** 3:
        return 50
    return 20


def time_gpu(fn, iters, trials=7):
    """(best, median) ms per call.  The `iters` launches are captured into one CUDA graph and replayed, so that the
    figure is device time and not the Python/ctypes cost of issuing a call (which exceeds the run time of the small
    shapes); torch's caching allocator serves the outputs inside the capture."""
    for _ in range(max(3, iters // 5)):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    out = []
    for _ in range(trials):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / iters)
    del graph
    return min(out), statistics.median(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("out", nargs="?", default="matmul_benchmark.json", help="output JSON (default: in the current directory)")
    ap.add_argument("--cpu", action="store_true", help="time the reference CPU matmul beside the GPU numbers")
    ap.add_argument("--quick", action="store_true", help="skip 16384^3")
    args = ap.parse_args()

    be = ops.Backend(0, workspace_bytes=6 << 30)
    tf32_peak, hbm_peak, peak_src = peaks()
    gpu_name = torch.cuda.get_device_name(0)
    torch.backends.cuda.matmul.allow_tf32 = True
    gen = torch.Generator(device="cuda").manual_seed(42)
    rnd = lambda *s: torch.rand(*s, device="cuda", generator=gen) * 2 - 1
    results = []

    cpu_rate = None
    if args.cpu:
        from oracle import binding
        ref = binding.Reference() if binding.Reference.available() else None
        rng = binding.SeededRng(42)
        a, b = rng.uniform((1024, 1024)), rng.uniform((1024, 1024))
        t0 = time.perf_counter()
        if ref:
            ref.matmul(a, binding.ref_view(a.shape), b, binding.ref_view(b.shape), out_shape=(1024, 1024))
        else:
            binding.Oracle().matmul(a, b)
        cpu_rate = 2.0 * 1024 ** 3 / (time.perf_counter() - t0)      # FLOP/s of one host core

    def record(name, mode, M, K, N, batch, t_best, t_med, cublas_ms=None, extra_bytes=0):
        flops = 2.0 * M * K * N * batch
        byts = 4.0 * (M * K + K * N + M * N) * batch + extra_bytes
        r = {"kernel_name": name, "dtype": "float32", "mode": mode, "M": M, "K": K, "N": N, "batch": batch,
             "time_ms": t_med, "time_ms_best": t_best, "tflops": flops / t_med / 1e9,
             "bandwidth_gb_s": byts / t_med / 1e6,
             "pct_of_cublas": (100.0 * cublas_ms / t_med) if cublas_ms else None,
             "pct_of_tensor_peak": 100.0 * flops / t_med / 1e9 / tf32_peak,
             "pct_of_hbm_peak": 100.0 * byts / t_med / 1e6 / hbm_peak, "peak_source": peak_src,
             "gpus": 1, "gpu_name": gpu_name}
        if cpu_rate:
            r["cpu_time_ms"] = flops / cpu_rate * 1e3
            r["cpu_cores"] = 1
            r["cpu_time_note"] = "extrapolated from the reference CPU matmul at 1024^3 (one core)"
        results.append(r)
        print("%-28s %-7s %6dx%6dx%6d b=%-4d %9.3f ms %8.1f TFLOP/s %8.1f GB/s %s" %
              (name, mode, M, K, N, batch, t_med, r["tflops"], r["bandwidth_gb_s"],
               ("%.0f%% of cuBLAS-TF32" % r["pct_of_cublas"]) if cublas_ms else ""), flush=True)

    # ---- GEMM sweep: squares and skinny shapes, given as (M, K, N) like the reference ----
    shapes = [(512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
              (8192, 512, 8192), (8192, 8192, 512), (16, 8192, 8192)]
    if not args.quick:
        shapes.append((16384, 16384, 16384))
    for (M, K, N) in shapes:
        a, b = rnd(M, K), rnd(K, N)
        it = iters_for(2.0 * M * K * N)
        it = max(it, 20) if M * K * N >= 4096 ** 3 else it
        if M >= 16384:
            it = 5
        _, cub = time_gpu(lambda: torch.matmul(a, b), it, trials=3)
        for mode in ("tf32", "3xtf32"):
            tb, tm = time_gpu(lambda: be.matmul(a, b, precision=mode), it)
            record("b200_tcgen05_gemm", mode, M, K, N, 1, tb, tm, cub)
            results[-1]["kernel_form"] = plan(M, K, N, mode)
        del a, b
        torch.cuda.empty_cache()

    # ---- attention: S = Q.K^T / 8, softmax, O = P.V  over [16, 12, 256, 64] ----
    q, k, v = (torch.randn(16, 12, 256, 64, device="cuda", generator=gen) for _ in range(3))
    for mode in ("tf32", "3xtf32"):
        tb, tm = time_gpu(lambda: be.scaled_dot(q, k, v, precision=mode), 50)
        # algorithmic traffic: fused kernel (TF32 mode) reads Q, K, V once and writes P and O once = 100.7 MB;
        # the unfused form (3xTF32 mode) also writes S and passes it through the softmax = 251.7 MB
        record("b200_attention_qk_softmax_pv", mode, 256, 64, 256, 192 * 2, tb, tm, None)
        byts = 100.7e6 if mode == "tf32" else 251.7e6
        results[-1]["bandwidth_gb_s"] = byts / (tm * 1e-3) / 1e9
        results[-1]["pct_of_hbm_peak"] = 100.0 * (byts / (tm * 1e-3) / 1e9) / hbm_peak
        results[-1]["note"] = ("one fused kernel, S stays in tensor memory; bytes = 100.7 MB" if mode == "tf32" else
                               "two batched GEMMs + row softmax; bytes = 251.7 MB (unfused)")

    # ---- attention backward: dQ, dK, dV from dO, P, O over the same [16, 12, 256, 64] operands ----
    d_o = torch.randn(16, 12, 256, 64, device="cuda", generator=gen)
    o_f, p_f = be.scaled_dot(q, k, v, precision="tf32")
    for mode, o_arg in (("tf32", o_f), ("3xtf32", None)):
        tb, tm = time_gpu(lambda: be.scaled_dot_backward(q, k, v, p_f, d_o, o=o_arg, precision=mode), 50)
        # four products of 2*T*T*d FLOP per head (dV, dP, dQ, dK; S is not recomputed, P is read back)
        record("b200_attention_backward", mode, 256, 64, 256, 192 * 4, tb, tm, None)
        # algorithmic traffic, fused: P, Q, K, V, O, dO read once, dQ, dK, dV written once = 151.0 MB;
        # unfused: P read twice, dP written, read and rewritten as dS, dS read twice (6 x 50.3 MB) + the [B,H,T,d] operands
        byts = 151.0e6 if mode == "tf32" else 6 * 50.3e6 + 9 * 12.6e6
        results[-1]["bandwidth_gb_s"] = byts / (tm * 1e-3) / 1e9
        results[-1]["pct_of_hbm_peak"] = 100.0 * (byts / (tm * 1e-3) / 1e9) / hbm_peak
        results[-1]["note"] = ("row-dot pre-pass + one fused kernel, dP and dS stay in tensor memory; bytes = 151.0 MB"
                               if mode == "tf32" else "four batched GEMMs + softmax-backward kernel (unfused)")

    # ---- MLP Linear: X [4096,768], W [3072,768] ----
    x, w, dy = torch.randn(4096, 768, device="cuda", generator=gen), torch.randn(3072, 768, device="cuda", generator=gen) * 0.02, \
        torch.randn(4096, 3072, device="cuda", generator=gen)
    bias = torch.zeros(3072, device="cuda")
    _, cub = time_gpu(lambda: torch.nn.functional.linear(x, w, bias), 50, trials=3)
    for mode in ("tf32", "3xtf32"):
        tb, tm = time_gpu(lambda: be.linear_forward(x, w, bias, gelu=True, precision=mode), 50)
        record("b200_linear_bias_gelu_fwd", mode, 4096, 768, 3072, 1, tb, tm, cub)
        tb, tm = time_gpu(lambda: be.linear_backward(x, w, dy, precision=mode), 50)
        record("b200_linear_bwd_dx_dw_db", mode, 4096, 3072, 768, 2, tb, tm, None)
    # ---- the Linear shapes of the GPT configuration (16 384 tokens, d_model 384, ffDim 1536), TF32 mode ----
    for (rows, inf, outf, gelu) in [(16384, 384, 384, False), (16384, 384, 1536, True), (16384, 1536, 384, False)]:
        xg, wg = torch.randn(rows, inf, device="cuda", generator=gen), torch.randn(outf, inf, device="cuda", generator=gen) * 0.02
        bg, dyg = torch.zeros(outf, device="cuda"), torch.randn(rows, outf, device="cuda", generator=gen)
        _, cub = time_gpu(lambda: torch.nn.functional.linear(xg, wg, bg), 50, trials=3)
        tb, tm = time_gpu(lambda: be.linear_forward(xg, wg, bg, gelu=gelu, precision="tf32"), 50)
        record("b200_linear_bias%s_fwd" % ("_gelu" if gelu else ""), "tf32", rows, inf, outf, 1, tb, tm, cub)
        tb, tm = time_gpu(lambda: be.linear_backward(xg, wg, dyg, precision="tf32"), 50)
        record("b200_linear_bwd_dx_dw_db", "tf32", rows, outf, inf, 2, tb, tm, None)
        del xg, wg, bg, dyg
    # ---- Linear on a thin batch (16 and 8 rows through an 8192 -> 8192 layer): bound by reading the weight once ----
    wt, bt = torch.randn(8192, 8192, device="cuda", generator=gen) * 0.02, torch.zeros(8192, device="cuda")
    for rows in (16, 8):
        xt = torch.randn(rows, 8192, device="cuda", generator=gen)
        _, cub = time_gpu(lambda: torch.nn.functional.linear(xt, wt, bt), 30, trials=3)
        for mode in ("tf32", "3xtf32"):
            tb, tm = time_gpu(lambda: be.linear_forward(xt, wt, bt, precision=mode), 30)
            record("b200_linear_bias_fwd_thin", mode, rows, 8192, 8192, 1, tb, tm, cub)
    del wt, bt
    torch.cuda.empty_cache()
    # ---- HBM-bound helpers around the GEMMs: softmax rows, GELU, bias-gradient column sum, 3xTF32 packing ----
    def record_stream(name, byts, tb, tm, shape):
        r = {"kernel_name": name, "dtype": "float32", "mode": "-", "shape": shape, "time_ms": tm, "time_ms_best": tb,
             "bandwidth_gb_s": byts / (tm * 1e-3) / 1e9, "pct_of_hbm_peak": 100.0 * byts / (tm * 1e-3) / 1e9 / hbm_peak,
             "peak_source": peak_src, "gpus": 1, "gpu_name": gpu_name}
        results.append(r)
        print("%-28s %-24s %9.3f ms %8.1f GB/s  %5.1f%% of HBM peak" % (name, shape, tm, r["bandwidth_gb_s"], r["pct_of_hbm_peak"]), flush=True)

    s_in = torch.randn(32 * 12 * 256, 256, device="cuda", generator=gen)          # 100.7 MB, larger than... read + write
    tb, tm = time_gpu(lambda: be.softmax(s_in), 20)
    record_stream("b200_softmax_rows", 2 * 4.0 * s_in.numel(), tb, tm, "98304x256")
    dy_s = torch.randn_like(s_in)
    p_s = be.softmax(s_in)
    tb, tm = time_gpu(lambda: be.softmax_backward(p_s, dy_s), 20)
    record_stream("b200_softmax_backward_rows", 3 * 4.0 * s_in.numel(), tb, tm, "98304x256")
    act = torch.randn(16384, 3072, device="cuda", generator=gen)                   # 201 MB
    tb, tm = time_gpu(lambda: be.gelu(act), 20)
    record_stream("b200_gelu", 2 * 4.0 * act.numel(), tb, tm, "16384x3072")
    dact = torch.randn_like(act)
    tb, tm = time_gpu(lambda: be.gelu_backward(act, dact), 20)
    record_stream("b200_gelu_backward", 3 * 4.0 * act.numel(), tb, tm, "16384x3072")
    tb, tm = time_gpu(lambda: be.colsum(act), 20)
    record_stream("b200_colsum", 4.0 * act.numel(), tb, tm, "16384x3072")
    # ---- the GPT step's kernels around the matmuls, at the GPT configuration's sizes scaled past L2 where it matters ----
    xn = torch.randn(65536, 384, device="cuda", generator=gen)                      # 100.7 MB
    gam, bet = torch.ones(384, device="cuda"), torch.zeros(384, device="cuda")
    tb, tm = time_gpu(lambda: be.layernorm(xn, gam, bet), 20)
    record_stream("b200_layernorm", 2 * 4.0 * xn.numel(), tb, tm, "65536x384")
    dyn = torch.randn_like(xn)
    tb, tm = time_gpu(lambda: be.layernorm_backward(xn, gam, dyn), 20)
    record_stream("b200_layernorm_backward", 3 * 4.0 * xn.numel(), tb, tm, "65536x384")
    res_n = torch.randn_like(xn)
    tb, tm = time_gpu(lambda: be.layernorm_backward(xn, gam, dyn, dx_residual=res_n, want_dx_colsum=True), 20)
    record_stream("b200_layernorm_backward_residual_colsum", 4 * 4.0 * xn.numel(), tb, tm, "65536x384")
    del res_n
    lg = torch.randn(16384, 65, device="cuda", generator=gen)
    tg = torch.randint(0, 65, (16384,), device="cuda", generator=gen)
    tb, tm = time_gpu(lambda: be.cross_entropy(lg, tg), 50)
    record_stream("b200_cross_entropy_fwd_bwd", 2 * 4.0 * lg.numel() + 8.0 * tg.numel(), tb, tm, "16384x65")
    table = torch.randn(65, 384, device="cuda", generator=gen)
    tok = torch.randint(0, 65, (64, 256), device="cuda", generator=gen)
    pe = torch.randn(256, 384, device="cuda", generator=gen)
    tb, tm = time_gpu(lambda: be.embedding(table, tok, pe), 50)
    record_stream("b200_embedding_plus_pos", 4.0 * 16384 * 384 + 8.0 * 16384, tb, tm, "16384 tokens x 384")
    d_emb = torch.randn(64, 256, 384, device="cuda", generator=gen)
    tb, tm = time_gpu(lambda: be.embedding_backward(tok, d_emb, 65), 50)
    record_stream("b200_embedding_backward", 4.0 * 16384 * 384 + 8.0 * 16384, tb, tm, "16384 tokens x 384, vocab 65")
    be.check_device_status()
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out, "w") as f:
        json.dump(results, f, indent=1)
    print("wrote %d results to %s" % (len(results), args.out))


if __name__ == "__main__":
    main()
