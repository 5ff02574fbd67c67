"""GPT training-step timing with every matmul on this backend: the counterpart of
src/benchmarks/gpt_benchmark_gpu.cpp of the reference (same JSON sections: model_config, training_config with
gemm_backend, metrics with tokens_per_sec / time_per_step_ms / final_loss).  Forward + loss + backward per step on
synthetic token ids (uniform in [0, vocab)); the optimizer update is not part of the matmul path and is left out,
which the output states.  Environment variables as in the reference (:110-123): TENSOR_EMBED_DIM, TENSOR_NUM_HEADS,
TENSOR_NUM_LAYERS, TENSOR_FF_DIM, TENSOR_BATCH_SIZE, TENSOR_SEQ_LEN, TENSOR_MEASURED_STEPS, TENSOR_WARMUP_STEPS,
plus TENSOR_GEMM_PRECISION (tf32 | 3xtf32) and TENSOR_CUDA_GRAPH=1, which captures one whole step (forward, loss,
backward: ~300 kernels of this backend and ~150 small torch kernels) into a CUDA graph and replays it, so that the
host's per-launch cost drops out of the step time (single GPU only).  Defaults are benchmark configuration 4.

    python torch-engine_b200/benchmarks/gpt_benchmark.py [out.json]

Under torchrun (one process per GPU) the step runs data-parallel: every rank takes TENSOR_BATCH_SIZE sequences of its
own (weak scaling), the ranks exchange one all-reduce of the flat gradient per step (NCCL), time is the maximum over
ranks and tokens/s the whole job's; rank 0 writes the result.
"""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import torch.distributed as dist  # noqa: E402

from torch_engine_b200 import gpt, ops, sharding  # noqa: E402


def env_int(name, default):
    return int(os.environ.get(name, default))


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else "gpt_benchmark_b200.json"   # beside the caller, like the reference's benchmark
    E, H, L = env_int("TENSOR_EMBED_DIM", 384), env_int("TENSOR_NUM_HEADS", 6), env_int("TENSOR_NUM_LAYERS", 6)
    ff = env_int("TENSOR_FF_DIM", 4 * E)
    B, T = env_int("TENSOR_BATCH_SIZE", 64), env_int("TENSOR_SEQ_LEN", 256)
    steps, warm = env_int("TENSOR_MEASURED_STEPS", 10), env_int("TENSOR_WARMUP_STEPS", 3)
    vocab = 65
    prec = os.environ.get("TENSOR_GEMM_PRECISION", "tf32")
    world, rank, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = ops.Backend(local, workspace_bytes=2 << 30)
    # the step's one exchange goes through the library's own communicator (csrc/dist.cu, te_b200_all_reduce_batch_mean)
    comm = sharding.Communicator(be, world, rank) if world > 1 else None
    sync = (lambda grads, rows: comm.all_reduce_batch_mean_(grads, rows)) if world > 1 else None
    g = torch.Generator(device="cuda").manual_seed(42)
    n_params = vocab * E + L * (4 * E + 4 * (E * E + E) + 2 * E * ff + ff + E) + 2 * E + vocab * E + vocab
    flat = torch.randn(n_params, device="cuda", generator=g) * 0.02
    g.manual_seed(1000 + rank)            # same parameters on every rank, different token batches
    tokens = torch.randint(0, vocab, (B, T), device="cuda", generator=g)
    targets = torch.randint(0, vocab, (B, T), device="cuda", generator=g)
    use_graph = os.environ.get("TENSOR_CUDA_GRAPH", "0") == "1" and world == 1
    loss = None
    for _ in range(warm):
        loss, _, _ = gpt.gpt_step(be, flat, tokens, targets, vocab, E, H, L, ff, prec, grad_sync=sync)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    n0 = be.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            gpt.gpt_step(be, flat, tokens, targets, vocab, E, H, L, ff, prec)        # allocator warm-up on this stream
            with torch.cuda.graph(graph, stream=side):
                loss, _, grads = gpt.gpt_step(be, flat, tokens, targets, vocab, E, H, L, ff, prec)
        torch.cuda.synchronize()
        launches_per_step = be.launches - n0 - (be.launches - n0) // 2                 # the captured pass only
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(steps):
            loss, _, _ = gpt.gpt_step(be, flat, tokens, targets, vocab, E, H, L, ff, prec, grad_sync=sync)
        e1.record()
        launches_per_step = None
    torch.cuda.synchronize()
    be.check_device_status()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
        dist.destroy_process_group()
        if rank != 0:
            return
    B = B * world
    result = {
        "framework": "TENSOR", "device": "CUDA",
        "hardware": {"gpu": torch.cuda.get_device_name(0)},
        "model_config": {"vocab_size": vocab, "max_seq_len": T, "embed_dim": E, "num_heads": H, "num_layers": L, "ff_dim": ff},
        "training_config": {"batch_size": B, "seq_len": T, "measured_steps": steps, "dropout": 0.0,
                            "gemm_backend": "b200", "gemm_precision": prec, "gpus": world,
                            "parallelism": "data-parallel, one gradient all-reduce per step" if world > 1 else "single GPU",
                            "step": "forward + loss + backward (no optimizer update)"},
        "metrics": {"timing_mode": "throughput", "total_time_s": ms * steps / 1e3, "total_tokens": B * T * steps,
                    "tokens_per_sec": B * T / (ms / 1e3), "steps_per_sec": 1e3 / ms, "time_per_step_ms": ms,
                    "final_loss": float(loss), "backend_kernel_launches_per_step": launches_per_step if launches_per_step is not None else (be.launches - n0) / steps,
                    "cuda_graph": bool(use_graph)},
    }
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    with open(out_path, "w") as f:
        json.dump(result, f, indent=1)
    print(json.dumps(result["metrics"]))


if __name__ == "__main__":
    main()
