"""The multi-rank path on CPU: two gloo ranks shard a product by N columns and attention by batch index,
compute their shards (the oracle stands in for the GPU kernel), all-gather, and must reproduce the
single-rank result bit for bit.  Also covers ragged splits and a rank that owns nothing."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle.binding import Oracle
    from torch_engine_b200 import sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        o = Oracle()
        mm = lambda a, b: torch.from_numpy(o.matmul(a.numpy(), b.numpy()))
        sd = lambda q, k, v: torch.from_numpy(o.scaled_dot(q.numpy(), k.numpy(), v.numpy())[0])
        g = torch.Generator().manual_seed(11)
        results = {}
        for (M, K, N, align) in [(48, 40, 96, 16), (33, 20, 50, 16), (8, 8, 8, 16)]:
            a = torch.rand(M, K, generator=g) * 2 - 1
            b = torch.rand(K, N, generator=g) * 2 - 1
            c_loc, (n0, cnt) = sharding.matmul_column_shard(mm, a, b, world, rank, align)
            assert c_loc.shape == (M, cnt)
            full = sharding.all_gather_columns(c_loc, N, world, rank, align)
            assert torch.equal(full, mm(a, b)), (M, K, N)
            results[f"mm_{M}_{K}_{N}"] = (n0, cnt)
        for B in (4, 3, 1):
            q, k, v = (torch.randn(B, 2, 8, 4, generator=g) for _ in range(3))
            o_loc, (b0, cnt) = sharding.attention_batch_shard(sd, q, k, v, world, rank)
            full = sharding.all_gather_batches(o_loc, B, world, rank)
            assert torch.equal(full, sd(q, k, v)), B
            results[f"attn_{B}"] = (b0, cnt)
        # data-parallel gradient averaging with unequal batch slices: rank r holds r + 1 rows whose per-row
        # gradients are known, so the batch mean is known too
        rows = rank + 1
        per_row = [torch.full((5,), float(10 * r + i)) for r in range(world) for i in range(r + 1)]
        mine = torch.stack([torch.full((5,), float(10 * rank + i)) for i in range(rows)]).mean(0)
        total = sharding.all_reduce_batch_mean_(mine, rows)
        assert total == sum(r + 1 for r in range(world))
        assert torch.allclose(mine, torch.stack(per_row).mean(0))
        torch.save(results, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_and_batch_sharding(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r0 = torch.load(os.path.join(tmp_path, "rank0.pt"))
    r1 = torch.load(os.path.join(tmp_path, "rank1.pt"))
    assert r0["mm_48_40_96"] == (0, 48) and r1["mm_48_40_96"] == (48, 48)
    assert r0["mm_33_20_50"] == (0, 32) and r1["mm_33_20_50"] == (32, 18)     # ragged tail on the last rank
    assert r0["mm_8_8_8"] == (0, 8) and r1["mm_8_8_8"] == (8, 0)              # a rank with no columns
    assert r0["attn_3"] == (0, 2) and r1["attn_3"] == (2, 1)
    assert r1["attn_1"] == (1, 0)
