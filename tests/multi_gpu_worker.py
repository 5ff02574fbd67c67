"""One rank of the multi-GPU checks (launched by tests/test_multi_gpu.py through torch.distributed.run, one process
per GPU).  Everything that crosses GPUs goes through the library's NCCL driver (te_b200_all_gather_*,
te_b200_gemm_f32_host_sharded); no kernel reads a peer's memory.  Prints "rank R ok" on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from torch_engine_b200 import lib as L  # noqa: E402
from torch_engine_b200 import ops, sharding  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    be = ops.Backend(local, workspace_bytes=1 << 30)
    comm = sharding.Communicator(be, world, rank)
    g = torch.Generator(device="cuda").manual_seed(5)          # the same operands on every rank

    # ---- a large product split by N column blocks, C reassembled on every rank (ragged: 1000 columns, align 256)
    for (M, K, N, align) in [(512, 384, 1024, 256), (300, 200, 1000, 256), (64, 96, 130, 1)]:
        a = torch.rand(M, K, device="cuda", generator=g) * 2 - 1
        b = torch.rand(K, N, device="cuda", generator=g) * 2 - 1
        whole = be.matmul(a, b, precision="3xtf32")
        n0, cnt = sharding.column_shard(N, world, rank, align)
        mine = be.matmul(a, b[:, n0:n0 + cnt], precision="3xtf32") if cnt else a.new_empty(M, 0)
        if cnt:
            assert torch.equal(mine, whole[:, n0:n0 + cnt]), "a column shard differs from the slice of the whole product"
        full = comm.all_gather_columns(mine, N, align=align)
        torch.cuda.synchronize()
        assert torch.equal(full, whole), ("all_gather_columns", M, K, N)

    # ---- row blocks gathered in place (how A is replicated after a sharded upload)
    rows, cols = 1000, 96
    src = torch.rand(rows, cols, device="cuda", generator=g)
    r0, rc = sharding.batch_shard(rows, world, rank)
    part = torch.zeros_like(src)
    part[r0:r0 + rc] = src[r0:r0 + rc]
    comm.all_gather_rows(part)
    torch.cuda.synchronize()
    assert torch.equal(part, src), "all_gather_rows"

    # ---- the host-buffer product for `world` ranks: each uploads its share, A replicated over NVLink
    M, K, N = 1024, 512, 1024
    gen = torch.Generator().manual_seed(11)
    ha = (torch.rand(M, K, generator=gen) * 2 - 1).pin_memory()
    hb = (torch.rand(K, N, generator=gen) * 2 - 1).pin_memory()
    hc = torch.zeros(M, N).pin_memory()
    d = L.GemmDesc()
    d.M, d.N, d.K = M, N, K
    d.a, d.b, d.c = ha.data_ptr(), hb.data_ptr(), hc.data_ptr()
    d.lda, d.ldb, d.ldc = K, N, N
    d.batch_outer = d.batch_inner = 1
    d.alpha, d.precision = 1.0, L.TE_PREC_3XTF32
    for _ in range(2):
        hc.zero_()
        comm.gemm_host_sharded(d)
        n0, cnt = sharding.column_shard(N, world, rank)
        ref = ha.double() @ hb.double()
        err = float((hc[:, n0:n0 + cnt].double() - ref[:, n0:n0 + cnt]).abs().max() / ref.abs().max())
        assert err <= 1e-5, ("gemm_host_sharded", err)
        if world > 1:
            other = torch.ones(N, dtype=torch.bool)
            other[n0:n0 + cnt] = False
            assert float(hc[:, other].abs().max()) == 0.0, "a rank wrote columns it does not own"

    # ---- attention sharded by batch index (configuration 2's shapes, smaller batch), outputs gathered
    B, H, T, dh = 2 * world + 1, 3, 128, 64
    q, k, v = (torch.randn(B, H, T, dh, device="cuda", generator=g) for _ in range(3))
    o_whole, _ = be.scaled_dot(q, k, v, precision="tf32")
    # (2 * world + 1 batches: with four ranks the last one owns nothing, and still takes part in the gather)
    o_mine, (b0, bc) = sharding.attention_batch_shard(lambda *t: be.scaled_dot(*t, precision="tf32")[0], q, k, v, world, rank)
    assert torch.equal(o_mine, o_whole[b0:b0 + bc]), "a batch shard differs from the slice of the whole call"
    gathered = o_whole.new_zeros(B, H * T * dh)
    if bc:
        gathered[b0:b0 + bc] = o_mine.reshape(bc, -1)
    comm.all_gather_rows(gathered)
    torch.cuda.synchronize()
    assert torch.equal(gathered.view(B, H, T, dh), o_whole), "batch-sharded attention after the gather"

    # ---- the data-parallel step's gradient exchange: row-weighted average over ranks with unequal (one empty) slices
    n = 100003
    rows_of = [37 * (r + 1) if r != world - 1 or world == 1 else 0 for r in range(world)]      # the last rank averaged over nothing
    gs = [torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 + r)) for r in range(world)]
    want = sum(g_.double() * rows_of[r] for r, g_ in enumerate(gs)) / float(sum(rows_of))
    mine = gs[rank].clone()
    comm.all_reduce_batch_mean_(mine, rows_of[rank])
    via_torch = gs[rank].clone()
    sharding.all_reduce_batch_mean_(via_torch, rows_of[rank])
    torch.cuda.synchronize()
    assert float((mine.double() - want).abs().max()) <= 1e-6 * float(want.abs().max()) + 1e-7, "native gradient all-reduce"
    assert float((mine - via_torch).abs().max()) <= 2e-6 * float(want.abs().max()), "native and torch.distributed exchanges differ"

    be.check_device_status()
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    be.close()
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
