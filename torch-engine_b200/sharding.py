"""Multi-GPU form of the matmul path: one process per GPU, no collective inside the data path.

A large product C = A.B is split by N column blocks (each rank holds all of A and its own columns of B and
produces its own columns of C); batched products and attention are split by the outermost batch index.  The
shards are independent, so ranks never exchange data while computing.  Only when the caller wants the
whole result on every rank is one all-gather issued (NCCL over NVLink on GPUs, gloo in the CPU tests).
The reference has no multi-device code at all (its README lists distributed training as planned), so this
layer has no counterpart there; it wraps whatever matmul callable it is given.
"""
import torch
import torch.distributed as dist

from . import lib as L

COLUMN_ALIGN = 256   # one GEMM tile width: shards start on tile boundaries


def column_shard(n_total, world, rank, align=COLUMN_ALIGN):
    """(first column, column count) owned by `rank`."""
    return L.shard_range(n_total, world, rank, align)


def batch_shard(b_total, world, rank):
    """(first batch index, batch count) owned by `rank`."""
    return L.shard_range(b_total, world, rank, 1)


def matmul_column_shard(matmul, a, b, world, rank, align=COLUMN_ALIGN):
    """This rank's column block of a @ b.  `b[..., n0:n0+cnt]` is a strided view (row pitch N), read in place."""
    n0, cnt = column_shard(b.shape[-1], world, rank, align)
    if cnt == 0:
        return a.new_empty(a.shape[:-1] + (0,)), (n0, cnt)
    return matmul(a, b[..., n0:n0 + cnt]), (n0, cnt)


def attention_batch_shard(scaled_dot, q, k, v, world, rank):
    """This rank's batch slice of scaled-dot attention over [B,H,T,d] operands."""
    b0, cnt = batch_shard(q.shape[0], world, rank)
    if cnt == 0:
        return q.new_empty((0,) + tuple(q.shape[1:])), (b0, cnt)
    return scaled_dot(q[b0:b0 + cnt], k[b0:b0 + cnt], v[b0:b0 + cnt]), (b0, cnt)


def _all_gather_padded(local, dim, total, world, rank, shard_fn, group):
    counts = [shard_fn(total, world, r)[1] for r in range(world)]
    width = max(counts)
    shape = list(local.shape)
    shape[dim] = width
    send = local.new_zeros(shape)
    if counts[rank]:
        send.narrow(dim, 0, counts[rank]).copy_(local)
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send.contiguous(), group=group)
    return torch.cat([recv[r].narrow(dim, 0, counts[r]) for r in range(world)], dim=dim)


def all_gather_columns(c_local, n_total, world, rank, align=COLUMN_ALIGN, group=None):
    """Reassembles the full [.., M, N] result on every rank from the column blocks."""
    return _all_gather_padded(c_local, c_local.dim() - 1, n_total, world, rank,
                              lambda t, w, r: column_shard(t, w, r, align), group)


def all_gather_batches(o_local, b_total, world, rank, group=None):
    """Reassembles a batch-sharded result on every rank."""
    return _all_gather_padded(o_local, 0, b_total, world, rank, batch_shard, group)


def all_reduce_batch_mean_(grads, local_rows, group=None):
    """Data-parallel form of the GPT training step: every rank ran the step on its own slice of the batch (a mean loss
    over `local_rows` token rows), and the gradient of the mean loss over the whole batch is the row-weighted average
    of the ranks' gradients.  This is the step's one real exchange: a single all-reduce of the flat gradient (NCCL over
    NVLink on GPUs, gloo in the CPU tests), in place.  Returns the total row count."""
    world = dist.get_world_size(group)
    total = torch.tensor([float(local_rows)], dtype=torch.float64, device=grads.device)
    if world > 1:
        grads.mul_(float(local_rows))
        dist.all_reduce(grads, op=dist.ReduceOp.SUM, group=group)
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
        grads.div_(float(total.item()))
    return int(total.item())
