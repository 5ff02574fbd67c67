"""Multi-GPU form of the matmul path: one process per GPU, no collective inside the data path.

A large product C = A.B is split by N column blocks (each rank holds all of A and its own columns of B and
produces its own columns of C); batched products and attention are split by the outermost batch index.  The
shards are independent, so ranks never exchange data while computing.  Only when the caller wants the
whole result on every rank is one all-gather issued (NCCL over NVLink on GPUs, gloo in the CPU tests).
The reference has no multi-device code at all (its README lists distributed training as planned), so this
layer has no counterpart there; it wraps whatever matmul callable it is given.
"""
import ctypes as C

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


class Communicator:
    """The library's own NCCL communicator for one rank (csrc/dist.cu): the all-gathers of the data plane and the
    sharded host-buffer GEMM run through the C ABI, not through torch.  torch.distributed is used once, to hand rank 0's
    communicator id to the other ranks."""

    def __init__(self, backend, world, rank, group=None):
        self.be, self.world, self.rank = backend, world, rank
        self._lib = backend._lib
        ident = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            buf = (C.c_ubyte * 128)()
            L.check(self._lib.te_b200_comm_unique_id(buf))
            ident = torch.tensor(list(buf), dtype=torch.uint8)
        if world > 1:
            ident = ident.to(backend.torch_device) if dist.get_backend(group) == "nccl" else ident
            dist.broadcast(ident, src=0, group=group)
        raw = (C.c_ubyte * 128)(*ident.cpu().tolist())
        h = C.c_void_p()
        L.check(self._lib.te_b200_comm_init(backend._ctx, raw, world, rank, C.byref(h)))
        self._comm = h

    def close(self):
        if getattr(self, "_comm", None):
            self._lib.te_b200_comm_destroy(self._comm)
            self._comm = None

    def all_gather_columns(self, c_local, n_total, align=COLUMN_ALIGN, out=None, staging=None):
        """[M, N] on every rank from the ranks' dense [M, n_r] column blocks: one NCCL all-gather + one re-tile kernel."""
        M = c_local.shape[0]
        c_local = c_local.contiguous()
        out = out if out is not None else torch.empty(M, n_total, dtype=torch.float32, device=c_local.device)
        staging = staging if staging is not None else torch.empty(M * n_total, dtype=torch.float32, device=c_local.device)
        L.check(self._lib.te_b200_all_gather_columns(self._comm, C.c_void_p(c_local.data_ptr()), M, n_total, align,
                                                     C.c_void_p(staging.data_ptr()), C.c_void_p(out.data_ptr()), out.stride(0),
                                                     self.be._stream()))
        return out

    def all_reduce_batch_mean_(self, grads, local_rows):
        """te_b200_all_reduce_batch_mean: the data-parallel step's gradient exchange through the library's own
        communicator (the counterpart of all_reduce_batch_mean_ above, which goes through torch.distributed); in place."""
        assert grads.is_contiguous() and grads.dtype == torch.float32
        L.check(self._lib.te_b200_all_reduce_batch_mean(self._comm, C.c_void_p(grads.data_ptr()), grads.numel(), int(local_rows),
                                                        self.be._stream()))
        return grads

    def all_gather_rows(self, full, align=1):
        """In place: every rank filled its own row block of the dense [rows, cols] tensor `full`."""
        rows = full.shape[0]
        cols = full.numel() // rows if rows else 0
        L.check(self._lib.te_b200_all_gather_rows(self._comm, C.c_void_p(full.data_ptr()), rows, cols, align, self.be._stream()))
        return full

    def gemm_host_sharded(self, desc, align=COLUMN_ALIGN):
        """te_b200_gemm_f32_host_sharded on a descriptor holding HOST pointers; collective."""
        L.check(self._lib.te_b200_gemm_f32_host_sharded(self._comm, C.byref(desc), align))
