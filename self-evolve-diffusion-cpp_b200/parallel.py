"""Multi-GPU plumbing of the quantized linear: one process per GPU, torch.distributed.

Two exact partitions exist (see sharding.py).  The row split needs no exchange at
all.  The column split is the one place where the path has a real exchange step:
every rank computes out[:, n0:n1] from its slice of the weight rows and the blocks
are all-gathered so that each rank ends with the full row-major [M, N].  The
collective is NCCL on GPUs (gloo on CPU in the tests); tensors may be CPU or CUDA.
"""
import torch
import torch.distributed as dist

from .sharding import col_shard, row_shard


def max_over_ranks(value, device="cpu", group=None):
    """A timing taken on every rank, reduced to the slowest one."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def local_rows(M, group=None):
    """[begin, end) of the token rows this rank owns under the row split."""
    if not dist.is_initialized():
        return 0, M
    return row_shard(M, dist.get_world_size(group), dist.get_rank(group))


def local_cols(N, group=None):
    """[begin, end) of the output columns (weight rows) this rank owns under the column split."""
    if not dist.is_initialized():
        return 0, N
    return col_shard(N, dist.get_world_size(group), dist.get_rank(group))


def allgather_columns(local_block, N, group=None):
    """local_block: [M, n1-n0] of this rank's columns -> full [M, N] on every rank.

    NCCL/gloo gather equal-sized contiguous chunks, not column blocks, so the blocks are
    padded to the common width, gathered as [world, M, width] and laid out once.
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        assert local_block.shape[1] == N
        return local_block
    world = dist.get_world_size(group)
    M = local_block.shape[0]
    width = col_shard(N, world, 0)[1]
    n0, n1 = col_shard(N, world, dist.get_rank(group))
    assert local_block.shape[1] == n1 - n0
    send = local_block
    if n1 - n0 != width:
        send = local_block.new_zeros((M, width))
        send[:, : n1 - n0] = local_block
    flat = local_block.new_empty((world * M, width))       # rank-major concatenation
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    gathered = flat.view(world, M, width)
    out = local_block.new_empty((M, N))
    for r in range(world):
        b, e = col_shard(N, world, r)
        if e > b:
            out[:, b:e] = gathered[r][:, : e - b]
    return out


def gather_rows(local_rows_block, M, group=None):
    """Row-split outputs stay sharded in production; tests use this to compare with one GPU."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local_rows_block
    world = dist.get_world_size(group)
    N = local_rows_block.shape[1]
    per = row_shard(M, world, 0)[1]
    send = local_rows_block.new_zeros((per, N))
    send[: local_rows_block.shape[0]] = local_rows_block
    flat = local_rows_block.new_empty((world * per, N))
    dist.all_gather_into_tensor(flat, send, group=group)
    gathered = flat.view(world, per, N)
    parts = []
    for r in range(world):
        b, e = row_shard(M, world, r)
        parts.append(gathered[r][: e - b])
    return torch.cat(parts, dim=0)


class SharedOutput:
    """One [M, N] fp32 result buffer per rank, each mapped into every other rank (CUDA IPC),
    for the fused column split: a rank's GEMM epilogue stores its column block into all of
    them, so no separate all-gather runs.  Collective: every rank of `group` constructs it."""

    def __init__(self, sdq, nbytes, group=None):
        self.sdq, self.group = sdq, group
        self.local = sdq.alloc(nbytes)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.opened = []
        if self.world == 1:
            self.ptrs = [self.local.ptr]
            return
        handles = [None] * self.world
        dist.all_gather_object(handles, sdq.ipc_export(self.local.ptr), group=group)
        by_rank = {}
        for r in range(self.world):
            if r == self.rank:
                by_rank[r] = self.local.ptr
            else:
                by_rank[r] = sdq.ipc_open(handles[r])
                self.opened.append(by_rank[r])
        # start with the own buffer, then the peers in ring order, so that at any moment the
        # ranks are not all storing into the same GPU
        self.ptrs = [by_rank[(self.rank + i) % self.world] for i in range(self.world)]

    def close(self):
        if dist.is_initialized() and self.world > 1:
            dist.barrier(group=self.group)      # nobody still stores into a buffer about to go
        for p in self.opened:
            self.sdq.ipc_close(p)
        self.opened = []
        self.local.free()


def qgemm_colsplit_fused(sdq, w_block, A_ptr, M, N_total, shared, bias_ptr=None, flags=0, stream=None):
    """This rank's column block of the linear, stored by the GEMM epilogue into every rank's
    buffer of `shared`.  The result is complete on a rank once all ranks' calls have finished:
    follow with a barrier (or any collective) before reading shared.local."""
    n0, _ = col_shard(N_total, shared.world, shared.rank)
    sdq.qgemm_colsplit(w_block, A_ptr, M, n0, N_total, shared.ptrs, bias_ptr, flags, stream)
