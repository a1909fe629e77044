"""Host side of the sharded matmul: one process per GPU (torchrun), `torch.distributed` only as plumbing
(exchange of CUDA IPC handles, barriers). The data path is the fused GEMM + peer-store kernel of the library
(b200_gemm_allgather / b200_gemm_reduce_scatter_partials); no NCCL collective carries matrix data.

Mirrors the reference's distributed benchmark: A replicated, B sharded on dim 1, local matmul, all-gather of C
(scripts/matmul_2dev_distributed.py:49-76; bench/metal/matmul_tensor_parallel.cpp:70-92), generalised to g ranks,
plus the K-split / reduce-scatter variant of the distributed-matmul configuration."""
from __future__ import annotations

from . import capi
from .capi import BF16, F32


# ---- pure host logic (no GPU): shard geometry -------------------------------------------------------------------------
def column_shard(n_total: int, world: int, rank: int) -> tuple[int, int]:
    """(offset, width) of rank's slice of the N dimension — `shard_tensor_to_mesh_mapper(mesh, 1)`. The fused
    all-gather needs equal shards of a multiple of 8 columns."""
    if n_total % world:
        raise ValueError(f"N = {n_total} is not divisible by {world} ranks")
    width = n_total // world
    if width % 8:
        raise ValueError(f"shard width {width} is not a multiple of 8 columns (16 bytes)")
    return rank * width, width


def k_shard(k_total: int, world: int, rank: int) -> tuple[int, int]:
    """(offset, depth) of rank's slice of the K dimension for the row-parallel product."""
    if k_total % world:
        raise ValueError(f"K = {k_total} is not divisible by {world} ranks")
    depth = k_total // world
    if depth % 8:
        raise ValueError(f"K shard {depth} is not a multiple of 8")
    return rank * depth, depth


def row_block(m_total: int, world: int, rank: int) -> tuple[int, int]:
    """(offset, rows) of the row block a rank owns after the reduce-scatter (multiples of the 128-row tile)."""
    if m_total % world or (m_total // world) % 128:
        raise ValueError(f"M / ranks = {m_total}/{world} must be a multiple of 128")
    rows = m_total // world
    return rank * rows, rows


def exchange(obj, group=None) -> list:
    """All ranks' `obj` in rank order (IPC handles are 64-byte strings)."""
    import torch.distributed as dist
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


class _PeerBuffers:
    """A device buffer per rank, allocated through the library and opened on every other rank via CUDA IPC."""

    def __init__(self, ctx: capi.Context, nbytes: int, rank: int, world: int, group=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        self.local = ctx.malloc(nbytes)
        handles = exchange(ctx.ipc_get_handle(self.local), group) if world > 1 else [None]
        self.ptrs = [self.local if r == rank else ctx.ipc_open_handle(handles[r]) for r in range(world)]

    def close(self) -> None:
        for r, p in enumerate(self.ptrs):
            if r != self.rank and p:
                self.ctx.ipc_close_handle(p)
        self.ptrs = []
        if self.local:
            self.ctx.free(self.local)
            self.local = 0


class ColumnParallelMatmul:
    """C = A . B with B split on N: every rank computes its column slice and stores it into every rank's C."""

    def __init__(self, ctx, M: int, N: int, K: int, rank: int, world: int, group=None):
        self.ctx, self.M, self.N, self.K, self.rank, self.world = ctx, M, N, K, rank, world
        self.offset, self.width = column_shard(N, world, rank)
        self.c = _PeerBuffers(ctx, M * N * 2, rank, world, group)

    @property
    def c_ptr(self) -> int:
        return self.c.local

    def launch(self, a, b_shard, stream) -> None:
        """a: [M, K] bf16 (replicated); b_shard: [K, N/g] bf16. Asynchronous; call the ranks' barrier afterwards."""
        d = self.ctx.gemm_desc(a, b_shard, None, self.M, self.width, self.K, ldb=self.width, ldc=self.N)
        self.ctx.gemm_allgather(d, self.c.ptrs, self.rank, stream)

    def close(self) -> None:
        self.c.close()


class RowParallelMatmul:
    """C = A . B with A split on K columns and B on K rows: fp32 partial tiles go to the owner of each row block,
    which sums the g slices and rounds to bf16 once."""

    def __init__(self, ctx, M: int, N: int, K: int, rank: int, world: int, group=None):
        self.ctx, self.M, self.N, self.K, self.rank, self.world = ctx, M, N, K, rank, world
        self.k_offset, self.k_depth = k_shard(K, world, rank)
        self.row_offset, self.rows = row_block(M, world, rank)
        self.slots = _PeerBuffers(ctx, world * self.rows * N * 4, rank, world, group)
        self.out = ctx.malloc(self.rows * N * 2)

    def launch_partials(self, a_shard, b_shard, stream, lda=None) -> None:
        """a_shard: [M, K/g] bf16 (lda = its leading dimension), b_shard: [K/g, N] bf16."""
        d = self.ctx.gemm_desc(a_shard, b_shard, None, self.M, self.N, self.k_depth, lda=lda or self.k_depth, ldb=self.N,
                               ldc=self.N, c_dtype=F32)
        self.ctx.gemm_reduce_scatter_partials(d, self.slots.ptrs, self.rank, stream)

    def launch_reduce(self, stream) -> None:
        """After the ranks' barrier: out[rows, N] (bf16) = sum of this rank's g slices."""
        d = self.ctx.gemm_desc(None, None, self.out, self.rows, self.N, 0, lda=8, ldb=self.N, c_dtype=BF16)
        self.ctx.reduce_slices(self.slots.local, self.world, d, stream)

    def close(self) -> None:
        self.slots.close()
        if self.out:
            self.ctx.free(self.out)
            self.out = 0
