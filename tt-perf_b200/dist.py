"""Host side of the sharded matmul: one process per GPU. The ranks talk through a communicator of the library
(`capi.Comm`: b200_comm_* over NCCL) for the exchange of CUDA IPC handles and for rank barriers; the data path is the
fused GEMM + peer-store kernel (b200_gemm_allgather / b200_gemm_reduce_scatter_partials): no collective carries matrix
data. Any object with `world`, `rank`, `exchange(bytes) -> list[bytes]` and `barrier(stream)` can stand in for the
communicator (the CPU tests use one over gloo).

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


def exchange(comm, blob: bytes) -> list:
    """All ranks' `blob` in rank order (IPC handles are 64-byte strings); a single rank needs no communicator."""
    if comm is None:
        return [blob]
    out = comm.exchange(blob)
    if len(out) != comm.world:
        raise RuntimeError(f"exchange returned {len(out)} blobs for {comm.world} ranks")
    return out


class _PeerBuffers:
    """A device buffer per rank, allocated through the library and opened on every other rank via CUDA IPC."""

    def __init__(self, ctx: capi.Context, nbytes: int, rank: int, world: int, comm=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        if world > 1 and comm is None:
            raise ValueError("more than one rank needs a communicator to exchange the buffer handles")
        self.local = ctx.malloc(nbytes)
        handles = exchange(comm, ctx.ipc_get_handle(self.local)) if world > 1 else [None]
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
    """C = A . B with B split on N: every rank computes its column slice and stores it into every rank's C.

    Two transports for the stores of the GEMM epilogue. With NVLink multicast (`multicast=True`, or "auto" when the
    GPUs offer it and there is more than one rank) every rank's C is bound to one multicast object and a finished box
    is written once, with multimem.st: the switch replicates it, so a rank's egress is its slice once. Otherwise the
    epilogue stores the box into each peer's C in turn (CUDA IPC mappings, one TMA store per peer)."""

    def __init__(self, ctx, M: int, N: int, K: int, rank: int, world: int, comm=None, multicast="auto"):
        self.ctx, self.M, self.N, self.K, self.rank, self.world = ctx, M, N, K, rank, world
        self.offset, self.width = column_shard(N, world, rank)
        self.mc = self.c = None
        want_mc = world > 1 and comm is not None and (multicast is True or (multicast == "auto" and ctx.mc_supported()))
        if want_mc and M >= 256 and self.width >= 256:
            try:
                self.mc = capi.MulticastBuffer(comm, M * N * 2)
            except capi.B200Error:
                if multicast is True:
                    raise
                self.mc = None                      # every rank fails together (the allocation is collective)
        if self.mc is None:
            self.c = _PeerBuffers(ctx, M * N * 2, rank, world, comm)

    @property
    def transport(self) -> str:
        return "NVLink multicast (multimem.st)" if self.mc is not None else "unicast peer stores (TMA store per peer)"

    @property
    def c_ptr(self) -> int:
        return self.mc.local if self.mc is not None else self.c.local

    def launch(self, a, b_shard, stream) -> None:
        """a: [M, K] bf16 (replicated); b_shard: [K, N/g] bf16. Asynchronous; call the ranks' barrier afterwards."""
        d = self.ctx.gemm_desc(a, b_shard, None, self.M, self.width, self.K, ldb=self.width, ldc=self.N)
        if self.mc is not None:
            self.ctx.gemm_allgather_mc(d, self.mc.multicast, self.world, self.rank, use_multimem=True, stream=stream)
        else:
            self.ctx.gemm_allgather(d, self.c.ptrs, self.rank, stream)

    def close(self) -> None:
        """Collective when the multicast transport is in use: every rank must call it before any rank exits."""
        if self.mc is not None:
            self.mc.close()
            self.mc = None
        if self.c is not None:
            self.c.close()
            self.c = None


class RowParallelMatmul:
    """C = A . B with A split on K columns and B on K rows: fp32 partial tiles go to the owner of each row block,
    which sums the g slices and rounds to bf16 once."""

    def __init__(self, ctx, M: int, N: int, K: int, rank: int, world: int, comm=None):
        self.ctx, self.M, self.N, self.K, self.rank, self.world = ctx, M, N, K, rank, world
        self.k_offset, self.k_depth = k_shard(K, world, rank)
        self.row_offset, self.rows = row_block(M, world, rank)
        self.slots = _PeerBuffers(ctx, world * self.rows * N * 4, rank, world, comm)
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
