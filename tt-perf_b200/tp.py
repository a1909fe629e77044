"""Tensor-parallel pre-LN transformer block (the GPT-2-XL-shaped configuration: D 1600, 25 heads, F 6400) over g ranks,
Megatron pairing with sequence-sharded activations:

  * QKV and FC1 are column-parallel (a rank owns whole heads / a slice of the hidden units; 25 heads do not divide by g,
    so the head counts differ by at most one), attention-out and FC2 are row-parallel;
  * the row-parallel products end in a reduce-scatter that is fused into the GEMM epilogue (fp32 partial tiles go
    straight to the owner of each row block, b200_gemm_reduce_scatter_partials), which leaves residual stream, LayerNorm
    and their gradients sharded by rows (T / g rows per rank);
  * the LayerNorm output is all-gathered (peer stores of the rank's row block) before the next column-parallel GEMM;
  * weight shards and their Adam state never leave the rank; only the LayerNorm parameters are replicated and their
    gradients summed over the ranks.

The reference has no tensor-parallel block (its distributed code stops at the column-parallel matmul of
bench/metal/matmul_tensor_parallel.cpp:54-123); the arithmetic is that of its single-device block
(autograd/traced/transformer_train.hpp:183-262, verify/compare_grads.py:37-97), against which the parity tests compare.

Every rank runs the same generator; each `yield` is a point where all ranks must have finished what they queued
(stores into peers' memory become visible only then). `run_emulated` steps the generators of g ranks that live in one
process on one GPU in lockstep (one stream orders everything); `run_process` is the one-process-per-GPU form, where
peer buffers are CUDA IPC mappings and a yield is a barrier between the ranks queued on the stream (b200_peer_barrier)
or, optionally, the same barrier bracketed by host-side synchronisations."""
from __future__ import annotations

import numpy as np

from . import capi, nn
from .capi import BF16, F32
from .tensor import DeviceTensor

HEAD_DIM = 64


def split_counts(total: int, world: int) -> list[int]:
    """Sizes of `world` nearly equal parts of `total` (the first total % world parts are one larger)."""
    base, rem = divmod(total, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def shard_weights(w: dict, heads: int, world: int, rank: int) -> dict:
    """Host-side shards of a full block's weights (numpy, keyed like the single-device block) for one rank."""
    hc = split_counts(heads, world)
    h0 = sum(hc[:rank]) * HEAD_DIM
    h1 = h0 + hc[rank] * HEAD_DIM
    f_total = w["w1"].shape[0]
    fc = split_counts(f_total // 8, world)          # hidden units in groups of 8 (16-byte rows)
    f0 = sum(fc[:rank]) * 8
    f1 = f0 + fc[rank] * 8
    return {
        "heads": hc[rank], "h0": h0, "h1": h1, "f0": f0, "f1": f1,
        "wqkv": np.concatenate([w["wq"][h0:h1], w["wk"][h0:h1], w["wv"][h0:h1]], axis=0),
        "bqkv": np.concatenate([w["bq"][h0:h1], w["bk"][h0:h1], w["bv"][h0:h1]], axis=0),
        "wo": np.ascontiguousarray(w["wo"][:, h0:h1]), "bo": w["bo"],
        "w1": np.ascontiguousarray(w["w1"][f0:f1]), "b1": w["b1"][f0:f1],
        "w2": np.ascontiguousarray(w["w2"][:, f0:f1]), "b2": w["b2"],
        "ln1_g": w["ln1_g"], "ln1_b": w["ln1_b"], "ln2_g": w["ln2_g"], "ln2_b": w["ln2_b"],
    }


class EmulatedFabric:
    """g ranks in one process on one GPU: shared buffers are plain allocations, a barrier is the stream order."""

    def __init__(self, ctx, world: int):
        self.ctx, self.world = ctx, world
        self._bufs = []

    def shared(self, nbytes: int) -> list[list[int]]:
        """per_rank[r] = the pointers by which rank r reaches every rank's buffer."""
        ptrs = [self.ctx.malloc(nbytes) for _ in range(self.world)]
        self._bufs += ptrs
        return [list(ptrs) for _ in range(self.world)]

    def close(self) -> None:
        for p in self._bufs:
            self.ctx.free(p)
        self._bufs = []


class ProcessFabric:
    """One process per GPU: a rank allocates its buffer, the others map it through CUDA IPC. `comm` is the ranks'
    communicator (capi.Comm)."""

    def __init__(self, ctx, rank: int, world: int, comm=None):
        self.ctx, self.rank, self.world, self.comm = ctx, rank, world, comm
        self._bufs = []
        self._flags = self._epoch = None
        if comm is not None and world > 1:
            self._flag_barrier_setup()     # collective, and not something to do while a trace is being recorded

    def _flag_barrier_setup(self) -> None:
        """Flag words for b200_peer_barrier: one array per rank, mapped by every rank, all zero before anybody stores."""
        self._flags = self.shared(4 * self.world)
        self._epoch = self.ctx.malloc(4)
        self.ctx.memset(self._flags[self.rank], 0, 4 * self.world)
        self.ctx.memset(self._epoch, 0, 4)
        self.barrier()

    def shared(self, nbytes: int) -> list[int]:
        from .dist import _PeerBuffers
        b = _PeerBuffers(self.ctx, nbytes, self.rank, self.world, self.comm)
        self._bufs.append(b)
        return b.ptrs

    def shared_multicast(self, nbytes: int):
        """(local pointer, multicast pointer) of a buffer that every rank holds a copy of and that one store to the
        multicast address updates everywhere; None when the GPUs offer no NVLink multicast (collective either way)."""
        if self.world < 2 or self.comm is None or not self.ctx.mc_supported():
            return None
        try:
            b = capi.MulticastBuffer(self.comm, nbytes)
        except capi.B200Error:
            return None
        self._bufs.append(b)
        return b.local, b.multicast

    def barrier(self) -> None:
        """Host-side: wait for this rank's stream, then for every rank."""
        self.ctx.synchronize()
        if self.comm is not None:
            self.comm.barrier()
            self.ctx.synchronize()

    def stream_barrier(self) -> None:
        """Device-side: a flag barrier kernel (b200_peer_barrier) queued on the context's stream. It starts only after the
        kernels and peer copies this rank queued before it and completes only when every rank has reached it, so whatever
        runs after it on this stream sees all peers' stores. No host synchronisation, no library collective: about one
        NVLink round trip instead of the ~25 us of a communicator barrier."""
        if self.comm is None or self.world < 2:
            return
        self.ctx.peer_barrier(self._flags, self.rank, self._epoch)

    def close(self) -> None:
        for b in self._bufs:
            b.close()
        self._bufs = []
        if self._epoch:
            self.ctx.free(self._epoch)
        self._flags = self._epoch = None


# Peer-visible buffers of a block, as (name, bytes per rank) given T rows, Tr rows per rank, D columns.
def _shared_layout(T: int, Tr: int, D: int, world: int):
    full = T * D * 2
    slots = world * Tr * D * 4
    return [("ln1_full", full), ("ln2_full", full), ("dout_full", full), ("dres1_full", full), ("slots0", slots),
            ("slots1", slots), ("ln_slots", world * 4 * D * 4)]


class TPBlockRank:
    """One rank's share of the block. `ptrs[name][p]` is this rank's pointer to rank p's buffer `name`."""

    def __init__(self, ctx, rank: int, world: int, *, batch: int, seq: int, d_model: int, heads: int, host_w: dict, ptrs: dict,
                 multicast: dict | None = None, partial_dtype: int = F32):
        """multicast: {buffer name: multicast address} for the all-gathered buffers that live in NVLink multicast
        memory (their row blocks are then broadcast with one store instead of one copy per peer).
        partial_dtype: F32, or BF16 to send the partial tiles of the row-parallel products as bf16 (half the bytes on
        the links, one more rounding per partial sum)."""
        self.ctx, self.rank, self.world = ctx, rank, world
        self.mc = multicast or {}
        self.pdt = partial_dtype
        self.B, self.S, self.D, self.H = batch, seq, d_model, heads
        self.T = batch * seq
        if self.T % world or (self.T // world) % 128:
            raise ValueError(f"rows per rank {self.T}/{world} must be a multiple of 128")
        if d_model != heads * HEAD_DIM:
            raise ValueError("the tensor-parallel block uses the fused attention kernels: head dimension 64")
        if heads < world:
            raise ValueError(f"{heads} heads cannot be spread over {world} ranks (every rank needs at least one)")
        self.Tr = self.T // world
        self.row0 = rank * self.Tr
        self.ptrs = ptrs
        sh = shard_weights(host_w, heads, world, rank)
        self.hr = sh["heads"]
        self.Kr = self.hr * HEAD_DIM
        self.Fr = sh["f1"] - sh["f0"]
        self.shard = sh
        self.w = {k: DeviceTensor.from_numpy(ctx, sh[k]) for k in ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2", "ln1_g",
                                                                   "ln1_b", "ln2_g", "ln2_b")}
        self.cache = {}
        self.out = None       # forward result: local rows [Tr, D]
        self.d_x = None       # backward result: local rows [Tr, D]
        self.grads = {}
        self.opt = None

    # -- helpers ----------------------------------------------------------------------------------------------------
    def _view(self, name: str, owner: int, rows: int, row0: int = 0, shape=None) -> DeviceTensor:
        base = self.ptrs[name][owner]
        return DeviceTensor(self.ctx, shape or (rows, self.D), BF16, ptr=base + row0 * self.D * 2, owner=self)

    def _push_rows(self, name: str) -> None:
        """Copies this rank's row block of its own `name` buffer into the same rows of every peer's buffer."""
        off = self.row0 * self.D * 2
        pitch = self.D * 2
        if name in self.mc:     # one multimem.st per 16 bytes reaches every rank (this one included)
            self.ctx.mc_broadcast(self.mc[name] + off, self.ptrs[name][self.rank] + off, self.Tr * pitch)
            return
        for step in range(1, self.world):
            p = (self.rank + step) % self.world     # ranks start at different peers
            capi.check(capi.lib().b200_peer_copy_2d(self.ctx._h, self.ptrs[name][p] + off, pitch, self.ctx._h,
                                                    self.ptrs[name][self.rank] + off, pitch, pitch, self.Tr))

    def _scatter_partials(self, slots: str, a, b, n: int, k: int, *, transpose_b: bool, lda: int, ldb: int) -> None:
        """fp32 partial of a [T, k] x (b) product, row block j stored into slot `rank` of rank j's staging buffer."""
        d = self.ctx.gemm_desc(a, b, None, self.T, n, k, transpose_b=transpose_b, lda=lda, ldb=ldb, ldc=n, c_dtype=self.pdt)
        self.ctx.gemm_reduce_scatter_partials(d, self.ptrs[slots], self.rank)

    def _reduce_slots(self, slots: str, out: DeviceTensor, n: int, bias=None) -> None:
        d = self.ctx.gemm_desc(None, None, out, self.Tr, n, 0, lda=8, ldb=n, bias=bias)
        self.ctx.reduce_slices(self.ptrs[slots][self.rank], self.world, d, slices_dtype=self.pdt)

    # -- forward ----------------------------------------------------------------------------------------------------
    def forward(self, x_r: DeviceTensor):
        ctx, w, c = self.ctx, self.w, self.cache
        T, Tr, D, B, S = self.T, self.Tr, self.D, self.B, self.S
        c["x"] = x_r
        c["mean1"], c["rstd1"] = DeviceTensor(ctx, (Tr,), F32), DeviceTensor(ctx, (Tr,), F32)
        ctx.layernorm_forward(x_r, w["ln1_g"], w["ln1_b"], self._view("ln1_full", self.rank, Tr, self.row0), c["mean1"],
                              c["rstd1"], Tr, D)
        self._push_rows("ln1_full")
        yield
        ln1 = self._view("ln1_full", self.rank, T, shape=(B, S, D))
        qkv = nn.linear_forward(ctx, ln1, w["wqkv"], w["bqkv"])                     # [B, S, 3 * Kr], this rank's heads
        q_op, k_op, v_op = nn._head_operands(ctx, qkv, self.hr, 3)
        merged = DeviceTensor(ctx, (B, S, self.Kr), BF16)
        lse = DeviceTensor(ctx, (B, self.hr, S), F32)
        merged_lo = DeviceTensor(ctx, (B, S, self.Kr), BF16)
        (o_op,), (olo_op,) = nn._head_operands(ctx, merged, self.hr), nn._head_operands(ctx, merged_lo, self.hr)
        ctx.attention_forward(q_op, k_op, v_op, o_op, lse, B, self.hr, S, causal=True, o_lo=olo_op)
        c.update(qkv=qkv, merged=merged, merged_lo=merged_lo, lse=lse)
        self._scatter_partials("slots0", merged, w["wo"], D, self.Kr, transpose_b=True, lda=self.Kr, ldb=self.Kr)
        yield
        attn_out = DeviceTensor(ctx, (Tr, D), BF16)
        self._reduce_slots("slots0", attn_out, D, bias=w["bo"])
        res1 = DeviceTensor(ctx, (Tr, D), BF16)
        c["mean2"], c["rstd2"] = DeviceTensor(ctx, (Tr,), F32), DeviceTensor(ctx, (Tr,), F32)
        ctx.add_layernorm_forward(x_r, attn_out, res1, w["ln2_g"], w["ln2_b"], self._view("ln2_full", self.rank, Tr, self.row0),
                                  c["mean2"], c["rstd2"], Tr, D)
        c["res1"] = res1
        self._push_rows("ln2_full")
        yield
        ln2 = self._view("ln2_full", self.rank, T, shape=(B, S, D))
        h1 = nn.linear_forward(ctx, ln2, w["w1"], w["b1"])                           # [B, S, Fr]
        h1g = DeviceTensor(ctx, h1.shape, BF16)
        ctx.unary(capi.U_GELU, h1, h1g, h1g.numel)
        c.update(h1=h1, h1g=h1g)
        self._scatter_partials("slots1", h1g, w["w2"], D, self.Fr, transpose_b=True, lda=self.Fr, ldb=self.Fr)
        yield
        mlp = DeviceTensor(ctx, (Tr, D), BF16)
        self._reduce_slots("slots1", mlp, D, bias=w["b2"])
        self.out = nn.add(ctx, res1, mlp)

    # -- backward ---------------------------------------------------------------------------------------------------
    def backward(self, d_out_r: DeviceTensor):
        ctx, w, c, g = self.ctx, self.w, self.cache, self.grads
        T, Tr, D, B, S = self.T, self.Tr, self.D, self.B, self.S
        # the row-parallel FC2 needs every row of d_out: all-gather it
        mine = self._view("dout_full", self.rank, Tr, self.row0)
        ctx.unary(capi.U_COPY, d_out_r, mine, Tr * D)
        self._push_rows("dout_full")
        yield
        d_y = self._view("dout_full", self.rank, T, shape=(B, S, D))
        h1g2, dy2 = c["h1g"].reshape(T, self.Fr), d_y.reshape(T, D)
        d_h1g = nn.matmul(ctx, d_y, w["w2"])                                          # [B,S,D] . [D,Fr]
        g["w2"] = nn.matmul(ctx, dy2, h1g2, True, False)                             # [D, Fr]
        g["b2"] = DeviceTensor(ctx, (D,), BF16)
        ctx.reduce(capi.R_SUM, dy2, 1, T, D, g["b2"])
        d_h1, g["b1"] = nn.gelu_backward(ctx, d_h1g, c["h1"], want_colsum=True)      # b1's gradient from the same pass
        ln2 = self._view("ln2_full", self.rank, T, shape=(B, S, D))
        _, g["w1"], _ = nn.linear_backward(ctx, ln2, w["w1"], d_h1, need_dx=False, need_db=False)
        self._scatter_partials("slots0", d_h1, w["w1"], D, self.Fr, transpose_b=False, lda=self.Fr, ldb=D)
        yield
        d_ln2 = DeviceTensor(ctx, (Tr, D), BF16)
        self._reduce_slots("slots0", d_ln2, D)
        d_res1, g["ln2_g"], g["ln2_b"] = nn.layernorm_backward(ctx, d_ln2, c["res1"], w["ln2_g"], c["mean2"], c["rstd2"],
                                                                upstream=d_out_r)
        mine = self._view("dres1_full", self.rank, Tr, self.row0)
        ctx.unary(capi.U_COPY, d_res1, mine, Tr * D)
        self._push_rows("dres1_full")
        yield
        d_r = self._view("dres1_full", self.rank, T, shape=(B, S, D))
        dr2, merged2 = d_r.reshape(T, D), c["merged"].reshape(T, self.Kr)
        d_merged = nn.matmul(ctx, d_r, w["wo"])                                       # [B,S,D] . [D,Kr]
        g["wo"] = nn.matmul(ctx, dr2, merged2, True, False)                           # [D, Kr]
        g["bo"] = DeviceTensor(ctx, (D,), BF16)
        ctx.reduce(capi.R_SUM, dr2, 1, T, D, g["bo"])
        q_op, k_op, v_op = nn._head_operands(ctx, c["qkv"], self.hr, 3)
        (o_op,), (do_op,) = nn._head_operands(ctx, c["merged"], self.hr), nn._head_operands(ctx, d_merged, self.hr)
        d_qkv = DeviceTensor(ctx, (B, S, 3 * self.Kr), BF16)
        dq_op, dk_op, dv_op = nn._head_operands(ctx, d_qkv, self.hr, 3)
        (olo_op,) = nn._head_operands(ctx, c["merged_lo"], self.hr)
        ctx.attention_backward(q_op, k_op, v_op, o_op, do_op, c["lse"], dq_op, dk_op, dv_op, B, self.hr, S, causal=True,
                               o_lo=olo_op)
        ln1 = self._view("ln1_full", self.rank, T, shape=(B, S, D))
        _, g["wqkv"], g["bqkv"] = nn.linear_backward(ctx, ln1, w["wqkv"], d_qkv, need_dx=False)
        self._scatter_partials("slots1", d_qkv, w["wqkv"], D, 3 * self.Kr, transpose_b=False, lda=3 * self.Kr, ldb=D)
        yield
        d_ln1 = DeviceTensor(ctx, (Tr, D), BF16)
        self._reduce_slots("slots1", d_ln1, D)
        self.d_x, g["ln1_g"], g["ln1_b"] = nn.layernorm_backward(ctx, d_ln1, c["x"], w["ln1_g"], c["mean1"], c["rstd1"],
                                                                  upstream=d_res1)
        # LayerNorm parameters are replicated: sum their gradients (computed over the local rows) over the ranks
        names = ("ln1_g", "ln1_b", "ln2_g", "ln2_b")
        for p in range(self.world):
            for i, n in enumerate(names):
                dst = self.ptrs["ln_slots"][p] + (self.rank * 4 + i) * D * 4
                capi.check(capi.lib().b200_peer_copy_2d(ctx._h, dst, D * 4, ctx._h, g[n].ptr, D * 4, D * 4, 1))
        yield
        total = DeviceTensor(ctx, (4, D), F32)
        d = ctx.gemm_desc(None, None, total, 1, 4 * D, 0, lda=8, ldb=4 * D, c_dtype=F32)
        ctx.reduce_slices(self.ptrs["ln_slots"][self.rank], self.world, d)
        for i, n in enumerate(names):
            g[n] = total.narrow0(i, 1).reshape(D)

    # -- optimiser: every rank updates what it owns -------------------------------------------------------------------
    def adam_step(self, *, lr=3e-4, betas=(0.9, 0.95), eps=1e-8):
        bf = ("wqkv", "bqkv", "wo", "bo", "w1", "b1", "w2", "b2")
        f32 = ("ln1_g", "ln1_b", "ln2_g", "ln2_b")
        if self.opt is None:
            self.opt = (nn.Adam(self.ctx, [self.w[k] for k in bf], lr=lr, betas=betas, eps=eps),
                        nn.Adam(self.ctx, [self.w[k] for k in f32], lr=lr, betas=betas, eps=eps))
        self.opt[0].step([self.grads[k] for k in bf])
        self.opt[1].step([self.grads[k] for k in f32])


def make_emulated(ctx, world: int, *, batch: int, seq: int, d_model: int, heads: int, host_w: dict, partial_dtype: int = F32):
    """g ranks of one block in this process (one GPU). Returns (ranks, fabric)."""
    T = batch * seq
    fabric = EmulatedFabric(ctx, world)
    per_rank = [dict() for _ in range(world)]
    for name, nbytes in _shared_layout(T, T // world, d_model, world):
        views = fabric.shared(nbytes)
        for r in range(world):
            per_rank[r][name] = views[r]
    ranks = [TPBlockRank(ctx, r, world, batch=batch, seq=seq, d_model=d_model, heads=heads, host_w=host_w, ptrs=per_rank[r],
                         partial_dtype=partial_dtype)
             for r in range(world)]
    return ranks, fabric


def run_emulated(generators) -> None:
    """Steps the ranks' generators in lockstep: everybody's work up to a yield is queued before anybody continues."""
    live = list(generators)
    while live:
        nxt = []
        for gen in live:
            try:
                next(gen)
                nxt.append(gen)
            except StopIteration:
                pass
        if nxt and len(nxt) != len(live):
            raise RuntimeError("ranks disagree on the number of exchange points")
        live = nxt


def make_process(ctx, rank: int, world: int, *, batch: int, seq: int, d_model: int, heads: int, host_w: dict, comm=None,
                 multicast: bool = True, partial_dtype: int = F32):
    """This process's rank of the block (one process per GPU). Returns (rank object, fabric). With `multicast` the four
    all-gathered activations / gradients live in NVLink multicast memory when the GPUs offer it."""
    T = batch * seq
    fabric = ProcessFabric(ctx, rank, world, comm)
    ptrs, mc = {}, {}
    for name, nbytes in _shared_layout(T, T // world, d_model, world):
        pair = fabric.shared_multicast(nbytes) if (multicast and name.endswith("_full")) else None
        if pair is not None:
            ptrs[name] = [pair[0]] * world       # only this rank's copy is ever addressed directly
            mc[name] = pair[1]
        else:
            ptrs[name] = fabric.shared(nbytes)
    rk = TPBlockRank(ctx, rank, world, batch=batch, seq=seq, d_model=d_model, heads=heads, host_w=host_w, ptrs=ptrs,
                     multicast=mc, partial_dtype=partial_dtype)
    return rk, fabric


def run_process(generator, fabric: ProcessFabric, *, host_barriers: bool = False) -> None:
    """Runs one rank's generator; every exchange point is a barrier between the ranks — on the stream (default: nothing
    blocks the host, the ranks' kernels simply queue up) or on the host (`host_barriers`, the conservative form)."""
    wait = fabric.barrier if host_barriers else fabric.stream_barrier
    for _ in generator:
        wait()
    wait()
