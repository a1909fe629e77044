"""Host side of the sharded matmul on CPU: shard geometry, and a world_size-2 gloo run of the exchange helper plus
the column-parallel / row-parallel algebra (each rank computes its shard with the oracle, the gathered / reduced
result must equal the unsharded product)."""
import os
import socket

import numpy as np
import pytest

from oracle import matmul_oracle as mo


def test_shard_geometry(pkg):
    d = pkg.dist
    assert [d.column_shard(16384, 8, r) for r in (0, 3, 7)] == [(0, 2048), (6144, 2048), (14336, 2048)]
    assert d.k_shard(16384, 4, 1) == (4096, 4096)
    assert d.row_block(16384, 8, 7) == (14336, 2048)
    for bad in (lambda: d.column_shard(100, 8, 0), lambda: d.column_shard(24, 2, 0), lambda: d.k_shard(100, 3, 0),
                lambda: d.row_block(1024, 16, 0)):
        with pytest.raises(ValueError):
            bad()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)

    class GlooComm:
        """Stands in for the library's communicator on a machine without GPUs: same interface, gloo underneath."""
        def __init__(self):
            self.world, self.rank = world, rank

        def exchange(self, blob):
            out = [None] * world
            dist.all_gather_object(out, blob)
            return out

        def barrier(self, stream=None):
            dist.barrier()

    try:
        # the same exchange helper that carries CUDA IPC handles on the GPU path
        handles = pkg.dist.exchange(GlooComm(), bytes([rank]) * 64)
        assert handles == [bytes([r]) * 64 for r in range(world)]
        assert pkg.dist.exchange(None, b"x") == [b"x"]
        rng = np.random.default_rng(7)
        M, N, K = 256, 64, 96
        a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
        b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
        full = mo.matmul(a, b)
        # N-split + all-gather
        off, width = pkg.dist.column_shard(N, world, rank)
        mine = torch.from_numpy(mo.matmul(a, b[:, off:off + width]))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        gathered = torch.cat(parts, dim=1).numpy()
        assert mo.rel_frobenius(gathered, full) < 1e-6
        # K-split + reduce-scatter (all-reduce then keep the owned row block)
        koff, kdepth = pkg.dist.k_shard(K, world, rank)
        partial = torch.from_numpy(mo.matmul(a[:, koff:koff + kdepth], b[koff:koff + kdepth]))
        dist.all_reduce(partial)
        roff, rows = pkg.dist.row_block(M, world, rank)
        assert mo.rel_frobenius(partial.numpy()[roff:roff + rows], full[roff:roff + rows]) < 1e-5
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_column_and_row_parallel():
    import torch.multiprocessing as mp
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(results) == {0: "ok", 1: "ok"}


def test_tensor_parallel_shard_geometry():
    """Host logic of the tensor-parallel block: uneven head counts, hidden-unit slices, weight shards."""
    import numpy as np
    from __graft_entry__ import load_package
    tp = load_package().tp
    assert tp.split_counts(25, 8) == [4, 3, 3, 3, 3, 3, 3, 3] and tp.split_counts(25, 2) == [13, 12]
    assert sum(tp.split_counts(6400 // 8, 8)) * 8 == 6400
    heads, d, f = 5, 320, 1280
    rng = np.random.default_rng(0)
    w = {k: rng.standard_normal(s).astype(np.float32) for k, s in dict(wq=(d, d), wk=(d, d), wv=(d, d), wo=(d, d), w1=(f, d),
                                                                         w2=(d, f), bq=(d,), bk=(d,), bv=(d,), bo=(d,), b1=(f,),
                                                                         b2=(d,), ln1_g=(d,), ln1_b=(d,), ln2_g=(d,), ln2_b=(d,)).items()}
    cover_h, cover_f = np.zeros(d, int), np.zeros(f, int)
    for r in range(4):
        sh = tp.shard_weights(w, heads, 4, r)
        kr = sh["heads"] * 64
        assert sh["wqkv"].shape == (3 * kr, d) and sh["wo"].shape == (d, kr)
        assert np.array_equal(sh["wqkv"][kr:2 * kr], w["wk"][sh["h0"]:sh["h1"]])
        assert np.array_equal(sh["w2"], w["w2"][:, sh["f0"]:sh["f1"]]) and sh["w1"].shape[0] % 8 == 0
        cover_h[sh["h0"]:sh["h1"]] += 1
        cover_f[sh["f0"]:sh["f1"]] += 1
    assert (cover_h == 1).all() and (cover_f == 1).all()   # every head and hidden unit owned exactly once
