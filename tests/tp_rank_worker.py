"""One rank of the tensor-parallel block job (launched by torchrun from tests/test_tp_gpu.py): one process per GPU,
CUDA-IPC peer buffers, fused GEMM + reduce-scatter epilogues and peer-store all-gathers; the rank checks its rows of the
output and of dx and its weight-gradient shards against the single-device CPU oracle. With TP_BENCH=1 it times the full
step (forward, backward, Adam) of the GPT-2-XL-shaped block instead and rank 0 prints one JSON line."""
import json
import os
import sys
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))
from __graft_entry__ import load_package  # noqa: E402
from oracle import matmul_oracle as mo  # noqa: E402
sys.path.insert(0, str(REPO / "tests"))
import rank_common  # noqa: E402


def weights(rng, d, f, std=0.03):
    shapes = dict(wq=(d, d), wk=(d, d), wv=(d, d), wo=(d, d), w1=(f, d), w2=(d, f))
    w = {k: mo.bf16_round(rng.standard_normal(sh).astype(np.float32) * std) for k, sh in shapes.items()}
    for k, n in (("bq", d), ("bk", d), ("bv", d), ("bo", d), ("b1", f), ("b2", d), ("ln1_b", d), ("ln2_b", d)):
        w[k] = mo.bf16_round(rng.standard_normal(n).astype(np.float32) * 0.02)
    w["ln1_g"] = mo.bf16_round(1 + 0.1 * rng.standard_normal(d).astype(np.float32))
    w["ln2_g"] = mo.bf16_round(1 + 0.1 * rng.standard_normal(d).astype(np.float32))
    return w


def main():
    pkg = load_package()
    tp, DT = pkg.tp, pkg.DeviceTensor
    rank, world, local, ctx, comm = rank_common.start(pkg)
    rng = np.random.default_rng(11)                       # identical on every rank
    bench = os.environ.get("TP_BENCH") == "1"
    if bench:
        b, s, heads = 16, 1024, 25                        # GPT-2-XL-shaped block: D 1600, F 6400, T = 16384
    else:
        b, s, heads = 2, 128 * world, max(5, world + 1)   # one head more than ranks (5 on 2 or 4 ranks): uneven head counts
    d, f = heads * 64, 4 * heads * 64
    w = weights(rng, d, f, std=0.02 if bench else 0.03)
    t, tr = b * s, b * s // world
    x = mo.bf16_round(rng.standard_normal((b, s, d)).astype(np.float32) * 0.5)
    d_out = mo.bf16_round(rng.standard_normal((b, s, d)).astype(np.float32) * 0.1)
    rk, fabric = tp.make_process(ctx, rank, world, batch=b, seq=s, d_model=d, heads=heads, host_w=w, comm=comm)
    x_r = DT.from_numpy(ctx, x.reshape(t, d)[rank * tr:(rank + 1) * tr])
    do_r = DT.from_numpy(ctx, d_out.reshape(t, d)[rank * tr:(rank + 1) * tr])
    fabric.barrier()

    def step():
        tp.run_process(rk.forward(x_r), fabric)
        tp.run_process(rk.backward(do_r), fabric)
        rk.adam_step()

    if bench:
        for _ in range(3):
            step()
        fabric.barrier()
        run, executor = step, "eager launches"
        if os.environ.get("TP_GRAPH", "1") == "1":
            # the whole step of this rank — kernels, peer copies and the on-stream NCCL barriers — as one CUDA graph
            tid = ctx.trace_begin()
            step()
            ctx.trace_end(tid)
            run, executor = (lambda: ctx.trace_execute(tid)), "trace replay (CUDA graph per rank, NCCL barriers inside)"
            run()
            fabric.barrier()
        n = 20
        t0 = time.perf_counter()
        for _ in range(n):
            run()
        fabric.barrier()
        ms_t = DT.from_numpy(ctx, np.array([(time.perf_counter() - t0) / n * 1e3], np.float32), pkg.F32)
        comm.allreduce(ms_t, 1, pkg.F32, pkg.capi.COMM_MAX)
        ms = float(ms_t.numpy()[0])
        if rank == 0:
            print(json.dumps({"metric": "TP GPT-2-XL block step", "ms_per_step": ms, "n_gpus": world,
                              "executor": executor,
                              "tokens_per_s": t / ms * 1e3, "config": {"batch": b, "seq": s, "d_model": d,
                                                                                      "heads": heads, "d_ff": f}}))
    else:
        # the oracle block with bf16 storage points: the reference's math, rounded where a bf16 executor stores a tensor
        ref_out, ref_cache = mo.transformer_block_forward(x, w, heads, quantize=mo.bf16_round)
        ref_dx, ref_g = mo.transformer_block_backward(d_out, w, ref_cache, heads, quantize=mo.bf16_round)
        tp.run_process(rk.forward(x_r), fabric)
        tp.run_process(rk.backward(do_r), fabric)
        rows = slice(rank * tr, (rank + 1) * tr)
        err = mo.rel_frobenius(rk.out.numpy(), ref_out.reshape(t, d)[rows])
        assert err <= 1e-2, f"rank {rank}: output {err}"
        err = mo.rel_frobenius(rk.d_x.numpy(), ref_dx.reshape(t, d)[rows])
        assert err <= 1e-2, f"rank {rank}: dx {err}"
        sh = rk.shard
        kr = sh["h1"] - sh["h0"]
        g = {k: v.numpy() for k, v in rk.grads.items()}
        checks = {"wq": (g["wqkv"][:kr], ref_g["wq"][sh["h0"]:sh["h1"]]), "wv": (g["wqkv"][2 * kr:], ref_g["wv"][sh["h0"]:sh["h1"]]),
                  "wo": (g["wo"], ref_g["wo"][:, sh["h0"]:sh["h1"]]), "w1": (g["w1"], ref_g["w1"][sh["f0"]:sh["f1"]]),
                  "w2": (g["w2"], ref_g["w2"][:, sh["f0"]:sh["f1"]]), "b1": (g["b1"], ref_g["b1"][sh["f0"]:sh["f1"]]),
                  "bo": (g["bo"], ref_g["bo"]), "b2": (g["b2"], ref_g["b2"]), "ln1_g": (g["ln1_g"], ref_g["ln1_g"]),
                  "ln2_b": (g["ln2_b"], ref_g["ln2_b"])}
        for k, (got, ref) in checks.items():
            err = mo.rel_frobenius(got, ref)
            assert err <= 1e-2, f"rank {rank}: grad {k} {err}"
        rk.adam_step()
        ctx.synchronize()
        if rank == 0:
            print("TP_PARITY_OK", world)
    fabric.barrier()
    fabric.close()
    rank_common.stop(ctx, comm)


if __name__ == "__main__":
    main()
