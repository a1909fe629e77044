"""Tensor-parallel transformer block (the GPT-2-XL-shaped configuration, scaled down) against the single-device oracle.
The ranks are emulated in one process on one GPU: every rank's kernels, peer stores and fused reduce-scatter epilogues
run for real, a barrier is the stream order. Tolerance: relative Frobenius error <= 1e-2 on the output, on dx and on
every weight gradient, against the oracle block with bf16 storage points (the reference's math, rounded where a bf16
executor stores a tensor between ops); the output is also held to 1e-2 against the oracle without rounding."""
import numpy as np
import pytest

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu


def _weights(rng, d, f):
    shapes = dict(wq=(d, d), wk=(d, d), wv=(d, d), wo=(d, d), w1=(f, d), w2=(d, f))
    w = {k: mo.bf16_round(rng.standard_normal(sh).astype(np.float32) * 0.03) for k, sh in shapes.items()}
    for k, n in (("bq", d), ("bk", d), ("bv", d), ("bo", d), ("b1", f), ("b2", d), ("ln1_b", d), ("ln2_b", d)):
        w[k] = mo.bf16_round(rng.standard_normal(n).astype(np.float32) * 0.02)
    w["ln1_g"] = mo.bf16_round(1 + 0.1 * rng.standard_normal(d).astype(np.float32))
    w["ln2_g"] = mo.bf16_round(1 + 0.1 * rng.standard_normal(d).astype(np.float32))
    return w


def _gather_grads(ranks, w, heads):
    """Full-shape gradients reassembled from the ranks' shards."""
    d = w["wq"].shape[0]
    out = {k: np.zeros_like(w[k]) for k in ("wq", "wk", "wv", "bq", "bk", "bv", "wo", "w1", "b1", "w2")}
    for r in ranks:
        sh, g = r.shard, {k: v.numpy() for k, v in r.grads.items()}
        kr = sh["h1"] - sh["h0"]
        for i, n in enumerate("qkv"):
            out["w" + n][sh["h0"]:sh["h1"]] = g["wqkv"][i * kr:(i + 1) * kr]
            out["b" + n][sh["h0"]:sh["h1"]] = g["bqkv"][i * kr:(i + 1) * kr]
        out["wo"][:, sh["h0"]:sh["h1"]] = g["wo"]
        out["w1"][sh["f0"]:sh["f1"]] = g["w1"]
        out["b1"][sh["f0"]:sh["f1"]] = g["b1"]
        out["w2"][:, sh["f0"]:sh["f1"]] = g["w2"]
    for k in ("bo", "b2", "ln1_g", "ln1_b", "ln2_g", "ln2_b"):
        out[k] = ranks[0].grads[k].numpy()
        for r in ranks[1:]:   # replicated parameters: every rank must hold the same gradient
            assert np.array_equal(r.grads[k].numpy(), out[k]), k
    return out


@pytest.mark.parametrize("world,partials", [(2, "f32"), (4, "f32"), (4, "bf16")])
def test_tp_block_matches_single_device_oracle(pkg, ctx, world, partials):
    """partials = "bf16": the partial tiles of the row-parallel products cross the links as bf16 (half the bytes)."""
    DT, tp = pkg.DeviceTensor, pkg.tp
    rng = np.random.default_rng(7)
    b, s, heads = 2, 256, 5                       # 5 heads do not divide by 2 or 4: uneven head counts
    d, f = heads * 64, 4 * heads * 64
    w = _weights(rng, d, f)
    x = mo.bf16_round(rng.standard_normal((b, s, d)).astype(np.float32) * 0.5)
    d_out = mo.bf16_round(rng.standard_normal((b, s, d)).astype(np.float32) * 0.1)
    fp32_out, _ = mo.transformer_block_forward(x, w, heads)
    ref_out, ref_cache = mo.transformer_block_forward(x, w, heads, quantize=mo.bf16_round)
    ref_dx, ref_g = mo.transformer_block_backward(d_out, w, ref_cache, heads, quantize=mo.bf16_round)

    ranks, fabric = tp.make_emulated(ctx, world, batch=b, seq=s, d_model=d, heads=heads, host_w=w,
                                     partial_dtype=pkg.BF16 if partials == "bf16" else pkg.F32)
    try:
        t, tr = b * s, b * s // world
        xs = [DT.from_numpy(ctx, x.reshape(t, d)[r * tr:(r + 1) * tr]) for r in range(world)]
        dos = [DT.from_numpy(ctx, d_out.reshape(t, d)[r * tr:(r + 1) * tr]) for r in range(world)]
        tp.run_emulated([rk.forward(xs[i]) for i, rk in enumerate(ranks)])
        out = np.concatenate([rk.out.numpy() for rk in ranks]).reshape(b, s, d)
        assert mo.rel_frobenius(out, ref_out) <= 1e-2 and mo.rel_frobenius(out, fp32_out) <= 1e-2
        tp.run_emulated([rk.backward(dos[i]) for i, rk in enumerate(ranks)])
        ctx.synchronize()
        dx = np.concatenate([rk.d_x.numpy() for rk in ranks]).reshape(b, s, d)
        assert mo.rel_frobenius(dx, ref_dx) <= 1e-2
        got = _gather_grads(ranks, w, heads)
        scale = max(np.linalg.norm(ref_g[k]) for k in got)
        for k, gk in got.items():
            if k == "bk":   # key bias: mathematically zero (softmax is invariant to it); only rounding noise on both sides
                assert np.linalg.norm(gk) <= 1e-2 * scale and np.linalg.norm(ref_g[k]) <= 1e-2 * scale, k
            else:
                err = mo.rel_frobenius(gk, ref_g[k])
                assert err <= 1e-2, (k, err)
        # one Adam step on a shard equals the oracle's update of the same rows
        before = ranks[1].w["w1"].numpy().copy()
        for rk in ranks:
            rk.adam_step()
        ctx.synchronize()
        g1 = mo.bf16_round(ranks[1].grads["w1"].numpy())
        expect, _, _ = mo.adam_update(before, g1, 0, 0, 1, lr=3e-4, beta1=0.9, beta2=0.95)
        assert mo.rel_frobenius(ranks[1].w["w1"].numpy(), expect) <= 1e-2
    finally:
        ctx.synchronize()
        fabric.close()


def test_tp_block_rejects_bad_geometry(pkg, ctx):
    rng = np.random.default_rng(1)
    w = _weights(rng, 128, 512)
    with pytest.raises(ValueError):
        pkg.tp.make_emulated(ctx, 4, batch=1, seq=256, d_model=128, heads=2, host_w=w)   # 64 rows per rank


def test_tp_block_one_process_per_gpu():
    """The real peer path: torchrun over the visible GPUs (2, 4 or 8), CUDA-IPC peer buffers, one rank per GPU."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    repo = Path(__file__).resolve().parent.parent
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
                        "--master-addr", "127.0.0.1", "--master-port", "29566", str(repo / "tests" / "tp_rank_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and f"TP_PARITY_OK {n}" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])
