"""Parity of the fused attention kernels (b200_attention_forward / b200_attention_backward) with the CPU oracle's
materialised form S = q k^T * scale, mask, P = softmax(S), O = P v and its backward, through the C ABI.
Tolerance: relative Frobenius error <= 1e-2 on O, dQ, dK, dV (bf16); lse absolute 2e-2. Where the softmax is nearly
one-hot, dS is the small remainder of a cancellation and the bf16 storage of P and dS dominates dQ and dK: that case
is compared with the oracle that stores P and dS in bf16 too, at the same 1e-2, and runs through the _hp entry points,
which carry the part of O that bf16 drops to the backward pass so that the row term rowsum(dO * O) is not the limit."""
import numpy as np
import pytest

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rnd(shape, seed, scale=1.0):
    return mo.bf16_round(np.random.default_rng(seed).standard_normal(shape).astype(np.float32) * scale)


def _lse(q, k, scale, causal):
    s = np.einsum("bhid,bhjd->bhij", q.astype(np.float64), k.astype(np.float64)) * scale
    if causal:
        s = np.where(np.triu(np.ones(s.shape[-2:], dtype=bool), k=1), -np.inf, s)
    m = s.max(-1, keepdims=True)
    return (m + np.log(np.exp(s - m).sum(-1, keepdims=True)))[..., 0]


def _run(pkg, ctx, B, H, S, causal, layout, seed=0, qscale=1.0, bf16_storage=False):
    """layout 'bhsd': separate [B,H,S,64] tensors. layout 'bsd3': q, k, v are column blocks of one [B,S,3*H*64] matrix
    (the output of a fused QKV projection) and o / gradients are [B,S,H*64] (no head split or merge copies)."""
    DT = pkg.DeviceTensor
    dh = 64
    q, k, v, d_o = (rnd((B, H, S, dh), seed + i, s) for i, s in enumerate((qscale, qscale, 1.0, 1.0)))
    lse = DT(ctx, (B, H, S), pkg.F32)
    if layout == "bhsd":
        tq, tk, tv, tdo = (DT.from_numpy(ctx, t) for t in (q, k, v, d_o))
        to, tdq, tdk, tdv, tlo = (DT(ctx, (B, H, S, dh)) for _ in range(5))
        op = lambda t: ctx.attn_operand(t, H * S * dh, S * dh, dh)
        oq, ok, ov, odo, oo, odq, odk, odv, olo = (op(t) for t in (tq, tk, tv, tdo, to, tdq, tdk, tdv, tlo))
        unpack = lambda t: t.numpy()
    else:
        D = H * dh
        merged = lambda t: np.ascontiguousarray(t.transpose(0, 2, 1, 3)).reshape(B, S, D)
        qkv = DT.from_numpy(ctx, np.concatenate([merged(q), merged(k), merged(v)], axis=-1))
        tdo = DT.from_numpy(ctx, merged(d_o))
        to, tlo = DT(ctx, (B, S, D)), DT(ctx, (B, S, D))
        tdqkv = DT(ctx, (B, S, 3 * D))
        oq, ok, ov = (ctx.attn_operand(qkv, S * 3 * D, dh, 3 * D, offset=i * D) for i in range(3))
        odq, odk, odv = (ctx.attn_operand(tdqkv, S * 3 * D, dh, 3 * D, offset=i * D) for i in range(3))
        oo, odo, olo = (ctx.attn_operand(t, S * D, dh, D) for t in (to, tdo, tlo))
        unpack = lambda t: t.numpy().reshape(B, S, H, dh).transpose(0, 2, 1, 3)
    # bf16_storage cases also carry the low part of O to the backward pass (the _hp entry points)
    ctx.attention_forward(oq, ok, ov, oo, lse, B, H, S, causal=causal, o_lo=olo if bf16_storage else None)
    ctx.attention_backward(oq, ok, ov, oo, odo, lse, odq, odk, odv, B, H, S, causal=causal, o_lo=olo if bf16_storage else None)
    ctx.synchronize()
    scale = dh ** -0.5
    o_ref, p_ref = mo.causal_attention_forward(q, k, v, scale, causal=causal)
    dq_ref, dk_ref, dv_ref = mo.causal_attention_backward(q, k, v, p_ref, d_o, scale,
                                                          quantize=mo.bf16_round if bf16_storage else None)
    if layout == "bhsd":
        got = dict(o=unpack(to), dq=unpack(tdq), dk=unpack(tdk), dv=unpack(tdv))
    else:
        g = tdqkv.numpy()
        D = H * dh
        split = lambda i: g[..., i * D:(i + 1) * D].reshape(B, S, H, dh).transpose(0, 2, 1, 3)
        got = dict(o=unpack(to), dq=split(0), dk=split(1), dv=split(2))
    ref = dict(o=o_ref, dq=dq_ref, dk=dk_ref, dv=dv_ref)
    for name in ("o", "dq", "dk", "dv"):
        assert np.isfinite(got[name]).all(), name
        err = mo.rel_frobenius(got[name], ref[name])
        assert err <= TOL, f"{name}: relative Frobenius error {err:.3e} > {TOL}"
    assert np.abs(lse.numpy() - _lse(q, k, scale, causal)).max() <= 2e-2


@pytest.mark.parametrize("B,H,S", [(1, 1, 128), (2, 3, 256), (1, 2, 384), (1, 1, 1024), (2, 2, 200), (1, 1, 77), (1, 3, 129)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_bhsd(pkg, ctx, B, H, S, causal):
    _run(pkg, ctx, B, H, S, causal, "bhsd", seed=10 * S + H)


@pytest.mark.parametrize("B,H,S", [(2, 4, 256), (1, 12, 320), (3, 2, 100)])
def test_attention_on_unpermuted_projection_output(pkg, ctx, B, H, S):
    _run(pkg, ctx, B, H, S, True, "bsd3", seed=S)


@pytest.mark.parametrize("B,H,S,causal", [(2, 3, 640, True), (1, 2, 300, False), (1, 1, 100, True)])
def test_attention_backward_deterministic_option(pkg, ctx, B, H, S, causal):
    """B200_ATTN_DETERMINISTIC: dQ from per-key-tile slabs summed in key order. Same parity as the default form, and
    three runs give the same bits (the default form adds the key tiles' contributions in arrival order)."""
    DT = pkg.DeviceTensor
    dh = 64
    q, k, v, d_o = (rnd((B, H, S, dh), 900 + S + i, 1.0) for i in range(4))
    tq, tk, tv, tdo = (DT.from_numpy(ctx, t) for t in (q, k, v, d_o))
    to, tdk, tdv = (DT(ctx, (B, H, S, dh)) for _ in range(3))
    lse = DT(ctx, (B, H, S), pkg.F32)
    op = lambda t: ctx.attn_operand(t, H * S * dh, S * dh, dh)
    ctx.attention_forward(op(tq), op(tk), op(tv), op(to), lse, B, H, S, causal=causal)
    runs = []
    for _ in range(3):
        tdq = DT(ctx, (B, H, S, dh))
        ctx.attention_backward(op(tq), op(tk), op(tv), op(to), op(tdo), lse, op(tdq), op(tdk), op(tdv), B, H, S, causal=causal,
                               deterministic=True)
        ctx.synchronize()
        runs.append(tdq.numpy().copy())
    assert np.array_equal(runs[0], runs[1]) and np.array_equal(runs[0], runs[2])
    scale = dh ** -0.5
    _, p_ref = mo.causal_attention_forward(q, k, v, scale, causal=causal)
    dq_ref, dk_ref, dv_ref = mo.causal_attention_backward(q, k, v, p_ref, d_o, scale)
    assert mo.rel_frobenius(runs[0], dq_ref) <= TOL
    assert mo.rel_frobenius(tdk.numpy(), dk_ref) <= TOL and mo.rel_frobenius(tdv.numpy(), dv_ref) <= TOL


def test_attention_large_scores(pkg, ctx):
    # scores of magnitude ~ 8 * 8 * sqrt(64) / 8: the running maximum has to keep exp() in range. The softmax is then
    # nearly one-hot, dS = P * (dP - sum(dP * P)) is the small remainder of a cancellation, and the bf16 storage of P and
    # dS that any tensor-core attention applies shows in dQ and dK: compared with the oracle that stores them in bf16.
    _run(pkg, ctx, 1, 2, 256, True, "bhsd", seed=5, qscale=8.0, bf16_storage=True)


def test_attention_rejects_other_head_dims(pkg, ctx):
    DT = pkg.DeviceTensor
    t = DT(ctx, (1, 1, 128, 128))
    lse = DT(ctx, (1, 1, 128), pkg.F32)
    op = ctx.attn_operand(t, 128 * 128, 128 * 128, 128)
    with pytest.raises(pkg.B200Error):
        ctx.attention_forward(op, op, op, op, lse, 1, 1, 128, head_dim=128)


def test_attention_empty(pkg, ctx):
    DT = pkg.DeviceTensor
    t = DT(ctx, (1, 1, 128, 64))
    lse = DT(ctx, (1, 1, 128), pkg.F32)
    op = ctx.attn_operand(t, 0, 0, 64)
    ctx.attention_forward(op, op, op, op, lse, 0, 1, 128)
    ctx.attention_backward(op, op, op, op, op, lse, op, op, op, 1, 1, 0)
