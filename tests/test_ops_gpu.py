"""Parity of the bandwidth-bound neighbours of the matmul (row softmax family, cross-entropy, LayerNorm, element-wise
and broadcast ops, reductions, layout, embedding, SGD/Adam) with the CPU oracle, through the C ABI.
Tolerances: bf16 outputs relative Frobenius <= 1e-2; fp32 losses relative <= 1e-3."""
import json

import numpy as np
import pytest

from oracle import matmul_oracle as mo
from conftest import GOLDEN

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rnd(shape, seed, scale=1.0):
    return mo.bf16_round(np.random.default_rng(seed).standard_normal(shape).astype(np.float32) * scale)


@pytest.fixture()
def DT(pkg):
    return pkg.DeviceTensor


@pytest.mark.parametrize("rows,cols", [(32, 64), (96, 1024), (7, 10), (33, 257), (16, 520), (5, 50257), (3, 4100)])
def test_softmax_and_log_softmax_forward_backward(pkg, ctx, DT, rows, cols):
    x = rnd((rows, cols), 1, 2.0)
    dy = rnd((rows, cols), 2)
    dx_ = DT.from_numpy(ctx, x)
    y = DT(ctx, (rows, cols))
    ctx.softmax(dx_, y, rows, cols)
    ref = mo.softmax(x)
    got = y.numpy()
    assert mo.rel_frobenius(got, ref) <= TOL
    d = DT(ctx, (rows, cols))
    ctx.softmax_backward(DT.from_numpy(ctx, dy), y, d, rows, cols)
    assert mo.rel_frobenius(d.numpy(), mo.softmax_backward(dy, got)) <= TOL
    ly = DT(ctx, (rows, cols))
    ctx.log_softmax(dx_, ly, rows, cols)
    lgot = ly.numpy()
    assert mo.rel_frobenius(lgot, mo.log_softmax(x)) <= TOL
    ctx.log_softmax_backward(DT.from_numpy(ctx, dy), ly, d, rows, cols)
    assert mo.rel_frobenius(d.numpy(), mo.log_softmax_backward(dy, lgot)) <= TOL


def test_softmax_known_answer(pkg, ctx, DT):
    """autograd/tests/test_softmax.cpp:17-35: softmax(ones[32,64]) = 1/64, backward of ones = 0."""
    gold = json.loads((GOLDEN / "verify_autograd.json").read_text())["softmax"]
    x = DT.from_numpy(ctx, np.ones((32, 64), np.float32))
    y = DT(ctx, (32, 64))
    ctx.softmax(x, y, 32, 64)
    assert np.all(y.numpy() == np.float32(gold["y"]))
    d = DT(ctx, (32, 64))
    ctx.softmax_backward(x, y, d, 32, 64)
    assert np.all(np.abs(d.numpy()) <= 1e-6)


@pytest.mark.parametrize("S", [64, 200, 1024, 1536])
def test_scaled_causal_softmax(pkg, ctx, DT, S):
    """scores * scale + (-1e9 upper triangle) -> softmax (traced/nn.hpp:166-170) in one pass."""
    bh = 3
    x = rnd((bh, S, S), 5, 3.0)
    y = DT(ctx, (bh, S, S))
    ctx.softmax(DT.from_numpy(ctx, x), y, bh * S, S, alpha=0.125, causal_period=S)
    masked = np.where(np.triu(np.ones((S, S), bool), 1), np.float32(-np.inf), x * np.float32(0.125))
    got = y.numpy()
    assert mo.rel_frobenius(got, mo.softmax(masked)) <= TOL
    assert np.all(got[:, np.triu(np.ones((S, S), bool), 1)] == 0)


@pytest.mark.parametrize("rows,classes", [(64, 10), (96, 64), (40, 1000), (16, 50257)])
def test_cross_entropy_loss_and_gradient(pkg, ctx, DT, rows, classes):
    logits = rnd((rows, classes), 11, 2.0)
    labels = np.random.default_rng(12).integers(0, classes, rows).astype(np.uint32)
    dl = DT(ctx, (rows, classes))
    loss = DT(ctx, (1,), pkg.F32)
    row_loss = DT(ctx, (rows,), pkg.F32)
    ctx.cross_entropy(DT.from_numpy(ctx, logits), DT.from_numpy(ctx, labels, pkg.U32), rows, classes, loss_sum=loss,
                      row_loss=row_loss, d_logits=dl)
    ref_loss, ref_grad = mo.cross_entropy(logits, labels)
    assert abs(float(loss.numpy()[0]) - ref_loss) <= 1e-3 * abs(ref_loss)
    assert abs(float(row_loss.numpy().mean()) - ref_loss) <= 1e-3 * abs(ref_loss)
    assert mo.rel_frobenius(dl.numpy(), ref_grad) <= TOL


@pytest.mark.parametrize("rows,cols", [(64, 128), (100, 768), (33, 1600), (8, 3000), (5, 24)])
def test_layernorm_forward_backward(pkg, ctx, DT, rows, cols):
    x = rnd((rows, cols), 21, 1.5) + np.float32(0.3)
    x = mo.bf16_round(x)
    gamma = mo.bf16_round(1.0 + 0.1 * np.random.default_rng(22).standard_normal(cols).astype(np.float32))
    beta = rnd((cols,), 23, 0.1)
    dy = rnd((rows, cols), 24)
    y, mean, rstd = pkg.nn.layernorm_forward(ctx, DT.from_numpy(ctx, x), DT.from_numpy(ctx, gamma), DT.from_numpy(ctx, beta))
    ry, rmean, rrstd = mo.layernorm_forward(x, gamma, beta)
    assert mo.rel_frobenius(y.numpy(), ry) <= TOL
    assert mo.rel_frobenius(mean.numpy(), rmean.ravel()) <= 1e-4 and mo.rel_frobenius(rstd.numpy(), rrstd.ravel()) <= 1e-4
    d_x, dg, db = pkg.nn.layernorm_backward(ctx, DT.from_numpy(ctx, dy), DT.from_numpy(ctx, x), DT.from_numpy(ctx, gamma),
                                            mean, rstd)
    rdx, rdg, rdb = mo.layernorm_backward(dy, x, gamma, rmean, rrstd)
    assert mo.rel_frobenius(d_x.numpy(), rdx) <= TOL
    assert mo.rel_frobenius(dg.numpy(), rdg) <= 1e-3 and mo.rel_frobenius(db.numpy(), rdb) <= 1e-3


def test_unary_and_scalar_ops(pkg, ctx, DT):
    c = pkg.capi
    x = rnd((37, 129), 31)
    xd = DT.from_numpy(ctx, x)
    y = DT(ctx, x.shape)
    pos = np.abs(x) + np.float32(0.5)
    cases = [(c.U_NEG, x, -x, 0), (c.U_RELU, x, mo.relu(x), 0), (c.U_GTZ, x, (x > 0).astype(np.float32), 0),
             (c.U_GELU, x, mo.gelu(x), 0), (c.U_RSQRT, pos, 1 / np.sqrt(pos), 0), (c.U_EXP, x, np.exp(x), 0),
             (c.U_LOG, pos, np.log(pos), 0), (c.U_TANH, x, np.tanh(x), 0), (c.U_SQRT, pos, np.sqrt(pos), 0),
             (c.U_ADD_SCALAR, x, x + np.float32(1.5), 1.5), (c.U_MUL_SCALAR, x, x * np.float32(-0.25), -0.25),
             (c.U_RSUB_SCALAR, x, np.float32(2.0) - x, 2.0), (c.U_COPY, x, x, 0), (c.U_RECIP, pos, 1 / pos, 0),
             (c.U_SQUARE, x, x * x, 0)]
    for op, inp, ref, s in cases:
        inp = mo.bf16_round(inp)
        xd.copy_from_numpy(inp)
        ctx.unary(op, xd, y, inp.size, scalar=s)
        refv = {c.U_RSQRT: 1 / np.sqrt(inp), c.U_LOG: np.log(inp), c.U_SQRT: np.sqrt(inp), c.U_RECIP: 1 / inp}.get(op, ref)
        assert mo.rel_frobenius(y.numpy(), refv) <= TOL, op


@pytest.mark.parametrize("a_shape,b_shape", [((64, 128), (64, 128)), ((64, 128), (1, 128)), ((2, 3, 16, 16), (1, 1, 16, 16)),
                                              ((4, 8, 24), (4, 8, 1)), ((5, 7), (1, 1)), ((3, 10), (1, 10)), ((1, 9), (6, 9))])
def test_binary_broadcast(pkg, ctx, DT, a_shape, b_shape):
    c = pkg.capi
    a, b = rnd(a_shape, 41), np.abs(rnd(b_shape, 42)) + np.float32(1.0)
    b = mo.bf16_round(b)
    out_shape = np.broadcast_shapes(a_shape, b_shape)
    out = DT(ctx, out_shape)
    ad, bd = DT.from_numpy(ctx, a), DT.from_numpy(ctx, b)
    for op, ref in ((c.B_ADD, a + b), (c.B_SUB, a - b), (c.B_MUL, a * b), (c.B_DIV, a / b), (c.B_MAX, np.maximum(a, b))):
        ctx.binary(op, ad, a_shape, bd, b_shape, out)
        assert mo.rel_frobenius(out.numpy(), np.broadcast_to(ref, out_shape)) <= TOL, op
    with pytest.raises(pkg.B200Error):
        ctx.binary(c.B_ADD, ad, (3, 5), bd, (4, 5), out)


def test_relu_and_gelu_backward(pkg, ctx, DT):
    x, dy = rnd((50, 72), 51), rnd((50, 72), 52)
    got = pkg.nn.relu_backward(ctx, DT.from_numpy(ctx, dy), DT.from_numpy(ctx, x)).numpy()
    np.testing.assert_array_equal(got, mo.relu_backward(dy, x))
    got = pkg.nn.gelu_backward(ctx, DT.from_numpy(ctx, dy), DT.from_numpy(ctx, x)).numpy()
    assert mo.rel_frobenius(got, mo.gelu_backward(dy, x)) <= TOL


@pytest.mark.parametrize("rows,cols", [(50, 72), (1, 8), (333, 3072), (4096, 1600), (37, 10), (8192, 768)])
def test_gelu_backward_with_column_sums(pkg, ctx, DT, rows, cols):
    """One pass writes dx and the bias gradient of the Linear layer in front of the GELU: dx must equal the separate
    kernel's bit for bit, the sums must be those of the stored dx."""
    x, dy = rnd((rows, cols), 53), rnd((rows, cols), 54)
    xd, dyd = DT.from_numpy(ctx, x), DT.from_numpy(ctx, dy)
    plain = pkg.nn.gelu_backward(ctx, dyd, xd).numpy()
    dx, colsum = pkg.nn.gelu_backward(ctx, dyd, xd, want_colsum=True)
    np.testing.assert_array_equal(dx.numpy(), plain)
    assert mo.rel_frobenius(plain, mo.gelu_backward(dy, x)) <= TOL
    want = plain.astype(np.float64).sum(axis=0)
    assert mo.rel_frobenius(colsum.numpy(), want) <= 4e-3   # one bf16 rounding of an fp32 sum
    # twice in a row: the ticket counters are back at zero
    dx2, colsum2 = pkg.nn.gelu_backward(ctx, dyd, xd, want_colsum=True)
    np.testing.assert_array_equal(colsum2.numpy(), colsum.numpy())


@pytest.mark.parametrize("outer,R,inner", [(1, 1024, 128), (1, 64, 10), (16, 768, 1), (3, 50, 7), (1, 8192, 768), (4, 9, 1), (1, 524288, 1),
                                            (5, 100003, 1)])
def test_reductions(pkg, ctx, DT, outer, R, inner):
    c = pkg.capi
    x = rnd((outer, R, inner), 61)
    xd = DT.from_numpy(ctx, x)
    y = DT(ctx, (outer, inner))
    for op, ref in ((c.R_SUM, x.sum(1)), (c.R_MEAN, x.mean(1)), (c.R_MAX, x.max(1))):
        ctx.reduce(op, xd, outer, R, inner, y)
        got = y.numpy()
        # a sum of R bf16 values of unit variance has magnitude ~sqrt(R); compare against that scale
        assert np.linalg.norm(got - ref) <= TOL * max(np.linalg.norm(ref), np.sqrt(R * ref.size) * 0.05), op


def test_mean_gradient_known_answer(pkg, ctx, DT):
    """autograd/tests/test_mean_debug.cpp:29-41: d(mean)/dx over 16 elements is 1/16."""
    x = DT.full(ctx, (4, 4), 1.0)
    y = DT(ctx, (1,))
    ctx.reduce(pkg.capi.R_MEAN, x, 1, 16, 1, y)
    assert float(y.numpy()[0]) == 1.0
    g = DT.full(ctx, (4, 4), 1.0 / 16)
    assert np.all(g.numpy() == np.float32(0.0625))


def test_permute_triu_fill_cast(pkg, ctx, DT):
    x = rnd((2, 6, 4, 16), 71)
    xd = DT.from_numpy(ctx, x)
    for perm in ((0, 2, 1, 3), (0, 1, 3, 2), (3, 2, 1, 0), (1, 0, 2, 3)):
        out = DT(ctx, tuple(x.shape[p] for p in perm))
        ctx.permute(xd, x.shape, perm, out)
        np.testing.assert_array_equal(out.numpy(), x.transpose(perm))
    w = rnd((1, 1, 40, 72), 72)
    wt = DT(ctx, (1, 1, 72, 40))
    ctx.permute(DT.from_numpy(ctx, w), w.shape, (0, 1, 3, 2), wt)
    np.testing.assert_array_equal(wt.numpy(), w.transpose(0, 1, 3, 2))
    m = DT.full(ctx, (2, 9, 9), -1e9)
    t = DT(ctx, (2, 9, 9))
    ctx.triu(m, t, 2, 9, 9, 1)
    ref = np.triu(np.full((9, 9), mo.bf16_round(np.array([-1e9], np.float32))[0]), 1)
    np.testing.assert_array_equal(t.numpy()[0], ref)
    f = DT(ctx, (100,), pkg.F32)
    ctx.fill(f, 100, pkg.F32, 0.3)
    b = DT(ctx, (100,))
    ctx.cast(f, pkg.F32, b, pkg.BF16, 100)
    assert np.all(b.numpy() == mo.bf16_round(np.array([0.3], np.float32))[0])


def test_embedding_forward_backward(pkg, ctx, DT):
    vocab, dim, n = 97, 64, 300
    table = rnd((vocab, dim), 81)
    ids = np.random.default_rng(82).integers(0, vocab, n).astype(np.uint32)
    dy = rnd((n, dim), 83)
    idd = DT.from_numpy(ctx, ids, pkg.U32)
    out = DT(ctx, (n, dim))
    ctx.embedding_forward(idd, n, DT.from_numpy(ctx, table), vocab, dim, out)
    np.testing.assert_array_equal(out.numpy(), mo.embedding_forward(ids, table))
    dt = DT(ctx, (vocab, dim), pkg.F32)
    ctx.embedding_backward(idd, n, DT.from_numpy(ctx, dy), vocab, dim, dt)
    assert mo.rel_frobenius(dt.numpy(), mo.embedding_backward(ids, dy, vocab)) <= 1e-5


def test_sgd_known_answer_and_random(pkg, ctx, DT):
    """autograd/tests/test_sgd.cpp:46-70: bias 0 with gradient 32 and lr 0.01 -> -0.32 -> -0.64 (bf16 tolerance 0.1)."""
    gold = json.loads((GOLDEN / "verify_autograd.json").read_text())["sgd"]
    bias = DT.zeros(ctx, (32,))
    grad = DT.full(ctx, (32,), 32.0)
    pkg.nn.sgd_step(ctx, [bias], [grad], gold["lr"])
    assert np.allclose(bias.numpy(), gold["bias_after_1"], atol=5e-3)
    pkg.nn.sgd_step(ctx, [bias], [grad], gold["lr"])
    assert np.allclose(bias.numpy(), gold["bias_after_2"], atol=5e-3)
    shapes = [(128, 784), (128,), (10, 128), (10,), (7,), (1000, 3)]
    ps = [rnd(s, 90 + i) for i, s in enumerate(shapes)]
    gs = [rnd(s, 190 + i) for i, s in enumerate(shapes)]
    pd = [DT.from_numpy(ctx, p) for p in ps]
    pkg.nn.sgd_step(ctx, pd, [DT.from_numpy(ctx, g) for g in gs], 0.05)
    for p, g, d in zip(ps, gs, pd):
        assert mo.rel_frobenius(d.numpy(), mo.sgd_update(p, g, 0.05)) <= TOL


def test_adam_two_steps_golden_and_validation(pkg, ctx, DT):
    """tests/adam_optimizer.py:15-22 recurrence, fp32 parameters so the comparison is tight; then bf16 parameters."""
    z = np.load(GOLDEN / "adam_two_step.npz")
    p = DT.from_numpy(ctx, z["w0"], pkg.F32)
    opt = pkg.nn.Adam(ctx, [p], lr=float(z["lr"]), betas=(float(z["beta1"]), float(z["beta2"])), eps=float(z["eps"]))
    opt.step([DT.from_numpy(ctx, z["g1"], pkg.F32)])
    np.testing.assert_allclose(p.numpy(), z["w1"], rtol=1e-4, atol=1e-6)
    opt.step([DT.from_numpy(ctx, z["g2"], pkg.F32)])
    np.testing.assert_allclose(p.numpy(), z["w2"], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(opt.m[0].numpy(), z["m2"], rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(opt.v[0].numpy(), z["v2"], rtol=1e-5, atol=1e-7)
    pb = DT.from_numpy(ctx, z["w0"])
    optb = pkg.nn.Adam(ctx, [pb], lr=0.1)
    optb.step([DT.from_numpy(ctx, z["g1"])])
    w1, _, _ = mo.adam_update(mo.bf16_round(z["w0"]), mo.bf16_round(z["g1"]), 0, 0, 1, lr=0.1)
    assert mo.rel_frobenius(pb.numpy(), w1) <= TOL
    for bad in (dict(lr=0.0), dict(eps=0.0), dict(betas=(1.0, 0.9)), dict(betas=(0.9,))):
        with pytest.raises(ValueError):   # tests/adam_optimizer.py:126-151
            pkg.nn.Adam(ctx, [p], **bad)


def test_adam_step_in_parts_equals_one_step(pkg, ctx, DT):
    """A step applied to parameter subsets (the second part without advancing the step number) leaves parameters and
    moments bit for bit as the undivided step does, over two steps."""
    rng = np.random.default_rng(77)
    shapes = [(300, 40), (17,), (64, 64)]
    w0 = [rng.standard_normal(sh).astype(np.float32) for sh in shapes]
    gs = [[rng.standard_normal(sh).astype(np.float32) for sh in shapes] for _ in range(2)]
    whole = [DT.from_numpy(ctx, w, pkg.F32) for w in w0]
    parts = [DT.from_numpy(ctx, w, pkg.F32) for w in w0]
    opt_w = pkg.nn.Adam(ctx, whole, lr=1e-2, betas=(0.9, 0.95))
    opt_p = pkg.nn.Adam(ctx, parts, lr=1e-2, betas=(0.9, 0.95))
    for g in gs:
        gd = [DT.from_numpy(ctx, x, pkg.F32) for x in g]
        opt_w.step(gd)
        opt_p.step(gd[1:], indices=range(1, 3))
        opt_p.step(gd[:1], indices=[0], advance=False)
    assert opt_p.t == opt_w.t == 2
    for a, b in zip(whole, parts):
        np.testing.assert_array_equal(a.numpy(), b.numpy())
    for a, b in zip(opt_w.m + opt_w.v, opt_p.m + opt_p.v):
        np.testing.assert_array_equal(a.numpy(), b.numpy())


@pytest.mark.parametrize("rows,cols", [(64, 768), (33, 520), (17, 100), (40, 1024), (9, 1600), (5, 2304)])
def test_layernorm_with_fused_residual_add(pkg, ctx, DT, rows, cols):
    """b200_add_layernorm_forward / b200_layernorm_backward_add against the separate oracle steps: the sum is rounded to
    bf16 before it is normalised, as a separate add would leave it."""
    x, res, dy, up = (rnd((rows, cols), s) for s in (11, 12, 13, 14))
    gamma = rnd((cols,), 15) * 0.1 + 1
    beta = rnd((cols,), 16) * 0.1
    total, y = DT(ctx, (rows, cols)), DT(ctx, (rows, cols))
    mean, rstd = DT(ctx, (rows,), pkg.F32), DT(ctx, (rows,), pkg.F32)
    ctx.add_layernorm_forward(DT.from_numpy(ctx, x), DT.from_numpy(ctx, res), total, DT.from_numpy(ctx, gamma),
                              DT.from_numpy(ctx, beta), y, mean, rstd, rows, cols)
    ref_total = mo.bf16_round(x + res)
    assert np.array_equal(total.numpy(), ref_total)
    ref_y, ref_mean, ref_rstd = mo.layernorm_forward(ref_total, gamma, beta)
    assert mo.rel_frobenius(y.numpy(), ref_y) <= TOL
    assert np.allclose(mean.numpy(), ref_mean.ravel(), atol=1e-4) and np.allclose(rstd.numpy(), ref_rstd.ravel(), rtol=1e-3)
    dx, dg, db = DT(ctx, (rows, cols)), DT(ctx, (cols,), pkg.F32), DT(ctx, (cols,), pkg.F32)
    ctx.layernorm_backward_add(DT.from_numpy(ctx, dy), total, DT.from_numpy(ctx, gamma), mean, rstd, DT.from_numpy(ctx, up), dx,
                               dg, db, rows, cols)
    ref_dx, ref_dg, ref_db = mo.layernorm_backward(dy, ref_total, gamma, ref_mean, ref_rstd)
    assert mo.rel_frobenius(dx.numpy(), mo.bf16_round(ref_dx) + up) <= TOL
    assert mo.rel_frobenius(dg.numpy(), ref_dg) <= TOL and mo.rel_frobenius(db.numpy(), ref_db) <= TOL


@pytest.mark.parametrize("rows,cols,with_upstream", [(256, 768, True), (100, 520, False), (64, 1600, True), (31, 100, True)])
def test_layernorm_backward_emits_column_sums_of_dx(pkg, ctx, DT, rows, cols, with_upstream):
    """b200_layernorm_backward_full: the column sums of dx (the bias gradient of the layer that feeds the residual stream)
    come out of the same kernel and equal a reduction over the stored bf16 dx."""
    x, dy, up = (rnd((rows, cols), s) for s in (21, 22, 23))
    gamma = rnd((cols,), 24) * 0.1 + 1
    ref_y, ref_mean, ref_rstd = mo.layernorm_forward(x, gamma, np.zeros(cols, np.float32))
    mean, rstd = DT.from_numpy(ctx, ref_mean.ravel(), pkg.F32), DT.from_numpy(ctx, ref_rstd.ravel(), pkg.F32)
    dx, dg, db, cs = DT(ctx, (rows, cols)), DT(ctx, (cols,), pkg.F32), DT(ctx, (cols,), pkg.F32), DT(ctx, (cols,))
    ctx.layernorm_backward_full(DT.from_numpy(ctx, dy), DT.from_numpy(ctx, x), DT.from_numpy(ctx, gamma), mean, rstd,
                                DT.from_numpy(ctx, up) if with_upstream else None, dx, dg, db, cs, rows, cols)
    ref_dx, ref_dg, ref_db = mo.layernorm_backward(dy, x, gamma, ref_mean, ref_rstd)
    want = mo.bf16_round(ref_dx) + (up if with_upstream else 0)
    assert mo.rel_frobenius(dx.numpy(), want) <= TOL
    assert mo.rel_frobenius(cs.numpy(), dx.numpy().sum(axis=0)) <= TOL
    assert mo.rel_frobenius(dg.numpy(), ref_dg) <= TOL and mo.rel_frobenius(db.numpy(), ref_db) <= TOL
