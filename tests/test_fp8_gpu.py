"""8-bit (e4m3) operand path of b200_gemm, through the C ABI. The product of the quantised operands is compared with
the oracle's float64 product of the same codes (the only error left is fp32 accumulation order, so the bound is tight);
the quantiser and the absmax reduction are compared bit for bit; and the end-to-end error against the bf16 product is
bounded by what three mantissa bits allow."""
import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu


def codes(shape, seed):
    """Random finite e4m3 codes with magnitudes up to 4 (keeps fp32 partial sums far from cancellation noise)."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape).astype(np.float32)
    return mo.quantize_e4m3(x)


def run(pkg, ctx, stream, a, b, M, N, K, *, batch=1, c_dtype=None, **kw):
    c_dtype = pkg.F32 if c_dtype is None else c_dtype
    tdt = torch.float32 if c_dtype == pkg.F32 else torch.bfloat16
    shape = (batch, M, N) if batch > 1 else (M, N)
    c = torch.full(shape, float("nan"), dtype=tdt, device="cuda")
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    ctx.gemm(ctx.gemm_desc(da, db, c, M, N, K, transpose_b=True, batch=batch, c_dtype=c_dtype,
                           ab_dtype=pkg.FP8_E4M3, **kw), stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    return c.float().cpu().numpy()


SHAPES = [
    (128, 256, 128),     # one tile, one K block
    (128, 64, 32),       # a single MMA K slice
    (256, 256, 512),
    (200, 136, 208),     # ragged everywhere; K ends inside a K block
    (1000, 520, 784),
    (513, 72, 1040),
    (8, 8, 16),
    (2600, 2824, 784),   # CTA-pair kernel, ragged
    (4096, 2560, 384),
    (128, 256, 8192),    # the planner slices K
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_fp8_gemm_matches_oracle(pkg, ctx, stream, M, N, K):
    a, b = codes((M, K), 1 + M), codes((N, K), 2 + N)
    got = run(pkg, ctx, stream, a, b, M, N, K, alpha=0.25)
    assert not np.isnan(got).any(), "output tile left unwritten"
    assert mo.rel_frobenius(got, mo.matmul_e4m3(a, b, 0.25)) <= 2e-6


@pytest.mark.parametrize("split_k", [1, 2, 4, 7])
def test_fp8_gemm_k_slices(pkg, ctx, stream, split_k):
    M, N, K = 256, 512, 2048
    a, b = codes((M, K), 11), codes((N, K), 12)
    got = run(pkg, ctx, stream, a, b, M, N, K, split_k=split_k)
    assert mo.rel_frobenius(got, mo.matmul_e4m3(a, b)) <= 2e-6


def test_fp8_gemm_batched_bias_gelu_bf16_out(pkg, ctx, stream):
    B, M, N, K = 3, 192, 320, 256
    a, b = codes((B, M, K), 21), codes((B, N, K), 22)
    bias = mo.bf16_round(np.random.default_rng(23).standard_normal(N).astype(np.float32))
    dbias = torch.from_numpy(bias).bfloat16().cuda()
    got = run(pkg, ctx, stream, a, b, M, N, K, batch=B, c_dtype=pkg.BF16, bias=dbias, activation=pkg.ACT_GELU,
              alpha=1.0 / 16)
    ref = mo.gelu(mo.matmul_e4m3(a, b, 1.0 / 16) + bias)
    assert mo.rel_frobenius(got, ref) <= 1e-2


def test_fp8_gemm_shared_weight_across_batch(pkg, ctx, stream):
    B, M, N, K = 4, 128, 128, 128
    a, b = codes((B, M, K), 31), codes((N, K), 32)
    got = run(pkg, ctx, stream, a, b, M, N, K, batch=B, stride_b=0)
    assert mo.rel_frobenius(got, mo.matmul_e4m3(a, b)) <= 2e-6


def test_fp8_rejects_what_the_tensor_cores_cannot_read(pkg, ctx, stream):
    a = torch.zeros(64 * 64, dtype=torch.uint8, device="cuda")
    c = torch.zeros(64, 64, dtype=torch.float32, device="cuda")
    for kw in (dict(transpose_b=False), dict(transpose_a=True, transpose_b=True), dict(transpose_b=True, lda=72),
               dict(transpose_b=True, algo=pkg.ALGO_SIMT)):
        with pytest.raises(pkg.B200Error) as e:
            ctx.gemm(ctx.gemm_desc(a, a, c, 64, 64, 64, c_dtype=pkg.F32, ab_dtype=pkg.FP8_E4M3, **kw), stream.cuda_stream)
        assert e.value.code == pkg.capi.ERR_INVALID_ARG
    with pytest.raises(pkg.B200Error):
        ctx.gemm(ctx.gemm_desc(a, a, c, 64, 64, 64, transpose_b=True, c_dtype=pkg.F32, ab_dtype=7), stream.cuda_stream)


@pytest.mark.parametrize("n,offset", [(1 << 20, 0), (100003, 0), (4099, 1), (7, 0), (16, 0)])
def test_absmax_and_quantise_are_bit_exact(pkg, ctx, stream, n, offset):
    rng = np.random.default_rng(n)
    x = mo.bf16_round((rng.standard_normal(n + offset) * rng.choice([1e-3, 0.1, 1.0, 40.0], n + offset)).astype(np.float32))
    dx = torch.from_numpy(x).bfloat16().cuda()[offset:]   # offset 1: a 2-byte aligned start, scalar path
    x = x[offset:]
    amax = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    ctx.absmax(dx, n, amax, stream=stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    want = float(np.abs(x).max())
    assert float(amax.item()) == want
    scale = float(np.float32(448.0) / np.float32(want))
    y = torch.full((n + 16,), 0xAB, dtype=torch.uint8, device="cuda")
    ctx.quantize_fp8(dx, n, scale, y, stream=stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    got = y.cpu().numpy()
    assert np.array_equal(got[:n], mo.quantize_e4m3(x, scale))
    assert (got[n:] == 0xAB).all(), "wrote past the end"
    # out-of-range products saturate instead of becoming NaN
    ctx.quantize_fp8(dx, n, scale * 8, y, stream=stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    assert np.array_equal(y.cpu().numpy()[:n], mo.quantize_e4m3(x, scale * 8))


def test_fp8_linear_close_to_the_bf16_product(pkg, ctx, stream):
    """x . W^T with per-tensor scales: the 8-bit result stays within the error three mantissa bits give (about 2^-4
    per operand, averaged down over K)."""
    M, N, K = 512, 768, 1024
    rng = np.random.default_rng(5)
    x = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    w = mo.bf16_round(rng.standard_normal((N, K)).astype(np.float32) * 0.02)
    dx, dw = torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(w).bfloat16().cuda()
    amax = torch.zeros(2, dtype=torch.float32, device="cuda")
    ctx.absmax(dx, M * K, amax[0:], stream=stream.cuda_stream)
    ctx.absmax(dw, N * K, amax[1:], stream=stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    sx, sw = 448.0 / float(amax[0]), 448.0 / float(amax[1])
    qx = torch.empty(M * K, dtype=torch.uint8, device="cuda")
    qw = torch.empty(N * K, dtype=torch.uint8, device="cuda")
    ctx.quantize_fp8(dx, M * K, sx, qx, stream=stream.cuda_stream)
    ctx.quantize_fp8(dw, N * K, sw, qw, stream=stream.cuda_stream)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ctx.gemm(ctx.gemm_desc(qx, qw, c, M, N, K, transpose_b=True, ab_dtype=pkg.FP8_E4M3, alpha=1.0 / (sx * sw)),
             stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    got = c.float().cpu().numpy()
    assert mo.rel_frobenius(got, mo.matmul(x, w, False, True)) <= 6e-2
    # and exactly what the oracle gives for those codes
    ref = mo.matmul_e4m3(qx.cpu().numpy().reshape(M, K), qw.cpu().numpy().reshape(N, K), 1.0 / (sx * sw))
    assert mo.rel_frobenius(got, ref) <= 1e-2


def test_fp8_linear_layer_helpers(pkg, ctx):
    """nn.quantize_fp8 + nn.linear_forward_fp8 on device tensors: codes equal the oracle's, the layer output equals
    the oracle's product of those codes, and stays close to the bf16 Linear."""
    nn, DT = pkg.nn, pkg.DeviceTensor
    rng = np.random.default_rng(9)
    B, S, D_in, D_out = 4, 96, 256, 384
    x = mo.bf16_round(rng.standard_normal((B, S, D_in)).astype(np.float32))
    w = mo.bf16_round(rng.standard_normal((D_out, D_in)).astype(np.float32) * 0.05)
    bias = mo.bf16_round(rng.standard_normal(D_out).astype(np.float32) * 0.1)
    dx, dw, db = DT.from_numpy(ctx, x), DT.from_numpy(ctx, w), DT.from_numpy(ctx, bias)
    xq, sx = nn.quantize_fp8(ctx, dx)
    wq, sw = nn.quantize_fp8(ctx, dw)
    assert xq.shape == dx.shape and xq.nbytes == dx.numel
    assert sx == 448.0 / float(np.abs(x).max()) and sw == 448.0 / float(np.abs(w).max())
    np.testing.assert_array_equal(xq.numpy(), mo.quantize_e4m3(x, sx))
    y = nn.linear_forward_fp8(ctx, xq, sx, wq, sw, db, "relu").numpy()
    ref = mo.relu(mo.matmul_e4m3(xq.numpy().reshape(B * S, D_in), wq.numpy(), 1.0 / (sx * sw)) + bias).reshape(B, S, D_out)
    assert mo.rel_frobenius(y, ref) <= 1e-2
    y16 = nn.linear_forward(ctx, dx, dw, db, "relu").numpy()
    assert mo.rel_frobenius(y, y16) <= 8e-2
    # a caller-supplied scale keeps the call asynchronous and saturates what it does not cover
    xq2, s2 = nn.quantize_fp8(ctx, dx, scale=1000.0)
    assert s2 == 1000.0
    np.testing.assert_array_equal(xq2.numpy(), mo.quantize_e4m3(x, 1000.0))


@pytest.mark.parametrize("rows,cols,off", [(64, 64, 0), (512, 768, 0), (200, 136, 0), (67, 33, 0), (1, 5, 0), (130, 70, 1)])
def test_transposed_quantiser_is_bit_exact(pkg, ctx, stream, rows, cols, off):
    rng = np.random.default_rng(rows * 1000 + cols)
    ld = cols + 6 + off                      # padded rows; an odd pitch takes the scalar load path
    x = mo.bf16_round((rng.standard_normal((rows, ld)) * 3.0).astype(np.float32))
    dx = torch.from_numpy(x).bfloat16().cuda()
    ldy = rows + (4 - rows % 4) % 4 + 4 * off + off   # off: a pitch the 4-byte stores cannot use
    y = torch.full((cols + 1, ldy), 0xAB, dtype=torch.uint8, device="cuda")
    ctx.quantize_fp8_transposed(dx, rows, cols, 7.5, y, ldx=ld, ldy=ldy, stream=stream.cuda_stream)
    ctx.synchronize(stream.cuda_stream)
    got = y.cpu().numpy()
    np.testing.assert_array_equal(got[:cols, :rows], mo.quantize_e4m3(x[:, :cols], 7.5).T)
    assert (got[:cols, rows:] == 0xAB).all() and (got[cols:] == 0xAB).all(), "wrote outside the matrix"


def test_fp8_linear_backward_products_through_transposed_copies(pkg, ctx):
    """dX = dY . W and dW = dY^T . X on 8-bit operands: each reads a transposed quantised copy as its K-major B (and A)."""
    nn, DT = pkg.nn, pkg.DeviceTensor
    rng = np.random.default_rng(13)
    T, D_in, D_out = 384, 256, 320
    x = mo.bf16_round(rng.standard_normal((T, D_in)).astype(np.float32))
    w = mo.bf16_round(rng.standard_normal((D_out, D_in)).astype(np.float32) * 0.05)
    dy = mo.bf16_round(rng.standard_normal((T, D_out)).astype(np.float32) * 0.01)
    dx_, dw_, ddy = DT.from_numpy(ctx, x), DT.from_numpy(ctx, w), DT.from_numpy(ctx, dy)
    dyq, sdy = nn.quantize_fp8(ctx, ddy)
    wtq, sw = nn.quantize_fp8(ctx, dw_, transposed=True)         # [in, out]
    dytq, _ = nn.quantize_fp8(ctx, ddy, scale=sdy, transposed=True)  # [out, T]
    xtq, sx = nn.quantize_fp8(ctx, dx_, transposed=True)         # [in, T]
    assert wtq.shape == (D_in, D_out) and dytq.shape == (D_out, T) and xtq.shape == (D_in, T)
    d_x = nn.linear_forward_fp8(ctx, dyq, sdy, wtq, sw, out_dtype=pkg.F32).numpy()
    d_w = nn.linear_forward_fp8(ctx, dytq, sdy, xtq, sx, out_dtype=pkg.F32).numpy()
    ref_dx = mo.matmul_e4m3(dyq.numpy(), wtq.numpy(), 1.0 / (sdy * sw))
    ref_dw = mo.matmul_e4m3(dytq.numpy(), xtq.numpy(), 1.0 / (sdy * sx))
    assert mo.rel_frobenius(d_x, ref_dx) <= 2e-6 and mo.rel_frobenius(d_w, ref_dw) <= 2e-6
    assert mo.rel_frobenius(d_x, mo.matmul(dy, w)) <= 6e-2
    assert mo.rel_frobenius(d_w, mo.matmul(dy, x, True, False)) <= 6e-2


def test_fidelity_sweep_small(pkg, ctx):
    """The operand-precision study at a small size: all levels learn, the bf16 levels agree closely, FP8 drifts
    within what three mantissa bits allow; with constant tensors (the reference's setting) FP8 quantises exactly."""
    from importlib import import_module
    fs = import_module(pkg.__name__ + ".fidelity_sweep")
    res = fs.run(pkg, ctx, "random", batch=128, dims=(512, 256, 128), lr=5.0, steps=5, warmup=1, timed=2, seed=3)
    base = res["HiFi4"]["loss"]
    assert base[-1] < base[0]
    for level in ("HiFi2", "LoFi", "FP8"):
        loss = res[level]["loss"]
        assert loss[-1] < loss[0] and res[level]["ms_per_step"] > 0
        tol = 0.08 if level == "FP8" else 0.02
        assert all(abs(a - b) <= tol * abs(b) for a, b in zip(loss, base)), (level, loss, base)
    const = fs.run(pkg, ctx, "constant", batch=64, dims=(512, 256, 128), lr=0.1, steps=3, warmup=1, timed=1,
                   levels=("HiFi4", "FP8"))
    assert all(abs(a - b) <= 0.02 * abs(b) for a, b in zip(const["FP8"]["loss"], const["HiFi4"]["loss"]))


def test_fp8_training_steps_follow_the_oracle(pkg, ctx):
    """Four FP8 training steps of the sweep's MLP (all five matmuls on e4m3 operands, per-tensor scales) against the
    oracle's emulation of the same arithmetic: the loss at every step and the weight updates."""
    from importlib import import_module
    fs = import_module(pkg.__name__ + ".fidelity_sweep")
    DT = pkg.DeviceTensor
    batch, dims, lr = 128, (512, 256, 128), 5.0
    x, t, w1, b1, w2, b2 = fs.make_problem("random", batch, dims, 3)
    model = fs.FidelityMLP(pkg, ctx, "FP8", w1, b1, w2, b2, lr)
    dx, dt = DT.from_numpy(ctx, x), DT.from_numpy(ctx, t)
    params = (w1, b1, w2, b2)
    for step in range(4):
        loss_dev = float(model.train_step(dx, dt).numpy()[0])
        loss_ref, params, _ = mo.mlp_train_step_e4m3(x, t, params, lr)
        assert abs(loss_dev - loss_ref) <= 1e-2 * loss_ref, (step, loss_dev, loss_ref)
    start = (mo.bf16_round(w1), mo.bf16_round(b1), mo.bf16_round(w2), mo.bf16_round(b2))
    for dev, ref, init, name in zip(model.params, params, start, ("w1", "b1", "w2", "b2")):
        got = dev.numpy().reshape(ref.shape)
        assert mo.rel_frobenius(got, ref) <= 5e-3, name
        assert mo.rel_frobenius(got - init, ref - init) <= 8e-2, name     # the updates themselves, not just the weights
