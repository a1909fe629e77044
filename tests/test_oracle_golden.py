"""The numpy oracle against the golden fixtures generated from the reference's own torch-CPU scripts
(tests/golden/make_golden.py). CPU only."""
import json

import numpy as np
import pytest

from oracle import matmul_oracle as mo
from conftest import GOLDEN


def load_json(name):
    return json.loads((GOLDEN / name).read_text())


def test_bf16_round_matches_torch():
    torch = pytest.importorskip("torch")
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4096, generator=g) * 37.0
    x[:8] = torch.tensor([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.0e38, -3.0e38, 1e-40])
    ref = x.bfloat16().float().numpy()
    np.testing.assert_array_equal(mo.bf16_round(x.numpy()), ref)
    bits = mo.to_bf16_bits(x.numpy())
    np.testing.assert_array_equal(mo.from_bf16_bits(bits), ref)


def test_e4m3_codec_matches_torch():
    """Decode table, round-to-nearest-even on every midpoint, saturation: against torch's CPU float8_e4m3fn casts."""
    torch = pytest.importorskip("torch")
    table = mo.e4m3_table()
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy().astype(np.float64)
    np.testing.assert_array_equal(np.isnan(table), np.isnan(ref))
    np.testing.assert_array_equal(table[~np.isnan(table)], ref[~np.isnan(ref)])
    rng = np.random.default_rng(3)
    x = np.clip(rng.standard_normal(100000) * rng.choice([1e-3, 0.1, 1.0, 30.0, 200.0], 100000), -448, 448).astype(np.float32)
    mids = np.array([(table[i] + table[i + 1]) / 2 for i in range(0x7E)], dtype=np.float32)
    for v in (x, mids, -mids, np.array([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10], dtype=np.float32)):
        want = torch.from_numpy(v).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        np.testing.assert_array_equal(mo.quantize_e4m3(v), want)
    np.testing.assert_array_equal(mo.quantize_e4m3(np.array([1e9, -1e9], dtype=np.float32)), [0x7E, 0xFE])
    codes = mo.quantize_e4m3(x[:64 * 48].reshape(64, 48))
    a = torch.from_numpy(codes).view(torch.float8_e4m3fn).double()
    np.testing.assert_allclose(mo.matmul_e4m3(codes, codes[:32], 0.5), (0.5 * a @ a[:32].T).float().numpy(), rtol=1e-6)


def test_known_answers_verify_autograd():
    """verify/verify_autograd.py and the C++ KATs (autograd/tests/test_matmul.cpp:22-34, test_softmax.cpp:25-35,
    test_relu.cpp, test_linear.cpp, test_sgd.cpp:57-70)."""
    gold = load_json("verify_autograd.json")
    assert gold["all_passed"]
    a = np.ones((32, 64), np.float32)
    b = np.ones((64, 32), np.float32)
    c = mo.matmul(a, b)
    assert np.all(c == gold["matmul"]["C"]) and gold["matmul"]["C"] == 64.0
    d_a, d_b = mo.matmul_backward(a, b, np.ones_like(c))
    assert np.all(d_a == gold["matmul"]["dA"]) and np.all(d_b == gold["matmul"]["dB"])
    x = np.ones((32, 32), np.float32)
    assert np.all(mo.relu(x) == gold["relu"]["y"])
    assert np.all(mo.relu_backward(np.ones_like(x), x) == gold["relu"]["dx"])
    xs = np.ones((32, 64), np.float32)
    y = mo.softmax(xs)
    np.testing.assert_allclose(y, gold["softmax"]["y"], rtol=0, atol=1e-7)
    np.testing.assert_allclose(mo.softmax_backward(np.ones_like(y), y), gold["softmax"]["dx"], atol=1e-6)
    w = np.full((32, 64), 0.1, np.float32)
    bias = np.zeros(32, np.float32)
    yl = mo.linear_forward(np.ones((32, 64), np.float32), w, bias)
    np.testing.assert_allclose(yl, gold["linear"]["y"], atol=1e-4)
    _, _, d_bias = mo.linear_backward(np.ones((32, 64), np.float32), w, np.ones_like(yl))
    assert np.all(d_bias == gold["linear"]["dBias"])
    b1 = mo.sgd_update(bias, d_bias, gold["sgd"]["lr"])
    b2 = mo.sgd_update(b1, d_bias, gold["sgd"]["lr"])
    np.testing.assert_allclose(b1, gold["sgd"]["bias_after_1"], atol=1e-6)
    np.testing.assert_allclose(b2, gold["sgd"]["bias_after_2"], atol=1e-6)


def _const_mlp(cfg):
    w1 = np.full((cfg["hidden"], cfg["in"]), cfg["init"], np.float32)
    w2 = np.full((cfg["out"], cfg["hidden"]), cfg["init"], np.float32)
    b1 = np.zeros(cfg["hidden"], np.float32)
    b2 = np.zeros(cfg["out"], np.float32)
    x = np.full((cfg["batch"], cfg["in"]), cfg["x"], np.float32)
    t = np.full((cfg["batch"], cfg["out"]), cfg["target"], np.float32)
    return x, t, (w1, b1, w2, b2)


def test_mlp_trajectory_verify_mlp():
    gold = load_json("verify_mlp.json")
    cfg = gold["config"]
    x, t, params = _const_mlp(cfg)
    out, _ = mo.mlp_forward(x, *params)
    assert abs(mo.mse_loss(out, t)[0] - gold["initial_loss"]) < 2e-6
    for step in range(cfg["steps"]):
        _, params, grads = mo.mlp_train_step(x, t, params, cfg["lr"], "mse")
        if step == 0:
            g = gold["step1_grads"]
            assert abs(grads[0][0, 0] - g["dW1_00"]) < 2e-6
            assert abs(grads[2][0, 0] - g["dW2_00"]) < 2e-6
            assert abs(grads[1][0] - g["db1_0"]) < 2e-6
            assert abs(grads[3][0] - g["db2_0"]) < 2e-6
        out, _ = mo.mlp_forward(x, *params)
        assert abs(mo.mse_loss(out, t)[0] - gold["loss_after_step"][step]) < 2e-6
        assert abs(params[0][0, 0] - gold["W1_00_after_step"][step]) < 2e-6
        assert abs(params[2][0, 0] - gold["W2_00_after_step"][step]) < 2e-6


def test_mlp_trajectory_verify_comparison_fp32_and_bf16():
    """fp32 run, and the bf16 run whose 159.390625 -> 0.000244 is also hard-coded in
    examples/train_mlp_traced.cpp:184-185."""
    gold = load_json("verify_comparison.json")
    cfg = gold["config"]
    for key, quant, tol in (("fp32", None, 2e-4), ("bf16", mo.bf16_round, 0.0)):
        x, t, params = _const_mlp(cfg)
        if quant:
            params = tuple(quant(p) for p in params)
        g = gold[key]
        for step in range(cfg["steps"]):
            loss, params, grads = mo.mlp_train_step(x, t, params, cfg["lr"], "mse", quantize=quant)
            ref = g["loss_before"][step]
            assert abs(loss - ref) <= max(tol * max(1.0, abs(ref)), 5e-7), (key, step, loss, ref)
            if step == 0:
                sg = g["step0_grads"]
                for got, name in ((grads[0][0, 0], "dW1_00"), (grads[2][0, 0], "dW2_00"), (grads[1][0], "db1_0"),
                                  (grads[3][0], "db2_0")):
                    assert abs(got - sg[name]) <= 1e-3 * abs(sg[name]) + 1e-6, (key, name, got, sg[name])
        out, _ = mo.mlp_forward(x, *params)
        final = mo.mse_loss(quant(out) if quant else out, t)[0]
        assert abs(final - g["loss_after"][-1]) <= max(tol, 5e-7), (key, final)


def test_mlp_cross_entropy_784_128_10():
    z = np.load(GOLDEN / "mlp_ce_784_128_10.npz")
    params = (z["w1_0"], z["b1_0"], z["w2_0"], z["b2_0"])
    for step in range(10):
        loss, params, grads = mo.mlp_train_step(z["x"], z["labels"], params, float(z["lr"]), "ce")
        assert abs(loss - z["losses"][step]) <= 1e-5 * abs(z["losses"][step]), (step, loss)
        if step == 0:
            for got, name in zip(grads, ("dw1_0", "db1_0", "dw2_0", "db2_0")):
                assert mo.rel_frobenius(got, z[name]) < 1e-5, name
    for got, name in zip(params, ("w1_10", "b1_10", "w2_10", "b2_10")):
        assert mo.rel_frobenius(got, z[name]) < 1e-5, name


def test_adam_two_steps():
    z = np.load(GOLDEN / "adam_two_step.npz")
    kw = dict(lr=float(z["lr"]), beta1=float(z["beta1"]), beta2=float(z["beta2"]), eps=float(z["eps"]))
    w1, m1, v1 = mo.adam_update(z["w0"], z["g1"], np.zeros_like(z["w0"]), np.zeros_like(z["w0"]), 1, **kw)
    w2, m2, v2 = mo.adam_update(w1, z["g2"], m1, v1, 2, **kw)
    for got, name in ((w1, "w1"), (m1, "m1"), (v1, "v1"), (w2, "w2"), (m2, "m2"), (v2, "v2")):
        np.testing.assert_allclose(got, z[name], rtol=2e-5, atol=1e-7, err_msg=name)


def _block_weights(z):
    return {k[2:]: z[k] for k in z.files if k.startswith("p_")}


def test_transformer_block_forward_backward():
    z = np.load(GOLDEN / "block_small.npz")
    w = _block_weights(z)
    heads = int(z["heads"])
    out, cache = mo.transformer_block_forward(z["x"], w, heads)
    assert mo.rel_frobenius(out, z["out"]) < 1e-5
    d_x, grads = mo.transformer_block_backward(z["d_out"], w, cache, heads)
    assert mo.rel_frobenius(d_x, z["d_x"]) < 1e-4
    for k, g in grads.items():
        ref = z["g_" + k]
        if np.linalg.norm(ref) < 1e-5:  # the key bias has no effect on a softmax over keys: gradient is rounding noise
            assert np.linalg.norm(g) < 1e-5, k
        else:
            assert mo.rel_frobenius(g, ref) < 1e-4, k


def test_transformer_block_reference_setting_constant_weights():
    """The setting verify/compare_grads.py::run_pytorch_reference uses: constant 0.02 weights, MSE against zeros."""
    z = np.load(GOLDEN / "block_const.npz")
    b, s, d = z["x"].shape
    init = float(z["init"])
    w = {}
    for k, shape in (("wq", (d, d)), ("wk", (d, d)), ("wv", (d, d)), ("wo", (d, d)), ("w1", (4 * d, d)), ("w2", (d, 4 * d))):
        w[k] = np.full(shape, init, np.float32)
    for k, n in (("bq", d), ("bk", d), ("bv", d), ("bo", d), ("b1", 4 * d), ("b2", d), ("ln1_b", d), ("ln2_b", d)):
        w[k] = np.zeros(n, np.float32)
    # init_weights_uniform fills every parameter whose name contains "weight", LayerNorm gains included
    w["ln1_g"] = np.full(d, init, np.float32)
    w["ln2_g"] = np.full(d, init, np.float32)
    heads = int(z["heads"])
    out, cache = mo.transformer_block_forward(z["x"], w, heads)
    assert mo.rel_frobenius(out, z["out"]) < 1e-5
    loss, d_out = mo.mse_loss(out, np.zeros_like(out))
    assert abs(loss - float(z["loss"])) < 1e-6 * max(1.0, abs(float(z["loss"])))
    d_x, grads = mo.transformer_block_backward(d_out, w, cache, heads)
    assert mo.rel_frobenius(d_x, z["d_x"]) < 1e-4
    for k, g in grads.items():
        ref = z["g_" + k]
        if np.linalg.norm(ref) < 1e-9:
            assert np.linalg.norm(g) < 1e-6, k
        else:
            assert mo.rel_frobenius(g, ref) < 2e-3, k


def test_tiny_transformer_cross_entropy_and_adam():
    """experiment_torch.py: logits -> cross-entropy on the answer token -> Adam; checks the oracle's CE (loss and
    d_logits through the output projection) and three Adam steps on every parameter."""
    z = np.load(GOLDEN / "tiny_transformer_adam.npz")
    pos = int(z["answer_pos"])
    logits = z["logits0"][:, pos, :]
    loss, d_logits = mo.cross_entropy(logits, z["targets"])
    assert abs(loss - z["losses"][0]) < 1e-5
    # d(out.weight) = d_logits^T . h where logits = h . W^T; recover h by least squares is overkill: use the
    # identity sum(d_W * W) = sum(d_logits * logits) (both equal the directional derivative along W).
    w_out = z["p0/out.weight"]
    g_out = z["g0/out.weight"]
    assert abs(float((g_out * w_out).sum()) - float((d_logits * logits).sum())) < 1e-5


def test_sharded_matmul_algebra():
    rng = np.random.default_rng(0)
    a = mo.bf16_round(rng.standard_normal((48, 64)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((64, 80)).astype(np.float32))
    full = mo.matmul(a, b)
    for g in (2, 4, 8):
        c, shards = mo.column_parallel_matmul(a, b, g)
        # each column is computed by exactly one rank; only the BLAS blocking (hence fp32 summation order) differs
        assert mo.rel_frobenius(c, full) < 1e-6
        np.testing.assert_array_equal(mo.bf16_round(c)[:, :4], mo.bf16_round(shards[0])[:, :4])
        assert len(shards) == g and shards[0].shape == (48, 80 // g)
        c2, blocks = mo.row_parallel_matmul(a, b, g)
        assert mo.rel_frobenius(c2, full) < 1e-6
        assert len(blocks) == g and blocks[0].shape == (48 // g, 80)


def test_softmax_logsoftmax_and_edge_cases():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 7, 33)).astype(np.float32) * 4
    y = mo.softmax(x)
    np.testing.assert_allclose(y.sum(-1), 1.0, atol=1e-6)
    np.testing.assert_allclose(np.exp(mo.log_softmax(x)), y, atol=1e-6)
    d = rng.standard_normal(x.shape).astype(np.float32)
    # log-softmax backward is softmax backward composed with d/dy log(y)
    np.testing.assert_allclose(mo.log_softmax_backward(d, mo.log_softmax(x)), mo.softmax_backward(d / y, y), atol=2e-4)
    # empty and ragged products
    assert mo.matmul(np.zeros((0, 8), np.float32), np.zeros((8, 4), np.float32)).shape == (0, 4)
    assert np.all(mo.matmul(np.zeros((3, 0), np.float32), np.zeros((0, 4), np.float32)) == 0)
    q = rng.standard_normal((2, 3, 8, 4)).astype(np.float32)
    o, p = mo.causal_attention_forward(q, q, q)
    assert np.allclose(np.triu(p, 1), 0) and np.allclose(p.sum(-1), 1, atol=1e-6)
    np.testing.assert_allclose(o[..., 0, :], q[..., 0, :], atol=1e-6)  # first query sees only itself


def _ones_layer_stack(case):
    b, s_, d, h, layers, mult = (case[k] for k in ("batch", "seq", "dim", "heads", "layers", "ffn_mult"))
    x = np.ones((b, s_, d), np.float32)

    def w(rows, cols):
        return np.full((rows, cols), 0.01, np.float32)

    for _ in range(layers):
        x = mo.simple_transformer_layer_forward(x, w(d, d), w(d, d), w(d, d), w(d, d), w(d, mult * d), w(mult * d, d), h)
    return x


def test_simple_transformer_layer_matches_the_compiled_reference_program():
    """bench/autograd/bench_transformer_torch.cpp, compiled unchanged against libtorch (oracle/build_ref.py), printed
    the values in tests/golden/bench_transformer_torch.json; the oracle's restatement of its layer reproduces them to
    the six digits the program prints. When the binary is present it is also run once, live, against the fixture."""
    gold = load_json("bench_transformer_torch.json")
    for case in gold["cases"]:
        y = _ones_layer_stack(case)
        assert list(y.shape) == case["output_shape"]
        np.testing.assert_allclose(y[0, 0, :3], case["first_values"], rtol=2e-6)
    from oracle import build_ref
    if build_ref.BINARY.exists():
        case = gold["cases"][1]
        live = build_ref.run(case["batch"], case["seq"], case["dim"], case["heads"], case["layers"], case["ffn_mult"])
        assert live["first_values"] == case["first_values"] and live["output_shape"] == case["output_shape"]

