"""Operand-precision study of a 2-layer MLP training step: loss drift against step time.

The reference trains Linear -> ReLU -> Linear with MSE and SGD under three TT math fidelities and prints the loss of
each after every step next to the HiFi4 one, then the average step time of each (verify/verify_fidelity.cpp:31-127
the model, :130-208 the protocol: batch 512, 8192 -> 4096 -> 2048, lr 0.1, 10 recorded steps, then 2 warm-up and 20
timed steps). This script runs the same protocol over the C ABI with four levels:

    HiFi4, HiFi2, LoFi   bf16 operands; the library's fidelity knob (rounding of split-K partial sums, tanh GELU)
    FP8                  e4m3 operands with one scale per tensor (448 / max|x|) for all five matmuls of the step:
                         y = x.W^T reads x and W as stored; dX = dY.W and dW = dY^T.X read transposed 8-bit copies,
                         because 8-bit operands reach the tensor cores K-major only

`--init constant` is the reference's setting (every tensor a constant, verify_fidelity.cpp:60-63, 142-144): a constant
tensor quantises exactly, so it isolates accumulation effects. `--init random` (seeded) shows the drift real data gives.

    python tt-perf_b200/fidelity_sweep.py [--init constant|random] [--batch 512] [--dims 8192 4096 2048] [--json]
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import math
import pathlib
import sys

import numpy as np

LEVELS = ("HiFi4", "HiFi2", "LoFi", "FP8")


def load_pkg():
    here = pathlib.Path(__file__).resolve().parent
    spec = importlib.util.spec_from_file_location("ttperf_b200", here / "__init__.py", submodule_search_locations=[str(here)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ttperf_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


class FidelityMLP:
    """Weights are kept [out, in] (ttnn::linear's layout), biases [out]; everything bf16 on the device."""

    def __init__(self, pkg, ctx, level, w1, b1, w2, b2, lr):
        self.pkg, self.ctx, self.level, self.lr = pkg, ctx, level, lr
        DT = pkg.DeviceTensor
        self.params = [DT.from_numpy(ctx, p) for p in (w1, b1, w2, b2)]
        self.fid = {"HiFi4": pkg.HIFI4, "HiFi2": pkg.HIFI2, "LoFi": pkg.LOFI, "FP8": pkg.HIFI4}[level]
        # FP8 scales per tensor role. calibrate = True: each quantisation measures max|x| first (a reduction and a host
        # read) and remembers the scale; False: the remembered scale is reused, nothing waits on the host ("delayed
        # scaling"; values that outgrew it saturate at +-448).
        self.scales = {}
        self.calibrate = True

    # x . w^T, dy . w, dy^T . x in the level's operand format -------------------------------------------------------
    def _q(self, role, t, transposed=False):
        scale = None if self.calibrate else self.scales[role]
        q, scale = self.pkg.nn.quantize_fp8(self.ctx, t, scale=scale, transposed=transposed)
        self.scales[role] = scale
        return q, scale

    def forward_product(self, role, x, w, bias):
        nn = self.pkg.nn
        if self.level != "FP8":
            return nn.matmul(self.ctx, x, w, False, True, bias=bias, fidelity=self.fid)
        (xq, sx), (wq, sw) = self._q(role + ".x", x), self._q(role + ".w", w)
        return nn.linear_forward_fp8(self.ctx, xq, sx, wq, sw, bias)

    def dx_product(self, role, dy, w):
        nn = self.pkg.nn
        if self.level != "FP8":
            return nn.matmul(self.ctx, dy, w, False, False, fidelity=self.fid)
        (dq, sd), (wtq, sw) = self._q(role + ".dy", dy), self._q(role + ".w", w, transposed=True)
        return nn.linear_forward_fp8(self.ctx, dq, sd, wtq, sw)

    def dw_product(self, role, dy, x):
        nn = self.pkg.nn
        if self.level != "FP8":
            return nn.matmul(self.ctx, dy, x, True, False, fidelity=self.fid)
        (dtq, sd), (xtq, sx) = self._q(role + ".dy", dy, transposed=True), self._q(role + ".x", x, transposed=True)
        return nn.linear_forward_fp8(self.ctx, dtq, sd, xtq, sx)

    # one step ----------------------------------------------------------------------------------------------------------
    def loss_and_cache(self, x, target):
        pkg, ctx, c = self.pkg, self.ctx, self.pkg.capi
        DT = pkg.DeviceTensor
        w1, b1, w2, b2 = self.params
        h_pre = self.forward_product("l1", x, w1, b1)
        h = DT(ctx, h_pre.shape)
        ctx.unary(c.U_RELU, h_pre, h, h.numel)
        pred = self.forward_product("l2", h, w2, b2)
        diff = DT(ctx, pred.shape)
        ctx.binary(c.B_SUB, pred, pred.shape, target, target.shape, diff)
        sq = DT(ctx, pred.shape)
        ctx.unary(c.U_SQUARE, diff, sq, sq.numel)
        loss = DT(ctx, (1,))
        ctx.reduce(c.R_MEAN, sq, 1, sq.numel, 1, loss)
        return loss, (h_pre, h, diff)

    def train_step(self, x, target):
        pkg, ctx, c, nn = self.pkg, self.ctx, self.pkg.capi, self.pkg.nn
        DT = pkg.DeviceTensor
        w1, b1, w2, b2 = self.params
        loss, (h_pre, h, diff) = self.loss_and_cache(x, target)
        d_pred = DT(ctx, diff.shape)
        ctx.unary(c.U_MUL_SCALAR, diff, d_pred, d_pred.numel, scalar=2.0 / diff.numel)
        d_w2 = self.dw_product("l2", d_pred, h)
        d_b2 = DT(ctx, b2.shape)
        ctx.reduce(c.R_SUM, d_pred, 1, d_pred.shape[0], d_pred.shape[1], d_b2)
        d_h = self.dx_product("l2", d_pred, w2)
        d_hpre = nn.relu_backward(ctx, d_h, h_pre)
        d_w1 = self.dw_product("l1", d_hpre, x)
        d_b1 = DT(ctx, b1.shape)
        ctx.reduce(c.R_SUM, d_hpre, 1, d_hpre.shape[0], d_hpre.shape[1], d_b1)
        nn.sgd_step(ctx, self.params, [d_w1, d_b1, d_w2, d_b2], self.lr)
        return loss


def make_problem(init, batch, dims, seed=0):
    d_in, d_hid, d_out = dims
    if init == "constant":
        x = np.full((batch, d_in), 1.0 / math.sqrt(d_in), np.float32)
        target = np.full((batch, d_out), 0.5, np.float32)
        w1, w2 = np.full((d_hid, d_in), 0.001, np.float32), np.full((d_out, d_hid), 0.001, np.float32)
    else:
        rng = np.random.default_rng(seed)
        x = rng.standard_normal((batch, d_in), dtype=np.float32)
        target = 0.5 * rng.standard_normal((batch, d_out), dtype=np.float32)
        w1 = rng.uniform(-1, 1, (d_hid, d_in)).astype(np.float32) / math.sqrt(d_in)
        w2 = rng.uniform(-1, 1, (d_out, d_hid)).astype(np.float32) / math.sqrt(d_hid)
    return x, target, w1, np.zeros(d_hid, np.float32), w2, np.zeros(d_out, np.float32)


def run(pkg, ctx, init="constant", batch=512, dims=(8192, 4096, 2048), lr=0.1, steps=10, warmup=2, timed=20, seed=0,
        levels=LEVELS):
    """Returns {level: {"loss": [steps + 1 values], "ms_per_step": t}}. The recorded steps of the FP8 level scale every
    tensor by its current range; its timed steps reuse the last scales, so that no step waits on the host."""
    DT = pkg.DeviceTensor
    x_h, t_h, w1, b1, w2, b2 = make_problem(init, batch, dims, seed)
    x, target = DT.from_numpy(ctx, x_h), DT.from_numpy(ctx, t_h)
    out = {}
    for level in levels:
        model = FidelityMLP(pkg, ctx, level, w1, b1, w2, b2, lr)
        losses = [float(model.loss_and_cache(x, target)[0].numpy()[0])]
        for _ in range(steps):
            model.train_step(x, target)
            losses.append(float(model.loss_and_cache(x, target)[0].numpy()[0]))
        model.calibrate = False   # the timed steps reuse the scales of the last recorded step
        for _ in range(warmup):
            model.train_step(x, target)
        ctx.synchronize()
        t = ctx.timer_start()
        for _ in range(timed):
            model.train_step(x, target)
        out[level] = {"loss": losses, "ms_per_step": ctx.timer_stop(t) / timed}
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--init", choices=("constant", "random"), default="constant")
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--dims", type=int, nargs=3, default=(8192, 4096, 2048))
    ap.add_argument("--lr", type=float, default=0.1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    pkg = load_pkg()
    ctx = pkg.Context(0)
    res = run(pkg, ctx, args.init, args.batch, tuple(args.dims), args.lr, args.steps)
    if args.json:
        print(json.dumps({"init": args.init, "batch": args.batch, "dims": list(args.dims), "results": res}))
    else:
        print(f"batch {args.batch}, {args.dims[0]} -> {args.dims[1]} -> {args.dims[2]}, lr {args.lr}, init {args.init}")
        print(f"{'step':>5}" + "".join(f"{lv:>13}" for lv in LEVELS) + "".join(f"{lv + ' diff':>12}" for lv in LEVELS[1:]))
        base = res["HiFi4"]["loss"]
        for s in range(args.steps + 1):
            row = f"{s:>5}" + "".join(f"{res[lv]['loss'][s]:>13.6f}" for lv in LEVELS)
            for lv in LEVELS[1:]:
                d = abs(res[lv]["loss"][s] - base[s]) / base[s] * 100 if base[s] else 0.0
                row += f"{d:>11.2f}%"
            print(row)
        for lv in LEVELS:
            t = res[lv]["ms_per_step"]
            print(f"  {lv:6s} {t:8.3f} ms/step  ({res['HiFi4']['ms_per_step'] / t:.2f} x HiFi4)")
    ctx.close()


if __name__ == "__main__":
    main()
