#!/usr/bin/env python3
"""Times the bandwidth-bound kernels of the hot path (softmax family, cross-entropy, LayerNorm with and without the
fused residual add, element-wise, reductions, embedding, SGD / Adam) and the fused attention kernels at the GPT-2-small
training shapes and reports achieved HBM GB/s against the measured copy bandwidth (for the attention kernels, which
are not HBM-bound, the GB/s column only says how little memory traffic they need).

    python tt-perf_b200/kernel_bench.py [--only NAME] [--iters 20] [--json]

"Algorithmic bytes" = every operand read once + every result written once at its storage type. Inputs are larger
than the 126 MiB L2 (LayerNorm and the [T, D] element-wise ops use 16x the GPT-2 token count for that reason; the
kernels are row-independent, so the per-row figures carry over). Timing: CUDA events on the stream around `iters`
back-to-back launches after 3 warm-up launches."""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent.parent


def load_pkg():
    spec = importlib.util.spec_from_file_location("__graft_entry__", REPO / "__graft_entry__.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.load_package()


def hbm_peak() -> tuple[float, str]:
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    pkg = load_pkg()
    c = pkg.capi
    ctx = pkg.Context(0)
    DT = pkg.DeviceTensor
    rng = np.random.default_rng(0)

    def rand(shape, dtype=pkg.BF16, scale=1.0):
        t = DT(ctx, shape, dtype)
        # fill on the device: a uniform value is enough for bandwidth, but softmax-like kernels get a ramp via two fills
        ctx.fill(t, t.numel, dtype, scale)
        return t

    B, H, S, D, V, T = 8, 12, 1024, 768, 50257, 8192
    Vp = (V + 7) // 8 * 8
    T16 = 16 * T
    cases = []

    def case(name, nbytes, fn, flops=None):
        cases.append((name, nbytes, fn, flops))

    # the matmul cases at the end allocate their own operands; a run restricted to them skips everything else
    if not (args.only and args.only.startswith("gemm ")):
        rows = B * H * S
        x_s, y_s, d_s = rand((rows, S)), DT(ctx, (rows, S)), rand((rows, S), scale=0.01)
        case("softmax_fwd_causal [B*H*S, S]", rows * S * 4, lambda: ctx.softmax(x_s, y_s, rows, S, alpha=0.125, causal_period=S))
        case("softmax_bwd [B*H*S, S]", rows * S * 6, lambda: ctx.softmax_backward(d_s, y_s, x_s, rows, S, alpha=0.125))
        logits = rand((T, Vp), scale=0.5)
        dlog = DT(ctx, (T, Vp))
        labels = DT.from_numpy(ctx, rng.integers(0, V, T).astype(np.uint32), pkg.U32)
        loss = DT(ctx, (1,), pkg.F32)
        case("cross_entropy fwd+bwd [T, 50257]", T * V * 4 + T * 4,
             lambda: ctx.cross_entropy(logits, labels, T, V, ld=Vp, loss_sum=loss, d_logits=dlog, ldd=Vp))
        case("log_softmax [T, 50257] (ld 50264)", T * V * 4, lambda: lib_log_softmax(ctx, c, logits, dlog, T, V, Vp))
        xl, yl, dyl = rand((T16, D)), DT(ctx, (T16, D)), rand((T16, D), scale=0.1)
        gam, bet = rand((D,)), rand((D,), scale=0.0)
        mean, rstd = DT(ctx, (T16,), pkg.F32), DT(ctx, (T16,), pkg.F32)
        dg, db = DT(ctx, (D,), pkg.F32), DT(ctx, (D,), pkg.F32)
        case("layernorm_fwd [16T, 768]", T16 * D * 4 + T16 * 8, lambda: ctx.layernorm_forward(xl, gam, bet, yl, mean, rstd, T16, D))
        case("layernorm_bwd dx+dgamma+dbeta [16T, 768]", T16 * D * (6 + 4) + T16 * 8,
             lambda: ctx.layernorm_backward(dyl, xl, gam, mean, rstd, yl, dg, db, T16, D))
        res_l, sum_l = rand((T16, D), scale=0.1), DT(ctx, (T16, D))
        case("add + layernorm_fwd [16T, 768]", T16 * D * 8 + T16 * 8,
             lambda: ctx.add_layernorm_forward(xl, res_l, sum_l, gam, bet, yl, mean, rstd, T16, D))
        case("layernorm_bwd + residual add [16T, 768]", T16 * D * (8 + 4) + T16 * 8,
             lambda: ctx.layernorm_backward_add(dyl, xl, gam, mean, rstd, res_l, yl, dg, db, T16, D))
        case("add [16T, 768] (residual)", T16 * D * 6, lambda: ctx.binary(c.B_ADD, xl, (T16, D), dyl, (T16, D), yl))
        case("bias add [16T, 768] + [1, 768]", T16 * D * 4, lambda: ctx.binary(c.B_ADD, xl, (T16, D), gam, (1, D), yl))
        case("gelu [16T, 768]", T16 * D * 4, lambda: ctx.unary(c.U_GELU, xl, yl, T16 * D))
        case("gelu_bw [16T, 768]", T16 * D * 6, lambda: ctx.binary(c.B_GELU_BW, dyl, (T16 * D,), xl, (T16 * D,), yl))
        case("gelu_bw + column sums of dx [16T, 768] (one pass)", T16 * D * 6,
             lambda: ctx.gelu_backward(dyl, xl, yl, gam, T16, D))
        case("column sum (bias grad) [16T, 768] -> [768]", T16 * D * 2, lambda: ctx.reduce(c.R_SUM, xl, 1, T16, D, gam))
        case("mean over all [16T*768] -> [1]", T16 * D * 2, lambda: ctx.reduce(c.R_MEAN, xl, 1, T16 * D, 1, gam))
        xh = rand((16 * B, S, H, 64))
        yh = DT(ctx, (16 * B, H, S, 64))
        case("head split permute [16B, S, H, 64] -> [16B, H, S, 64]", xh.numel * 4,
             lambda: ctx.permute(xh, (16 * B, S, H, 64), (0, 2, 1, 3), yh))
        table = rand((V, D))
        ids = DT.from_numpy(ctx, rng.integers(0, V, T16).astype(np.uint32), pkg.U32)
        case("embedding gather [16T] x [50257, 768]", T16 * D * 4 + T16 * 4, lambda: ctx.embedding_forward(ids, T16, table, V, D, yl))
        n_par = 163_037_184
        p_, g_ = rand((n_par,), scale=0.02), rand((n_par,), scale=1e-3)
        m_, v_ = DT.zeros(ctx, (n_par,), pkg.F32), DT.zeros(ctx, (n_par,), pkg.F32)
        case("adam 163M params (bf16 p, g; fp32 m, v): 22 B/param", n_par * 22,
             lambda: ctx.adam_step([p_], [g_], [m_], [v_], [n_par], 1, lr=3e-4, beta1=0.9, beta2=0.95))
        case("sgd 163M params (bf16 p, g): 6 B/param", n_par * 6, lambda: ctx.sgd_step([p_], [g_], [n_par], 0.01))

        # fused attention at the GPT-2-small shape: q, k, v read in place from a stacked [B, S, 3D] projection output
        qkv_a, o_a, do_a, dqkv_a = rand((B, S, 3 * D), scale=0.5), DT(ctx, (B, S, D)), rand((B, S, D), scale=0.1), DT(ctx, (B, S, 3 * D))
        lse_a = DT(ctx, (B, H, S), pkg.F32)
        op3 = [ctx.attn_operand(qkv_a, S * 3 * D, 64, 3 * D, offset=i * D) for i in range(3)]
        dop3 = [ctx.attn_operand(dqkv_a, S * 3 * D, 64, 3 * D, offset=i * D) for i in range(3)]
        o_op, do_op = ctx.attn_operand(o_a, S * D, 64, D), ctx.attn_operand(do_a, S * D, 64, D)
        case("attention_fwd causal [B8, H12, S1024, 64]", B * S * D * 2 * 4 + B * H * S * 4,
             lambda: ctx.attention_forward(op3[0], op3[1], op3[2], o_op, lse_a, B, H, S))
        case("attention_bwd causal [B8, H12, S1024, 64]", B * S * D * 2 * 8 + B * H * S * 4,
             lambda: ctx.attention_backward(op3[0], op3[1], op3[2], o_op, do_op, lse_a, dop3[0], dop3[1], dop3[2], B, H, S))

    # 8-bit (e4m3) operands: quantisation kernels and the matmul beside its bf16 form (x . W^T, bf16 output)
    if not (args.only and args.only.startswith("gemm ")):
        q8 = DT(ctx, (T16 * D,), pkg.FP8_E4M3)
        amax = DT(ctx, (1,), pkg.F32)
        case("absmax [16T, 768]", T16 * D * 2, lambda: ctx.absmax(xl, T16 * D, amax))
        case("quantize_fp8 [16T, 768]", T16 * D * 3, lambda: ctx.quantize_fp8(xl, T16 * D, 2.0, q8))
    for (gm, gn, gk) in ((8192, 8192, 8192), (4096, 4096, 4096), (8192, 3072, 768), (8192, 768, 3072)):
        names = (f"gemm bf16 x.W^T {gm}x{gn}x{gk}", f"gemm fp8 e4m3 x.W^T {gm}x{gn}x{gk}")
        if args.only and not any(args.only in n for n in names):
            continue
        # random operands: a matmul of constants toggles few bits, draws less power and clocks higher than real data
        a16 = DT.from_numpy(ctx, rng.standard_normal((gm, gk), dtype=np.float32))
        b16 = DT.from_numpy(ctx, rng.standard_normal((gn, gk), dtype=np.float32))
        c16 = DT(ctx, (gm, gn))
        a8, b8 = DT(ctx, (gm, gk), pkg.FP8_E4M3), DT(ctx, (gn, gk), pkg.FP8_E4M3)
        ctx.quantize_fp8(a16, gm * gk, 1.0, a8)
        ctx.quantize_fp8(b16, gn * gk, 1.0, b8)
        d16 = ctx.gemm_desc(a16, b16, c16, gm, gn, gk, transpose_b=True)
        d8 = ctx.gemm_desc(a8, b8, c16, gm, gn, gk, transpose_b=True, ab_dtype=pkg.FP8_E4M3)
        case(names[0], (gm * gk + gn * gk + gm * gn) * 2, lambda d=d16: ctx.gemm(d), 2.0 * gm * gn * gk)
        case(names[1], gm * gk + gn * gk + gm * gn * 2, lambda d=d8: ctx.gemm(d), 2.0 * gm * gn * gk)

    peak, peak_src = hbm_peak()
    results = []
    for name, nbytes, fn, flops in cases:
        if args.only and args.only not in name:
            continue
        for _ in range(3):
            fn()
        ctx.synchronize()
        t = ctx.timer_start()
        for _ in range(args.iters):
            fn()
        ms = ctx.timer_stop(t) / args.iters
        gbs = nbytes / (ms * 1e-3) / 1e9
        results.append({"kernel": name, "ms": ms, "algorithmic_bytes": nbytes, "gb_per_s": gbs, "frac_of_hbm_peak": gbs / peak})
        if flops:
            results[-1]["tflops"] = flops / (ms * 1e-3) / 1e12
    if args.json:
        print(json.dumps({"hbm_peak_gbs": peak, "peak_source": peak_src, "results": results}))
    else:
        print(f"HBM peak {peak:.0f} GB/s ({peak_src})")
        for r in results:
            tail = f"  {r['tflops']:7.0f} TFLOP/s" if "tflops" in r else ""
            print(f"{r['kernel']:58s} {r['ms']*1e3:9.1f} us  {r['gb_per_s']:8.0f} GB/s  {100*r['frac_of_hbm_peak']:5.1f} %{tail}")
    ctx.close()


def lib_log_softmax(ctx, c, x, y, rows, cols, ld):
    c.check(c.lib().b200_log_softmax(ctx.handle, c.ptr(x), ld, c.ptr(y), ld, rows, cols, None))


if __name__ == "__main__":
    main()
