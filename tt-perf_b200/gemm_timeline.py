"""Per-tile timeline of the tcgen05 GEMM kernels from clock stamps written inside the kernels.

Needs the development variant of the library (`python tt-perf_b200/build.py --profile`, which compiles the sources with
-DB200_GEMM_PROFILE into lib/libb200ttperf_prof.so); the product build carries no stamps. For the first 8 tiles of a
few CTAs it prints, in SM clocks from the CTA's start: when the MMA warp issued the tile's first and last MMA, when the
epilogue began (the accumulator was complete) and when epilogue warps 2..5 finished (all four of the single-CTA kernel;
in the CTA-pair kernel the four that take the first half of the columns). For the CTA-pair kernel the two CTAs of a
pair are listed on one time axis (each CTA's clock is taken right after the cluster-wide start-up barrier).

    python tt-perf_b200/gemm_timeline.py --m 8192 --n 3072 --k 768 [--ta] [--tb] [--kernel single|pair] [--bn 256]
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib.util
import os
import pathlib
import sys

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent


def load_pkg():
    spec = importlib.util.spec_from_file_location("ttperf_b200", HERE / "__init__.py", submodule_search_locations=[str(HERE)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ttperf_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--ta", action="store_true", help="A stored [K, M]")
    ap.add_argument("--tb", action="store_true", help="B stored [N, K]")
    ap.add_argument("--kernel", choices=("auto", "single", "pair"), default="auto")
    ap.add_argument("--bn", type=int, default=0, help="tile width of the single-CTA kernel (64, 128, 192, 256)")
    ap.add_argument("--ctas", type=int, nargs="*", default=None, help="CTAs to print (default: 0, 1 and the last two)")
    args = ap.parse_args()

    prof_lib = HERE / "lib" / "libb200ttperf_prof.so"
    if not prof_lib.exists():
        raise SystemExit(f"{prof_lib} is missing: build it with `python tt-perf_b200/build.py --profile`")
    os.environ["B200_TTPERF_LIB"] = str(prof_lib)
    # the tuning switches pin kernel and tile width; they are read by the library at every call
    os.environ["B200_GEMM_TUNE"] = "1"
    if args.kernel == "pair":
        os.environ["B200_GEMM_KERNEL"] = "pair"
    elif args.kernel == "single":
        os.environ["B200_GEMM_2CTA"] = "0"
    if args.bn:
        os.environ["B200_GEMM_BLOCK_N"] = str(args.bn)

    pkg = load_pkg()
    lib = pkg.lib()
    lib.b200_debug_gemm_stamps_prepare.restype = C.c_int
    lib.b200_debug_gemm_stamps_prepare.argtypes = [C.c_void_p]
    lib.b200_debug_gemm_stamps.restype = C.c_int
    lib.b200_debug_gemm_stamps.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    ctx = pkg.Context(0)
    DT = pkg.DeviceTensor
    rng = np.random.default_rng(0)
    M, N, K = args.m, args.n, args.k
    a = DT.from_numpy(ctx, rng.standard_normal((K, M) if args.ta else (M, K), dtype=np.float32))
    b = DT.from_numpy(ctx, rng.standard_normal((N, K) if args.tb else (K, N), dtype=np.float32))
    c = DT(ctx, (M, N))
    d = ctx.gemm_desc(a, b, c, M, N, K, transpose_a=args.ta, transpose_b=args.tb, algo=pkg.ALGO_TCGEN05, split_k=1)
    for _ in range(3):
        ctx.gemm(d)
    ctx.synchronize()
    pkg.capi.check(lib.b200_debug_gemm_stamps_prepare(ctx._h))
    t = ctx.timer_start()
    ctx.gemm(d)
    ms = ctx.timer_stop(t)
    sms = ctx.sm_count
    host = np.zeros(sms * 64, dtype=np.int64)
    pkg.capi.check(lib.b200_debug_gemm_stamps(ctx._h, host.ctypes.data, host.size))
    st = host.reshape(sms, 8, 8)
    pair = bool((st[1::2, :, 0] == 0).all() and (st[1, :, 2] != 0).any())   # odd CTAs of a pair issue no MMAs
    print(f"{M} x {N} x {K}  ta={int(args.ta)} tb={int(args.tb)}  kernel: {'CTA pair' if pair else 'single CTA'}  "
          f"{ms * 1e3:.1f} us for the stamped launch")
    ctas = args.ctas if args.ctas else [0, 1, sms - 2, sms - 1]
    for cta in ctas:
        base = st[cta, 0, 7]
        if base == 0:
            print(f"cta {cta}: no stamps (CTA not launched)")
            continue
        print(f"cta {cta}" + (f" ({'leader' if cta % 2 == 0 else 'peer'} of pair {cta // 2})" if pair else ""))
        prev_end = None
        for slot in range(8):
            row = st[cta, slot]
            if row[2] == 0:
                break
            rel = [int(v - base) if v else None for v in row[:7]]
            ends = [v for v in rel[3:7] if v is not None]
            line = f"  tile {slot}:"
            if rel[0] is not None:
                gap = f" (+{rel[0] - prev_end} after the last issue)" if prev_end is not None else ""
                line += f" mma issue {rel[0]}..{rel[1]} = {rel[1] - rel[0]} clk{gap};"
                prev_end = rel[1]
            line += f" epilogue from {rel[2]}, warps done at {ends} ({max(ends) - rel[2]} clk)"
            print(line)
    ctx.close()


if __name__ == "__main__":
    main()
