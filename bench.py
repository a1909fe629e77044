#!/usr/bin/env python3
"""Benchmark of the dense-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1   one bf16 GEMM C = A.B with M = N = K = 8192 per step (the shape the headline metric is quoted on),
        inputs resident in HBM, through the C ABI (b200_gemm). Extra objects on the same line: `sustained` (the
        same product looped for seconds under the power cap), `sweep` (the matmul sweep's other shapes:
        512^3 .. 16384^3 and the HBM-bound 128 x 8192 x 8192), `gpt2_small_train` (the GPT-2-small step).
N > 1   launched by torchrun, one rank per GPU: the distributed matmul M = N = K = 16384 with B split on N
        across the ranks and C all-gathered (scripts/matmul_2dev_distributed.py generalised), strong scaling.
        Extra objects: `reduce_scatter` (the K-split variant of the same product, checked against the N-split
        result), `tp_block` (the tensor-parallel GPT-2-XL-shaped block step, checked against the one-rank run of
        the same library), `gpt2_small_train` (data parallel).

Prints ONE JSON line on rank 0. `value` is whole-job TFLOP/s (2.M.N.K per product, counted once for the
sharded product). `e2e` repeats the measurement with host buffers: pinned host operands -> device, GEMM, C -> host.
`--impl reference` times the reference's CPU path for the same workload (torch CPU fp32 matmul, the baseline
scripts/matmul_sweep.py:84-108 uses) on a bounded slab of rows.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum of one 8192^3 launch of the CTA-pair kernel, from an ncu capture
# (1.072 GB read + 0.128 GB written).
GEMM_8192_DRAM_TRAFFIC_BYTES = 1.200e9


def load_peaks() -> dict:
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        # one streaming nvidia-smi process: a sample every 100 ms until stop()
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                           "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                          stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        for line in self._proc.stdout:
            if self._stop.is_set():
                break
            if line.strip():
                self.samples.append([c.strip() for c in line.strip().split(",")])

    def start(self):
        self._proc = None
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
        if self._thread:
            self._thread.join(timeout=6)
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class L2Flush:
    """Evicts the 126 MiB L2 between timed iterations by overwriting a 256 MiB device buffer."""

    def __init__(self, ctx):
        self.ctx, self.nbytes = ctx, 2 * 128 * 1024 * 1024
        self.buf = ctx.malloc(self.nbytes)
        self.value = 0

    def __call__(self, stream):
        self.value = (self.value + 1) & 0x7F
        self.ctx.memset(self.buf, self.value, self.nbytes, stream)

    def close(self):
        if self.buf:
            self.ctx.free(self.buf)
            self.buf = 0


def time_each(torch, st, fn, iters, flush=None):
    """Milliseconds of each of `iters` calls of fn(), CUDA events on stream `st`; flush() runs untimed between them."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in evs:
        if flush is not None:
            flush(st.cuda_stream)
        e0.record(st)
        fn()
        e1.record(st)
    torch.cuda.synchronize()
    return [e0.elapsed_time(e1) for e0, e1 in evs]


def sweep_bench(torch, pkg, ctx, st, peaks, quick=False) -> dict:
    """The single-GPU matmul sweep (bench/metal/matmul_sweep.cpp:85, scripts/matmul_inflection.py:63-85, extended to
    the configured sizes): C = A . B, bf16 ~ N(0,1) from seed 42, fp32 accumulate, bf16 out, square M = N = K in
    {512 .. 16384} plus the skinny M = 128, K = N = 8192 product. Two timings per shape:
      isolated      one launch per pair of events with the L2 flushed before it (includes the launch latency, which
                    dominates the small shapes);
      back to back  `reps` launches between one pair of events, each on its own operand set, the sets together larger
                    than 2 x L2 (so no launch finds its operands cached): the per-launch figure a loop of matmuls sees,
                    as the reference's sweep measures (matmul_sweep.cpp:44-79). This is the figure `tflops` and `frac`
                    are computed from.
    Square products are reported against the tensor peak, the skinny one (138.4 MB of algorithmic traffic for 17
    GFLOP) against the HBM copy bandwidth. A row sample of every result is checked against fp32 on the device."""
    s = st.cuda_stream
    flush = L2Flush(ctx)
    shapes = [(n, n, n) for n in (512, 1024, 2048, 4096, 8192, 16384)] + [(128, 8192, 8192)]
    if quick:
        shapes = [(512, 512, 512), (128, 8192, 8192)]
    points = []
    g = torch.Generator(device="cuda").manual_seed(42)
    for M, N, K in shapes:
        set_bytes = 2 * (M * K + K * N + M * N)
        n_sets = max(1, min(128, -(-2 * L2_BYTES // set_bytes)))       # enough sets to exceed 2 x L2 (1 for the big shapes)
        sets = []
        for _ in range(n_sets):
            a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).bfloat16()
            b = torch.randn(K, N, generator=g, device="cuda", dtype=torch.float32).bfloat16()
            c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
            sets.append((a, b, c, ctx.gemm_desc(a, b, c, M, N, K)))
        a, b, c, desc = sets[0]
        plan = ctx.gemm_plan(desc)
        for _ in range(3):
            ctx.gemm(desc, s)
        ctx.synchronize(s)
        iters = 5 if M >= 16384 else 10
        ms_iso = time_each(torch, st, lambda: ctx.gemm(desc, s), iters, flush)
        reps = max(iters, 2 * n_sets)

        def burst():
            for i in range(reps):
                ctx.gemm(sets[i % n_sets][3], s)

        burst()
        ms_b2b = [t / reps for t in time_each(torch, st, burst, 3, flush)]
        rows = torch.arange(0, M, max(1, M // 16), device="cuda")
        for (ai, bi, ci, _) in (sets[0], sets[-1]):
            ref = ai[rows].float() @ bi.float()
            err = ((ci[rows].float() - ref).norm() / ref.norm()).item()
            if not err < 1e-2:
                raise RuntimeError(f"bench sweep: {M}x{N}x{K} fails parity (relative Frobenius error {err:.3e})")
        med = statistics.median(ms_b2b)
        flops, nbytes = 2.0 * M * N * K, 2.0 * (M * K + K * N + M * N)
        tflops, gbs = flops / (med * 1e-3) / 1e12, nbytes / (med * 1e-3) / 1e9
        hbm_bound = M < 512
        points.append({"M": M, "N": N, "K": K, "ms_back_to_back": med, "ms_isolated_median": statistics.median(ms_iso),
                       "ms_isolated_min": min(ms_iso), "operand_sets": n_sets, "launches_per_timing": reps,
                       "tflops": tflops, "gb_per_s": gbs, "bound": "hbm" if hbm_bound else "tensor",
                       "frac": gbs / peaks["hbm_gbs"] if hbm_bound else tflops / peaks["bf16_tflops"],
                       "algorithmic_bytes": nbytes, "kernel": ctx.gemm_plan_text(desc, plan),
                       "parity_sample_rel_frobenius": err})
        del sets, a, b, c
    flush.close()
    return {"what": "matmul sweep; tflops / frac from back-to-back launches on rotating operand sets (> 2 x L2 in total), "
                    "isolated single-launch times (L2 flushed by a 256 MiB overwrite) beside them",
            "peaks": {"tensor_tflops": peaks["bf16_tflops"], "hbm_gbs": peaks["hbm_gbs"], "source": peaks["source"]},
            "points": points}


def sustained_bench(torch, ctx, st, desc, flops, peaks, seconds=2.5) -> dict:
    """The headline product launched back to back for `seconds`: what the kernel holds once the part sits on its
    power cap, against the measured sustained cuBLAS figure."""
    s = st.cuda_stream
    for _ in range(20):
        ctx.gemm(desc, s)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    time.sleep(0.15)
    launches, t_end = 0, time.perf_counter() + seconds
    e0.record(st)
    while time.perf_counter() < t_end:
        for _ in range(50):
            ctx.gemm(desc, s)
        launches += 50
        st.synchronize()            # keeps the queue shallow; 50 launches (tens of ms) between host round trips
    e1.record(st)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    tflops = flops * launches / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"]
    mhz = clocks.get("sm_mhz")
    return {"seconds": ms * 1e-3, "launches": launches, "ms_per_step": ms / launches, "tflops": tflops,
            "peak_sustained_tflops": peak, "frac_of_sustained_peak": tflops / peak, "clocks": clocks,
            "ms_per_step_x_sm_mhz": (ms / launches) * mhz if mhz else None}


def cpu_matmul_baseline(M: int, N: int, K: int, target_s: float = 12.0) -> dict:
    """The reference's CPU path for this workload — torch CPU fp32 matmul on bf16-rounded inputs, as
    scripts/matmul_sweep.py:84-108 times it — on a slab of rows of A sized for about `target_s` seconds."""
    import torch
    if torch.get_num_threads() < (os.cpu_count() or 1):
        torch.set_num_threads(os.cpu_count() or 1)   # torchrun pins OMP_NUM_THREADS=1; the baseline uses every core
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(42)
    rows = min(M, 256)
    b = torch.randn(K, N, generator=g).bfloat16().float()
    a = torch.randn(rows, K, generator=g).bfloat16().float()
    torch.matmul(a, b)  # warm-up
    t0 = time.perf_counter()
    torch.matmul(a, b)
    dt = time.perf_counter() - t0
    rate = 2.0 * rows * N * K / dt
    rows_big = int(min(M, max(rows, (target_s * rate) / (2.0 * N * K))))
    rows_big = max(64, rows_big // 64 * 64)
    a = torch.randn(rows_big, K, generator=g).bfloat16().float()
    reps = max(1, int(round(target_s * rate / (2.0 * rows_big * N * K))))
    t0 = time.perf_counter()
    for _ in range(reps):
        torch.matmul(a, b)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows_big * N * K * reps / dt / 1e12
    return {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
            "sample": f"torch CPU fp32 matmul of a {rows_big}-row slab of A[{M},{K}] against the full B[{K},{N}], "
                      f"{reps} repetitions ({dt:.2f} s, {threads} threads of {os.cpu_count()} cpus)",
            "seconds": dt}


def run_reference_arm(args) -> None:
    """`--impl reference`: the reference's own CPU implementation of the path (torch CPU fp32 matmul) with all
    host threads, each step a bounded slab of the workload. Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    if torch.get_num_threads() < (os.cpu_count() or 1):
        torch.set_num_threads(os.cpu_count() or 1)
    n = args.gpus
    size = 8192 if n == 1 else 16384
    M = N = K = size
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(42)
    b = torch.randn(K, N, generator=g).bfloat16().float()
    probe = torch.randn(128, K, generator=g).bfloat16().float()
    torch.matmul(probe, b)
    t0 = time.perf_counter()
    torch.matmul(probe, b)
    rate = 2.0 * 128 * N * K / (time.perf_counter() - t0)
    total_steps = max(1, args.steps + args.warmup)
    per_step_s = min(10.0, 120.0 / total_steps)
    rows = int(min(M, max(64, per_step_s * rate / (2.0 * N * K))) // 64 * 64) or 64
    a = torch.randn(rows, K, generator=g).bfloat16().float()
    for _ in range(args.warmup):
        torch.matmul(a, b)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch.matmul(a, b)
    dt = time.perf_counter() - t0
    tflops = 2.0 * rows * N * K * args.steps / dt / 1e12
    sample = (f"torch CPU fp32 matmul, {rows}-row slab of A[{M},{K}] x B[{K},{N}] per step, {threads} threads of "
              f"{os.cpu_count()} cpus")
    line = {
        "impl": "reference", "metric": "bf16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": n,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if n > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(n),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n: int) -> dict:
    if n == 1:
        return {"workload": "matmul_sweep M=N=K=8192: C[M,N] = A[M,K] . B[K,N], bf16 in, fp32 accumulate, bf16 out",
                "M": 8192, "N": 8192, "K": 8192, "seed": 42,
                "l2_policy": "inputs (A+B = 256 MiB) larger than the 126 MiB L2; no flush between steps"}
    return {"workload": f"distributed matmul M=N=K=16384, B column-sharded on N across {n} GPUs, all-gather of C",
            "M": 16384, "N": 16384, "K": 16384, "seed": 42, "shards": n,
            "l2_policy": "inputs larger than the 126 MiB L2; no flush between steps"}


def gpt2_train_bench(steps: int = 10, warmup: int = 3, device: int = 0, rank: int = 0, world: int = 1, comm=None) -> dict:
    """GPT-2-small-shaped training step (12 layers, d_model 768, 12 heads, d_ff 3072, seq 1024, batch 8 per GPU, vocab
    50257, random N(0, 0.02) weights, uniform random token ids, Adam lr 3e-4 betas (0.9, 0.95)): forward, cross-entropy,
    backward and the Adam update. Every kernel comes from the C ABI; the host side is tt-perf_b200/nn.py.

    One GPU: the whole step is recorded once as a trace (CUDA graph) and replayed, as the reference's traced executor
    does (bench/autograd/bench_gpt2_full.cpp). N GPUs (data parallel, weak scaling): each rank replays forward +
    backward on its own batch as a chain of traces (LM head, then groups of two blocks, then the embeddings); every trace packs its
    gradients into a bucket that NCCL (b200_comm_allreduce on `comm`, a communicator of this context) averages over
    the ranks on a second stream while the next trace runs; a last trace applies Adam from the buckets. Returns
    whole-job tokens/s and ms/step."""
    import numpy as np
    from __graft_entry__ import load_package
    pkg = load_package()
    ctx = comm.ctx if comm is not None else pkg.Context(device)
    DT = pkg.DeviceTensor
    L, D, H, S, V, B = 12, 768, 12, 1024, 50257, 8
    model = pkg.nn.GPT2(ctx, layers=L, d_model=D, heads=H, seq=S, vocab=V)
    model.init_random(42)                               # same weights on every rank
    rng = np.random.default_rng(42 + rank)              # a different batch per rank
    ids = rng.integers(0, V, (B, S)).astype(np.uint32)
    targets = np.roll(ids, -1, axis=1)
    idd = DT.from_numpy(ctx, ids, pkg.U32)
    tgd = DT.from_numpy(ctx, targets.ravel(), pkg.U32)
    pos = DT.from_numpy(ctx, np.arange(S, dtype=np.uint32), pkg.U32)

    def step():
        loss, grads = model.forward_backward(idd, tgd, pos)
        model.adam_step(grads)
        return loss

    losses = []
    for _ in range(max(2, warmup)):          # eager steps: allocate the pool and scratch, check the loss moves
        losses.append(float(step().numpy()[0]))
    if world == 1:
        tid = ctx.trace_begin()
        loss = step()
        ctx.trace_end(tid)
        ctx.trace_execute(tid)
        ctx.synchronize()
        timer = ctx.timer_start()                       # CUDA events on the context stream
        for _ in range(steps):
            ctx.trace_execute(tid)
        dt = ctx.timer_stop(timer) * 1e-3 / steps
        executor = "trace replay (CUDA graph)"
        traces = [tid]
    else:
        import torch
        # The backward pass is recorded as several traces (LM head, then groups of two blocks, the last one with the
        # embeddings). Each trace ends by packing its gradients into its own bf16 / fp32 bucket; while the next trace
        # runs on the compute stream, the bucket is averaged over the ranks by NCCL on a second stream (events order
        # the two, no host synchronisation). A last trace applies Adam straight from the buckets.
        c = pkg.capi
        specs = []
        SEG = 2   # blocks per backward trace: the last block trace's bucket (all that no later trace hides) stays small
        model.forward_backward(idd, tgd, pos, blocks_per_segment=SEG,
                               segment_hook=lambda pairs: specs.append([(g.numel, g.dtype) for _, g in pairs]))
        ctx.synchronize()
        buckets = []
        for spec in specs:
            offs, n_bf, n_f32 = [], 0, 0
            for numel, dtype in spec:
                if dtype == pkg.BF16:
                    offs.append(n_bf)
                    n_bf += (numel + 7) // 8 * 8
                else:
                    offs.append(n_f32)
                    n_f32 += (numel + 3) // 4 * 4
            buckets.append((DT.zeros(ctx, (max(n_bf, 8),), pkg.BF16), DT.zeros(ctx, (max(n_f32, 4),), pkg.F32), offs, n_bf, n_f32))
        ctx.synchronize()
        slice_of, seg_traces, cur = {}, [], [ctx.trace_begin()]

        def pack_and_cut(pairs):
            flat_bf, flat_f32, offs, _, _ = buckets[len(seg_traces)]
            for (prm, g), off in zip(pairs, offs):
                if g.dtype == pkg.BF16:
                    sl = DT(ctx, g.shape, pkg.BF16, ptr=flat_bf.ptr + 2 * off, owner=flat_bf)
                    ctx.unary(c.U_COPY, g, sl, g.numel)
                else:
                    sl = DT(ctx, g.shape, pkg.F32, ptr=flat_f32.ptr + 4 * off, owner=flat_f32)
                    ctx.unary(c.U_COPY, g, sl, 2 * g.numel)      # a pure copy: fp32 moved as pairs of 16-bit words
                slice_of[id(prm)] = sl
            ctx.trace_end(cur[0])
            seg_traces.append(cur[0])
            if len(seg_traces) < len(specs):
                cur[0] = ctx.trace_begin()

        loss, grads = model.forward_backward(idd, tgd, pos, blocks_per_segment=SEG, segment_hook=pack_and_cut)
        bf, f32 = model._flat(grads)
        # The last bucket holds the token-embedding gradient (fp32, 154 MB), which exists only when the backward pass
        # ends: nothing is left to hide its all-reduce under except the optimiser itself. So Adam runs in two parts:
        # every other parameter as soon as its bucket is averaged, the token embedding after its own all-reduce.
        tok = model.params["tok_emb"]
        split_tok = f32[0][0] is tok and sum(1 for _, dt in specs[-1] if dt == pkg.F32) == 1
        t_opt = ctx.trace_begin()
        model.opt[0].step([slice_of[id(prm)] for prm, _ in bf])
        if split_tok:
            model.opt[1].step([slice_of[id(prm)] for prm, _ in f32[1:]], indices=range(1, len(f32)))
        else:
            model.opt[1].step([slice_of[id(prm)] for prm, _ in f32])
        ctx.trace_end(t_opt)
        t_opt_tok = None
        if split_tok:
            t_opt_tok = ctx.trace_begin()
            model.opt[1].step([slice_of[id(tok)]], indices=[0], advance=False)
            ctx.trace_end(t_opt_tok)
        seg_views = []
        for flat_bf, flat_f32, _, n_bf, n_f32 in buckets:
            v = []
            if n_bf:
                v.append((flat_bf.ptr, n_bf, pkg.BF16))
            if n_f32:
                v.append((flat_f32.ptr, n_f32, pkg.F32))
            seg_views.append(v)
        comp, comm_st = torch.cuda.Stream(), torch.cuda.Stream()

        def dp_step():
            rest_done = None
            for k, (tid, views) in enumerate(zip(seg_traces, seg_views)):
                ctx.trace_execute_on(tid, comp.cuda_stream)
                ev = torch.cuda.Event()
                ev.record(comp)
                comm_st.wait_event(ev)                         # this segment's gradients are packed
                for ptr_, count, dtype in views:
                    if t_opt_tok is not None and k == len(seg_traces) - 1 and dtype == pkg.F32:
                        rest_done = torch.cuda.Event()         # everything but the token embedding is averaged
                        rest_done.record(comm_st)
                    comm.allreduce(ptr_, count, dtype, c.COMM_AVG, stream=comm_st.cuda_stream)
            if rest_done is not None:
                comp.wait_event(rest_done)
                ctx.trace_execute_on(t_opt, comp.cuda_stream)  # runs beside the last all-reduce
                comp.wait_stream(comm_st)
                ctx.trace_execute_on(t_opt_tok, comp.cuda_stream)
            else:
                comp.wait_stream(comm_st)                      # every bucket is averaged before Adam reads it
                ctx.trace_execute_on(t_opt, comp.cuda_stream)

        def rank_barrier():
            comp.synchronize()
            comm.barrier(comp.cuda_stream)
            comp.synchronize()

        ctx.synchronize()
        dp_step()
        rank_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(comp)
        for _ in range(steps):
            dp_step()
        e1.record(comp)
        comp.synchronize()
        dt = max_over_ranks(pkg, comm, e0.elapsed_time(e1) / steps) * 1e-3
        executor = (f"{len(seg_traces)} backward traces on a compute stream, each followed by the NCCL all-reduce of its gradient "
                    "bucket on a second stream (overlapping the next trace), then an Adam trace"
                    + (" beside the all-reduce of the token-embedding gradient and a second one for that parameter" if t_opt_tok is not None else ""))
        traces = seg_traces + [t_opt] + ([t_opt_tok] if t_opt_tok is not None else [])
    final = float(loss.numpy()[0])
    for t in traces:
        ctx.trace_release(t)
    flops = 3 * (12 * 24 * B * S * D * D + 2 * B * S * D * V) + 12 * 12 * B * H * 64 * (S * (S + 1) // 2)
    if comm is None:
        ctx_to_close = ctx
    else:
        ctx_to_close = None
    out = {"metric": "GPT-2-small train tokens/s", "tokens_per_s": world * B * S / dt, "ms_per_step": dt * 1e3,
           "model_tflops_per_s": world * flops / dt / 1e12, "params": model.num_params(), "batch_per_gpu": B, "seq": S,
           "n_gpus": world, "scaling": "weak (data parallel)" if world > 1 else None, "first_losses": losses,
           "loss_after_replays": final, "executor": executor,
           "data": "synthetic: uniform token ids, targets = ids shifted by one"}
    del model, idd, tgd, pos
    if ctx_to_close is not None:
        ctx_to_close.close()
    return out


def max_over_ranks(pkg, comm, value: float) -> float:
    """Largest `value` over the ranks (device-side all-reduce through the communicator)."""
    t = pkg.DeviceTensor.from_numpy(comm.ctx, __import__("numpy").array([value], dtype="float32"), pkg.F32)
    comm.allreduce(t, 1, pkg.F32, pkg.capi.COMM_MAX)
    comm.ctx.synchronize()
    return float(t.numpy()[0])


def run_b200_single(args) -> None:
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    torch.cuda.set_device(0)
    ctx = pkg.Context(0)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s = st.cuda_stream
    M = N = K = 8192
    g = torch.Generator().manual_seed(42)
    a_h = torch.randn(M, K, generator=g).bfloat16().pin_memory()
    b_h = torch.randn(K, N, generator=g).bfloat16().pin_memory()
    c_h = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    a = a_h.cuda(non_blocking=True)
    b = b_h.cuda(non_blocking=True)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    desc = ctx.gemm_desc(a, b, c, M, N, K)
    flops = 2.0 * M * N * K

    for _ in range(max(args.warmup, 3)):
        ctx.gemm(desc, s)
    ctx.synchronize(s)

    sampler = ClockSampler(0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(st)
    for _ in range(args.steps):
        ctx.gemm(desc, s)
    e1.record(st)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # keep the sampler over a region long enough to see clocks under load
    t_end = time.perf_counter() + (0.0 if args.quick else 1.5)
    while time.perf_counter() < t_end:
        for _ in range(20):
            ctx.gemm(desc, s)
        torch.cuda.synchronize()
    clocks = sampler.stop()
    ctx.synchronize(s)
    ms_per_step = ms / args.steps
    tflops = flops / (ms_per_step * 1e-3) / 1e12

    # sanity: the timed kernel really computed the product (a sample of rows against fp32 torch on the device)
    rows = torch.arange(0, M, 257, device="cuda")
    ref = a[rows].float() @ b.float()
    err = ((c[rows].float() - ref).norm() / ref.norm()).item()
    if not err < 1e-2:
        raise RuntimeError(f"bench: GEMM output fails parity (relative Frobenius error {err:.3e})")

    # end to end through the C ABI with host buffers: b200_matmul_host takes pinned host A and B and leaves C in pinned
    # host memory (upload, compute and download pipelined over row panels)
    e2e_steps = max(1, min(args.steps, 5))
    nbytes = M * K * 2
    hdesc = ctx.gemm_desc(a_h, b_h, c_h, M, N, K)
    for _ in range(0 if args.quick else 2):
        ctx.matmul_host(hdesc)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(0 if args.quick else e2e_steps):
        ctx.matmul_host(hdesc)   # returns when C is complete in host memory
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_tflops = flops / e2e_s / 1e12 if not args.quick else 0.0
    if not args.quick:
        ref_rows = a[rows].float() @ b.float()
        err_h = ((c_h[rows.cpu()].float().cuda() - ref_rows).norm() / ref_rows.norm()).item()
        if not err_h < 1e-2:
            raise RuntimeError(f"bench: host-buffer matmul fails parity (relative Frobenius error {err_h:.3e})")

    peaks = load_peaks()
    peak = peaks["bf16_tflops"]
    cpu = cpu_matmul_baseline(M, N, K, 0.2 if args.quick else 12.0)
    cpu.pop("seconds", None)
    line = {
        "metric": "bf16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(1),
        "pct_of_peak": tflops / peak,
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                     "traffic": GEMM_8192_DRAM_TRAFFIC_BYTES if ctx.gemm_plan(desc).kernel == pkg.capi.KERNEL_TCGEN05_PAIR else None,
                     "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json bf16_tflops, burst: kernel timed alone)",
                     "kernel": ctx.gemm_plan_text(desc, ctx.gemm_plan(desc)), "flops_per_launch": flops},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": nbytes,
                "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
        "gpu_launches": args.steps,
        "clocks": clocks,
        "parity_sample_rel_frobenius": err,
    }
    if args.quick:
        line["quick"] = True
        line["e2e"] = None
    else:
        mhz = clocks.get("sm_mhz")
        line["ms_per_step_x_sm_mhz"] = ms_per_step * mhz if mhz else None
        line["sustained"] = sustained_bench(torch, ctx, st, desc, flops, peaks)
        line["sweep"] = sweep_bench(torch, pkg, ctx, st, peaks)
        line["gpt2_small_train"] = gpt2_train_bench()
    print(json.dumps(line), flush=True)
    ctx.close()


def start_ranks(pkg):
    """torchrun's environment -> (rank, world, local device, context, communicator). A gloo group only ships the
    communicator id from rank 0; everything the ranks exchange afterwards goes through b200_comm_* (NCCL)."""
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local_rank)
    dist.init_process_group("gloo")
    ctx = pkg.Context(local_rank)
    box = [pkg.capi.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = pkg.capi.Comm(ctx, box[0], world, rank)
    return rank, world, local_rank, ctx, comm


def reduce_scatter_bench(torch, pkg, ctx, comm, st, a, b_full, c_gathered_ptr, steps, peaks) -> dict:
    """The K-split variant of the distributed matmul: rank r holds A[:, K_r] and B[K_r, :], its fp32 partial tiles go
    from the GEMM epilogue straight into slot r of the row-block owner's staging buffer (peer stores over NVLink, tile
    by tile under the tensor-core work), and after a rank barrier every rank sums its g slots and rounds to bf16 once.
    Checked against the rows this rank owns of the N-split result of the same run."""
    s = st.cuda_stream
    rank, world = comm.rank, comm.world
    M, K = a.shape
    N = b_full.shape[1]
    row = pkg.dist.RowParallelMatmul(ctx, M, N, K, rank, world, comm)
    a_sh = a[:, row.k_offset:row.k_offset + row.k_depth].contiguous()
    b_sh = b_full[row.k_offset:row.k_offset + row.k_depth].contiguous()

    def step():
        row.launch_partials(a_sh, b_sh, s)
        comm.barrier(s)                 # all peers' partial tiles have landed in this rank's slots
        row.launch_reduce(s)
        comm.barrier(s)                 # nobody overwrites slots that a peer is still summing

    for _ in range(3):
        step()
    ctx.synchronize(s)
    comm.barrier(s)
    ctx.synchronize(s)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for _ in range(steps):
        step()
    e1.record(st)
    torch.cuda.synchronize()
    ms = max_over_ranks(pkg, comm, e0.elapsed_time(e1) / steps)
    # parity: this rank's row block against the same rows of the all-gathered C (same inputs, other sharding)
    mine = torch.empty(row.rows, N, dtype=torch.bfloat16, device="cuda")
    ctx.memcpy_d2d(mine, row.out, row.rows * N * 2, s)
    ref = torch.empty(row.rows, N, dtype=torch.bfloat16, device="cuda")
    ctx.memcpy_d2d(ref, c_gathered_ptr + row.row_offset * N * 2, row.rows * N * 2, s)
    ctx.synchronize(s)
    err = ((mine.float() - ref.float()).norm() / ref.float().norm()).item()
    err = max_over_ranks(pkg, comm, err)
    if not err < 1e-2:
        raise RuntimeError(f"bench: K-split result differs from the N-split result (relative Frobenius error {err:.3e})")
    d = ctx.gemm_desc(a_sh, b_sh, None, M, N, row.k_depth, lda=row.k_depth, ldb=N, ldc=N, c_dtype=pkg.F32)
    kernel = ctx.gemm_plan_text(d, ctx.gemm_dist_plan(d, world, True))
    row.close()
    flops = 2.0 * M * N * K
    link_bytes = (world - 1) / world * M * N * 4
    t_compute = flops / world / (peaks["bf16_tflops"] * 1e12)
    t_link = link_bytes / 770e9
    return {"workload": f"distributed matmul M=N=K={M}, A split on K columns and B on K rows across {world} GPUs, fp32 partial "
                        "tiles reduce-scattered from the GEMM epilogue, bf16 cast after the sum",
            "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "steps": steps,
            "nvlink_bytes_sent_per_rank": link_bytes, "target_ms": max(t_compute, t_link) * 1e3,
            "target_bound": "tensor" if t_compute >= t_link else "nvlink (770 GB/s per direction measured peer copy)",
            "frac_of_target": max(t_compute, t_link) * 1e3 / ms, "kernel": kernel + " + splitk_reduce_kernel over the rank slots",
            "parity_vs_n_split_rel_frobenius": err}


def tp_block_bench(pkg, ctx, comm, steps=10) -> dict:
    """The tensor-parallel GPT-2-XL-shaped block (d_model 1600, 25 heads, d_ff 6400, seq 1024, batch 16): forward,
    backward and Adam of one block across the ranks (tt-perf_b200/tp.py), the step of every rank replayed as one CUDA
    graph. Parity: the rank's rows of the output and of dx and two of its weight-gradient shards against the one-rank
    run of the same library on the same seeded inputs (relative Frobenius error <= 1e-2)."""
    import numpy as np
    tp, DT = pkg.tp, pkg.DeviceTensor
    rank, world = comm.rank, comm.world
    b, s, heads = 16, 1024, 25
    d, f = heads * 64, 4 * heads * 64
    t, tr = b * s, b * s // world
    rng = np.random.default_rng(11)                       # identical on every rank

    def bf16r(x):
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
        return ((((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint32) << 16).view(np.float32)

    shapes = dict(wq=(d, d), wk=(d, d), wv=(d, d), wo=(d, d), w1=(f, d), w2=(d, f))
    w = {k: bf16r(rng.standard_normal(sh, dtype=np.float32) * 0.02) for k, sh in shapes.items()}
    for k, n in (("bq", d), ("bk", d), ("bv", d), ("bo", d), ("b1", f), ("b2", d), ("ln1_b", d), ("ln2_b", d)):
        w[k] = np.zeros(n, np.float32)
    w["ln1_g"], w["ln2_g"] = np.ones(d, np.float32), np.ones(d, np.float32)
    x = bf16r(rng.standard_normal((t, d), dtype=np.float32) * 0.1)
    d_out = bf16r(rng.standard_normal((t, d), dtype=np.float32) * 0.1)

    # one-rank run of the same library (this GPU alone): the parity reference
    ranks1, fabric1 = tp.make_emulated(ctx, 1, batch=b, seq=s, d_model=d, heads=heads, host_w=w)
    x_full, do_full = DT.from_numpy(ctx, x), DT.from_numpy(ctx, d_out)
    tp.run_emulated([ranks1[0].forward(x_full)])
    tp.run_emulated([ranks1[0].backward(do_full)])
    ctx.synchronize()
    rows = slice(rank * tr, (rank + 1) * tr)
    ref = {"out": ranks1[0].out.numpy()[rows], "dx": ranks1[0].d_x.numpy()[rows],
           "w1": ranks1[0].grads["w1"].numpy(), "wo": ranks1[0].grads["wo"].numpy()}
    del ranks1, x_full, do_full
    fabric1.close()

    # From 4 ranks on the links, not the tensor cores, bound the step: the partial tiles then travel as bf16.
    partials = pkg.BF16 if world >= 4 else pkg.F32
    rk, fabric = tp.make_process(ctx, rank, world, batch=b, seq=s, d_model=d, heads=heads, host_w=w, comm=comm,
                                 partial_dtype=partials)
    mc_names = sorted(rk.mc)
    try:   # the fabric may hold NVLink multicast buffers: every rank releases them, also when a check raises
        x_r, do_r = DT.from_numpy(ctx, x[rows]), DT.from_numpy(ctx, d_out[rows])
        fabric.barrier()

        def step(update=True):
            tp.run_process(rk.forward(x_r), fabric)
            tp.run_process(rk.backward(do_r), fabric)
            if update:
                rk.adam_step()

        step(update=False)
        ctx.synchronize()
        sh = rk.shard

        def rel(got, want):
            return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want.astype(np.float64)), 1e-30))

        errs = {"out": rel(rk.out.numpy(), ref["out"]), "dx": rel(rk.d_x.numpy(), ref["dx"]),
                "dW1_shard": rel(rk.grads["w1"].numpy(), ref["w1"][sh["f0"]:sh["f1"]]),
                "dWo_shard": rel(rk.grads["wo"].numpy(), ref["wo"][:, sh["h0"]:sh["h1"]])}
        errs = {k: max_over_ranks(pkg, comm, v) for k, v in errs.items()}
        bad = {k: v for k, v in errs.items() if not v <= 1e-2}
        if bad:
            raise RuntimeError(f"bench: tensor-parallel block differs from the one-rank run: {bad}")
        for _ in range(2):
            step()
        fabric.barrier()
        tid = ctx.trace_begin()                               # kernels, peer copies and the rank barriers of one step
        step()
        ctx.trace_end(tid)
        ctx.trace_execute(tid)
        fabric.barrier()
        timer = ctx.timer_start()
        for _ in range(steps):
            ctx.trace_execute(tid)
        ms = max_over_ranks(pkg, comm, ctx.timer_stop(timer) / steps)
        fabric.barrier()
        ctx.trace_release(tid)
    finally:
        ctx.synchronize()
        fabric.close()
    flops = 3 * 24 * t * d * d + 3 * 4 * b * heads * 64 * (s * (s + 1) // 2)
    return {"workload": f"tensor-parallel GPT-2-XL-shaped block, d_model {d}, {heads} heads, d_ff {f}, seq {s}, batch {b}, "
                        f"forward + backward + Adam over {world} GPUs (QKV and FC1 column-parallel, attention-out and FC2 "
                        "row-parallel with the reduce-scatter fused into the GEMM epilogue)",
            "ms_per_step": ms, "tokens_per_s": t / (ms * 1e-3), "model_tflops_per_s": flops / (ms * 1e-3) / 1e12,
            "steps": steps, "executor": "trace replay (one CUDA graph per rank, rank barriers inside)",
            "heads_per_rank": tp.split_counts(heads, world), "partial_tiles": "bf16" if partials == pkg.BF16 else "fp32",
            "all_gather_transport": "NVLink multicast (multimem.st broadcast of row blocks)" if mc_names else "peer copies",
            "parity_vs_one_rank_rel_frobenius": errs}


def run_b200_distributed(args) -> None:
    """N > 1 (torchrun, one rank per GPU): C = A . B at 16384^3 with B split on N; the all-gather of C is fused into
    the GEMM epilogue (stores of finished tiles into every peer's C over NVLink). Per step: one fused launch per rank,
    then a stream-ordered rank barrier so that every rank holds the complete C before the next step starts."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    # NCCL prints its version banner on stdout; keep stdout for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    rank, world, local_rank, ctx, comm = start_ranks(pkg)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s = st.cuda_stream
    M = N = K = 16384
    off, width = pkg.dist.column_shard(N, world, rank)
    g = torch.Generator(device="cuda").manual_seed(42)           # same seed on every rank: A and B are replicated inputs
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    b_full = torch.randn(K, N, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    b = b_full[:, off:off + width].contiguous()
    mc_env = os.environ.get("B200_BENCH_MULTICAST", "auto")      # "0" forces the unicast transport for comparison runs
    mm = pkg.dist.ColumnParallelMatmul(ctx, M, N, K, rank, world, comm, multicast=False if mc_env == "0" else "auto")
    flops = 2.0 * M * N * K
    try:   # the multicast buffer must be released by every rank, also when a check below raises (all ranks raise together)

        def step():
            mm.launch(a, b, s)
            comm.barrier(s)            # rank barrier on the stream: all peers' stores have landed after it

        def host_barrier():
            ctx.synchronize(s)
            comm.barrier(s)
            ctx.synchronize(s)

        for _ in range(max(args.warmup, 3)):
            step()
        host_barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(st)
        for _ in range(args.steps):
            step()
        e1.record(st)
        torch.cuda.synchronize()
        ms_per_step = max_over_ranks(pkg, comm, e0.elapsed_time(e1)) / args.steps
        clocks = None
        # keep all ranks busy together while rank 0 samples clocks
        for _ in range(0 if args.quick else max(30, int(1500.0 / ms_per_step))):
            step()
        torch.cuda.synchronize()
        if rank == 0:
            clocks = sampler.stop()
        tflops = flops / (ms_per_step * 1e-3) / 1e12

        # parity: rows of the gathered C (every rank's copy) against fp32 torch on this GPU
        rows = torch.arange(rank, M, 1013, device="cuda")
        c_dev = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        ctx.memcpy_d2d(c_dev, mm.c_ptr, M * N * 2, s)
        ctx.synchronize(s)
        ref = a[rows].float() @ b_full.float()
        err = ((c_dev[rows].float() - ref).norm() / ref.norm()).item()
        err = max_over_ranks(pkg, comm, err)
        del c_dev, ref
        if not err < 1e-2:
            raise RuntimeError(f"bench: gathered C fails parity on some rank (relative Frobenius error {err:.3e})")

        # End to end with host buffers. One product, so every byte crosses PCIe once over the whole job: a rank uploads its
        # row block of A and its column shard of B from pinned host memory, the row blocks of A are all-gathered over NVLink
        # (peer copies into every rank's A), the fused product runs, and the rank downloads its row block of the gathered C.
        e2e = None
        if not args.quick:
            roff, rws = pkg.dist.row_block(M, world, rank)
            a_peer = pkg.dist._PeerBuffers(ctx, M * K * 2, rank, world, comm)
            a_h = a[roff:roff + rws].cpu().pin_memory()
            b_h = b.cpu().pin_memory()
            c_h = torch.empty(rws, N, dtype=torch.bfloat16).pin_memory()
            blk = rws * K * 2

            def e2e_step():
                ctx.h2d(a_peer.local + roff * K * 2, a_h, blk, s)
                ctx.h2d(b, b_h, K * width * 2, s)
                for k in range(1, world):                       # ranks start at different peers
                    peer = (rank + k) % world
                    ctx.memcpy_d2d(a_peer.ptrs[peer] + roff * K * 2, a_peer.local + roff * K * 2, blk, s)
                comm.barrier(s)                                 # every rank's A is complete
                mm.launch(a_peer.local, b, s)
                comm.barrier(s)                                 # every rank's C is complete
                ctx.d2h(c_h, mm.c_ptr + roff * N * 2, rws * N * 2, s)

            e2e_steps = 3
            e2e_step()
            host_barrier()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                e2e_step()
            torch.cuda.synchronize()
            e2e_s = max_over_ranks(pkg, comm, (time.perf_counter() - t0) / e2e_steps)
            ref = (a[roff:roff + rws:97].float() @ b_full.float()).cpu()
            err_h = max_over_ranks(pkg, comm, ((c_h[::97].float() - ref).norm() / ref.norm()).item())
            if not err_h < 1e-2:
                raise RuntimeError(f"bench: host-buffer sharded matmul fails parity (relative Frobenius error {err_h:.3e})")
            host_barrier()
            a_peer.close()
            e2e = {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": (rws * K + K * width) * 2,
                   "d2h_bytes_per_step": rws * N * 2, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                   "parity_sample_rel_frobenius": err_h,
                   "note": "bytes are per rank: its row block of A and its column shard of B host->device, all-gather of A over "
                           "NVLink, fused GEMM + all-gather of C, its row block of C device->host; the job moves A, B and C "
                           "over PCIe once"}

        transport = mm.transport
        d_local = ctx.gemm_desc(a, b, None, M, width, K, ldb=width, ldc=N)
        kernel = ctx.gemm_plan_text(d_local, ctx.gemm_dist_plan(d_local, world, False))
        peaks = load_peaks()
        rs = None
        if not args.quick:
            rs = reduce_scatter_bench(torch, pkg, ctx, comm, st, a, b_full, mm.c_ptr, max(3, min(args.steps, 10)), peaks)
        host_barrier()
    finally:
        mm.close()
    del a, b, b_full
    torch.cuda.empty_cache()
    tpb = gpt2 = None
    if not args.quick:
        tpb = tp_block_bench(pkg, ctx, comm)
        gpt2 = gpt2_train_bench(steps=5, warmup=2, device=local_rank, rank=rank, world=world, comm=comm)
    if rank == 0:
        peak = peaks["bf16_tflops"] * world
        # bytes each rank puts on its links: its slice once per peer, or once in all when the switch replicates it
        nvlink_bytes = (M * N * 2 / world) * (1 if "multicast" in transport else world - 1)
        nvlink_bytes_in = (world - 1) / world * M * N * 2       # bytes each rank receives, whatever the transport
        t_compute = flops / world / (peaks["bf16_tflops"] * 1e12)
        t_link = max(nvlink_bytes, nvlink_bytes_in) / 770e9
        mhz = clocks.get("sm_mhz") if clocks else None
        line = {
            "metric": "bf16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "pct_of_peak": tflops / peak,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                         "traffic": None,
                         "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json bf16_tflops x {world} GPUs)",
                         "kernel": kernel + " with the all-gather fused into its epilogue; transport: " + transport,
                         "flops_per_launch": flops / world, "nvlink_bytes_sent_per_rank": nvlink_bytes,
                         "nvlink_bytes_received_per_rank": nvlink_bytes_in,
                         "target_ms": max(t_compute, t_link) * 1e3, "target_bound": "tensor" if t_compute >= t_link else "nvlink",
                         "frac_of_target": max(t_compute, t_link) * 1e3 / ms_per_step},
            "cpu_baseline": None,
            "e2e": e2e,
            "gpu_launches": args.steps * world,
            "clocks": clocks,
            "ms_per_step_x_sm_mhz": ms_per_step * mhz if mhz else None,
            "parity_sample_rel_frobenius": err,
        }
        if not args.quick:
            cpu = cpu_matmul_baseline(M, N, K)
            cpu.pop("seconds", None)
            line["cpu_baseline"] = cpu
            line["reduce_scatter"] = rs
            line["tp_block"] = tpb
            line["gpt2_small_train"] = gpt2
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    comm.barrier()
    ctx.synchronize()
    comm.close()
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="gemm", choices=["gemm", "gpt2"],
                    help="gemm: the headline matmul line (default). gpt2: only the GPT-2-small training step "
                         "(its own JSON object; used for profiling that workload)")
    ap.add_argument("--quick", action="store_true",
                    help="timed region only: skip the CPU baseline, the host-buffer leg and the clock soak "
                         "(for runs under a profiler; its line is not a bench result)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "gpt2":
        print(json.dumps(gpt2_train_bench(steps=args.steps, warmup=args.warmup)), flush=True)
        return
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_b200_single(args)
    else:
        run_b200_distributed(args)


if __name__ == "__main__":
    main()
