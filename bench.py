#!/usr/bin/env python3
"""Benchmark of the dense-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

N = 1   one bf16 GEMM C = A.B with M = N = K = 8192 per step (the shape the headline metric is quoted on),
        inputs resident in HBM, through the C ABI (b200_gemm).
N > 1   launched by torchrun, one rank per GPU: the distributed matmul M = N = K = 16384 with B split on N
        across the ranks and C all-gathered (scripts/matmul_2dev_distributed.py generalised), strong scaling.

Prints ONE JSON line on rank 0. `value` is whole-job TFLOP/s (2.M.N.K per product, counted once for the
sharded product). `e2e` repeats the measurement with host buffers: pinned host A/B -> device, GEMM, C -> host.
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


class _DevBytes:
    """CUDA array interface over a raw device pointer, so that torch.distributed (NCCL) can all-reduce buffers that
    the library's pool owns."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def gpt2_train_bench(steps: int = 10, warmup: int = 3, device: int = 0, rank: int = 0, world: int = 1) -> dict:
    """GPT-2-small-shaped training step (12 layers, d_model 768, 12 heads, d_ff 3072, seq 1024, batch 8 per GPU, vocab
    50257, random N(0, 0.02) weights, uniform random token ids, Adam lr 3e-4 betas (0.9, 0.95)): forward, cross-entropy,
    backward and the Adam update. Every kernel comes from the C ABI; the host side is tt-perf_b200/nn.py.

    One GPU: the whole step is recorded once as a trace (CUDA graph) and replayed, as the reference's traced executor
    does (bench/autograd/bench_gpt2_full.cpp). N GPUs (data parallel, weak scaling): each rank replays forward +
    backward on its own batch as a chain of traces (LM head, then groups of four blocks); every trace packs its
    gradients into a bucket that NCCL (through torch.distributed) averages over the ranks on a second stream while the
    next trace runs; a last trace applies Adam from the buckets. Returns whole-job tokens/s and ms/step."""
    import numpy as np
    from __graft_entry__ import load_package
    pkg = load_package()
    ctx = pkg.Context(device)
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
        t0 = time.perf_counter()
        for _ in range(steps):
            ctx.trace_execute(tid)
        ctx.synchronize()
        dt = (time.perf_counter() - t0) / steps
        executor = "trace replay (CUDA graph)"
        traces = [tid]
    else:
        import torch
        import torch.distributed as dist
        # The backward pass is recorded as several traces (LM head, then groups of four blocks, the last one with the
        # embeddings). Each trace ends by packing its gradients into its own bf16 / fp32 bucket; while the next trace
        # runs on the compute stream, the bucket is averaged over the ranks by NCCL on a second stream (events order
        # the two, no host synchronisation). A last trace applies Adam straight from the buckets.
        c = pkg.capi
        specs = []
        model.forward_backward(idd, tgd, pos, segment_hook=lambda pairs: specs.append([(g.numel, g.dtype) for _, g in pairs]))
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

        loss, grads = model.forward_backward(idd, tgd, pos, segment_hook=pack_and_cut)
        bf, f32 = model._flat(grads)
        t_opt = ctx.trace_begin()
        model.opt[0].step([slice_of[id(prm)] for prm, _ in bf])
        model.opt[1].step([slice_of[id(prm)] for prm, _ in f32])
        ctx.trace_end(t_opt)
        seg_views = []
        for flat_bf, flat_f32, _, n_bf, n_f32 in buckets:
            v = []
            if n_bf:
                v.append(torch.as_tensor(_DevBytes(flat_bf.ptr, 2 * n_bf), device="cuda").view(torch.bfloat16))
            if n_f32:
                v.append(torch.as_tensor(_DevBytes(flat_f32.ptr, 4 * n_f32), device="cuda").view(torch.float32))
            seg_views.append(v)
        comp, comm = torch.cuda.Stream(), torch.cuda.Stream()

        def dp_step():
            for tid, views in zip(seg_traces, seg_views):
                ctx.trace_execute_on(tid, comp.cuda_stream)
                ev = torch.cuda.Event()
                ev.record(comp)
                comm.wait_event(ev)                            # this segment's gradients are packed
                with torch.cuda.stream(comm):
                    for v in views:
                        dist.all_reduce(v, op=dist.ReduceOp.AVG)
            comp.wait_stream(comm)                             # every bucket is averaged before Adam reads it
            ctx.trace_execute_on(t_opt, comp.cuda_stream)

        ctx.synchronize()
        dp_step()
        comp.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            dp_step()
        comp.synchronize()
        t = torch.tensor([(time.perf_counter() - t0) / steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = t.item()
        executor = (f"{len(seg_traces)} backward traces on a compute stream, each followed by the NCCL all-reduce of its gradient "
                    "bucket on a second stream (overlapping the next trace), then an Adam trace")
        traces = seg_traces + [t_opt]
    final = float(loss.numpy()[0])
    for t in traces:
        ctx.trace_release(t)
    flops = 3 * (12 * 24 * B * S * D * D + 2 * B * S * D * V) + 12 * 12 * B * H * 64 * (S * (S + 1) // 2)
    out = {"metric": "GPT-2-small train tokens/s", "tokens_per_s": world * B * S / dt, "ms_per_step": dt * 1e3,
           "model_tflops_per_s": world * flops / dt / 1e12, "params": model.num_params(), "batch_per_gpu": B, "seq": S,
           "n_gpus": world, "scaling": "weak (data parallel)" if world > 1 else None, "first_losses": losses,
           "loss_after_replays": final, "executor": executor,
           "data": "synthetic: uniform token ids, targets = ids shifted by one"}
    ctx.close()
    return out


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
                     "traffic": GEMM_8192_DRAM_TRAFFIC_BYTES,
                     "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json bf16_tflops, burst: kernel timed alone)",
                     "kernel": "gemm_tcgen05_2cta_kernel<K-major A,MN-major B> (cta_group::2, 256x256x64 tiles)", "flops_per_launch": flops},
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
        line["gpt2_small_train"] = gpt2_train_bench()
    print(json.dumps(line), flush=True)
    ctx.close()


def run_b200_distributed(args) -> None:
    """N > 1 (torchrun, one rank per GPU): C = A . B at 16384^3 with B split on N; the all-gather of C is fused into
    the GEMM epilogue (TMA stores into every peer's C over NVLink). Per step: one fused launch per rank, then a
    rank barrier (tiny NCCL all-reduce) so that every rank holds the complete C before the next step starts."""
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local_rank)
    # NCCL prints its version banner on stdout; keep stdout for the one JSON line
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = pkg.Context(local_rank)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s = st.cuda_stream
    M = N = K = 16384
    off, width = pkg.dist.column_shard(N, world, rank)
    g = torch.Generator(device="cuda").manual_seed(42)           # same seed on every rank: A and B are replicated inputs
    a = torch.randn(M, K, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    b_full = torch.randn(K, N, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    b = b_full[:, off:off + width].contiguous()
    mm = pkg.dist.ColumnParallelMatmul(ctx, M, N, K, rank, world)
    flag = torch.zeros(1, device="cuda")
    flops = 2.0 * M * N * K

    def step():
        mm.launch(a, b, s)
        dist.all_reduce(flag)      # rank barrier on the stream: all peers' stores have landed after it

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
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
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t.item() / args.steps
    clocks = None
    # keep all ranks busy together while rank 0 samples clocks
    for _ in range(0 if args.quick else max(30, int(1500.0 / ms_per_step))):
        step()
    torch.cuda.synchronize()
    if rank == 0:
        clocks = sampler.stop()
    tflops = flops / (ms_per_step * 1e-3) / 1e12

    # parity: rows of the gathered C (every rank's copy) against fp32 torch on this GPU
    c_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
    ctx.d2h(c_host, mm.c_ptr, M * N * 2, s)
    rows = torch.arange(rank, M, 1013)
    ref = (a[rows.cuda()].float() @ b_full.float()).cpu()
    err = ((c_host[rows].float() - ref).norm() / ref.norm()).item()
    errs = torch.tensor([err], device="cuda")
    dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    if not errs.item() < 1e-2:
        raise RuntimeError(f"bench: gathered C fails parity on some rank (relative Frobenius error {errs.item():.3e})")

    # end to end with host buffers: A and the B shard from pinned host memory, fused GEMM + gather, full C to the host
    e2e = None
    if not args.quick:
        a_h = a.cpu().pin_memory()
        b_h = b.cpu().pin_memory()
        e2e_steps = 2
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ctx.h2d(a, a_h, M * K * 2, s)
            ctx.h2d(b, b_h, K * width * 2, s)
            step()
            ctx.d2h(c_host, mm.c_ptr, M * N * 2, s)
        torch.cuda.synchronize()
        t = torch.tensor([(time.perf_counter() - t0) / e2e_steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": flops / t.item() / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": (M * K + K * width) * 2,
               "d2h_bytes_per_step": M * N * 2, "ms_per_step": t.item() * 1e3, "steps": e2e_steps,
               "note": "per rank: A and the B shard host->device, fused GEMM + all-gather, the full C device->host"}

    mm.close()
    ctx.close()
    gpt2 = None
    if not args.quick:
        del a, b, b_full
        torch.cuda.empty_cache()
        gpt2 = gpt2_train_bench(steps=5, warmup=2, device=local_rank, rank=rank, world=world)
    if rank == 0:
        peaks = load_peaks()
        peak = peaks["bf16_tflops"] * world
        nvlink_bytes = (world - 1) / world * M * N * 2          # bytes each rank sends to its peers
        t_compute = flops / world / (peaks["bf16_tflops"] * 1e12)
        t_link = nvlink_bytes / 770e9
        line = {
            "metric": "bf16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "pct_of_peak": tflops / peak,
            "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                         "traffic": None,
                         "peak_source": f"{peaks['source']} (MEASURED_PEAKS.json bf16_tflops x {world} GPUs)",
                         "kernel": "gemm_tcgen05_kernel<256> with the all-gather fused into its TMA-store epilogue",
                         "flops_per_launch": flops / world, "nvlink_bytes_sent_per_rank": nvlink_bytes,
                         "target_ms": max(t_compute, t_link) * 1e3, "target_bound": "tensor" if t_compute >= t_link else "nvlink",
                         "frac_of_target": max(t_compute, t_link) * 1e3 / ms_per_step},
            "cpu_baseline": None,
            "e2e": e2e,
            "gpu_launches": args.steps * world,
            "clocks": clocks,
            "parity_sample_rel_frobenius": errs.item(),
        }
        if not args.quick:
            cpu = cpu_matmul_baseline(M, N, K)
            cpu.pop("seconds", None)
            line["cpu_baseline"] = cpu
            line["gpt2_small_train"] = gpt2
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
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
