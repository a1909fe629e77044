"""Runtime behaviour around the kernels, through the C ABI: the bounded-wait error path, the context's shared scratch
under traces and across streams, the device-resident Adam step of replayed traces, and explicit GEMM plans."""
import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _operands(M, N, K, ta, tb, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((K, M) if ta else (M, K), generator=g).bfloat16()
    b = torch.randn((N, K) if tb else (K, N), generator=g).bfloat16()
    ref = mo.matmul(a.float().numpy(), b.float().numpy(), ta, tb)
    return a.cuda(), b.cuda(), ref


def _err(c, ref):
    return mo.rel_frobenius(c.float().cpu().numpy(), ref)


def test_wait_that_runs_out_is_reported_and_the_context_recovers(pkg, ctx, stream):
    """A kernel whose bounded wait gives up raises the status word; b200_synchronize turns it into
    B200_ERR_DEVICE_TIMEOUT once, clears the status block (ticket counters included), and later kernels that rely
    on zeroed tickets — the K-sliced pair kernel, column sums — are correct."""
    s = stream.cuda_stream
    ctx.synchronize(s)                                   # clean start
    ctx.selftest_wait_timeout(1_000_000, s)              # 1 ms on a barrier nothing arrives at
    with pytest.raises(pkg.B200Error) as e:
        ctx.synchronize(s)
    assert e.value.code == pkg.capi.ERR_DEVICE_TIMEOUT
    ctx.synchronize(s)                                   # reported once, then clear
    M, N, K = 512, 512, 4096
    a, b, ref = _operands(M, N, K, True, False, 11)
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    plan = pkg.capi.GemmPlan(pkg.capi.KERNEL_TCGEN05_PAIR, 256, 3, 0)
    ctx.gemm_planned(ctx.gemm_desc(a, b, c, M, N, K, transpose_a=True), plan, s)
    x = torch.randn(4096, 768, generator=torch.Generator().manual_seed(3)).bfloat16().cuda()
    colsum = torch.empty(768, dtype=torch.bfloat16, device="cuda")
    ctx.reduce(pkg.capi.R_SUM, x, 1, 4096, 768, colsum, stream=s)
    ctx.synchronize(s)
    assert _err(c, ref) <= TOL
    assert mo.rel_frobenius(colsum.float().cpu().numpy(), x.float().cpu().numpy().sum(0)) <= TOL


def test_peer_barrier_alone_and_with_an_absent_peer(pkg, ctx, stream):
    """b200_peer_barrier on one GPU: with one rank it completes at once and advances its epoch on the device; with a
    second flag array that nobody writes (a peer that never arrives) the wait runs out, the status word is raised and
    the context stays usable. (Ranks that do arrive are covered by the one-process-per-GPU TP block tests.)"""
    s = stream.cuda_stream
    ctx.synchronize(s)
    mine = torch.zeros(2, dtype=torch.int32, device="cuda")
    absent = torch.zeros(2, dtype=torch.int32, device="cuda")
    epoch = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(3):
        ctx.peer_barrier([mine], 0, epoch, stream=s)
    ctx.synchronize(s)
    assert int(epoch.item()) == 3 and int(mine[0].item()) == 3
    ctx.peer_barrier([mine, absent], 0, epoch, stream=s)      # rank 1 never stores into `mine`
    with pytest.raises(pkg.B200Error) as e:
        ctx.synchronize(s)
    assert e.value.code == pkg.capi.ERR_DEVICE_TIMEOUT
    assert int(absent[0].item()) == 4                         # this rank did publish its epoch to the peer's array
    ctx.synchronize(s)                                        # reported once, then clear
    a, b, ref = _operands(256, 256, 512, False, False, 5)
    c = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    ctx.gemm(ctx.gemm_desc(a, b, c, 256, 256, 512), s)
    ctx.synchronize(s)
    assert _err(c, ref) <= TOL


def test_every_plan_gives_the_same_product(pkg, ctx, stream):
    """b200_gemm_plan_query reports the library's own choice; b200_gemm_planned runs any other kernel, tile width,
    slice count and tile order on the same operands."""
    s = stream.cuda_stream
    k = pkg.capi
    M, N, K = 768, 520, 2048
    a, b, ref = _operands(M, N, K, False, True, 21)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    desc = ctx.gemm_desc(a, b, c, M, N, K, transpose_b=True)
    own = ctx.gemm_plan(desc)
    assert own.kernel in (k.KERNEL_TCGEN05, k.KERNEL_TCGEN05_PAIR) and own.k_slices >= 1
    assert "tcgen05" in ctx.gemm_plan_text(desc, own)
    plans = [k.GemmPlan(k.KERNEL_SIMT, 0, 1, 0)]
    plans += [k.GemmPlan(k.KERNEL_TCGEN05, bn, ks, gm) for bn in (64, 128, 192, 256) for ks, gm in ((1, 0), (4, 3))]
    plans += [k.GemmPlan(k.KERNEL_TCGEN05_PAIR, 256, ks, gm) for ks, gm in ((1, 0), (2, 5))]
    for plan in plans:
        c.fill_(float("nan"))
        ctx.gemm_planned(desc, plan, s)
        ctx.synchronize(s)
        assert _err(c, ref) <= TOL, ctx.gemm_plan_text(desc, plan)
    with pytest.raises(pkg.B200Error):
        ctx.gemm_planned(desc, k.GemmPlan(k.KERNEL_TCGEN05, 100, 1, 0), s)      # not a tile width
    unaligned = ctx.gemm_desc(a, b, c, 64, 10, 128)                              # 20-byte rows: CUDA cores only
    assert ctx.gemm_plan(unaligned).kernel == k.KERNEL_SIMT
    assert "simt" in ctx.gemm_plan_text(unaligned, ctx.gemm_plan(unaligned))


def test_k_sliced_products_on_two_streams_do_not_corrupt_each_other(pkg, ctx, stream):
    """Both products keep their partial sums in the context's one scratch block; the library orders the streams."""
    s1 = stream.cuda_stream
    st2 = torch.cuda.Stream()
    s2 = st2.cuda_stream
    M, N, K = 512, 384, 8192
    a1, b1, ref1 = _operands(M, N, K, True, False, 31)
    a2, b2, ref2 = _operands(M, N, K, True, False, 32)
    c1 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    c2 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()
    for _ in range(4):
        ctx.gemm(ctx.gemm_desc(a1, b1, c1, M, N, K, transpose_a=True, split_k=8, algo=pkg.ALGO_TCGEN05), s1)
        ctx.gemm(ctx.gemm_desc(a2, b2, c2, M, N, K, transpose_a=True, split_k=8, algo=pkg.ALGO_TCGEN05), s2)
    ctx.synchronize(s1)
    ctx.synchronize(s2)
    assert _err(c1, ref1) <= TOL and _err(c2, ref2) <= TOL


def test_scratch_outgrown_after_a_trace_was_recorded_stays_valid_for_replays(pkg):
    """A recorded K-sliced product replays on the scratch address it saw. A later, larger request must not free that
    block while the trace exists."""
    import torch
    c = pkg.Context(0)
    try:
        DT = pkg.DeviceTensor
        M, N, K = 256, 256, 4096
        a, b, ref = _operands(M, N, K, True, False, 41)
        ad, bd = DT.from_numpy(c, a.float().cpu().numpy()), DT.from_numpy(c, b.float().cpu().numpy())
        out = DT(c, (M, N), pkg.BF16)
        desc = c.gemm_desc(ad, bd, out, M, N, K, transpose_a=True, split_k=4, algo=pkg.ALGO_TCGEN05)
        c.gemm(desc)                                   # untraced once: the scratch exists
        c.synchronize()
        tid = c.trace_begin()
        c.gemm(desc)
        c.trace_end(tid)
        # a much larger K-sliced product outgrows the 64 MiB block
        M2, N2, K2 = 2048, 2048, 4096
        a2, b2, ref2 = _operands(M2, N2, K2, True, False, 42)
        c2 = torch.empty(M2, N2, dtype=torch.bfloat16, device="cuda")
        big = c.gemm_desc(a2, b2, c2, M2, N2, K2, transpose_a=True, split_k=8, algo=pkg.ALGO_TCGEN05)
        assert c.gemm_scratch_bytes(big) > (64 << 20)
        c.gemm(big)
        c.synchronize()
        assert _err(c2, ref2) <= TOL
        c.fill(out, out.numel, pkg.BF16, 0.0)
        c.trace_execute(tid, blocking=True)
        c.synchronize()
        assert mo.rel_frobenius(out.numpy(), ref) <= TOL
        c.trace_release(tid)                           # last trace gone: the outgrown block is freed here
        c.gemm(desc)
        c.synchronize()
        assert mo.rel_frobenius(out.numpy(), ref) <= TOL
    finally:
        c.close()


def test_replayed_adam_steps_follow_the_eager_recurrence(pkg):
    """One optimiser step recorded into a trace and replayed k times must equal k eager steps: the step number and
    the bias corrections live in device memory (py/optim.py:73-84; tests/adam_optimizer.py:15-22)."""
    c = pkg.Context(0)
    try:
        DT = pkg.DeviceTensor
        rng = np.random.default_rng(7)
        n = 4096 + 5
        p0 = rng.standard_normal(n).astype(np.float32)
        g0 = rng.standard_normal(n).astype(np.float32)
        p = DT.from_numpy(c, p0, pkg.F32)
        g = DT.from_numpy(c, g0, pkg.F32)
        opt = pkg.nn.Adam(c, [p], lr=1e-2, betas=(0.9, 0.999), eps=1e-8)
        opt.step([g])                                   # eager step 1
        tid = c.trace_begin()
        opt.step([g])                                   # recorded, not run
        c.trace_end(tid)
        for _ in range(4):                              # replays: steps 2 .. 5
            c.trace_execute(tid)
        c.synchronize()
        steps = opt.t
        assert steps == 5
        ref_p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
        for t in range(1, steps + 1):
            ref_p, m, v = mo.adam_update(ref_p, g0, m, v, t, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8)
        got = p.numpy()
        assert mo.rel_frobenius(got - p0, ref_p - p0) <= 1e-4
        assert mo.rel_frobenius(opt.m[0].numpy(), m) <= 1e-4 and mo.rel_frobenius(opt.v[0].numpy(), v) <= 1e-4   # fp32 rounding
        c.trace_release(tid)
    finally:
        c.close()
