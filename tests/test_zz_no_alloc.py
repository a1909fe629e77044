"""b200_gemm_static_scratch — the split-K matmul for hosts that may not allocate device memory at call time
(arena-owning executors, latency-bound loops, processes with a device-memory cap): its partial sums live in a fixed
32 MiB array inside the library instead of cudaMalloc'ed context scratch.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other
test. The checks hold both in a fresh process and after the rest of the suite: the entry point must give
the same bits as b200_gemm with the same K slicing, on two calls in a row that share the array."""
import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo

pytestmark = pytest.mark.gpu


def _case(pkg, ctx, stream, M, N, K, ta, tb, split, seed, **kw):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((K, M) if ta else (M, K), generator=g).bfloat16().cuda()
    b = torch.randn((N, K) if tb else (K, N), generator=g).bfloat16().cuda()
    ref = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    s = stream.cuda_stream
    ctx.gemm(ctx.gemm_desc(a, b, ref, M, N, K, transpose_a=ta, transpose_b=tb, split_k=split,
                           algo=pkg.ALGO_TCGEN05, **kw), s)
    ctx.gemm_static_scratch(ctx.gemm_desc(a, b, got, M, N, K, transpose_a=ta, transpose_b=tb, split_k=split, **kw), s)
    ctx.synchronize(s)
    oracle = mo.matmul(a.float().cpu().numpy(), b.float().cpu().numpy(), ta, tb)
    return got, ref, oracle


def _same(got, ref):
    """b200_gemm may pick another kernel or slice count for the same product (its planner also knows the CTA-pair
    kernel), which changes the order of the fp32 additions: equal up to one bf16 rounding, not bit for bit."""
    return mo.rel_frobenius(got.float().cpu().numpy(), ref.float().cpu().numpy()) <= 2e-3


def test_static_scratch_matches_gemm_on_two_calls_in_a_row(pkg, ctx, stream):
    # call 1: dW-shaped product (reduction over 4096 tokens), 4 K slices
    got, ref, oracle = _case(pkg, ctx, stream, 384, 264, 4096, True, False, 4, seed=101)
    assert _same(got, ref), "first call differs from b200_gemm"
    assert mo.rel_frobenius(got.float().cpu().numpy(), oracle) <= 1e-2
    # call 2 straight after, other shape / form / slice count: must not see call 1's partial sums
    got, ref, oracle = _case(pkg, ctx, stream, 200, 512, 1536, False, True, 3, seed=202)
    assert _same(got, ref), "second call differs from b200_gemm"
    assert mo.rel_frobenius(got.float().cpu().numpy(), oracle) <= 1e-2
    # automatic slice choice, with a fused epilogue
    bias = torch.randn(256, generator=torch.Generator().manual_seed(5)).bfloat16().cuda()
    got, ref, oracle = _case(pkg, ctx, stream, 256, 256, 8192, True, False, 0, seed=303, bias=bias,
                             activation=pkg.ACT_RELU)
    assert _same(got, ref)
    assert mo.rel_frobenius(got.float().cpu().numpy(), mo.relu(oracle + bias.float().cpu().numpy())) <= 1e-2


def test_static_scratch_calls_leave_device_memory_untouched_and_report_their_status(pkg, ctx, stream):
    """After the set-up call of a shape class, further calls change neither the free device memory nor the caching
    pools of the process (the property arena-owning hosts need), and b200_static_scratch_status — this entry point's
    counterpart of b200_synchronize — reports a clean status."""
    s = stream.cuda_stream
    g = torch.Generator().manual_seed(404)
    M, N, K = 256, 384, 4096
    a = torch.randn(K, M, generator=g).bfloat16().cuda()
    b = torch.randn(K, N, generator=g).bfloat16().cuda()
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    desc = ctx.gemm_desc(a, b, c, M, N, K, transpose_a=True, split_k=4)
    ctx.gemm_static_scratch(desc, s)                    # set-up call: symbol addresses, kernel attributes
    assert ctx.static_scratch_status(s) == 0
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        ctx.gemm_static_scratch(desc, s)
    assert ctx.static_scratch_status(s) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    ref = mo.matmul(a.float().cpu().numpy(), b.float().cpu().numpy(), True, False)
    assert mo.rel_frobenius(c.float().cpu().numpy(), ref) <= 1e-2
    # the descriptor checks are those of b200_gemm
    bad = ctx.gemm_desc(a, b, c, M, N, K, transpose_a=True, split_k=4)
    bad.ab_dtype = 7
    with pytest.raises(pkg.B200Error):
        ctx.gemm_static_scratch(bad, s)


def test_static_scratch_rejects_what_does_not_fit(pkg, ctx, stream):
    a = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    s = stream.cuda_stream
    # 4 slices x 2048 x 2048 x 4 B = 64 MiB > 32 MiB
    with pytest.raises(pkg.B200Error) as e:
        ctx.gemm_static_scratch(ctx.gemm_desc(a, a, a, 2048, 2048, 4096, split_k=4), s)
    assert e.value.code == pkg.capi.ERR_INVALID_ARG and "static scratch holds" in str(e.value)
    # rows of 20 bytes cannot be TMA sources and there is no SIMT path here
    with pytest.raises(pkg.B200Error) as e:
        ctx.gemm_static_scratch(ctx.gemm_desc(a, a, a, 64, 10, 128), s)
    assert e.value.code == pkg.capi.ERR_INVALID_ARG
    with pytest.raises(pkg.B200Error):
        ctx.gemm_static_scratch(ctx.gemm_desc(a, a, a, 64, 64, 128), None)   # a stream is required
