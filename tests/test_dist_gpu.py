"""Sharded matmul on the GPU. With one GPU the ranks are emulated in one process: each "rank" launches its fused
GEMM + store kernel in turn, with every rank's buffer living on the same device (the kernels never wait on one
another, so running them back to back is legal). With two or more GPUs a torchrun job exercises the real CUDA-IPC
peer stores."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import matmul_oracle as mo
from conftest import REPO

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_column_parallel_allgather_emulated_ranks(pkg, ctx, stream, world):
    M, N, K = 384, 128 * world, 320
    rng = np.random.default_rng(world)
    a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    ad = torch.from_numpy(a).bfloat16().cuda()
    c_bufs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    s = stream.cuda_stream
    for r in range(world):
        off, width = pkg.dist.column_shard(N, world, r)
        b_shard = torch.from_numpy(b[:, off:off + width].copy()).bfloat16().cuda()
        d = ctx.gemm_desc(ad, b_shard, None, M, width, K, ldb=width, ldc=N)
        ctx.gemm_allgather(d, c_bufs, r, s)
        ctx.synchronize(s)
    ref = mo.matmul(a, b)
    for c in c_bufs:   # every rank ends with the whole C, like ttnn::all_gather(c, 1)
        got = c.float().cpu().numpy()
        assert not np.isnan(got).any()
        assert mo.rel_frobenius(got, ref) <= 1e-2
    assert all(torch.equal(c_bufs[0], c) for c in c_bufs[1:])


@pytest.mark.parametrize("world,dtype", [(2, "bf16"), (4, "bf16"), (2, "f32")])
def test_allgather_single_destination_epilogue_emulated_ranks(pkg, ctx, stream, world, dtype):
    """b200_gemm_allgather_mc: the epilogue that writes each staged box with 16-byte warp stores to ONE destination —
    on real ranks the NVLink multicast address of C (multimem.st), here an ordinary buffer (use_multimem = 0), which
    exercises the same addressing: ragged M, a shard width that is not a multiple of the 64-column box."""
    M, width, K = 712, 328, 320
    N = width * world
    rng = np.random.default_rng(20 + world)
    a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    ad = torch.from_numpy(a).bfloat16().cuda()
    f32 = dtype == "f32"
    c = torch.full((M, N), float("nan"), dtype=torch.float32 if f32 else torch.bfloat16, device="cuda")
    s = stream.cuda_stream
    for r in range(world):
        b_shard = torch.from_numpy(b[:, r * width:(r + 1) * width].copy()).bfloat16().cuda()
        d = ctx.gemm_desc(ad, b_shard, None, M, width, K, ldb=width, ldc=N, c_dtype=pkg.F32 if f32 else pkg.BF16)
        ctx.gemm_allgather_mc(d, c, world, r, use_multimem=False, stream=s)
    ctx.synchronize(s)
    got = c.float().cpu().numpy()
    assert not np.isnan(got).any(), "a box was left unwritten"
    assert mo.rel_frobenius(got, mo.matmul(a, b)) <= 1e-2
    with pytest.raises(pkg.B200Error):   # too small for the CTA-pair kernel: the caller falls back to b200_gemm_allgather
        ctx.gemm_allgather_mc(ctx.gemm_desc(ad, ad, None, 128, 128, K, transpose_b=True, ldc=256), c, 2, 0, use_multimem=False, stream=s)


@pytest.mark.parametrize("world", [1, 2, 4])
def test_row_parallel_reduce_scatter_emulated_ranks(pkg, ctx, stream, world):
    M, N, K = 128 * world * 2, 200, 64 * world
    rng = np.random.default_rng(10 + world)
    a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    rows = M // world
    slots = [torch.full((world, rows, N), float("nan"), dtype=torch.float32, device="cuda") for _ in range(world)]
    s = stream.cuda_stream
    for r in range(world):
        koff, kdepth = pkg.dist.k_shard(K, world, r)
        a_sh = torch.from_numpy(a[:, koff:koff + kdepth].copy()).bfloat16().cuda()
        b_sh = torch.from_numpy(b[koff:koff + kdepth].copy()).bfloat16().cuda()
        d = ctx.gemm_desc(a_sh, b_sh, None, M, N, kdepth, ldc=N, c_dtype=pkg.F32)
        ctx.gemm_reduce_scatter_partials(d, slots, r, s)
    ctx.synchronize(s)
    ref, blocks = mo.row_parallel_matmul(a, b, world)
    for r in range(world):
        out = torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        d = ctx.gemm_desc(None, None, out, rows, N, 0, lda=8, ldb=N)
        ctx.reduce_slices(slots[r], world, d, s)
        ctx.synchronize(s)
        assert mo.rel_frobenius(out.float().cpu().numpy(), blocks[r]) <= 1e-2


def test_dist_argument_validation(pkg, ctx, stream):
    a = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    s = stream.cuda_stream
    with pytest.raises(pkg.B200Error):   # ldc does not cover the gathered width
        ctx.gemm_allgather(ctx.gemm_desc(a, a, None, 256, 128, 64, transpose_b=True, ldc=128), [c, c], 0, s)
    with pytest.raises(pkg.B200Error):   # rank out of range
        ctx.gemm_allgather(ctx.gemm_desc(a, a, None, 256, 128, 64, transpose_b=True, ldc=256), [c, c], 2, s)
    with pytest.raises(pkg.B200Error):   # M / ranks not a multiple of the 128-row tile
        ctx.gemm_reduce_scatter_partials(ctx.gemm_desc(a, a, None, 192, 64, 64, transpose_b=True, ldc=64), [c, c], 0, s)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_torchrun_bench_line():
    """The real peer path: torchrun with 2 ranks, CUDA-IPC peer buffers, fused all-gather; bench.py checks the gathered
    C on every rank against fp32 torch before it prints its line."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(REPO / "bench.py"), "--gpus", "2",
                        "--steps", "3", "--warmup", "3", "--quick"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"n_gpus": 2' in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_multi_gpu_parity_all_gather_and_reduce_scatter():
    """torchrun over all visible GPUs (2, 4 or 8): fused all-gather and fused reduce-scatter against the oracle."""
    n = min(8, torch.cuda.device_count())
    n = 8 if n >= 8 else 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n),
                        "--master-addr", "127.0.0.1", "--master-port", "29544", str(REPO / "tests" / "dist_rank_worker.py")],
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and f"DIST_PARITY_OK {n}" in r.stdout, (r.stdout[-1500:], r.stderr[-3000:])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_reference_tensor_parallel_program_on_a_two_gpu_mesh():
    """bench/metal/matmul_tensor_parallel.cpp, compiled unchanged: 1x2 mesh in one process, A replicated, B sharded
    on dim 1, ttnn::matmul then ttnn::all_gather(c, 1)."""
    exe = REPO / "build" / "ref_mains" / "matmul_tensor_parallel"
    if not exe.exists():
        pytest.skip("reference mains not built")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [l for l in r.stdout.splitlines() if l and l[0].isdigit()]
    assert len(rows) >= 5 and "Error" not in r.stderr
