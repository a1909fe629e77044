"""One rank of the multi-GPU parity job (launched by torchrun from tests/test_dist_gpu.py): real CUDA-IPC peer
buffers, fused GEMM + all-gather and fused GEMM + reduce-scatter, each checked against the CPU oracle on this rank."""
import os
import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))
from __graft_entry__ import load_package  # noqa: E402
from oracle import matmul_oracle as mo  # noqa: E402
sys.path.insert(0, str(REPO / "tests"))
import rank_common  # noqa: E402


def main():
    pkg = load_package()
    rank, world, local, ctx, comm = rank_common.start(pkg)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s = st.cuda_stream

    def host_barrier():
        ctx.synchronize(s)
        comm.barrier(s)
        ctx.synchronize(s)

    rng = np.random.default_rng(123)                      # identical on every rank
    M, N, K = 128 * world * 2, 256 * world, 192 * world
    a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    full = mo.matmul(a, b)

    # N-split + all-gather
    col = pkg.dist.ColumnParallelMatmul(ctx, M, N, K, rank, world, comm)
    ad = torch.from_numpy(a).bfloat16().cuda()
    bd = torch.from_numpy(b[:, col.offset:col.offset + col.width].copy()).bfloat16().cuda()
    ctx.memset(col.c_ptr, 0xFF, M * N * 2, s)             # NaN pattern: an unwritten tile would show
    ctx.synchronize(s)
    host_barrier()
    col.launch(ad, bd, s)
    comm.barrier(s)               # stream-ordered: every peer's stores have landed after it
    host = np.empty(M * N, np.uint16)
    ctx.d2h(host.ctypes.data, col.c_ptr, host.nbytes, s)
    got = mo.from_bf16_bits(host).reshape(M, N)
    assert not np.isnan(got).any(), f"rank {rank}: unwritten tiles in the gathered C"
    err = mo.rel_frobenius(got, full)
    assert err <= 1e-2, f"rank {rank}: all-gather parity {err}"

    # The same all-gather through an NVLink multicast buffer: one multimem.st per box reaches every rank's C. Skipped
    # (with a note) where the GPUs or the driver offer no multicast.
    if ctx.mc_supported():
        mc = pkg.capi.MulticastBuffer(comm, M * N * 2)
        try:
            ctx.memset(mc.local, 0xFF, M * N * 2, s)
            host_barrier()
            d = ctx.gemm_desc(ad, bd, None, M, col.width, K, ldb=col.width, ldc=N)
            ctx.gemm_allgather_mc(d, mc.multicast, world, rank, use_multimem=True, stream=s)
            comm.barrier(s)
            host = np.empty(M * N, np.uint16)
            ctx.d2h(host.ctypes.data, mc.local, host.nbytes, s)
            got = mo.from_bf16_bits(host).reshape(M, N)
            assert not np.isnan(got).any(), f"rank {rank}: unwritten boxes in the multicast C"
            err = mo.rel_frobenius(got, full)
            assert err <= 1e-2, f"rank {rank}: multicast all-gather parity {err}"
            host_barrier()
        finally:
            mc.close()
        if rank == 0:
            print("MULTICAST_ALLGATHER_OK", world)
    elif rank == 0:
        print("MULTICAST_UNSUPPORTED")

    # K-split + reduce-scatter
    row = pkg.dist.RowParallelMatmul(ctx, M, N, K, rank, world, comm)
    a_sh = torch.from_numpy(a[:, row.k_offset:row.k_offset + row.k_depth].copy()).bfloat16().cuda()
    b_sh = torch.from_numpy(b[row.k_offset:row.k_offset + row.k_depth].copy()).bfloat16().cuda()
    host_barrier()
    row.launch_partials(a_sh, b_sh, s)
    comm.barrier(s)
    row.launch_reduce(s)
    host = np.empty(row.rows * N, np.uint16)
    ctx.d2h(host.ctypes.data, row.out, host.nbytes, s)
    got = mo.from_bf16_bits(host).reshape(row.rows, N)
    err = mo.rel_frobenius(got, full[row.row_offset:row.row_offset + row.rows])
    assert err <= 1e-2, f"rank {rank}: reduce-scatter parity {err}"

    host_barrier()
    col.close()
    row.close()
    rank_common.stop(ctx, comm)
    if rank == 0:
        print("DIST_PARITY_OK", world)


if __name__ == "__main__":
    main()
