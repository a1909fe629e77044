"""One rank of the multi-GPU parity job (launched by torchrun from tests/test_dist_gpu.py): real CUDA-IPC peer
buffers, fused GEMM + all-gather and fused GEMM + reduce-scatter, each checked against the CPU oracle on this rank."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))
from __graft_entry__ import load_package  # noqa: E402
from oracle import matmul_oracle as mo  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    ctx = pkg.Context(local)
    st = torch.cuda.Stream()
    torch.cuda.set_stream(st)
    s = st.cuda_stream
    flag = torch.zeros(1, device="cuda")
    rng = np.random.default_rng(123)                      # identical on every rank
    M, N, K = 128 * world * 2, 256 * world, 192 * world
    a = mo.bf16_round(rng.standard_normal((M, K)).astype(np.float32))
    b = mo.bf16_round(rng.standard_normal((K, N)).astype(np.float32))
    full = mo.matmul(a, b)

    # N-split + all-gather
    col = pkg.dist.ColumnParallelMatmul(ctx, M, N, K, rank, world)
    ad = torch.from_numpy(a).bfloat16().cuda()
    bd = torch.from_numpy(b[:, col.offset:col.offset + col.width].copy()).bfloat16().cuda()
    ctx.memset(col.c_ptr, 0xFF, M * N * 2, s)             # NaN pattern: an unwritten tile would show
    ctx.synchronize(s)
    dist.barrier()
    col.launch(ad, bd, s)
    dist.all_reduce(flag)
    host = np.empty(M * N, np.uint16)
    ctx.d2h(host.ctypes.data, col.c_ptr, host.nbytes, s)
    got = mo.from_bf16_bits(host).reshape(M, N)
    assert not np.isnan(got).any(), f"rank {rank}: unwritten tiles in the gathered C"
    err = mo.rel_frobenius(got, full)
    assert err <= 1e-2, f"rank {rank}: all-gather parity {err}"

    # K-split + reduce-scatter
    row = pkg.dist.RowParallelMatmul(ctx, M, N, K, rank, world)
    a_sh = torch.from_numpy(a[:, row.k_offset:row.k_offset + row.k_depth].copy()).bfloat16().cuda()
    b_sh = torch.from_numpy(b[row.k_offset:row.k_offset + row.k_depth].copy()).bfloat16().cuda()
    dist.barrier()
    row.launch_partials(a_sh, b_sh, s)
    dist.all_reduce(flag)
    row.launch_reduce(s)
    host = np.empty(row.rows * N, np.uint16)
    ctx.d2h(host.ctypes.data, row.out, host.nbytes, s)
    got = mo.from_bf16_bits(host).reshape(row.rows, N)
    err = mo.rel_frobenius(got, full[row.row_offset:row.row_offset + row.rows])
    assert err <= 1e-2, f"rank {rank}: reduce-scatter parity {err}"

    dist.barrier()
    col.close()
    row.close()
    ctx.close()
    dist.destroy_process_group()
    if rank == 0:
        print("DIST_PARITY_OK", world)


if __name__ == "__main__":
    main()
