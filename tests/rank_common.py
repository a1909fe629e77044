"""Shared start-up of the multi-GPU rank workers (tests/dist_rank_worker.py, tests/tp_rank_worker.py): the launcher's
environment gives rank and world size, a gloo group ships the communicator id from rank 0 to the others, and the
library's own communicator (b200_comm_* over NCCL) carries everything the ranks exchange afterwards."""
import os

import torch
import torch.distributed as dist


def start(pkg):
    """Returns (rank, world, local device ordinal, context, communicator)."""
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    ctx = pkg.Context(local)
    box = [pkg.capi.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = pkg.capi.Comm(ctx, box[0], world, rank)
    return rank, world, local, ctx, comm


def stop(ctx, comm):
    comm.close()
    ctx.close()
    dist.barrier()
    dist.destroy_process_group()
