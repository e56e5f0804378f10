"""Data-parallel plumbing: one process per GPU, batch rows sharded, table gradients all-reduced.

The reference has no distributed code.  Training shards the global batch into contiguous row
blocks; every rank holds the full tables and index maps; the only exchange per step is a sum
all-reduce of the flat table-gradient buffer.  Inference shards rows with no communication.
"""

import datetime
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist


def init_from_env(backend: Optional[str] = None, timeout_s: float = 180.0) -> Tuple[int, int, int]:
    """Initialise the default process group from RANK / WORLD_SIZE / LOCAL_RANK / MASTER_*.

    Returns (rank, world, local_rank).  Without WORLD_SIZE > 1 nothing is initialised.  A collective
    that a rank never joins ends with an error after `timeout_s` instead of waiting forever.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local),
                                    timeout=datetime.timedelta(seconds=timeout_s))
        else:
            dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s))
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return rank, world, local


def shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """[start, stop) of the contiguous row block of `rank`; the first `total % world` ranks get
    one extra row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(total_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allreduce_sum_(flat: torch.Tensor, group=None, async_op: bool = False):
    """In-place sum all-reduce of a flat gradient buffer (no-op outside a process group).

    Returns the tensor, or with `async_op` the work handle to `wait()` on (None when nothing ran)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)
        return work if async_op else flat
    return None if async_op else flat


def max_over_ranks(value: float, device=None) -> float:
    """Max of a host scalar over all ranks (used for timings)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
