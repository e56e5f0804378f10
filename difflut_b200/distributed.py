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


class PeerWindow:
    """A CUDA tensor of this rank together with the same-shaped tensor of every other rank of the node.

    The ranks exchange CUDA IPC handles (the mechanism torch.multiprocessing uses to pass CUDA tensors
    between processes) through the process group and every rank opens the others' handles with ITS OWN
    device current, which is what maps the memory into this GPU's address space and lets the driver set up
    peer access (opening it under the exporter's device index, as torch.multiprocessing does for a consumer
    that computes on the exporter's GPU, would leave the mapping in another context of this process, out
    of reach of this GPU's kernels).  `ptrs` is a host array of `world` device pointers indexed by rank,
    in the form the `dl_p2p_*` entry points take.  Plain peer mappings only: no multicast object is
    created.
    """

    def __init__(self, tensor: torch.Tensor, group=None):
        import ctypes

        from torch.multiprocessing.reductions import rebuild_cuda_tensor, reduce_tensor

        from . import _native

        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("PeerWindow needs a contiguous CUDA tensor")
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("PeerWindow supports at most 8 ranks (one node)")
        self.local = tensor
        # Every rank takes part in both exchanges whatever happens locally, and all ranks learn whether
        # every mapping succeeded: either all of them get a window or all of them raise (a caller can then
        # fall back to another exchange on all ranks at once instead of leaving some waiting in a collective).
        error = None
        args = None
        try:
            _, args = reduce_tensor(tensor)
        except Exception as e:  # export failed on this rank
            error = f"export: {e}"
        gathered = [None] * self.world
        dist.all_gather_object(gathered, (tensor.device.index, args), group=group)
        self.tensors = []
        if error is None:
            try:
                with torch.cuda.device(tensor.device):
                    for p, (dev, peer_args) in enumerate(gathered):
                        if p == self.rank:
                            self.tensors.append(tensor)
                            continue
                        if peer_args is None:
                            raise RuntimeError(f"rank {p} could not export its buffer")
                        if dev == tensor.device.index:
                            raise RuntimeError("two ranks share one GPU: peer windows need one GPU per rank")
                        rc = _native.lib().dl_p2p_enable_peer(dev)
                        if rc != 0:
                            raise RuntimeError(f"no peer access from cuda:{tensor.device.index} to cuda:{dev} "
                                               f"(code {rc})")
                        peer_args = list(peer_args)
                        peer_args[6] = tensor.device.index  # storage_device: open the handle on this rank's GPU
                        mapped = rebuild_cuda_tensor(*peer_args)
                        if mapped.numel() != tensor.numel() or mapped.dtype != tensor.dtype:
                            raise RuntimeError("peer tensor does not match the local one")
                        self.tensors.append(mapped)
            except Exception as e:
                error = f"map: {e}"
        ok = torch.tensor([0 if error else 1], device=tensor.device, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)  # also: every rank has mapped every buffer
        if int(ok.item()) == 0:
            self.tensors = []
            raise RuntimeError(f"peer window unavailable ({error or 'another rank failed'})")
        self._array = (ctypes.c_void_p * self.world)(*[t.data_ptr() for t in self.tensors])
        self.ptrs = ctypes.addressof(self._array)
