"""Batch sharding of independent particle systems over the GPUs of one node.

Every perception kernel indexes (system, particle) and never reads across systems, so a batch
of B systems shards over W ranks with no collective on the data path: rank r owns systems
``[r*B/W, (r+1)*B/W)`` and its own ``HashGrid(batch_size=B/W)``.  The only exchange of
data-parallel training is one all-reduce of the (tiny) MLP parameter gradients per optimizer
step, issued after ``loss.backward()`` and BEFORE the reference's per-parameter gradient
normalisation (``NPA.normalize_grads``, models/npa.py:162-165), which is non-linear.

One process per GPU (``torchrun`` / ``torch.distributed``); backend ``nccl`` on GPUs, ``gloo``
for CPU-side tests of this logic.
"""
from __future__ import annotations

import os
from typing import Iterable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(num_systems: int, rank: int, world: int) -> Tuple[int, int]:
    """Half-open range of the systems rank ``rank`` of ``world`` owns (contiguous, sizes differ by <= 1)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} of world {world}")
    if num_systems < 0:
        raise ValueError("num_systems must be non-negative")
    base, extra = divmod(num_systems, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's slice of a ``[B, ...]`` tensor (a view)."""
    lo, hi = shard_range(t.shape[0], rank, world)
    return t[lo:hi]


def init_from_env(backend: Optional[str] = None) -> Tuple[int, int, int]:
    """Join the process group described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* (torchrun's
    environment).  Returns ``(rank, world, local_rank)``; a single process needs no group."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
            kwargs["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, **kwargs)
    return rank, world, local_rank


def bind_to_gpu_cpus(device_index: int) -> Optional[set]:
    """Restrict this process to the CPU cores the driver reports as closest to the GPU (its NUMA
    node), so that the pinned host buffers allocated afterwards sit on that node and host <-> device
    copies of the ranks of one machine do not all cross the socket interconnect.  Read-only use of
    NVML; returns the core set, or None when it cannot be determined (nothing is changed then).
    ``device_index`` counts visible devices (CUDA_VISIBLE_DEVICES is honoured)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            if visible:
                ident = visible.split(",")[device_index].strip()
                handle = (pynvml.nvmlDeviceGetHandleByUUID(ident) if ident.startswith("GPU-")
                          else pynvml.nvmlDeviceGetHandleByIndex(int(ident)))
            else:
                handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            words = (os.cpu_count() + 63) // 64
            mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        finally:
            pynvml.nvmlShutdown()
        cpus = {64 * w + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return cpus
    except Exception:
        return None


def local_grid(rank: int, world: int, *, batch_size: int, **hashgrid_kwargs):
    """``HashGrid`` for this rank's share of a global batch of ``batch_size`` systems."""
    from .sphops import HashGrid

    lo, hi = shard_range(batch_size, rank, world)
    if hi == lo:
        raise ValueError(f"rank {rank} of {world} owns no system of a batch of {batch_size}")
    return HashGrid(batch_size=hi - lo, **hashgrid_kwargs)


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, average: bool = True,
                        weight: Optional[float] = None) -> int:
    """All-reduce the ``.grad`` of ``params`` as ONE flat buffer; returns the number of floats sent.

    ``average=True`` divides by the world size, which reproduces the single-process gradient when
    the loss is a batch mean and shards are equal.  For unequal shards pass ``weight`` = this
    rank's share of the global batch (its gradients are scaled by it and summed instead).
    Parameters without a gradient contribute zeros so that every rank sends the same layout.
    """
    params = [p for p in params if p.requires_grad]
    if not params or not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return 0
    flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float() for p in params])
    if weight is not None:
        flat.mul_(float(weight))
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    if weight is None and average:
        flat.div_(dist.get_world_size(group))
    off = 0
    for p in params:
        n = p.numel()
        g = flat[off:off + n].view_as(p).to(p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += n
    return int(flat.numel())
