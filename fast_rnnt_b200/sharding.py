"""Data-parallel plumbing of the loss: the path shards per utterance, so every
rank works on a contiguous slice of the batch and the only exchange is one
all-reduce of the scalar loss (NCCL over NVLink on GPUs; any torch.distributed
backend works, the CPU tests use gloo)."""
from typing import Dict, Sequence

import torch
import torch.distributed as dist


def shard_range(batch: int, rank: int, world: int):
    """Contiguous, balanced slice [lo, hi) of `batch` utterances for `rank`."""
    base, extra = divmod(batch, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(tensors: Dict[str, torch.Tensor], keys: Sequence[str], rank: int, world: int):
    """Slices the batch dimension (dim 0) of tensors[k] for k in keys; other
    entries (e.g. joiner weights) are passed through."""
    out = dict(tensors)
    for k in keys:
        lo, hi = shard_range(tensors[k].shape[0], rank, world)
        out[k] = tensors[k][lo:hi].contiguous()
    return out


def allreduce_loss(loss: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the per-rank loss sums (in place); a no-op without a process group."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(loss, op=dist.ReduceOp.SUM, group=group)
    return loss
