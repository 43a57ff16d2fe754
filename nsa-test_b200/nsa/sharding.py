"""Multi-GPU plumbing of the NSA layer: the path shards by batch / sequence with no collective in the
attention itself; only the compression-MLP and gate-MLP weight gradients are summed over ranks."""
from __future__ import annotations

from typing import Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist


def batch_shard(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced [start, stop) slice of `batch` sequences owned by `rank` (earlier ranks take the
    remainder)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(batch, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def allreduce_grads(grads: Iterable[torch.Tensor], group: Optional[dist.ProcessGroup] = None) -> List[torch.Tensor]:
    """Sum the given gradient tensors over all ranks with ONE all-reduce (flattened fp32 bucket); returns new
    tensors in the inputs' dtypes and shapes.  With no process group initialised it returns the inputs."""
    grads = list(grads)
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1 or not grads:
        return grads
    flat = torch.cat([g.detach().float().reshape(-1) for g in grads])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    out, off = [], 0
    for g in grads:
        n = g.numel()
        out.append(flat[off:off + n].view(g.shape).to(g.dtype))
        off += n
    return out
