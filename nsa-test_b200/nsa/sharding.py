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


# --------------------------------------------------------------------------------------------------
# long-context mode: queries sharded by position, K/V gathered (one exchange step each way)
# --------------------------------------------------------------------------------------------------

def query_shard(T: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """Contiguous [start, stop) slice of the T positions owned by `rank`; slices are equal and a multiple of the
    kernels' 128-row query tile."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if T % world or (T // world) % multiple:
        raise ValueError(f"T={T} does not split into {world} slices that are multiples of {multiple}")
    step = T // world
    return rank * step, (rank + 1) * step


class _AllGatherSeq(torch.autograd.Function):
    """All-gather of equal slices along `dim`.  Backward: the gradient of the gathered tensor is summed over the ranks
    in fp32 and every rank keeps its own slice (a reduce-scatter; all-reduce + slice where the backend has none)."""

    @staticmethod
    def forward(ctx, x, dim, group):
        world = dist.get_world_size(group)
        ctx.dim, ctx.group, ctx.world, ctx.rank = dim % x.dim(), group, world, dist.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=ctx.dim)

    @staticmethod
    def backward(ctx, g):
        chunks = [c.float().contiguous() for c in g.chunk(ctx.world, dim=ctx.dim)]
        if dist.get_backend(ctx.group) == "nccl":
            out = torch.empty_like(chunks[ctx.rank])
            dist.reduce_scatter(out, chunks, op=dist.ReduceOp.SUM, group=ctx.group)
        else:
            full = torch.cat(chunks, dim=ctx.dim)
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=ctx.group)
            out = full.chunk(ctx.world, dim=ctx.dim)[ctx.rank]
        return out.to(g.dtype), None, None


def all_gather_seq(x: torch.Tensor, dim: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Differentiable all-gather along `dim` (identity without a process group or with one rank)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return x
    return _AllGatherSeq.apply(x, dim, group)


def query_sharded_layer(q_local, k_local, v_local, gate_logits_local, phi_params, config, group=None, **kw):
    """The NSA layer with the sequence split by position over the ranks of `group`: every rank holds the q
    [B,H,T/N,dk], k [B,G,dk,T/N], v [B,G,T/N,dv] and gate-logit slices of its positions.  K and V are all-gathered
    (their gradients come back reduce-scattered), each rank then runs its query slice against the gathered keys; the
    compressed keys/values are recomputed from the gathered K/V on every rank (a few percent of the layer's work)
    instead of being exchanged.  Weight gradients (phi, gate MLP) still need `allreduce_grads`."""
    from .kernels import nsa_layer
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    Tl = q_local.shape[2]
    k_full = all_gather_seq(k_local, -1, group)
    v_full = all_gather_seq(v_local, 2, group)
    return nsa_layer(q_local, k_full, v_full, gate_logits_local, phi_params, config, q_pos0=rank * Tl, **kw)
