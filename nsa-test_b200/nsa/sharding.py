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


def balanced_query_bounds(T: int, world: int, per_query_fixed: float, d: int, multiple: int = 128) -> List[int]:
    """Slice boundaries [0 = b_0 < b_1 < ... < b_world = T] (multiples of the 128-row query tile) that give every rank about
    the same attention work when the cost of the query at position t is ``per_query_fixed + t / d`` keys: a constant for
    the sliding window and the selected blocks, plus the compressed keys it can see, which grow with t.  Equal slices
    would leave the last rank with most of the causal work."""
    if T % multiple or T // multiple < world:
        raise ValueError(f"T={T} does not split into {world} slices that are multiples of {multiple}")
    c0 = float(per_query_fixed)
    total = c0 * T + T * T / (2.0 * d)
    bounds = [0]
    for r in range(1, world):
        target = total * r / world
        s_ = d * (-c0 + (c0 * c0 + 2.0 * target / d) ** 0.5)
        b = int(round(s_ / multiple)) * multiple
        b = max(b, bounds[-1] + multiple)
        b = min(b, T - (world - r) * multiple)
        bounds.append(b)
    bounds.append(T)
    return bounds


class _AllGatherSeq(torch.autograd.Function):
    """All-gather of slices along `dim` (``sizes``: every rank's slice length; equal slices when None).  Backward: the
    gradient of the gathered tensor is summed over the ranks in fp32 and every rank keeps its own slice (a reduce-scatter;
    all-reduce + slice where the backend has none).  Uneven slices travel padded to the longest one."""

    @staticmethod
    def forward(ctx, x, dim, group, sizes=None):
        world = dist.get_world_size(group)
        dim = dim % x.dim()
        sizes = [x.shape[dim]] * world if sizes is None else [int(v_) for v_ in sizes]
        ctx.dim, ctx.group, ctx.world, ctx.rank, ctx.sizes = dim, group, world, dist.get_rank(group), sizes
        big = max(sizes)
        xp = x.contiguous()
        if xp.shape[dim] < big:
            pad_shape = list(xp.shape)
            pad_shape[dim] = big - xp.shape[dim]
            xp = torch.cat([xp, xp.new_zeros(pad_shape)], dim=dim)
        parts = [torch.empty_like(xp) for _ in range(world)]
        dist.all_gather(parts, xp, group=group)
        return torch.cat([p_.narrow(dim, 0, n_) for p_, n_ in zip(parts, sizes)], dim=dim)

    @staticmethod
    def backward(ctx, g):
        big = max(ctx.sizes)
        dim = ctx.dim
        # A gradient whose last two dimensions are swapped in memory (dK arrives as the transposed view of a time-major
        # buffer) is split, widened and summed in that layout: every pass then reads and writes whole lines.
        swapped = (not g.is_contiguous()) and g.dim() >= 2 and dim == g.dim() - 1 and g.transpose(-1, -2).is_contiguous()
        if swapped:
            g, dim = g.transpose(-1, -2), dim - 1
        chunks = []
        for c in g.split(ctx.sizes, dim=dim):
            c = c.float()
            if c.shape[dim] < big:
                pad_shape = list(c.shape)
                pad_shape[dim] = big - c.shape[dim]
                c = torch.cat([c, c.new_zeros(pad_shape)], dim=dim)
            chunks.append(c.contiguous())
        if dist.get_backend(ctx.group) == "nccl":
            out = torch.empty_like(chunks[ctx.rank])
            dist.reduce_scatter(out, chunks, op=dist.ReduceOp.SUM, group=ctx.group)
        else:
            full = torch.stack(chunks)
            dist.all_reduce(full, op=dist.ReduceOp.SUM, group=ctx.group)
            out = full[ctx.rank]
        out = out.narrow(dim, 0, ctx.sizes[ctx.rank]).to(g.dtype)
        return (out.transpose(-1, -2) if swapped else out), None, None, None


def all_gather_seq(x: torch.Tensor, dim: int, group: Optional[dist.ProcessGroup] = None, sizes=None) -> torch.Tensor:
    """Differentiable all-gather along `dim` (identity without a process group or with one rank)."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return x
    return _AllGatherSeq.apply(x, dim, group, sizes)


def owned_block_range(bounds: List[int], rank: int, l: int, d: int, T: int) -> Tuple[int, int]:
    """Compressed blocks [b0, b1) that `rank` computes in the long-context mode: block i covers tokens [i*d, i*d + l);
    it belongs to the rank whose position slice holds its first token.  Slice boundaries are multiples of d, and the
    sequence has (T - l) // d + 1 blocks (the last rank owns fewer: blocks that would reach beyond T do not exist)."""
    nb = (T - l) // d + 1 if T >= l else 0
    t0, t1 = bounds[rank], bounds[rank + 1]
    if t0 % d or t1 % d:
        raise ValueError(f"slice [{t0}, {t1}) does not start and end at multiples of the compression stride {d}")
    return min(t0 // d, nb), min(t1 // d, nb)


def sharded_compress(k_full, v_full, compress_fn, bounds: List[int], rank: int, l: int, d: int,
                     group: Optional[dist.ProcessGroup] = None):
    """Block compression with the work split over the ranks: every rank compresses the blocks it owns
    (`owned_block_range`) from the gathered keys/values (a block may reach up to l - d tokens into the next rank's
    slice) and the compressed keys/values are all-gathered (12.6 MB + 4.2 MB at T = 64K instead of every rank running
    phi over the whole sequence).  In backward the gradients of the gathered compressed tensors are reduce-scattered
    to the owners, whose phi backward then adds to the gradient of the gathered K/V.

    k_full [B,G,dk,T], v_full [B,G,T,dv]; ``compress_fn(keys [B,G,Tn,dk], values [B,G,Tn,dv]) -> (k_cmp [B,G,dk,>=n],
    v_cmp [B,G,>=n,dv])`` compresses a token range into its (Tn - l) // d + 1 blocks.  Returns k_cmp [B,G,dk,nb],
    v_cmp [B,G,nb,dv] of the whole sequence (not padded)."""
    T = k_full.shape[-1]
    world = len(bounds) - 1
    ranges = [owned_block_range(bounds, r, l, d, T) for r in range(world)]
    b0, b1 = ranges[rank]
    cnt = b1 - b0
    B, G, dk = k_full.shape[:3]
    dv = v_full.shape[-1]
    if cnt > 0:
        lo, hi = b0 * d, (b1 - 1) * d + l
        # (slice of the transposed view: the slice's backward then builds its zero-filled full-length gradient in the
        # time-major memory layout the attention branches' dK has, so autograd adds the two without a strided pass)
        kc, vc = compress_fn(k_full.transpose(-1, -2)[:, :, lo:hi], v_full[:, :, lo:hi])
        kc, vc = kc[..., :cnt], vc[:, :, :cnt]
    else:
        kc = k_full.new_zeros(B, G, dk, 0, dtype=torch.float32)
        vc = v_full.new_zeros(B, G, 0, dv)
    sizes = [r1 - r0 for r0, r1 in ranges]
    if max(sizes) == 0:
        return kc, vc
    return all_gather_seq(kc.contiguous(), -1, group, sizes), all_gather_seq(vc.contiguous(), 2, group, sizes)


def query_sharded_layer(q_local, k_local, v_local, gate_logits_local, phi_params, config, group=None, bounds=None, **kw):
    """The NSA layer with the sequence split by position over the ranks of `group`: every rank holds the q
    [B,H,Tr,dk], k [B,G,dk,Tr], v [B,G,Tr,dv] and gate-logit slices of its positions ``bounds[rank]:bounds[rank+1]``
    (equal slices when ``bounds`` is None; see `balanced_query_bounds`).  K and V are all-gathered (their gradients
    come back reduce-scattered); the block compression is split over the ranks too and its results all-gathered
    (`sharded_compress`); each rank then runs its query slice against the gathered keys.  Weight gradients (phi, gate
    MLP) still need `allreduce_grads`."""
    from .kernels import _PhiCompress, nsa_layer
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    if world == 1:
        return nsa_layer(q_local, k_local, v_local, gate_logits_local, phi_params, config, **kw)
    if bounds is None:
        step = q_local.shape[2]
        bounds = [r * step for r in range(world + 1)]
    sizes, q_pos0 = [bounds[i + 1] - bounds[i] for i in range(world)], bounds[rank]
    k_full = all_gather_seq(k_local, -1, group, sizes)
    v_full = all_gather_seq(v_local, 2, group, sizes)
    compress = lambda keys, values: _PhiCompress.apply(keys, values, *phi_params, config.l, config.d)
    k_cmp, v_cmp = sharded_compress(k_full, v_full, compress, bounds, rank, config.l, config.d, group)
    return nsa_layer(q_local, k_full, v_full, gate_logits_local, phi_params, config, q_pos0=q_pos0, compressed=(k_cmp, v_cmp),
                     **kw)
