"""CPU oracle for the NSA layer hot path.  TEST INFRASTRUCTURE ONLY.

This module is a CPU (PyTorch, fp32/fp64) restatement of the algorithms of the
reference project (Noumena-Network/NSA-Test).  It exists so that the CUDA path
can be checked against something that runs where no reference checkout exists.
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it; the shipped package never does.

Parity status: PINNED.  Every function below is compared against the reference's
own code (imported from a reference checkout) by ``tests/golden/make_golden.py``;
the outputs of that comparison run are committed as ``tests/golden/*.npz`` and
re-checked by ``tests/test_oracle_golden.py`` on every CPU test run.

Each function cites the reference lines it restates (paths are relative to the
reference project root).  The restatement is vectorised: the reference loops
over (batch, head, token) in Python, this code applies a boolean visibility
mask to chunked dense scores instead, which yields the same numbers up to fp32
re-association.  Backward passes come from autograd, exactly as the reference's
CPU path obtains them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch
import torch.utils.checkpoint

PAD_BLOCK_END = 999999  # sentinel block end of padded compressed blocks (nsa/kernels.py:2190)
LOW_MEMORY = False      # True: the dense score chunks are recomputed in backward (same numbers, a fraction of the memory)


# ----------------------------------------------------------------------------------------------
# generic masked attention
# ----------------------------------------------------------------------------------------------

def _expand_groups(x: torch.Tensor, H: int) -> torch.Tensor:
    """[B,G,...] -> [B,H,...] by repeating each KV group for its heads (nsa/reference.py:41-48)."""
    B, G = x.shape[:2]
    return x.unsqueeze(2).expand(B, G, H // G, *x.shape[2:]).reshape(B, H, *x.shape[2:])


def masked_attention(
    q: torch.Tensor,            # [B,H,T,dk]
    k: torch.Tensor,            # [B,G,dk,Tk]   (reference layout: dk before time)
    v: torch.Tensor,            # [B,G,Tk,dv]
    visible: Callable[[int, int], torch.Tensor],  # (t0,t1) -> bool [*,*,t1-t0,Tk] broadcastable to [B,H,.,.]
    scale: float,
    chunk: int = 256,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """softmax(q k * scale over visible keys) v, with the per-row statistics the kernels store.

    Returns (out [B,H,T,dv], M [B,H,T], L [B,H,T]) where M is the row maximum of the scaled
    logits and L = log(sum(exp(s - M))) (natural log), so that logsumexp = M + L.  A row with no
    visible key gives out = 0 and M = L = -inf (nsa/kernels.py:818-833, nsa/reference.py:133-141).
    """
    B, H, T, dk = q.shape
    ke = _expand_groups(k, H)
    ve = _expand_groups(v, H)

    def one_chunk(qc, ke_, ve_, vis):
        s = torch.matmul(qc * scale, ke_)                                   # [B,H,c,Tk]
        s = s.masked_fill(~vis, float("-inf"))
        m = s.amax(dim=-1, keepdim=True)
        has = torch.isfinite(m)
        m_safe = torch.where(has, m, torch.zeros_like(m))
        e = torch.exp(s - m_safe)                                           # masked -> exp(-inf) = 0
        l = e.sum(dim=-1, keepdim=True)
        p = e / torch.where(has, l, torch.ones_like(l))
        L_ = torch.where(has, torch.log(torch.where(has, l, torch.ones_like(l))), torch.full_like(l, float("-inf")))
        return torch.matmul(p, ve_), m.squeeze(-1), L_.squeeze(-1)

    outs, Ms, Ls = [], [], []
    for t0 in range(0, T, chunk):
        t1 = min(T, t0 + chunk)
        vis = visible(t0, t1)
        if LOW_MEMORY and torch.is_grad_enabled():
            # same operations, recomputed in the backward pass instead of kept: long sequences with many heads
            o_, m_, l_ = torch.utils.checkpoint.checkpoint(one_chunk, q[:, :, t0:t1], ke, ve, vis, use_reentrant=False)
        else:
            o_, m_, l_ = one_chunk(q[:, :, t0:t1], ke, ve, vis)
        outs.append(o_)
        Ms.append(m_)
        Ls.append(l_)
    return torch.cat(outs, 2), torch.cat(Ms, 2), torch.cat(Ls, 2)


def sliding_window_attention(q, k, v, window_size: int, scale: Optional[float] = None, *,
                             return_stats: bool = False):
    """Causal window attention: query t sees keys [max(0,t-w+1), t] (nsa/reference.py:13-78)."""
    T = q.shape[2]
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    kpos = torch.arange(k.shape[-1])

    def vis(t0, t1):
        t = torch.arange(t0, t1)[:, None]
        return ((kpos[None, :] <= t) & (kpos[None, :] > t - window_size))[None, None]

    o, M, L = masked_attention(q, k, v, vis, scale)
    return (o, M, L) if return_stats else o


def compression_attention(q, k_cmp, v_cmp, block_ends, scale: Optional[float] = None, *,
                          return_stats: bool = False):
    """Attention over compressed tokens; block i visible iff block_ends[i] <= t; rows that see no
    block output zero (nsa/reference.py:81-147; kernel mask nsa/kernels.py:1646)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    be = block_ends.to(torch.int64)

    def vis(t0, t1):
        t = torch.arange(t0, t1)[:, None]
        return (be[None, :] <= t)[None, None]

    o, M, L = masked_attention(q, k_cmp, v_cmp, vis, scale)
    return (o, M, L) if return_stats else o


def selection_fallback_indices(indices: torch.Tensor, l_prime: int) -> torch.Tensor:
    """Rows whose slots are all -1 fall back to the block holding the query (nsa/kernels.py:199-205)."""
    T = indices.shape[2]
    t_blocks = (torch.arange(T, dtype=indices.dtype) // l_prime).view(1, 1, T, 1)
    none_valid = (indices < 0).all(dim=-1, keepdim=True)
    return torch.where(none_valid, t_blocks, indices)


def selection_attention(q, k, v, indices, l_prime: int, scale: Optional[float] = None, *,
                        return_stats: bool = False):
    """Attention over the union of the selected l'-blocks of the query's KV group, causally masked;
    ids < 0 and blocks starting at or beyond the KV length are ignored (nsa/reference.py:205-254)."""
    B, H, T, _ = q.shape
    G = k.shape[1]
    Tk = k.shape[-1]
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    nblk = (Tk + l_prime - 1) // l_prime
    kblk = torch.arange(Tk) // l_prime
    kpos = torch.arange(Tk)

    def vis(t0, t1):
        idx = indices[:, :, t0:t1].to(torch.int64)                          # [B,G,c,n]
        ok = (idx >= 0) & (idx < nblk)
        sel = torch.zeros(B, G, t1 - t0, nblk + 1, dtype=torch.bool)
        sel.scatter_(-1, torch.where(ok, idx, torch.full_like(idx, nblk)), True)
        sel = sel[..., :nblk]                                                # block membership
        m = sel[..., kblk]                                                   # [B,G,c,Tk]
        m = m & (kpos[None, :] <= torch.arange(t0, t1)[:, None])[None, None]
        return _expand_groups(m, H)

    o, M, L = masked_attention(q, k, v, vis, scale)
    return (o, M, L) if return_stats else o


# ----------------------------------------------------------------------------------------------
# compression MLP phi, Eq. 8, Eq. 9, Eq. 10/11
# ----------------------------------------------------------------------------------------------

@dataclass
class PhiParams:
    """Weights of the block-compression MLP (nsa/kernels.py:2096-2102)."""
    pos_embed: torch.Tensor   # [l, l]
    w1: torch.Tensor          # [2dk, dk+l]
    b1: torch.Tensor          # [2dk]
    w2: torch.Tensor          # [dk, 2dk]
    b2: torch.Tensor          # [dk]


def next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def compress_tokens(keys: torch.Tensor, values: torch.Tensor, phi: PhiParams, l: int, d: int):
    """Block compression (nsa/kernels.py:2119-2208).

    keys [B,G,T,dk], values [B,G,T,dv] (time-major).  Block i covers tokens [i*d, i*d+l);
    k_cmp[i] = mean_j MLP([k_j || pos_embed(j - i*d)]), v_cmp[i] = mean_j v_j.  The block count is
    padded to the next power of two with zero blocks whose block end is 999999.
    Returns (k_cmp [B,G,dk,nbp], v_cmp [B,G,nbp,dv], block_ends [nbp] int32, n_blocks_actual).
    """
    B, G, T, dk = keys.shape
    dv = values.shape[-1]
    nb = max(0, (T - l) // d + 1)
    nbp = next_pow2(nb)
    if nb == 0:
        # a sequence shorter than one block: the reference's loop runs zero times and only the padding block is left
        # (nsa/kernels.py:2137-2142, 2181-2186); every row then falls back to block 0 in Eq. 8
        return (torch.zeros(B, G, dk, nbp, dtype=keys.dtype), torch.zeros(B, G, nbp, dv, dtype=values.dtype),
                torch.full((nbp,), PAD_BLOCK_END, dtype=torch.int32), 0)
    kb = keys.unfold(2, l, d)[:, :, :nb].permute(0, 1, 2, 4, 3)             # [B,G,nb,l,dk]
    vb = values.unfold(2, l, d)[:, :, :nb].permute(0, 1, 2, 4, 3)           # [B,G,nb,l,dv]
    pos = phi.pos_embed.to(keys.dtype).view(1, 1, 1, l, l).expand(B, G, nb, l, l)
    x = torch.cat([kb, pos], dim=-1)
    h = torch.relu(torch.nn.functional.linear(x, phi.w1, phi.b1))
    kc = torch.nn.functional.linear(h, phi.w2, phi.b2).mean(dim=3)          # [B,G,nb,dk]
    vc = vb.mean(dim=3)                                                     # [B,G,nb,dv]
    k_cmp = torch.zeros(B, G, dk, nbp, dtype=keys.dtype)
    v_cmp = torch.zeros(B, G, nbp, dv, dtype=values.dtype)
    k_cmp = torch.cat([kc.transpose(-1, -2), k_cmp[..., nb:]], dim=-1)
    v_cmp = torch.cat([vc, v_cmp[:, :, nb:]], dim=2)
    block_ends = torch.full((nbp,), PAD_BLOCK_END, dtype=torch.int32)
    block_ends[:nb] = torch.arange(nb, dtype=torch.int32) * d + (l - 1)
    return k_cmp, v_cmp, block_ends, nb


def compression_probabilities(q, k_cmp, block_ends, scale: float, positions=None) -> torch.Tensor:
    """Eq. 8 (nsa/kernels.py:2316-2343): softmax over visible compressed blocks; a row that sees no
    block falls back to block 0 alone (one-hot).  Returns [B,H,T,nbp].  ``positions`` [T] gives the
    sequence position of every query row when the rows are a sample of a longer sequence (row t sits
    at position t by default, as in the reference)."""
    B, H, T, _ = q.shape
    ke = _expand_groups(k_cmp, H)
    s = torch.matmul(q, ke) * scale
    t = torch.arange(T) if positions is None else positions.to(torch.int64)
    vis = block_ends.to(torch.int64)[None, :] <= t[:, None]                  # [T,nbp]
    first = torch.zeros_like(vis)
    first[:, 0] = True
    vis = vis | (first & ~vis.any(dim=-1, keepdim=True))
    s = s.masked_fill(~vis[None, None], float("-inf"))
    return torch.softmax(s, dim=-1)


def selection_scores_from_compression(p_cmp: torch.Tensor, l: int, d: int, l_prime: int) -> torch.Tensor:
    """Eq. 9 (nsa/kernels.py:1943-1960): sel[j] = sum_{m<s} sum_{n<a} p[s*j+m+n] with a=l/d,
    s=l'/d, n_sel = ceil(n_cmp/s) on the padded block count, out-of-range terms skipped, fp32 adds
    issued in (m outer, n inner) order starting from zero."""
    n_cmp = p_cmp.shape[-1]
    a, s = l // d, l_prime // d
    n_sel = (n_cmp + s - 1) // s
    base = s * torch.arange(n_sel)
    padded = torch.cat([p_cmp, torch.zeros(*p_cmp.shape[:-1], s + a, dtype=p_cmp.dtype)], dim=-1)
    out = torch.zeros(*p_cmp.shape[:-1], n_sel, dtype=p_cmp.dtype)
    for m in range(s):
        for n in range(a):
            out = out + padded[..., base + m + n]     # the zero padding stands for skipped terms
    return out


def select_top_n(sel_scores: torch.Tensor, G: int, n: int, l_prime: int,
                 include_fixed: bool = True, n_fixed: int = 3, positions=None) -> torch.Tensor:
    """Eq. 10/11 (nsa/kernels.py:1986-2040): sum the heads of each group, stable descending sort
    (ties to the lower block id), keep min(n, n_blocks); with fixed blocks, prepend
    [0, max(0,(t-l')//l'), t//l'], drop repeats keeping first occurrences, cut to n, pad with -1.
    Returns int64 [B,G,T,n].  ``positions`` as in compression_probabilities."""
    B, H, T, nb = sel_scores.shape
    agg = sel_scores.view(B, G, H // G, T, nb).sum(dim=2)
    order = torch.sort(agg, dim=-1, descending=True, stable=True).indices[..., : min(n, nb)]
    if not (include_fixed and n_fixed > 0):
        pad = torch.full((B, G, T, n - order.shape[-1]), -1, dtype=torch.int64)
        return torch.cat([order, pad], dim=-1)[..., :n]
    t = torch.arange(T) if positions is None else positions.to(torch.int64)
    fixed = torch.stack([torch.zeros_like(t), torch.clamp((t - l_prime) // l_prime, min=0), t // l_prime], -1)
    cand = torch.cat([fixed.view(1, 1, T, 3).expand(B, G, T, 3), order], dim=-1)   # [B,G,T,C]
    C = cand.shape[-1]
    same = cand.unsqueeze(-1) == cand.unsqueeze(-2)                          # [.,C,C]
    earlier = torch.tril(torch.ones(C, C, dtype=torch.bool), diagonal=-1)
    keep = ~(same & earlier).any(dim=-1)
    rank = torch.cumsum(keep.to(torch.int64), dim=-1) - 1
    out = torch.full((B, G, T, n + 1), -1, dtype=torch.int64)
    slot = torch.where(keep & (rank < n), rank, torch.full_like(rank, n))
    out.scatter_(-1, slot, cand)
    return out[..., :n]


# ----------------------------------------------------------------------------------------------
# the three branches for a SAMPLE of query rows of a long sequence (row-by-row, as the reference loops)
# ----------------------------------------------------------------------------------------------

def _row_attention(qr: torch.Tensor, keys: torch.Tensor, vals: torch.Tensor, scale: float) -> torch.Tensor:
    """One query position, the heads of one KV group: qr [hpg,dk], keys [dk,N], vals [N,dv] -> [hpg,dv];
    N = 0 gives zeros (nsa/reference.py:133-141)."""
    if keys.shape[-1] == 0:
        return qr.new_zeros(qr.shape[0], vals.shape[-1])
    p = torch.softmax((qr @ keys) * scale, dim=-1)
    return p @ vals


def branch_rows(q_rows, positions, k, v, k_cmp, v_cmp, block_ends, indices_rows, *, w: int, l_prime: int,
                scale: Optional[float] = None):
    """O_cmp, O_slc, O_win for sampled query rows of a sequence too long for the dense functions above.

    q_rows [B,H,S,dk] are the queries at ``positions`` [S]; k [B,G,dk,T], v [B,G,T,dv] the whole
    sequence; indices_rows [B,G,S,n] the selected blocks of those rows (all -1 falls back to the
    query's own block, nsa/kernels.py:199-205).  Follows the reference's per-(batch, head, token) loops:
    window keys [max(0,t-w+1), t] (nsa/reference.py:50-77), compressed blocks with block_ends <= t
    (nsa/reference.py:116-141), union of the selected blocks clipped causally, ids < 0 or starting
    beyond the keys ignored (nsa/reference.py:232-251).  Returns three [B,H,S,dv] tensors."""
    B, H, S, dk = q_rows.shape
    G, T = k.shape[1], k.shape[-1]
    hpg = H // G
    scale = 1.0 / math.sqrt(dk) if scale is None else scale
    dv = v.shape[-1]
    o_cmp, o_slc, o_win = (q_rows.new_zeros(B, H, S, dv) for _ in range(3))
    be = block_ends.to(torch.int64)
    for b in range(B):
        for g in range(G):
            hs = slice(g * hpg, (g + 1) * hpg)
            for i, t in enumerate(int(x) for x in positions):
                qr = q_rows[b, hs, i]
                lo = max(0, t - w + 1)
                o_win[b, hs, i] = _row_attention(qr, k[b, g, :, lo:t + 1], v[b, g, lo:t + 1], scale)
                vis = (be <= t).nonzero().flatten()
                o_cmp[b, hs, i] = _row_attention(qr, k_cmp[b, g][:, vis], v_cmp[b, g][vis], scale)
                ids = [int(x) for x in indices_rows[b, g, i]]
                if all(x < 0 for x in ids):
                    ids = [t // l_prime]
                keys = sorted({x for x in ids if x >= 0 and x * l_prime < T and x * l_prime <= t})   # future blocks hold no key <= t
                pos = torch.cat([torch.arange(x * l_prime, min((x + 1) * l_prime, T, t + 1)) for x in keys]) if keys \
                    else torch.zeros(0, dtype=torch.int64)
                o_slc[b, hs, i] = _row_attention(qr, k[b, g][:, pos], v[b, g][pos], scale)
    return o_cmp, o_slc, o_win


def score_rows(q_rows, positions, k_cmp, block_ends, *, l: int, d: int, l_prime: int, n: int, scale: float,
               include_fixed: bool = True, n_fixed: int = 3):
    """Eq. 8 -> 9 -> 10/11 for sampled query rows: returns (indices [B,G,S,n] int64, aggregated scores
    [B,G,S,n_sel]); the same three functions the layer composes, told the rows' positions."""
    B, H, S, _ = q_rows.shape
    G = k_cmp.shape[1]
    p = compression_probabilities(q_rows, k_cmp, block_ends, scale, positions)
    sel = selection_scores_from_compression(p, l, d, l_prime)
    idx = select_top_n(sel, G, n, l_prime, include_fixed, n_fixed if include_fixed else 0, positions)
    return idx, sel.view(B, G, H // G, S, -1).sum(dim=2)


# ----------------------------------------------------------------------------------------------
# gate + mix, and the whole layer
# ----------------------------------------------------------------------------------------------

@dataclass
class GateParams:
    """Weights of the branch-gate MLP (nsa/kernels.py:2105-2109)."""
    w1: torch.Tensor   # [d_model/2, d_model]
    b1: torch.Tensor
    w2: torch.Tensor   # [3H, d_model/2]
    b2: torch.Tensor


def gates_from_hidden(x: torch.Tensor, gp: GateParams, H: int, gate_mode: str) -> torch.Tensor:
    """[B,T,d_model] -> gates [B,H,T,3]; column 0 compression, 1 selection, 2 sliding
    (nsa/kernels.py:2446-2451)."""
    B, T, _ = x.shape
    logits = torch.nn.functional.linear(torch.relu(torch.nn.functional.linear(x, gp.w1, gp.b1)), gp.w2, gp.b2)
    g = logits.view(B, T, H, 3).permute(0, 2, 1, 3)
    return torch.softmax(g, dim=-1) if gate_mode == "softmax" else torch.sigmoid(g)


def mix_branches(gates, o_cmp, o_slc, o_win):
    """o = g0*o_cmp + g1*o_slc + g2*o_win (nsa/kernels.py:2461-2463)."""
    return o_cmp * gates[..., 0:1] + o_slc * gates[..., 1:2] + o_win * gates[..., 2:3]


def nsa_layer(q, k, v, x, phi: PhiParams, gp: GateParams, *, l=32, d=16, l_prime=64, n=16, w=512,
              include_fixed=True, n_fixed=3, gate_mode="sigmoid", scale=None,
              kv_compress=None, kv_sliding=None, indices=None) -> Dict[str, torch.Tensor]:
    """The layer between the q/k/v projections and o_proj.

    Composition of nsa/kernels.py:2298-2463 with the training-path fallback for all-(-1) index rows
    (nsa/kernels.py:199-205).  q [B,H,T,dk], k [B,G,dk,T], v [B,G,T,dv], x [B,T,d_model].  By
    default one k,v feeds the three branches; ``kv_compress`` / ``kv_sliding`` give the compression
    and sliding branches their own (k,v) as the reference module's separate projections do, (k,v)
    then being the selection branch's.  ``indices`` [B,G,T,n] replaces the layer's own top-n choice
    (used to compare implementations on identical selections; the scoring still runs and is returned).
    """
    B, H, T, dk = q.shape
    G = k.shape[1]
    scale = 1.0 / math.sqrt(dk) if scale is None else scale
    kc_src, vc_src = kv_compress if kv_compress is not None else (k, v)
    kw, vw = kv_sliding if kv_sliding is not None else (k, v)
    k_cmp, v_cmp, block_ends, nb = compress_tokens(kc_src.transpose(-1, -2), vc_src, phi, l, d)
    p_cmp = compression_probabilities(q, k_cmp, block_ends, scale)
    sel = selection_scores_from_compression(p_cmp, l, d, l_prime)
    idx_own = select_top_n(sel.detach(), G, n, l_prime, include_fixed, n_fixed if include_fixed else 0)
    idx = idx_own if indices is None else indices.to(torch.int64)
    o_cmp = compression_attention(q, k_cmp, v_cmp, block_ends, scale)
    o_slc = selection_attention(q, k, v, selection_fallback_indices(idx, l_prime), l_prime, scale)
    o_win = sliding_window_attention(q, kw, vw, w, scale)
    gates = gates_from_hidden(x, gp, H, gate_mode)
    out = mix_branches(gates, o_cmp, o_slc, o_win)
    return dict(out=out, o_cmp=o_cmp, o_slc=o_slc, o_win=o_win, indices=idx, gates=gates,
                k_cmp=k_cmp, v_cmp=v_cmp, block_ends=block_ends, p_cmp=p_cmp, sel_scores=sel, indices_own=idx_own)


# ----------------------------------------------------------------------------------------------
# what "bit-exact block ids" can mean between independent implementations
# ----------------------------------------------------------------------------------------------

def ambiguous_rows(sel_scores_grouped: torch.Tensor, n: int, tau: float = 1e-5) -> torch.Tensor:
    """Rows [B,G,T] whose top-(n+1) aggregated scores hold an adjacent pair closer than tau (relative): there the
    ranking depends on fp32 rounding order (the reference's own fp32 and fp64 runs disagree on such rows), so no
    independent implementation can be expected to agree bit for bit.  Exact ties are decided by block id
    (nsa/kernels.py:1986-1990, stable sort) and are not ambiguous."""
    k = min(n + 1, sel_scores_grouped.shape[-1])
    top = torch.sort(sel_scores_grouped.double(), dim=-1, descending=True).values[..., :k]
    gap = (top[..., :-1] - top[..., 1:]) / top[..., :-1].abs().clamp_min(1e-30)
    both_zero = (top[..., :-1] == 0) & (top[..., 1:] == 0)
    return ((gap < tau) & ~both_zero).any(dim=-1)


def sample_positions(T: int, count: int, l: int = 32, w: int = 512, l_prime: int = 64, n: int = 16, seed: int = 0) -> torch.Tensor:
    """`count` query positions of [0,T): the boundary rows of every branch (first rows, around the first compressed
    block, the window edge, the point where the selection blocks run out, the last row) plus seeded random ones;
    sorted, unique."""
    must = [0, l - 2, l - 1, l, w - 1, w, n * l_prime - 1, n * l_prime, n * l_prime + 1, T - 1]
    must = [t for t in must if 0 <= t < T]
    g = torch.Generator().manual_seed(seed)
    rnd = torch.randint(0, T, (max(0, count - len(must)),), generator=g).tolist()
    return torch.tensor(sorted(set(must + rnd)), dtype=torch.int64)


# ----------------------------------------------------------------------------------------------
# seeded inputs shared by tests, fixtures and the benchmark
# ----------------------------------------------------------------------------------------------

def make_inputs(B, H, G, T, dk, dv, d_model, l=32, *, seed=0, block_offset_std=0.0, l_prime=64,
                dtype=torch.float32):
    """q,k,v ~ N(0,1) (draw order q,k,v), then phi/gate weights ~ N(0,0.02) with zero biases from
    the same generator, dO from seed+1, gate input x from seed+2.  ``block_offset_std`` > 0 adds one
    N(0,std) [dk] vector per (b,g,l'-block) to the keys of that block.  Values are rounded to
    ``dtype`` and returned as fp32 so CPU oracle and GPU see identical numbers."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s, std=1.0: torch.randn(*s, generator=g) * std
    q, k, v = rn(B, H, T, dk), rn(B, G, dk, T), rn(B, G, T, dv)
    if block_offset_std > 0:
        nblk = (T + l_prime - 1) // l_prime
        off = rn(B, G, dk, nblk, std=block_offset_std)
        k = k + off.repeat_interleave(l_prime, dim=-1)[..., :T]
    phi = PhiParams(pos_embed=rn(l, l, std=0.02), w1=rn(2 * dk, dk + l, std=0.02), b1=torch.zeros(2 * dk),
                    w2=rn(dk, 2 * dk, std=0.02), b2=torch.zeros(dk))
    gp = GateParams(w1=rn(d_model // 2, d_model, std=0.02), b1=torch.zeros(d_model // 2),
                    w2=rn(3 * H, d_model // 2, std=0.02), b2=torch.zeros(3 * H))
    do = torch.randn(B, H, T, dv, generator=torch.Generator().manual_seed(seed + 1))
    x = torch.randn(B, T, d_model, generator=torch.Generator().manual_seed(seed + 2))
    rd = lambda t: t.to(dtype).float()
    return dict(q=rd(q), k=rd(k), v=rd(v), do=rd(do), x=rd(x), phi=phi, gate=gp)


PROJ_NAMES = ("q_proj", "k_compress", "v_compress", "k_select", "v_select", "k_sliding", "v_sliding", "o_proj")


def draw_projection_weights(seed, d_model, H, G, dk, dv):
    """Seeded weights (no biases) for the module's eight projections (nsa/kernels.py:2060-2114),
    N(0, 1/sqrt(fan_in)); used to pin the oracle against a whole-module run of the reference."""
    g = torch.Generator().manual_seed(seed)
    shapes = dict(q_proj=(H * dk, d_model), k_compress=(G * dk, d_model), v_compress=(G * dv, d_model),
                  k_select=(G * dk, d_model), v_select=(G * dv, d_model), k_sliding=(G * dk, d_model),
                  v_sliding=(G * dv, d_model), o_proj=(d_model, H * dv))
    return {n: torch.randn(*shapes[n], generator=g) / math.sqrt(shapes[n][1]) for n in PROJ_NAMES}


def nsa_module_forward(hidden, proj, phi, gp, *, H, G, dk, dv, **layer_kw):
    """hidden [B,T,d_model] -> (y [B,T,d_model], layer dict): projections (nsa/kernels.py:2256-2296),
    the layer, and o_proj (nsa/kernels.py:2466-2477)."""
    B, T, _ = hidden.shape
    lin = torch.nn.functional.linear
    q = lin(hidden, proj["q_proj"]).view(B, T, H, dk).transpose(1, 2)
    kv = lambda kn, vn: (lin(hidden, proj[kn]).view(B, T, G, dk).permute(0, 2, 3, 1),
                         lin(hidden, proj[vn]).view(B, T, G, dv).transpose(1, 2))
    ks, vs = kv("k_select", "v_select")
    r = nsa_layer(q, ks, vs, hidden, phi, gp, kv_compress=kv("k_compress", "v_compress"),
                  kv_sliding=kv("k_sliding", "v_sliding"), **layer_kw)
    y = lin(r["out"].transpose(1, 2).reshape(B, T, H * dv), proj["o_proj"])
    return y, r
