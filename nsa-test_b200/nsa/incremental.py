"""Incremental (prefill-in-chunks / decode) forward of the NSA layer against a key/value cache.

The reference has no incremental path (its module accepts and ignores ``attention_mask``,
nsa/kernels.py:2213, and always recomputes the whole sequence); this is the same layer arithmetic
(nsa/kernels.py:2298-2463) evaluated for the newest query rows only, so that the rows it returns equal the
corresponding rows of the full-sequence forward.  Forward only, no autograd.

``NSACache`` keeps, per layer, the three key/value streams of the module (selection, sliding window and the
source of the compression), zero-padded to a fixed capacity, and the compressed keys/values, which grow by
one block every ``d`` tokens once ``l`` tokens are there.  ``nsa_layer_incremental`` runs the scoring/top-n,
the three branches and the gate mix for the new rows with a query position offset; the kernels work on
128-row query tiles, so the new rows are padded to a tile with rows that are computed and dropped.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from . import ops
from .kernels import (NSAConfig, PAD_BLOCK_END, _PhiCompress, _next_pow2, _project_heads, _selection_fallback,
                      gate_logits_from_hidden)

__all__ = ["NSACache", "nsa_layer_incremental", "module_forward_incremental"]

_TILE = 128
_FEW_ROWS = 64       # (sequence, group, row) count up to which scoring takes the unpadded rows


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class NSACache:
    """Key/value cache of one NSA layer for ``batch`` sequences of up to ``capacity`` tokens.

    Layouts are the kernels' own: keys ``[B,G,dk,capacity]``, values ``[B,G,capacity,dv]`` (zeros beyond
    ``length``), compressed keys fp32 ``[B,G,dk,nbp]`` (+ a copy in the compute dtype for the compressed
    attention) and compressed values ``[B,G,nbp,dv]`` with ``n_blocks`` valid blocks.
    """

    def __init__(self, config: NSAConfig, batch: int, capacity: int, device, dtype=torch.bfloat16,
                 shared_kv: bool = False):
        c = config
        self.config, self.dtype, self.shared_kv = c, dtype, shared_kv
        self.capacity = _round_up(capacity, _TILE)
        G, dk, dv = c.n_kv_groups, c.head_dim_qk, c.head_dim_v

        def kv():
            return (torch.zeros(batch, G, dk, self.capacity, device=device, dtype=dtype),
                    torch.zeros(batch, G, self.capacity, dv, device=device, dtype=dtype))

        self.k_slc, self.v_slc = kv()
        (self.k_win, self.v_win) = (self.k_slc, self.v_slc) if shared_kv else kv()
        (self.k_src, self.v_src) = (self.k_slc, self.v_slc) if shared_kv else kv()
        nb_cap = max((self.capacity - c.l) // c.d + 1, 1)
        self.nbp = max(_next_pow2(nb_cap), _TILE)
        self.k_cmp = torch.zeros(batch, G, dk, self.nbp, device=device, dtype=torch.float32)
        self.k_cmp_lp = torch.zeros(batch, G, dk, self.nbp, device=device, dtype=dtype)
        self.v_cmp = torch.zeros(batch, G, self.nbp, dv, device=device, dtype=dtype)
        self.block_ends = torch.full((self.nbp,), PAD_BLOCK_END, device=device, dtype=torch.int32)
        self.length = 0
        self.n_blocks = 0

    @torch.no_grad()
    def append(self, phi_params, k_slc, v_slc, kv_compress=None, kv_sliding=None) -> int:
        """Add ``Tn`` tokens: k_* ``[B,G,dk,Tn]``, v_* ``[B,G,Tn,dv]`` (one pair feeds all branches unless the
        cache was built with separate streams).  Compresses the blocks the new tokens complete.  Returns the
        position of the first new token."""
        c = self.config
        Tn = k_slc.shape[-1]
        p0, p1 = self.length, self.length + Tn
        if p1 > self.capacity:
            raise ValueError(f"NSACache: {p1} tokens exceed the capacity {self.capacity}")
        if not self.shared_kv and (kv_compress is None or kv_sliding is None):
            raise ValueError("NSACache: built with separate streams, kv_compress and kv_sliding are required")
        self.k_slc[..., p0:p1] = k_slc
        self.v_slc[:, :, p0:p1] = v_slc
        if not self.shared_kv:
            self.k_src[..., p0:p1], self.v_src[:, :, p0:p1] = kv_compress[0], kv_compress[1]
            self.k_win[..., p0:p1], self.v_win[:, :, p0:p1] = kv_sliding[0], kv_sliding[1]
        self.length = p1
        nb_new = (p1 - c.l) // c.d + 1 if p1 >= c.l else 0
        if nb_new > self.n_blocks:
            b0, cnt = self.n_blocks, nb_new - self.n_blocks
            lo, hi = b0 * c.d, (nb_new - 1) * c.d + c.l
            keys = self.k_src[..., lo:hi].transpose(-1, -2).contiguous()
            vals = self.v_src[:, :, lo:hi].contiguous()
            kc, vc = _PhiCompress.apply(keys, vals, *phi_params, c.l, c.d)
            self.k_cmp[..., b0:nb_new] = kc[..., :cnt]
            self.k_cmp_lp[..., b0:nb_new] = kc[..., :cnt].to(self.dtype)
            self.v_cmp[:, :, b0:nb_new] = vc[:, :, :cnt].to(self.dtype)
            self.block_ends[b0:nb_new] = (torch.arange(b0, nb_new, device=self.block_ends.device, dtype=torch.int32)
                                          * c.d + (c.l - 1))
            self.n_blocks = nb_new
        return p0


def _pad_rows(x: torch.Tensor, dim: int, rows: int) -> torch.Tensor:
    have = x.shape[dim]
    if have == rows:
        return x.contiguous()
    shape = list(x.shape)
    shape[dim] = rows - have
    return torch.cat([x, x.new_zeros(shape)], dim=dim)


@torch.no_grad()
def nsa_layer_incremental(q_new: torch.Tensor, gate_logits_new: torch.Tensor, cache: NSACache,
                          scale: Optional[float] = None, return_info: bool = False):
    """Output rows ``[B,H,Tn,dv]`` of the NSA layer for the ``Tn`` newest tokens of ``cache`` (the keys/values
    of these tokens must have been appended already).  q_new ``[B,H,Tn,dk]``, gate_logits_new ``[B,Tn,3H]``.

    Row r is the query at position ``cache.length - Tn + r`` and sees exactly what the full-sequence forward
    shows it: the compressed blocks that end at or before it, its top-n selected blocks (causally clipped)
    and the last ``w`` keys.
    """
    c = cache.config
    B, H, Tn, dk = q_new.shape
    pos = cache.length - Tn
    if pos < 0:
        raise ValueError("nsa_layer_incremental: more query rows than cached tokens")
    if cache.n_blocks == 0:
        # The full-sequence layer lets rows without a visible compressed block attend block 0; before that
        # block exists there is nothing to reproduce, so the first chunk has to bring at least l tokens.
        raise ValueError(f"nsa_layer_incremental: the cache needs at least l={c.l} tokens")
    scale = 1.0 / math.sqrt(dk) if scale is None else scale
    rows = _round_up(Tn, _TILE)
    q = _pad_rows(q_new, 2, rows)
    n_fixed = c.n_fixed if c.include_fixed_in_selection else 0
    nb = cache.n_blocks

    G = c.n_kv_groups
    blocks = (c.l, c.d, nb)
    if Tn < rows and B * G * Tn <= _FEW_ROWS:
        # A handful of rows (decode): the tile kernel would run one CTA per (sequence, group) over all compressed
        # blocks; unpadded rows take the generic scoring path, whose q.k products spread over the whole GPU.
        real = ops.score_topn(q_new.contiguous(), cache.k_cmp, cache.block_ends, c.l, c.d, c.l_prime, c.n, n_fixed, scale,
                              nb, pos)
        indices = torch.cat([real, real.new_full((B, G, rows - Tn, c.n), -1)], dim=2)
        o_cmp, _, _ = ops.cmp_attn_fwd(q, cache.k_cmp_lp, cache.v_cmp, cache.block_ends, scale, blocks, pos)
    elif ops.cmp_exact_supported(q, cache.k_cmp_lp, cache.v_cmp):
        # as the full-sequence layer does it: the compressed attention runs on the fp32 keys (as bf16 hi + lo halves)
        # and hands its log-sum-exp to the scoring kernel, so the two agree on every row, near-ties included
        hi, lo = ops.split_keys(cache.k_cmp)
        o_cmp, _, _, lse2 = ops.cmp_attn_fwd(q, hi, cache.v_cmp, cache.block_ends, scale, blocks, pos, k_lo=lo)
        indices = ops.score_topn(q, cache.k_cmp, cache.block_ends, c.l, c.d, c.l_prime, c.n, n_fixed, scale, nb, pos,
                                 cmp_lse2=lse2)
    else:
        indices = ops.score_topn(q, cache.k_cmp, cache.block_ends, c.l, c.d, c.l_prime, c.n, n_fixed, scale, nb, pos)
        o_cmp, _, _ = ops.cmp_attn_fwd(q, cache.k_cmp_lp, cache.v_cmp, cache.block_ends, scale, blocks, pos)
    idx = _selection_fallback(indices, c.l_prime, pos).to(torch.int32).contiguous()
    o_slc, _, _ = ops.slc_fwd(q, cache.k_slc, cache.v_slc, idx, c.l_prime, scale, pos)

    # Sliding window: the window reaches w - 1 positions back, so the dense kernel runs on the key slice that
    # starts at a tile boundary at or before pos - (w - 1); the query rows sit at their offset inside it.
    lo = max(0, (pos - (c.w - 1)) // _TILE * _TILE)
    span = _round_up(pos - lo + Tn, _TILE)
    qw = q_new.new_zeros(B, H, span, dk)
    qw[:, :, pos - lo:pos - lo + Tn] = q_new
    ks = cache.k_win[..., lo:lo + span].contiguous()
    vs = cache.v_win[:, :, lo:lo + span].contiguous()
    o_win, _, _ = ops.sliding_fwd(qw, ks, vs, c.w, scale)
    o_win = _pad_rows(o_win[:, :, pos - lo:pos - lo + Tn], 2, rows)

    out, gates = ops.gate_mix_fwd(_pad_rows(gate_logits_new, 1, rows), o_cmp, o_slc, o_win, c.gate_mode)
    out = out[:, :, :Tn]
    if return_info:
        return out, dict(indices=indices[:, :, :Tn], gates=gates[:, :, :Tn], o_cmp=o_cmp[:, :, :Tn],
                         o_slc=o_slc[:, :, :Tn], o_win=o_win[:, :, :Tn])
    return out


@torch.no_grad()
def module_forward_incremental(module, hidden_new: torch.Tensor, cache: NSACache) -> torch.Tensor:
    """``NSAAttention`` applied to the ``Tn`` newest tokens ``hidden_new [B,Tn,d_model]``: projects them, appends
    their keys/values to ``cache`` (built with ``shared_kv=False``) and returns ``[B,Tn,d_model]``, equal to the
    last ``Tn`` rows of ``module(hidden_all)[0]`` in eval mode."""
    c = module.config
    B, Tn, _ = hidden_new.shape
    H, G, dk, dv = c.n_heads, c.n_kv_groups, c.head_dim_qk, c.head_dim_v
    q = _project_heads(hidden_new, module.q_proj, H, dk)

    def kv(kp, vp):
        return _project_heads(hidden_new, kp, G, dk, transposed=True), _project_heads(hidden_new, vp, G, dv)

    k_sel, v_sel = kv(module.k_select, module.v_select)
    cache.append(module._phi_params(), k_sel, v_sel, kv_compress=kv(module.k_compress, module.v_compress),
                 kv_sliding=kv(module.k_sliding, module.v_sliding))
    out = nsa_layer_incremental(q, gate_logits_from_hidden(hidden_new, module.gate_mlp), cache, module.scale)
    return module.o_proj(out.transpose(1, 2).reshape(B, Tn, H * dv))
