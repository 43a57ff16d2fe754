"""Host-side mirror of the reference project's ``nsa.kernels`` module, backed by sm_100a CUDA kernels.

Same names and call signatures as Noumena-Network/NSA-Test ``nsa/kernels.py``: ``NSAConfig``
(:516-591), the autograd wrappers ``CompressionAttention`` / ``SelectionAttention`` /
``SlidingWindowAttention`` (:34-513), the scoring functions (:1920-2040), the ``NSAAttention`` module
(:2043-2507) and the six ``_nsa_*_kernel`` objects, which here are launcher shims that accept the
reference's ``kernel[grid](*positional, **constexpr)`` call and forward it to the C ABI.

Deliberate differences from the reference:
* every path runs on the GPU; eval mode uses the same (deterministic) kernels as training instead of
  a float64 CPU detour (nsa/kernels.py:2366-2398), and CPU tensors raise;
* the [B,H,T,n_cmp] probability tensor is never materialised on the training path; it is produced
  only for ``output_attentions=True``;
* dK/dV are reduced in a fixed order (no atomics), so backward is bit-reproducible.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from . import ops

__all__ = [
    "NSAConfig", "NSAAttention", "CompressionAttention", "SelectionAttention", "SlidingWindowAttention",
    "derive_selection_from_compression_per_timestep", "select_top_k_blocks_per_query_with_gqa",
    "_nsa_sliding_window_fwd_kernel", "_nsa_sliding_window_bwd_kernel", "_nsa_compression_fwd_kernel",
    "_nsa_compression_bwd_kernel", "_nsa_sparse_selection_fwd_kernel", "_nsa_sparse_selection_bwd_kernel",
]

PAD_BLOCK_END = 999999  # block end of the padding blocks (nsa/kernels.py:2190)
_USE_C_LAYER = True      # False: nsa_layer composes the branch entry points itself (what the long-context mode always does)
_TILE_ROWS = 128         # query/key rows per tile of the tensor-core kernels
_PAD_FROM = 2048         # ragged bf16 sequences at least this long are padded to a whole tile


def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


# --------------------------------------------------------------------------------------------------
# configuration (nsa/kernels.py:516-591)
# --------------------------------------------------------------------------------------------------

@dataclass
class NSAConfig:
    """NSA layer configuration; field names and defaults are those of the reference (paper Sec. 4.1)."""

    d_model: int = 2560
    head_dim_qk: int = 192
    head_dim_v: int = 128
    l: int = 32           # compression block size
    d: int = 16           # compression stride
    l_prime: int = 64     # selection block size
    n: int = 16           # blocks selected per query
    include_fixed_in_selection: bool = True
    n_fixed: int = 3      # 1 initial + 2 local
    n_dynamic: int = 13
    w: int = 512          # sliding window
    n_heads: int = 64
    n_kv_groups: int = 4
    dropout_p: float = 0.0
    use_bias: bool = False
    block_m: int = 32     # accepted for compatibility; tile sizes are chosen by the CUDA kernels
    block_n: int = 32
    gate_mode: str = "sigmoid"

    def __post_init__(self):
        # The reference accepts l=0 / l_prime=0 by accident (0 % d == 0) although its own contract test
        # expects a rejection (tests/test_kernel_contracts.py:372-382); reject them explicitly.
        assert self.d > 0, "compression stride d must be positive"
        assert self.l > 0 and self.l_prime > 0, "block sizes l and l_prime must be positive"
        assert self.n > 0, "n must be positive"
        assert self.n_kv_groups > 0 and self.n_heads % self.n_kv_groups == 0
        assert self.l % self.d == 0
        assert self.l_prime % self.d == 0
        assert self.w > 0
        if not self.include_fixed_in_selection:
            self.n_fixed = 0
        self.n_dynamic = max(0, self.n - self.n_fixed)
        assert self.n_fixed + self.n_dynamic == self.n
        assert self.gate_mode in ("sigmoid", "softmax")

    @property
    def heads_per_group(self) -> int:
        return self.n_heads // self.n_kv_groups

    @property
    def head_dim_qk_padded(self) -> int:
        return _next_pow2(self.head_dim_qk)

    @property
    def head_dim_v_padded(self) -> int:
        return _next_pow2(self.head_dim_v)


# --------------------------------------------------------------------------------------------------
# autograd wrappers (nsa/kernels.py:34-513)
# --------------------------------------------------------------------------------------------------

class SlidingWindowAttention(torch.autograd.Function):
    """``apply(q [B,H,T,dk], k [B,G,dk,T], v [B,G,T,dv], scale, window_size, config) -> o [B,H,T,dv]``."""

    @staticmethod
    def forward(ctx, q, k, v, scale, window_size, config=None):
        o, L, M = ops.sliding_fwd(q, k, v, window_size, scale)
        ctx.save_for_backward(q, k, v, o, L, M)
        ctx.scale, ctx.window_size = scale, window_size
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, L, M = ctx.saved_tensors
        dq, dkey, dval = ops.sliding_bwd(q, k, v, o, do, L, M, ctx.window_size, ctx.scale)
        return dq, dkey.transpose(-1, -2), dval, None, None, None


class CompressionAttention(torch.autograd.Function):
    """``apply(q, k_compressed [B,G,dk,NB], v_compressed [B,G,NB,dv], block_ends [NB], scale, config)``."""

    @staticmethod
    def forward(ctx, q, k_compressed, v_compressed, block_ends, scale, config=None, blocks=None, q_pos0=0):
        o, L, M = ops.cmp_attn_fwd(q, k_compressed, v_compressed, block_ends, scale, blocks, q_pos0)
        ctx.save_for_backward(q, k_compressed, v_compressed, block_ends, o, L, M)
        ctx.scale, ctx.blocks, ctx.q_pos0 = scale, blocks, q_pos0
        return o

    @staticmethod
    def backward(ctx, do):
        q, kc, vc, block_ends, o, L, M = ctx.saved_tensors
        dq, dkc, dvc = ops.cmp_attn_bwd(q, kc, vc, block_ends, o, do, L, M, ctx.scale, ctx.blocks, ctx.q_pos0)
        return dq, dkc.transpose(-1, -2), dvc, None, None, None, None, None


def _selection_fallback(indices: torch.Tensor, l_prime: int, q_pos0: int = 0) -> torch.Tensor:
    """Rows whose slots are all -1 attend the block holding the query (nsa/kernels.py:199-205)."""
    if indices.numel() == 0:
        return indices
    T = indices.shape[2]
    t_blocks = ((torch.arange(T, device=indices.device, dtype=indices.dtype) + q_pos0) // l_prime).view(1, 1, T, 1)
    none_valid = (indices < 0).all(dim=-1, keepdim=True)
    return torch.where(none_valid, t_blocks, indices)


class SelectionAttention(torch.autograd.Function):
    """``apply(q, k [B,G,dk,T], v [B,G,T,dv], indices [B,G,T,n], scale, config) -> o``."""

    @staticmethod
    def forward(ctx, q, k, v, indices, scale, config, q_pos0=0):
        idx = _selection_fallback(indices, config.l_prime, q_pos0).to(torch.int32).contiguous()
        o, L, M = ops.slc_fwd(q, k, v, idx, config.l_prime, scale, q_pos0)
        ctx.save_for_backward(q, k, v, idx, o, L, M)
        ctx.scale, ctx.l_prime, ctx.q_pos0 = scale, config.l_prime, q_pos0
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, idx, o, L, M = ctx.saved_tensors
        dq, dkey, dval = ops.slc_bwd(q, k, v, idx, o, do, L, M, ctx.l_prime, ctx.scale, ctx.q_pos0)
        return dq, dkey.transpose(-1, -2), dval, None, None, None, None


def _window_slice(q_pos0: int, Tq: int, Tk: int, w: int):
    """Key range [lo, hi) and the number of zero query rows in front that let the sliding-window kernels (which take
    query row t as position t of their key tensor) serve queries at positions q_pos0 + [0, Tq): the window reaches
    w - 1 positions back, so the slice starts a tile-aligned margin before the first query."""
    if q_pos0 == 0 and Tk == Tq:
        return 0, Tk, 0
    pad = min(q_pos0, ((w - 1 + _TILE_ROWS - 1) // _TILE_ROWS) * _TILE_ROWS)
    return q_pos0 - pad, q_pos0 + Tq, pad


class _BranchesAndMix(torch.autograd.Function):
    """The three attention branches and the gate mix of one layer under a single autograd node
    (nsa/kernels.py:2401-2463), so that the backward can pass on what the reference leaves to separate kernels and to
    autograd: the gate/mix backward also produces the row sums dO_b.O_b that each branch backward needs, and the
    selection backward adds the dQ of the other two branches to its own before the one rounding of the sum.

    ``apply(q, k_cmp, v_cmp, block_ends, k_slc, v_slc, indices, k_win, v_win, gate_logits, scale, config, blocks, q_pos0,
    token_major)`` -> (out, gates, o_cmp, o_slc, o_win); only ``out`` is differentiable.  The selection branch runs
    last and does the gate + mix in its epilogue (north-star item: no separate pass over the three branch outputs in the
    forward); ``token_major`` lays the mixed output out as [B,T,H,dv] in memory for the output projection.  Same kernels and layouts as the separate
    wrappers above.  With ``q_pos0`` > 0 the query rows sit at positions q_pos0 + [0, Tq) of keys that start at
    position 0 (long-context mode); the sliding-window kernels then run on the key slice around the queries."""

    @staticmethod
    def forward(ctx, q, k_cmp, v_cmp, block_ends, k_slc, v_slc, indices, k_win, v_win, gate_logits, scale, config, blocks,
                q_pos0=0, token_major=False, k_cmp_f32=None):
        Tq = q.shape[2]
        # ``indices`` None: the blocks are chosen here (Eq. 8-11) from the fp32 compressed keys ``k_cmp_f32``.  Where the
        # tensor-core kernels apply, the compressed attention runs on the keys as a bf16 pair hi + lo and hands its
        # log-sum-exp to the scoring kernel, which then sweeps the compressed keys once instead of twice.
        lse2 = None
        if indices is None and k_cmp_f32 is not None and blocks is not None and ops.cmp_exact_supported(q, k_cmp, v_cmp):
            hi, lo = ops.split_keys(k_cmp_f32)
            o_cmp, Lc, Mc, lse2 = ops.cmp_attn_fwd(q, hi, v_cmp, block_ends, scale, blocks, q_pos0, k_lo=lo)
            k_cmp = hi
        else:
            o_cmp, Lc, Mc = ops.cmp_attn_fwd(q, k_cmp, v_cmp, block_ends, scale, blocks, q_pos0)
        if indices is None:
            n_fixed = config.n_fixed if config.include_fixed_in_selection else 0
            indices = ops.score_topn(q, k_cmp_f32, block_ends, config.l, config.d, config.l_prime, config.n, n_fixed, scale,
                                     blocks[2], q_pos0, cmp_lse2=lse2)
        ctx.chosen = indices
        idx = _selection_fallback(indices, config.l_prime, q_pos0).to(torch.int32).contiguous()
        lo, hi, pad = _window_slice(q_pos0, Tq, k_win.shape[-1], config.w)
        if pad or lo or hi != k_win.shape[-1]:
            kw_s, vw_s = k_win[..., lo:hi].contiguous(), v_win[:, :, lo:hi].contiguous()
            qw = torch.cat([q.new_zeros(q.shape[0], q.shape[1], pad, q.shape[3]), q], dim=2) if pad else q
        else:
            kw_s, vw_s, qw = k_win, v_win, q
        o_wp, Lw, Mw = ops.sliding_fwd(qw, kw_s, vw_s, config.w, scale)
        o_win = o_wp[:, :, pad:] if pad else o_wp
        o_slc, Ls, Ms, out, gates = ops.slc_fwd_mix(q, k_slc, v_slc, idx, config.l_prime, scale, gate_logits, o_cmp, o_win,
                                                    config.gate_mode, q_pos0, token_major)
        ctx.save_for_backward(q, k_cmp, v_cmp, block_ends, k_slc, v_slc, idx, kw_s, vw_s, qw, o_cmp, Lc, Mc, o_slc, Ls, Ms,
                              o_wp, Lw, Mw, gates)
        ctx.scale, ctx.l_prime, ctx.w, ctx.blocks = scale, config.l_prime, config.w, blocks
        ctx.gate_mode, ctx.ldtype = config.gate_mode, gate_logits.dtype
        ctx.q_pos0, ctx.win = q_pos0, (lo, hi, pad, tuple(k_win.shape), tuple(v_win.shape))
        # one k/v pair feeding both the selection and the sliding-window branch: their dK/dV are summed in the backward
        ctx.shared_win = (k_win.data_ptr() == k_slc.data_ptr() and v_win.data_ptr() == v_slc.data_ptr()
                          and k_win.shape == k_slc.shape and v_win.shape == v_slc.shape)
        ctx.mark_non_differentiable(gates, o_cmp, o_slc, o_win, indices)
        return out, gates, o_cmp, o_slc, o_win, indices

    @staticmethod
    def backward(ctx, dout, *_unused):
        (q, k_cmp, v_cmp, block_ends, k_slc, v_slc, idx, kw_s, vw_s, qw, o_cmp, Lc, Mc, o_slc, Ls, Ms, o_wp, Lw, Mw,
         gates) = ctx.saved_tensors
        lo, hi, pad, kshape, vshape = ctx.win
        o_win = o_wp[:, :, pad:] if pad else o_wp
        d_cmp, d_slc, d_win, dlogits, delta = ops.gate_mix_bwd(gates, o_cmp, o_slc, o_win, dout, ctx.gate_mode,
                                                               want_delta=True)
        dq_c, dkc, dvc = ops.cmp_attn_bwd(q, k_cmp, v_cmp, block_ends, o_cmp, d_cmp, Lc, Mc, ctx.scale, ctx.blocks,
                                          ctx.q_pos0, row_delta=delta[0])
        if pad:
            # the zero query rows in front get a zero upstream gradient and zero row sums: they add nothing to dK/dV
            F = torch.nn.functional
            d_wp, delta_w = F.pad(d_win, (0, 0, pad, 0)), F.pad(delta[2], (pad, 0))
        else:
            d_wp, delta_w = d_win, delta[2]
        dq_w, dkw, dvw = ops.sliding_bwd(qw, kw_s, vw_s, o_wp, d_wp, Lw, Mw, ctx.w, ctx.scale, row_delta=delta_w)
        if pad:
            dq_w = dq_w[:, :, pad:].contiguous()
        dq, dks, dvs = ops.slc_bwd(q, k_slc, v_slc, idx, o_slc, d_slc, Ls, Ms, ctx.l_prime, ctx.scale, ctx.q_pos0,
                                   dq_addends=(dq_c, dq_w), row_delta=delta[1])
        if ctx.shared_win:
            # the window's gradients (time-major, for the key slice [lo, hi)) go straight into the selection branch's
            # full-length buffers: no zero-filled full-length copies, no separate full-length additions by autograd
            dks[:, :, lo:hi] += dkw
            dvs[:, :, lo:hi] += dvw
            dkw = dvw = None
        else:
            dkw = dkw.transpose(-1, -2)
            if (lo, hi) != (0, kshape[-1]):
                full_k, full_v = dkw.new_zeros(kshape), dvw.new_zeros(vshape)
                full_k[..., lo:hi] = dkw
                full_v[:, :, lo:hi] = dvw
                dkw, dvw = full_k, full_v
        return (dq, dkc.transpose(-1, -2), dvc, None, dks.transpose(-1, -2), dvs, None, dkw, dvw,
                dlogits.to(ctx.ldtype), None, None, None, None, None, None)


class _LayerC(torch.autograd.Function):
    """The whole layer through the library's nsa_layer_fwd / nsa_layer_bwd (one C call each way).

    ``apply(q, k_slc, v_slc, k_cmp, v_cmp, k_win, v_win, gate_logits, pos_embed, w1, b1, w2, b2, desc, shared_kv, indices)``
    -> (out, ctx); only ``out`` is differentiable.  ``shared_kv``: the three k/v pairs are one pair (their gradients are
    accumulated in one pair of buffers inside the library and returned for k_slc/v_slc only)."""

    @staticmethod
    def forward(ctx, q, k_slc, v_slc, k_cmp, v_cmp, k_win, v_win, gate_logits, pos_embed, w1, b1, w2, b2, desc, shared_kv, indices):
        f32 = lambda p: None if p is None else p.detach().float().contiguous()
        phi = tuple(f32(p) for p in (pos_embed, w1, b1, w2, b2))
        lg = gate_logits.detach().float().contiguous()
        out, saved = ops.layer_fwd(desc, q, (k_slc, v_slc), (k_cmp, v_cmp), (k_win, v_win), lg, phi, indices)
        ctx.save_for_backward(q, k_slc, v_slc, k_cmp, k_win, v_win, phi[0], phi[1], phi[3], saved)
        ctx.desc, ctx.shared_kv = desc, shared_kv
        ctx.pdtypes = (gate_logits.dtype, pos_embed.dtype, w1.dtype, w2.dtype, b1 is not None, b2 is not None)
        ctx.mark_non_differentiable(saved)
        return out, saved

    @staticmethod
    def backward(ctx, dout, _dsaved):
        q, k_slc, v_slc, k_cmp, k_win, v_win, pos, w1, w2, saved = ctx.saved_tensors
        desc = ctx.desc
        tm = bool(desc.out_token_major)
        # the upstream gradient in the layout the forward wrote: read as it lies when it has it, copied otherwise
        if tm:
            if not dout.permute(0, 2, 1, 3).is_contiguous():
                dout = dout.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        else:
            dout = dout.contiguous()
        dq, g_slc, g_cmp, g_win, dlogits, (dpos, dw1, db1, dw2, db2) = ops.layer_bwd(
            desc, q, (k_slc, v_slc), (k_cmp, None), (k_win, v_win), (pos, w1, None, w2, None), saved, dout, ctx.shared_kv)
        ldt, pdt, w1dt, w2dt, has_b1, has_b2 = ctx.pdtypes
        tk = lambda g: g.transpose(-1, -2)            # dK comes back time-major; the keys are [B,G,dk,T]
        if ctx.shared_kv:
            gk = (tk(g_slc[0]), g_slc[1], None, None, None, None)
        else:
            gk = (tk(g_slc[0]), g_slc[1], tk(g_cmp[0]), g_cmp[1], tk(g_win[0]), g_win[1])
        return (dq, *gk, dlogits.to(ldt), dpos.to(pdt), dw1.to(w1dt), db1.to(w1dt) if has_b1 else None, dw2.to(w2dt),
                db2.to(w2dt) if has_b2 else None, None, None, None)


# --------------------------------------------------------------------------------------------------
# scoring functions (nsa/kernels.py:1920-2040)
# --------------------------------------------------------------------------------------------------

def derive_selection_from_compression_per_timestep(compression_scores: torch.Tensor, config: NSAConfig) -> torch.Tensor:
    """Eq. 9 on a materialised probability tensor [B,H,T,n_cmp] -> [B,H,T,n_sel]."""
    assert config.l % config.d == 0 and config.l_prime % config.d == 0
    out = ops.eq9_scores(compression_scores, config.l, config.d, config.l_prime)
    return out.to(compression_scores.dtype)


def select_top_k_blocks_per_query_with_gqa(selection_scores: torch.Tensor, config: NSAConfig,
                                           always_include_blocks: Optional[List[int]] = None) -> torch.Tensor:
    """Eq. 10/11: [B,H,T,n_blocks] scores -> int64 block ids [B,G,T,n] (-1 = empty slot).

    ``always_include_blocks`` is accepted and ignored, as in the reference."""
    n_fixed = config.n_fixed if config.include_fixed_in_selection else 0
    idx = ops.topn_from_scores(selection_scores, config.n_kv_groups, config.l_prime, config.n, n_fixed)
    return idx.to(torch.int64)


# --------------------------------------------------------------------------------------------------
# phi compression and gate/mix as autograd functions
# --------------------------------------------------------------------------------------------------

class _PhiCompress(torch.autograd.Function):
    """Block compression phi (nsa/kernels.py:2119-2208) with fp32 compressed keys, through the library's
    nsa_cmp_phi_fwd / nsa_cmp_phi_bwd.

    k_cmp[i] = W2 mean_j relu(W1k k_{id+j} + W1p pos_j + b1) + b2, which equals the reference's
    mean_j MLP([k_j || pos_j]) because the second linear layer commutes with the mean.  ``keys`` [B,G,T,dk] (usually the
    transposed view of K as it lies, [B,G,dk,T]), ``values`` [B,G,T,dv]."""

    @staticmethod
    def forward(ctx, keys, values, pos_embed, w1, b1, w2, b2, l, d):
        kt = keys.transpose(-1, -2)                                                 # [B,G,dk,T]
        kt = kt if kt.is_contiguous() else kt.contiguous()
        vals = values.to(kt.dtype).contiguous()
        f32 = lambda p: None if p is None else p.detach().float().contiguous()
        pe, w1f, b1f, w2f, b2f = f32(pos_embed), f32(w1), f32(b1), f32(w2), f32(b2)
        k_cmp, v_cmp, saved = ops.cmp_phi_fwd(kt, vals, pe, w1f, b1f, w2f, b2f, l, d)
        ctx.save_for_backward(kt, pe, w1f, w2f, saved)
        ctx.cfg = (l, d, vals.shape[-1], values.dtype, pos_embed.dtype, w1.dtype, w2.dtype, b1 is not None, b2 is not None)
        return k_cmp, v_cmp.to(values.dtype)

    @staticmethod
    def backward(ctx, dk_cmp, dv_cmp):
        kt, pe, w1f, w2f, saved = ctx.saved_tensors
        l, d, dv_dim, vdtype, pdtype, w1dtype, w2dtype, has_b1, has_b2 = ctx.cfg
        # block-major gradients in the I/O type, as the compressed attention's backward writes them
        dkc = dk_cmp.transpose(-1, -2).to(kt.dtype).contiguous()                    # [B,G,nbp,dk]
        dvc = dv_cmp.to(kt.dtype).contiguous()                                      # [B,G,nbp,dv]
        dkeys, dvals, dpos, dw1, db1, dw2, db2 = ops.cmp_phi_bwd(kt, pe, w1f, w2f, dkc, dvc, saved, dv_dim, l, d)
        return (dkeys, dvals.to(vdtype), dpos.to(pdtype), dw1.to(w1dtype), db1.to(w1dtype) if has_b1 else None,
                dw2.to(w2dtype), db2.to(w2dtype) if has_b2 else None, None, None)


class _GateMLP(torch.autograd.Function):
    """Branch-gate MLP (nsa/kernels.py:2105-2109) through the library's nsa_gate_mlp_fwd / nsa_gate_mlp_bwd:
    ``apply(x [B,T,d_model], w1, b1, w2, b2) -> logits [B,T,3H]`` in fp32 (what the gate/mix kernels take)."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        cast = lambda p: None if p is None else p.detach().to(x.dtype).contiguous()
        w1c, b1c, w2c, b2c = cast(w1), cast(b1), cast(w2), cast(b2)
        logits, hidden = ops.gate_mlp_fwd(x.detach(), w1c, b1c, w2c, b2c)
        ctx.save_for_backward(x, w1c, w2c, hidden)
        ctx.meta = (w1.dtype, w2.dtype, None if b1 is None else b1.dtype, None if b2 is None else b2.dtype)
        return logits

    @staticmethod
    def backward(ctx, dlogits):
        x, w1c, w2c, hidden = ctx.saved_tensors
        dx, dw1, db1, dw2, db2 = ops.gate_mlp_bwd(x, w1c, w2c, hidden, dlogits, ctx.needs_input_grad[0])
        w1d, w2d, b1d, b2d = ctx.meta
        return (dx, dw1.to(w1d), None if b1d is None else db1.to(b1d), dw2.to(w2d), None if b2d is None else db2.to(b2d))


def gate_logits_from_hidden(x: torch.Tensor, gate_mlp: torch.nn.Sequential) -> torch.Tensor:
    """The module's gate MLP (Linear, ReLU, Linear) applied through the library: fp32 logits [B,T,3H]."""
    return _GateMLP.apply(x, gate_mlp[0].weight, gate_mlp[0].bias, gate_mlp[2].weight, gate_mlp[2].bias)


class _GateMix(torch.autograd.Function):
    """out = g0*o_cmp + g1*o_slc + g2*o_win with gates from logits [B,T,3H] (nsa/kernels.py:2446-2463)."""

    @staticmethod
    def forward(ctx, logits, o_cmp, o_slc, o_win, gate_mode):
        out, gates = ops.gate_mix_fwd(logits, o_cmp, o_slc, o_win, gate_mode)
        ctx.save_for_backward(gates, o_cmp, o_slc, o_win)
        ctx.gate_mode, ctx.ldtype = gate_mode, logits.dtype
        ctx.mark_non_differentiable(gates)
        return out, gates

    @staticmethod
    def backward(ctx, dout, _dgates):
        gates, o_cmp, o_slc, o_win = ctx.saved_tensors
        d0, d1, d2, dlogits = ops.gate_mix_bwd(gates, o_cmp, o_slc, o_win, dout, ctx.gate_mode)
        return dlogits.to(ctx.ldtype), d0, d1, d2, None


_BLOCK_ENDS_CACHE: Dict[tuple, torch.Tensor] = {}


def _block_ends(nbp: int, nb: int, l: int, d: int, device) -> torch.Tensor:
    """int32 [nbp]: block i ends at i*d + l - 1 for i < nb, 999999 for the padding blocks (nsa/kernels.py:2185-2192).
    The same few tensors recur every step, so they are built once per (shape, device)."""
    key = (nbp, nb, l, d, str(device))
    be = _BLOCK_ENDS_CACHE.get(key)
    if be is None:
        be = torch.full((nbp,), PAD_BLOCK_END, device=device, dtype=torch.int32)
        be[:nb] = torch.arange(nb, device=device, dtype=torch.int32) * d + (l - 1)
        if len(_BLOCK_ENDS_CACHE) > 64:
            _BLOCK_ENDS_CACHE.clear()
        _BLOCK_ENDS_CACHE[key] = be
    return be


def nsa_layer(q, k_slc, v_slc, gate_logits, phi_params, config: NSAConfig, *, kv_compress=None, kv_sliding=None,
              scale: Optional[float] = None, return_info: bool = False, q_pos0: int = 0, indices=None, compressed=None,
              token_major_out: bool = False):
    """The NSA hot path between the q/k/v projections and o_proj (nsa/kernels.py:2298-2463).

    q [B,H,T,dk]; k_* [B,G,dk,T]; v_* [B,G,T,dv]; gate_logits [B,T,3H]; phi_params =
    (pos_embed [l,l], w1 [2dk,dk+l], b1, w2 [dk,2dk], b2).  One (k,v) feeds all branches unless
    ``kv_compress`` / ``kv_sliding`` are given.  Returns the mixed output [B,H,T,dv] (and a dict with
    indices, gates, k_cmp, v_cmp, block_ends when ``return_info``).

    Query-sharded long-context runs: q and gate_logits hold the Tq query rows at positions
    ``q_pos0 + [0, Tq)`` while k/v cover the sequence from position 0 (at least up to the last query); the
    gradients of k/v then hold this query slice's contribution only (summed over the ranks by the caller).

    ``compressed`` = (k_cmp fp32 [B,G,dk,nb], v_cmp [B,G,nb,dv]) of the whole sequence, when the caller has run the
    block compression already (the long-context mode splits it over the ranks); phi_params are then not used here.

    ``token_major_out``: the returned [B,H,T,dv] tensor is a view of a contiguous [B,T,H,dv] buffer (written that way by
    the mix epilogue), so that ``out.permute(0, 2, 1, 3).reshape(B, T, H*dv)`` feeds the output projection without the
    transposing copy of nsa/kernels.py:2466-2467; the upstream gradient is read in the same layout.

    ``indices`` [B,G,Tq,n] (int) replaces the layer's own Eq. 8-11 block choice, e.g. to evaluate two
    implementations on identical selections; the selection is not differentiable either way.
    """
    cfg = config
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    T_in = q.shape[2]
    if (q.dtype == torch.bfloat16 and q_pos0 == 0 and T_in % _TILE_ROWS and T_in >= _PAD_FROM
            and k_slc.shape[-1] == T_in):
        # The tensor-core kernels work on 128-row tiles; a long ragged sequence is padded with zero tokens to the next
        # tile instead of falling to the generic kernels.  The pad sits after every real token, so causality hides it:
        # real queries never see a pad key, a compressed block that reaches into the pad ends after the last real
        # query, and with T >= 2048 there are more selection blocks than slots, so the indices of the real rows do
        # not depend on the padded block count.  The pad rows are computed and dropped; autograd slices the gradients.
        pad = _TILE_ROWS - T_in % _TILE_ROWS
        F = torch.nn.functional
        pk = lambda kv: None if kv is None else (F.pad(kv[0], (0, pad)), F.pad(kv[1], (0, 0, 0, pad)))
        res = nsa_layer(F.pad(q, (0, 0, 0, pad)), *pk((k_slc, v_slc)), F.pad(gate_logits, (0, 0, 0, pad)), phi_params,
                        config, kv_compress=pk(kv_compress), kv_sliding=pk(kv_sliding), scale=scale,
                        return_info=return_info, token_major_out=token_major_out,
                        indices=None if indices is None else F.pad(indices, (0, 0, 0, pad), value=-1))
        if not return_info:
            return res[:, :, :T_in]
        out, info = res
        rows = ("indices", "gates", "o_cmp", "o_slc", "o_win")
        info = {k_: (v_[:, :, :T_in] if k_ in rows else v_) for k_, v_ in info.items()}
        # compressed blocks as the unpadded sequence has them: its block count, its power-of-two padding
        nb = (T_in - cfg.l) // cfg.d + 1
        nbp = _next_pow2(nb)
        info["k_cmp"], info["v_cmp"] = info["k_cmp"][..., :nbp], info["v_cmp"][:, :, :nbp]
        info["block_ends"] = info["block_ends"][:nbp].clone()
        info["block_ends"][nb:] = PAD_BLOCK_END
        return out[:, :, :T_in], info
    kc_src, vc_src = kv_compress if kv_compress is not None else (k_slc, v_slc)
    kw, vw = kv_sliding if kv_sliding is not None else (k_slc, v_slc)
    T = kc_src.shape[-1]   # sequence length covered by the keys (== query rows unless q_pos0 shards the queries)
    if q_pos0 == 0 and compressed is None and T == T_in and k_slc.shape[-1] == T_in and kw.shape[-1] == T_in and _USE_C_LAYER:
        # the common case: the whole layer is one call into the library each way (nsa_layer_fwd / nsa_layer_bwd)
        shared = kv_compress is None and kv_sliding is None
        cont = lambda t: t if t.is_contiguous() else t.contiguous()
        desc = ops.layer_desc(q, k_slc, v_slc, phi_params[1].shape[0], cfg.l, cfg.d, cfg.l_prime, cfg.n,
                              cfg.n_fixed if cfg.include_fixed_in_selection else 0, cfg.w, cfg.gate_mode, scale, token_major_out)
        forced = None if indices is None else indices.to(device=q.device, dtype=torch.int32).contiguous()
        out, saved = _LayerC.apply(cont(q), cont(k_slc), cont(v_slc), cont(kc_src), cont(vc_src), cont(kw), cont(vw), gate_logits,
                                   *phi_params, desc, shared, forced)
        if not return_info:
            return out
        v_ = ops.layer_ctx_views(desc, saved)
        return out, dict(indices=indices.to(torch.int32) if indices is not None else v_["indices"], gates=v_["gates"],
                         k_cmp=v_["k_cmp"], v_cmp=v_["v_cmp"], block_ends=v_["block_ends"], o_cmp=v_["o_cmp"], o_slc=v_["o_slc"],
                         o_win=v_["o_win"])
    nb = max(0, (T - cfg.l) // cfg.d + 1)
    if nb == 0:
        # shorter than one compression block: only the reference's padding block exists (nsa/kernels.py:2137-2142,
        # 2181-2186); the compressed branch outputs zero and every row's Eq. 8 falls back to block 0
        k_cmp = q.new_zeros(q.shape[0], k_slc.shape[1], q.shape[-1], 1, dtype=torch.float32)
        v_cmp = q.new_zeros(q.shape[0], k_slc.shape[1], 1, v_slc.shape[-1])
    elif compressed is None:
        pos_embed, w1, b1, w2, b2 = phi_params
        k_cmp, v_cmp = _PhiCompress.apply(kc_src.transpose(-1, -2), vc_src, pos_embed, w1, b1, w2, b2, cfg.l, cfg.d)
    else:
        k_cmp, v_cmp = compressed
        if k_cmp.shape[-1] < nb or v_cmp.shape[2] < nb:
            raise ValueError(f"compressed keys/values hold {k_cmp.shape[-1]}/{v_cmp.shape[2]} blocks, the sequence has {nb}")
        nbp = _next_pow2(nb)
        F = torch.nn.functional
        k_cmp = F.pad(k_cmp[..., :nb].float(), (0, nbp - nb))
        v_cmp = F.pad(v_cmp[:, :, :nb], (0, 0, 0, nbp - nb))
    block_ends = _block_ends(k_cmp.shape[-1], nb, cfg.l, cfg.d, q.device)
    if indices is not None:
        indices = indices.to(device=q.device, dtype=torch.int32).contiguous()
    out, gates, o_cmp, o_slc, o_win, indices = _BranchesAndMix.apply(q, k_cmp.to(q.dtype), v_cmp, block_ends, k_slc, v_slc, indices,
                                                                     kw, vw, gate_logits, scale, cfg, (cfg.l, cfg.d, nb), q_pos0,
                                                                     token_major_out, k_cmp.detach())
    if return_info:
        return out, dict(indices=indices, gates=gates, k_cmp=k_cmp, v_cmp=v_cmp, block_ends=block_ends,
                         o_cmp=o_cmp, o_slc=o_slc, o_win=o_win)
    return out


# --------------------------------------------------------------------------------------------------
# module (nsa/kernels.py:2043-2507)
# --------------------------------------------------------------------------------------------------

def _project_heads(x: torch.Tensor, linear: torch.nn.Linear, heads: int, dim: int, transposed: bool = False):
    """``linear(x)`` of x [B,T,d_model] written by the GEMM itself in the kernels' layout: [B,heads,T,dim], or
    [B,heads,dim,T] when ``transposed`` (keys).  The reference projects to [B,T,heads*dim] and then copies into these
    layouts (``transpose().contiguous()``, nsa/kernels.py:2361-2364).  Keys come out of one GEMM W x^T per batch
    element; queries and values out of a GEMM batched over the heads, with x shared by a zero batch stride."""
    w, b = linear.weight, linear.bias
    if transposed:
        y = torch.matmul(w, x.transpose(1, 2)).view(x.shape[0], heads, dim, x.shape[1])          # [B,heads,dim,T]
        return y if b is None else y + b.view(heads, dim, 1)
    wt = w.view(heads, dim, -1).transpose(1, 2)                                                  # [heads,d_model,dim]
    y = torch.stack([torch.matmul(xb, wt) for xb in x]) if x.shape[0] > 1 else torch.matmul(x[0], wt).unsqueeze(0)
    return y if b is None else y + b.view(heads, 1, dim)


class NSAAttention(torch.nn.Module):
    """Drop-in for the reference's ``NSAAttention``: same parameter names (so its state_dicts load),
    same ``forward(hidden_states, attention_mask=None, output_attentions=False) -> (out, info)``."""

    def __init__(self, config: NSAConfig):
        super().__init__()
        self.config = config
        c = config
        lin = torch.nn.Linear
        self.q_proj = lin(c.d_model, c.n_heads * c.head_dim_qk, bias=c.use_bias)
        self.k_compress = lin(c.d_model, c.n_kv_groups * c.head_dim_qk, bias=c.use_bias)
        self.v_compress = lin(c.d_model, c.n_kv_groups * c.head_dim_v, bias=c.use_bias)
        self.k_select = lin(c.d_model, c.n_kv_groups * c.head_dim_qk, bias=c.use_bias)
        self.v_select = lin(c.d_model, c.n_kv_groups * c.head_dim_v, bias=c.use_bias)
        self.k_sliding = lin(c.d_model, c.n_kv_groups * c.head_dim_qk, bias=c.use_bias)
        self.v_sliding = lin(c.d_model, c.n_kv_groups * c.head_dim_v, bias=c.use_bias)
        self.pos_embed = torch.nn.Embedding(c.l, c.l)
        self.compress_mlp = torch.nn.Sequential(lin(c.head_dim_qk + c.l, c.head_dim_qk * 2), torch.nn.ReLU(),
                                                lin(c.head_dim_qk * 2, c.head_dim_qk))
        self.gate_mlp = torch.nn.Sequential(lin(c.d_model, c.d_model // 2), torch.nn.ReLU(),
                                            lin(c.d_model // 2, 3 * c.n_heads))
        self.o_proj = lin(c.n_heads * c.head_dim_v, c.d_model, bias=c.use_bias)
        self.dropout = torch.nn.Dropout(c.dropout_p)
        self.scale = 1.0 / math.sqrt(c.head_dim_qk)

    def _phi_params(self):
        m = self.compress_mlp
        return (self.pos_embed.weight, m[0].weight, m[0].bias, m[2].weight, m[2].bias)

    def compress_tokens(self, keys: torch.Tensor, values: torch.Tensor):
        """keys [B,G,T,dk], values [B,G,T,dv] -> (k_cmp [B,G,dk,nbp], v_cmp [B,G,nbp,dv],
        block_ends [nbp] int32, n_blocks_actual); nbp = block count padded to a power of two with zero
        blocks whose block end is 999999."""
        c = self.config
        T = keys.shape[2]
        nb = max(0, (T - c.l) // c.d + 1)
        if nb == 0:
            k_cmp = keys.new_zeros(keys.shape[0], keys.shape[1], keys.shape[3], 1)
            v_cmp = values.new_zeros(values.shape[0], values.shape[1], 1, values.shape[3])
        else:
            k_cmp, v_cmp = _PhiCompress.apply(keys, values, *self._phi_params(), c.l, c.d)
        return k_cmp.to(keys.dtype), v_cmp, _block_ends(k_cmp.shape[-1], nb, c.l, c.d, keys.device).clone(), nb

    def forward(self, hidden_states: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                output_attentions: bool = False) -> Tuple[torch.Tensor, Optional[Dict]]:
        c = self.config
        B, T, _ = hidden_states.shape
        H, G, dk, dv = c.n_heads, c.n_kv_groups, c.head_dim_qk, c.head_dim_v
        q = _project_heads(hidden_states, self.q_proj, H, dk)                                    # [B,H,T,dk]

        def kv(kp, vp):
            return (_project_heads(hidden_states, kp, G, dk, transposed=True),                   # [B,G,dk,T]
                    _project_heads(hidden_states, vp, G, dv))                                    # [B,G,T,dv]

        k_sel, v_sel = kv(self.k_select, self.v_select)
        gate_logits = gate_logits_from_hidden(hidden_states, self.gate_mlp)                      # [B,T,3H] fp32
        out, info = nsa_layer(q, k_sel, v_sel, gate_logits, self._phi_params(), c,
                              kv_compress=kv(self.k_compress, self.v_compress),
                              kv_sliding=kv(self.k_sliding, self.v_sliding), scale=self.scale, return_info=True,
                              token_major_out=True)
        # the mix epilogue wrote [B,T,H,dv] in memory: this reshape is a view, not the copy of nsa/kernels.py:2466-2467
        y = self.o_proj(out.permute(0, 2, 1, 3).reshape(B, T, H * dv))
        y = self.dropout(y)
        attn_info = None
        if output_attentions:
            with torch.no_grad():
                p_cmp = ops.cmp_probs(q, info["k_cmp"], info["block_ends"], self.scale)
                sel = ops.eq9_scores(p_cmp, c.l, c.d, c.l_prime)
            attn_info = {
                "compression_scores": p_cmp.to(q.dtype),
                "selection_scores": sel.to(q.dtype),
                "selected_indices": info["indices"].to(torch.int64),
                "gates": info["gates"].permute(0, 2, 1, 3).to(q.dtype),                         # [B,T,H,3]
            }
        return y, attn_info


# --------------------------------------------------------------------------------------------------
# launcher shims for the raw kernel-call contract (README.md:55-101, examples/basic_usage.py:48-114)
# --------------------------------------------------------------------------------------------------

def _names(prefix, dims):
    return [f"stride_{prefix}{d}" for d in dims]


_Q, _K, _V, _O = _names("q", "zhmk"), _names("k", "zgnk"), _names("v", "zgnk"), _names("o", "zhmk")
_BI = _names("b", "zgmn")
_LM = _names("l", "zhm") + _names("m", "zhm")
_DG = _names("dq", "zhmk") + _names("dk", "zgnk") + _names("dv", "zgnk")


class _Launcher:
    """``launcher[grid](*positional, **constexpr)`` with the reference kernel's parameter order.

    ``grid`` is accepted and ignored (the CUDA kernels size their own grids), as are BLOCK_M/BLOCK_N.
    The strides passed by the caller are honoured as given.  Before any launch the extent every tensor's strides
    address is checked against its storage: a tensor the kernels read (Q, K, V, dOut, and Out/L/M in the backward) is
    served from a zero-padded copy when the strides reach past it (the contract tests pass wrong K strides on purpose
    and expect a different answer, not a fault); a tensor the kernels write (Out, L, M, dQ, dK, dV) or the index tensor
    raises ValueError instead, as do negative strides and a Block_ends shorter than N_BLOCKS.
    """

    def __init__(self, name: str, positional: List[str], kind: str, backward: bool):
        self.__name__ = name
        self.positional, self.kind, self.backward = positional, kind, backward

    def __getitem__(self, grid):
        def launch(*args, **kwargs):
            if len(args) > len(self.positional):
                raise TypeError(f"{self.__name__}: too many positional arguments")
            named = dict(zip(self.positional, args))
            dup = set(named) & set(kwargs)
            if dup:
                raise TypeError(f"{self.__name__}: got multiple values for {sorted(dup)}")
            named.update(kwargs)
            return self._run(named)
        return launch

    @staticmethod
    def _extent(name: str, strides, dims) -> int:
        """Elements from the first to one past the last one addressed through ``strides`` over ``dims``."""
        if any(int(s_) < 0 for s_ in strides):
            raise ValueError(f"{name}: negative strides are not supported")
        if any(int(n_) <= 0 for n_ in dims):
            return 0
        return 1 + sum((int(n_) - 1) * int(s_) for n_, s_ in zip(dims, strides))

    @staticmethod
    def _have(t: torch.Tensor) -> int:
        return t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()

    @classmethod
    def _safe(cls, name: str, t: torch.Tensor, strides, dims):
        """A tensor the kernels only READ: served from a zero-padded copy when the strides reach past its storage."""
        need, have = cls._extent(name, strides, dims), cls._have(t)
        if need <= have:
            return t
        buf = torch.zeros(need, device=t.device, dtype=t.dtype)
        buf[:have] = torch.as_strided(t, (have,), (1,))
        return buf

    @classmethod
    def _fits(cls, name: str, t: torch.Tensor, strides, dims):
        """A tensor the kernels WRITE: refused (before any launch) when the strides reach past its storage."""
        need, have = cls._extent(name, strides, dims), cls._have(t)
        if need > have:
            raise ValueError(f"{name}: strides {tuple(int(s_) for s_ in strides)} over shape {tuple(int(n_) for n_ in dims)} "
                             f"address {need} elements but the tensor's storage holds {have}")
        return t

    def _run(self, a):
        from ._lib import check, dtype_code, i64, lib, ptr, require_cuda, stream_ptr
        kind = self.kind
        Q, Out = a["Q"], a["Out"]
        if kind == "cmp":
            K = a["K_compressed"] if "K_compressed" in a else a["K_blocks"]
            V = a["V_compressed"] if "V_compressed" in a else a["V_blocks"]
        else:
            K, V = a["K"], a["V"]
        B, H, G = int(a["Z"]), int(a["H"]), int(a["N_KV_GROUPS"])
        dk, dv = Q.shape[-1], V.shape[-1]
        if kind == "win":
            Tq = Tk = int(a["N_CTX"])
        elif kind == "cmp":
            Tq, Tk = int(a["N_CTX_Q"]), int(a["N_BLOCKS"])
        else:
            Tq, Tk = int(a["N_CTX_Q"]), int(a["N_CTX_KV"])
        scale = float(a["sm_scale"])
        dev = require_cuda(Q, K, V, Out)
        sq, sk, sv, so = ([a[n] for n in names] for names in (_Q, _K, _V, _O))
        sl, sm = [a[n] for n in _LM[:3]], [a[n] for n in _LM[3:]]
        L, M = a["L"], a["M"]
        Q = self._safe("Q", Q, sq, (B, H, Tq, dk))
        K = self._safe("K", K, sk, (B, G, Tk, dk))
        V = self._safe("V", V, sv, (B, G, Tk, dv))
        if self.backward:      # read by the backward kernels
            Out = self._safe("Out", Out, so, (B, H, Tq, dv))
            L = self._safe("L", L, sl, (B, H, Tq))
            M = self._safe("M", M, sm, (B, H, Tq))
        else:                  # written by the forward kernels
            self._fits("Out", Out, so, (B, H, Tq, dv))
            self._fits("L", L, sl, (B, H, Tq))
            self._fits("M", M, sm, (B, H, Tq))
        strides = sq + sk + sv + so + sl + sm
        idx = None
        if self.backward:
            sdq, sdk, sdv = ([a[n] for n in names] for names in (_DG[:4], _DG[4:8], _DG[8:]))
            strides += sdq + sdk + sdv
            dO = self._safe("dOut", a["dOut"], so, (B, H, Tq, dv))     # dOut shares Out's strides
            dQ = self._fits("dQ", a["dQ"], sdq, (B, H, Tq, dk))
            dK = self._fits("dK", a["dK"], sdk, (B, G, Tk, dk))
            dV = self._fits("dV", a["dV"], sdv, (B, G, Tk, dv))
        if kind == "slc":
            idx = a["Block_indices"]
            if idx.dtype != torch.int32:
                raise TypeError("Block_indices must be int32")
            sb = [a[n] for n in _BI]
            self._fits("Block_indices", idx, sb, (B, G, Tq, int(a["N_BLOCKS"])))
            strides += sb
            if not bool(a.get("IS_CAUSAL", True)):
                raise NotImplementedError("selection kernels are causal")
        be = None
        if kind == "cmp":
            be = a["Block_ends"].to(torch.int32).contiguous()
            if be.numel() < Tk:
                raise ValueError(f"Block_ends holds {be.numel()} entries, N_BLOCKS is {Tk}")
        code = dtype_code(Q)
        st = stream_ptr(dev)
        with torch.cuda.device(dev):
            if not self.backward:
                if kind == "win":
                    rc = lib.nsa_sliding_fwd(ptr(Q), ptr(K), ptr(V), ptr(Out), ptr(L), ptr(M), i64(strides), B, H, G, Tq,
                                             dk, dv, int(a["WINDOW_SIZE"]), scale, code, 0, st)
                elif kind == "cmp":
                    rc = lib.nsa_cmp_attn_fwd(ptr(Q), ptr(K), ptr(V), ptr(be), ptr(Out), ptr(L), ptr(M), i64(strides), B, H,
                                              G, Tq, Tk, dk, dv, scale, code, 0, 0, 0, 0, 0, None, None, st)
                else:
                    n, lp = int(a["N_BLOCKS"]), int(a["BLOCK_SIZE_SELECTION"])
                    nbytes = lib.nsa_slc_fwd_workspace_bytes(B, H, G, Tq, Tk, dk, dv, n, lp, code, 0)
                    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
                    rc = lib.nsa_slc_fwd(ptr(Q), ptr(K), ptr(V), ptr(idx), ptr(Out), ptr(L), ptr(M), i64(strides), B, H, G,
                                         Tq, Tk, n, lp, dk, dv, scale, code, 0, 0, ptr(ws), nbytes, st)
            else:
                if kind == "win":
                    nbytes = lib.nsa_attn_bwd_workspace_bytes(B, H, G, Tq, Tk, dk, dv, 0, int(a["WINDOW_SIZE"]), 0)
                    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
                    rc = lib.nsa_sliding_bwd(ptr(Q), ptr(K), ptr(V), ptr(Out), ptr(dO), ptr(L), ptr(M), ptr(dQ), ptr(dK),
                                             ptr(dV), i64(strides), B, H, G, Tq, dk, dv, int(a["WINDOW_SIZE"]), scale, code,
                                             None, 0, ptr(ws), nbytes, st)
                elif kind == "cmp":
                    rc = lib.nsa_cmp_attn_bwd(ptr(Q), ptr(K), ptr(V), ptr(be), ptr(Out), ptr(dO), ptr(L), ptr(M), ptr(dQ),
                                              ptr(dK), ptr(dV), i64(strides), B, H, G, Tq, Tk, dk, dv, scale, code, 0, 0, 0,
                                              0, None, 0, None, 0, st)
                else:
                    n = int(a["N_BLOCKS"])
                    lp = int(a["BLOCK_SIZE_SELECTION"])
                    nbytes = lib.nsa_slc_bwd_workspace_bytes(B, H, G, Tq, Tk, dk, dv, n, lp, code, 0)
                    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
                    rc = lib.nsa_slc_bwd(ptr(Q), ptr(K), ptr(V), ptr(idx), ptr(Out), ptr(dO), ptr(L), ptr(M), ptr(dQ),
                                         ptr(dK), ptr(dV), i64(strides), B, H, G, Tq, Tk, n, lp, dk, dv, scale, code,
                                         0, None, None, None, 0, ptr(ws), nbytes, st)
        check(rc, self.__name__)


def _sig(kind: str, backward: bool) -> List[str]:
    kv = {"win": ["K", "V"], "cmp": ["K_compressed" if not backward else "K_blocks",
                                     "V_compressed" if not backward else "V_blocks", "Block_ends"],
          "slc": ["K", "V", "Block_indices"]}[kind]
    head = ["Q"] + kv + ["Out"] + (["dOut"] if backward else []) + ["sm_scale", "L", "M"]
    strides = _Q + _K + _V + _O + (_BI if kind == "slc" else []) + _LM
    tail = (["dQ", "dK", "dV"] + _DG) if backward else []
    return head + strides + tail


_nsa_sliding_window_fwd_kernel = _Launcher("_nsa_sliding_window_fwd_kernel", _sig("win", False), "win", False)
_nsa_sliding_window_bwd_kernel = _Launcher("_nsa_sliding_window_bwd_kernel", _sig("win", True), "win", True)
_nsa_compression_fwd_kernel = _Launcher("_nsa_compression_fwd_kernel", _sig("cmp", False), "cmp", False)
_nsa_compression_bwd_kernel = _Launcher("_nsa_compression_bwd_kernel", _sig("cmp", True), "cmp", True)
_nsa_sparse_selection_fwd_kernel = _Launcher("_nsa_sparse_selection_fwd_kernel", _sig("slc", False), "slc", False)
_nsa_sparse_selection_bwd_kernel = _Launcher("_nsa_sparse_selection_bwd_kernel", _sig("slc", True), "slc", True)
