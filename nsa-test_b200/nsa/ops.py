"""Tensor-level wrappers of the C-ABI entry points: compute strides, pick the stream, check status.

Each function launches asynchronously on the current CUDA stream of the tensors' device and returns
nothing but its outputs; shapes follow the reference project's kernel-call contract
(K is [B,G,dk,T] in memory, dK comes back time-major [B,G,T,dk]).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import check, dtype_code, i64, lib, ptr, require_cuda, stream_ptr


def _k_strides(k: torch.Tensor):
    """Strides of a [B,G,dk,T] key tensor in the contract's (z, g, n=time, k=dk) order."""
    return [k.stride(0), k.stride(1), k.stride(3), k.stride(2)]


def _fwd_strides(q, k, v, o, L, M):
    return list(q.stride()) + _k_strides(k) + list(v.stride()) + list(o.stride()) + list(L.stride()) + list(M.stride())


def _stats(q, o_dv):
    B, H, T, _ = q.shape
    o = torch.empty(B, H, T, o_dv, device=q.device, dtype=q.dtype)
    L = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    M = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    return o, L, M


# ------------------------------------------------------------------------------------------------
# the three branches
# ------------------------------------------------------------------------------------------------

def sliding_fwd(q, k, v, window: int, scale: float, generic: bool = False):
    """``generic=True`` forces the stride-generic kernels (cross-checks); same for the functions below."""
    dev = require_cuda(q, k, v)
    B, H, T, dk = q.shape
    G, dv = k.shape[1], v.shape[-1]
    o, L, M = _stats(q, dv)
    with torch.cuda.device(dev):
        check(lib.nsa_sliding_fwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(L), ptr(M), i64(_fwd_strides(q, k, v, o, L, M)),
                                  B, H, G, T, dk, dv, int(window), float(scale), dtype_code(q), _flags(generic),
                                  stream_ptr(dev)), "nsa_sliding_fwd")
    return o, L, M


def sliding_bwd(q, k, v, o, do, L, M, window: int, scale: float, row_delta=None, generic: bool = False,
                recompute: bool = False):
    """``row_delta``: the row sums dO.O [B,H,T] (fp32) when the caller has them, else they are computed here.
    ``recompute``: small scratch; the dQ kernel recomputes S and dP instead of taking dS from the dK/dV kernel."""
    dev = require_cuda(q, k, v, o, do, L, M)
    delta, dptr = _delta_ptr(row_delta, q)
    B, H, T, dk = q.shape
    G, dv = k.shape[1], v.shape[-1]
    if do.stride() != o.stride():
        do = do.contiguous()
        o = o.contiguous()
    dq = torch.empty_like(q)
    dkey = torch.zeros(B, G, T, dk, device=dev, dtype=q.dtype)
    dval = torch.zeros(B, G, T, dv, device=dev, dtype=q.dtype)
    s = _fwd_strides(q, k, v, o, L, M) + list(dq.stride()) + list(dkey.stride()) + list(dval.stride())
    nbytes = lib.nsa_attn_bwd_workspace_bytes(B, H, G, T, T, dk, dv, 0, int(window), _flags(generic, recompute))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_sliding_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(L), ptr(M), ptr(dq), ptr(dkey), ptr(dval),
                                  i64(s), B, H, G, T, dk, dv, int(window), float(scale), dtype_code(q), dptr, _flags(generic),
                                  ptr(ws), nbytes, stream_ptr(dev)), "nsa_sliding_bwd")
    return dq, dkey, dval


def _flags(generic: bool, recompute: bool = False) -> int:
    return (_lib.FLAG_GENERIC if generic else 0) | (_lib.FLAG_RECOMPUTE if recompute else 0)


def _delta_ptr(row_delta, q):
    """Row sums dO.O [B,H,T] fp32 handed to a backward call, or None."""
    if row_delta is None:
        return None, None
    d = row_delta.contiguous()
    if d.dtype != torch.float32 or d.shape != q.shape[:3] or d.device != q.device:
        raise ValueError("row_delta must be a float32 [B,H,T] tensor on the device of q")
    return d, ptr(d)


def cmp_exact_supported(q, k_cmp, v_cmp) -> bool:
    """Does this shape admit the hi + lo key form of the compressed attention's forward (bf16 tensor-core path)?"""
    B, H, T, dk = q.shape
    return q.dtype == torch.bfloat16 and bool(lib.nsa_cmp_attn_exact_supported(B, H, k_cmp.shape[1], T, k_cmp.shape[-1], dk,
                                                                              v_cmp.shape[-1], dtype_code(q)))


def split_keys(k_cmp_f32):
    """fp32 compressed keys -> (hi, lo) bf16 with hi + lo equal to the fp32 value to 16 mantissa bits."""
    dev = require_cuda(k_cmp_f32)
    x = k_cmp_f32.float().contiguous()
    hi = torch.empty(x.shape, device=dev, dtype=torch.bfloat16)
    lo = torch.empty(x.shape, device=dev, dtype=torch.bfloat16)
    with torch.cuda.device(dev):
        check(lib.nsa_split_keys_hi_lo(ptr(x), ptr(hi), ptr(lo), x.numel(), stream_ptr(dev)), "nsa_split_keys_hi_lo")
    return hi, lo


def cmp_attn_fwd(q, k_cmp, v_cmp, block_ends, scale: float, blocks=None, q_pos0: int = 0, generic: bool = False, k_lo=None):
    """``blocks=(l, d, n_blocks)`` asserts block_ends[i] == i*d + l - 1 for i < n_blocks and no later block
    ever visible; it lets the tensor-core kernel bound its key loop.  ``k_lo`` (the low-order bf16 part of the keys,
    k_cmp being the high-order one) selects the exact-key form; a fourth result, the log-sum-exp of the logits in log2
    units (+inf on rows that see no block), is then returned for score_topn's ``cmp_lse2``."""
    bl, bd, bn = blocks if blocks is not None else (0, 0, 0)
    dev = require_cuda(q, k_cmp, v_cmp, block_ends)
    B, H, T, dk = q.shape
    G, NB, dv = k_cmp.shape[1], k_cmp.shape[-1], v_cmp.shape[-1]
    be = block_ends.to(torch.int32).contiguous()
    o, L, M = _stats(q, dv)
    lse2 = torch.empty(B, H, T, device=dev, dtype=torch.float32) if k_lo is not None else None
    with torch.cuda.device(dev):
        check(lib.nsa_cmp_attn_fwd(ptr(q), ptr(k_cmp), ptr(v_cmp), ptr(be), ptr(o), ptr(L), ptr(M),
                                   i64(_fwd_strides(q, k_cmp, v_cmp, o, L, M)), B, H, G, T, NB, dk, dv, float(scale),
                                   dtype_code(q), int(bl), int(bd), int(bn), int(q_pos0), _flags(generic), ptr(k_lo), ptr(lse2),
                                   stream_ptr(dev)), "nsa_cmp_attn_fwd")
    return (o, L, M) if k_lo is None else (o, L, M, lse2)


def cmp_attn_bwd(q, k_cmp, v_cmp, block_ends, o, do, L, M, scale: float, blocks=None, q_pos0: int = 0, row_delta=None,
                 generic: bool = False, recompute: bool = False):
    bl, bd, bn = blocks if blocks is not None else (0, 0, 0)
    dev = require_cuda(q, k_cmp, v_cmp, block_ends, o, do, L, M)
    delta, dptr = _delta_ptr(row_delta, q)
    B, H, T, dk = q.shape
    G, NB, dv = k_cmp.shape[1], k_cmp.shape[-1], v_cmp.shape[-1]
    be = block_ends.to(torch.int32).contiguous()
    if do.stride() != o.stride():
        do = do.contiguous()
        o = o.contiguous()
    dq = torch.empty_like(q)
    dkc = torch.zeros(B, G, NB, dk, device=dev, dtype=q.dtype)
    dvc = torch.zeros(B, G, NB, dv, device=dev, dtype=q.dtype)
    s = _fwd_strides(q, k_cmp, v_cmp, o, L, M) + list(dq.stride()) + list(dkc.stride()) + list(dvc.stride())
    nbytes = lib.nsa_attn_bwd_workspace_bytes(B, H, G, T, NB, dk, dv, 1, 0, _flags(generic, recompute))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_cmp_attn_bwd(ptr(q), ptr(k_cmp), ptr(v_cmp), ptr(be), ptr(o), ptr(do), ptr(L), ptr(M), ptr(dq),
                                   ptr(dkc), ptr(dvc), i64(s), B, H, G, T, NB, dk, dv, float(scale), dtype_code(q),
                                   int(bl), int(bd), int(bn), int(q_pos0), dptr, _flags(generic), ptr(ws), nbytes,
                                   stream_ptr(dev)), "nsa_cmp_attn_bwd")
    return dq, dkc, dvc


def slc_fwd(q, k, v, indices_i32, l_prime: int, scale: float, q_pos0: int = 0, generic: bool = False):
    dev = require_cuda(q, k, v, indices_i32)
    B, H, Tq, dk = q.shape
    G, Tkv, dv = k.shape[1], k.shape[-1], v.shape[-1]
    assert indices_i32.dtype == torch.int32
    o, L, M = _stats(q, dv)
    s = _fwd_strides(q, k, v, o, L, M) + list(indices_i32.stride())
    n = indices_i32.shape[-1]
    nbytes = lib.nsa_slc_fwd_workspace_bytes(B, H, G, Tq, Tkv, dk, dv, n, int(l_prime), dtype_code(q), _flags(generic))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_slc_fwd(ptr(q), ptr(k), ptr(v), ptr(indices_i32), ptr(o), ptr(L), ptr(M), i64(s), B, H, G, Tq, Tkv,
                              n, int(l_prime), dk, dv, float(scale), dtype_code(q), int(q_pos0), _flags(generic), ptr(ws),
                              nbytes, stream_ptr(dev)), "nsa_slc_fwd")
    return o, L, M


def _mixed_empty(like: torch.Tensor, token_major: bool) -> torch.Tensor:
    """Buffer for the mixed output of shape [B,H,T,dv]: contiguous, or (token_major) a [B,H,T,dv] view of a contiguous
    [B,T,H,dv] buffer, which ``.permute(0, 2, 1, 3).reshape(B, T, H*dv)`` turns into o_proj's input without a copy."""
    B, H, T, dv = like.shape
    if not token_major:
        return torch.empty(B, H, T, dv, device=like.device, dtype=like.dtype)
    return torch.empty(B, T, H, dv, device=like.device, dtype=like.dtype).permute(0, 2, 1, 3)


def slc_fwd_mix(q, k, v, indices_i32, l_prime: int, scale: float, gate_logits, o_cmp, o_win, gate_mode: str, q_pos0: int = 0,
                token_major: bool = False, generic: bool = False):
    """Selection forward with the layer's gate + mix as its epilogue -> (o_slc, L, M, out_mixed, gates [B,H,T,3])."""
    dev = require_cuda(q, k, v, indices_i32, gate_logits, o_cmp, o_win)
    B, H, Tq, dk = q.shape
    G, Tkv, dv = k.shape[1], k.shape[-1], v.shape[-1]
    assert indices_i32.dtype == torch.int32
    o, L, M = _stats(q, dv)
    s = _fwd_strides(q, k, v, o, L, M) + list(indices_i32.stride())
    n = indices_i32.shape[-1]
    lg = gate_logits.float().contiguous()
    o_cmp, o_win = o_cmp.contiguous(), o_win.contiguous()
    out = _mixed_empty(o, token_major)
    gates = torch.empty(B, H, Tq, 3, device=dev, dtype=torch.float32)
    mode = _lib.GATE_SOFTMAX if gate_mode == "softmax" else _lib.GATE_SIGMOID
    nbytes = lib.nsa_slc_fwd_workspace_bytes(B, H, G, Tq, Tkv, dk, dv, n, int(l_prime), dtype_code(q), _flags(generic))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_slc_fwd_mix(ptr(q), ptr(k), ptr(v), ptr(indices_i32), ptr(o), ptr(L), ptr(M), i64(s), B, H, G, Tq, Tkv,
                                  n, int(l_prime), dk, dv, float(scale), dtype_code(q), int(q_pos0), _flags(generic), ptr(lg),
                                  ptr(o_cmp), ptr(o_win), ptr(out), ptr(gates), mode, 1 if token_major else 0, ptr(ws), nbytes,
                                  stream_ptr(dev)), "nsa_slc_fwd_mix")
    return o, L, M, out, gates


def slc_bwd(q, k, v, indices_i32, o, do, L, M, l_prime: int, scale: float, q_pos0: int = 0, dq_addends=(), row_delta=None,
            generic: bool = False):
    """``dq_addends``: up to two tensors shaped and typed like q (the dQ of the other branches) that the kernel adds
    to the selection branch's dQ before the one rounding of the sum."""
    dev = require_cuda(q, k, v, indices_i32, o, do, L, M)
    delta, dptr = _delta_ptr(row_delta, q)
    B, H, Tq, dk = q.shape
    G, Tkv, dv = k.shape[1], k.shape[-1], v.shape[-1]
    n = indices_i32.shape[-1]
    if do.stride() != o.stride():
        do = do.contiguous()
        o = o.contiguous()
    dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    dkey = torch.zeros(B, G, Tkv, dk, device=dev, dtype=q.dtype)
    dval = torch.zeros(B, G, Tkv, dv, device=dev, dtype=q.dtype)
    nbytes = lib.nsa_slc_bwd_workspace_bytes(B, H, G, Tq, Tkv, dk, dv, n, int(l_prime), dtype_code(q), _flags(generic))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    s = (_fwd_strides(q, k, v, o, L, M) + list(dq.stride()) + list(dkey.stride()) + list(dval.stride())
         + list(indices_i32.stride()))
    adds = [a.contiguous() for a in dq_addends]
    if any(a.shape != q.shape or a.dtype != q.dtype or a.device != q.device for a in adds) or len(adds) > 2:
        raise ValueError("slc_bwd: dq_addends must be at most two tensors shaped and typed like q")
    add0 = ptr(adds[0]) if len(adds) > 0 else None
    add1 = ptr(adds[1]) if len(adds) > 1 else None
    with torch.cuda.device(dev):
        check(lib.nsa_slc_bwd(ptr(q), ptr(k), ptr(v), ptr(indices_i32), ptr(o), ptr(do), ptr(L), ptr(M), ptr(dq),
                              ptr(dkey), ptr(dval), i64(s), B, H, G, Tq, Tkv, n, int(l_prime), dk, dv, float(scale),
                              dtype_code(q), int(q_pos0), dptr, add0, add1, _flags(generic), ptr(ws), nbytes,
                              stream_ptr(dev)), "nsa_slc_bwd")
    return dq, dkey, dval


# ------------------------------------------------------------------------------------------------
# phi pooling, scoring, gates
# ------------------------------------------------------------------------------------------------

def _next_pow2(n: int) -> int:
    p = 1
    while p < n:
        p *= 2
    return p


def cmp_phi_fwd(k, v, pos_embed, w1, b1, w2, b2, l: int, d: int):
    """Block compression phi through the C ABI.  k [B,G,dk,T], v [B,G,T,dv] (contiguous, one dtype); fp32 parameters.
    -> k_cmp fp32 [B,G,dk,nbp], v_cmp [B,G,nbp,dv], and the buffer the backward needs."""
    dev = require_cuda(k, v, pos_embed, w1, w2)
    B, G, dk, T = k.shape
    dv, U = v.shape[-1], w1.shape[0]
    if T < l:
        raise ValueError(f"sequence length {T} shorter than one compression block ({l})")
    nb = (T - l) // d + 1
    nbp = _next_pow2(nb)
    code = dtype_code(k)
    k_cmp = torch.empty(B, G, dk, nbp, device=dev, dtype=torch.float32)
    v_cmp = torch.empty(B, G, nbp, dv, device=dev, dtype=k.dtype)
    saved = torch.empty(lib.nsa_cmp_phi_saved_bytes(B, G, T, int(l), int(d), U), device=dev, dtype=torch.uint8)
    nbytes = lib.nsa_cmp_phi_workspace_bytes(B, G, T, dk, dv, int(l), int(d), U, nbp, code, 0)
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_cmp_phi_fwd(ptr(k), ptr(v), ptr(pos_embed), ptr(w1), ptr(b1), ptr(w2), ptr(b2), ptr(k_cmp), None, ptr(v_cmp),
                                  B, G, T, dk, dv, int(l), int(d), U, nbp, code, ptr(saved), saved.numel(), ptr(ws), nbytes,
                                  stream_ptr(dev)), "nsa_cmp_phi_fwd")
    return k_cmp, v_cmp, saved


def cmp_phi_bwd(k, pos_embed, w1, w2, dk_cmp, dv_cmp, saved, dv_dim: int, l: int, d: int):
    """dk_cmp [B,G,nbp,dk], dv_cmp [B,G,nbp,dv] in k's dtype -> (dk [B,G,T,dk], dv [B,G,T,dv] in k's dtype; dpos, dw1, db1,
    dw2, db2 fp32)."""
    dev = require_cuda(k, pos_embed, w1, w2, dk_cmp, dv_cmp, saved)
    B, G, dk, T = k.shape
    U, nbp = w1.shape[0], dk_cmp.shape[2]
    code = dtype_code(k)
    dkeys = torch.zeros(B, G, T, dk, device=dev, dtype=k.dtype)
    dvals = torch.zeros(B, G, T, dv_dim, device=dev, dtype=k.dtype)
    f32 = lambda *s_: torch.empty(*s_, device=dev, dtype=torch.float32)
    dpos, dw1, db1, dw2, db2 = f32(l, l), f32(U, dk + l), f32(U), f32(dk, U), f32(dk)
    nbytes = lib.nsa_cmp_phi_workspace_bytes(B, G, T, dk, dv_dim, int(l), int(d), U, nbp, code, 1)
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_cmp_phi_bwd(ptr(k), ptr(pos_embed), ptr(w1), ptr(w2), ptr(dk_cmp), ptr(dv_cmp), ptr(saved), saved.numel(),
                                  ptr(dkeys), ptr(dvals), ptr(dpos), ptr(dw1), ptr(db1), ptr(dw2), ptr(db2), B, G, T, dk, dv_dim,
                                  int(l), int(d), U, nbp, code, ptr(ws), nbytes, stream_ptr(dev)), "nsa_cmp_phi_bwd")
    return dkeys, dvals, dpos, dw1, db1, dw2, db2


def phi_pool_fwd(a, c, v, l: int, d: int, n_blocks: int, nbp: int):
    """a [B,G,T,U] fp32, c [l,U] fp32, v [B,G,T,dv] -> hbar [B,G,n_blocks,U] fp32, v_cmp [B,G,nbp,dv] (zero padded)."""
    dev = require_cuda(a, c, v)
    B, G, T, U = a.shape
    dv = v.shape[-1]
    a, c = a.contiguous(), c.contiguous()
    hbar = torch.empty(B, G, n_blocks, U, device=dev, dtype=torch.float32)
    v_cmp = torch.zeros(B, G, nbp, dv, device=dev, dtype=v.dtype)
    with torch.cuda.device(dev):
        check(lib.nsa_phi_pool_fwd(ptr(a), ptr(c), ptr(v), i64(v.stride()), ptr(hbar), ptr(v_cmp), B, G, T, U, dv, int(l),
                                   int(d), int(n_blocks), int(nbp), dtype_code(v), stream_ptr(dev)), "nsa_phi_pool_fwd")
    return hbar, v_cmp


def phi_pool_bwd(a, c, dhbar, dv_cmp, l: int, d: int, n_blocks: int):
    """-> da [B,G,T,U], dc [l,U] (summed over batch and group), dv [B,G,T,dv]; all fp32."""
    dev = require_cuda(a, c, dhbar, dv_cmp)
    B, G, T, U = a.shape
    nbp, dvd = dv_cmp.shape[2], dv_cmp.shape[3]
    a, c, dhbar, dv_cmp = a.contiguous(), c.contiguous(), dhbar.float().contiguous(), dv_cmp.float().contiguous()
    da = torch.empty_like(a)
    dc_part = torch.empty(B * G, int(l), U, device=dev, dtype=torch.float32)
    dv = torch.empty(B, G, T, dvd, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(lib.nsa_phi_pool_bwd(ptr(a), ptr(c), ptr(dhbar), ptr(dv_cmp), ptr(da), ptr(dc_part), ptr(dv), B, G, T, U,
                                   dvd, int(l), int(d), int(n_blocks), nbp, stream_ptr(dev)), "nsa_phi_pool_bwd")
    return da, dc_part.sum(0), dv


def score_topn(q, k_cmp_f32, block_ends, l: int, d: int, l_prime: int, n: int, n_fixed: int, scale: float,
               n_real_blocks: int = -1, q_pos0: int = 0, generic: bool = False, cmp_lse2=None):
    """q [B,H,T,dk], k_cmp fp32 [B,G,dk,nbp] -> int32 indices [B,G,T,n].  ``n_real_blocks >= 0`` asserts the
    canonical block ends (block i ends at i*d + l - 1 for i < n_real_blocks, later blocks never visible)."""
    dev = require_cuda(q, k_cmp_f32, block_ends)
    B, H, T, dk = q.shape
    G, nbp = k_cmp_f32.shape[1], k_cmp_f32.shape[-1]
    kc = k_cmp_f32.float().contiguous()
    be = block_ends.to(torch.int32).contiguous()
    out = torch.empty(B, G, T, n, device=dev, dtype=torch.int32)
    nbytes = lib.nsa_score_topn_workspace_bytes(B, H, G, T, dk, nbp, int(l), int(d), int(l_prime), int(n), dtype_code(q),
                                                _flags(generic))
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_score_topn(ptr(q), i64(q.stride()), ptr(kc), ptr(be), ptr(out), B, H, G, T, dk, nbp, int(l), int(d),
                                 int(l_prime), int(n), int(n_fixed), float(scale), dtype_code(q), int(n_real_blocks),
                                 int(q_pos0), _flags(generic), ptr(cmp_lse2), ptr(ws), nbytes, stream_ptr(dev)), "nsa_score_topn")
    return out


def topn_from_scores(scores, G: int, l_prime: int, n: int, n_fixed: int):
    """scores [B,H,T,n_sel] -> int32 indices [B,G,T,n]."""
    dev = require_cuda(scores)
    B, H, T, n_sel = scores.shape
    sc = scores.float().contiguous()
    out = torch.empty(B, G, T, n, device=dev, dtype=torch.int32)
    with torch.cuda.device(dev):
        check(lib.nsa_topn_from_scores(ptr(sc), ptr(out), B, H, G, T, n_sel, int(l_prime), int(n), int(n_fixed),
                                       stream_ptr(dev)), "nsa_topn_from_scores")
    return out


def cmp_probs(q, k_cmp_f32, block_ends, scale: float):
    """Eq. 8 probabilities materialised: [B,H,T,nbp] fp32 (diagnostics only)."""
    dev = require_cuda(q, k_cmp_f32, block_ends)
    B, H, T, dk = q.shape
    G, nbp = k_cmp_f32.shape[1], k_cmp_f32.shape[-1]
    kc = k_cmp_f32.float().contiguous()
    be = block_ends.to(torch.int32).contiguous()
    out = torch.empty(B, H, T, nbp, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(lib.nsa_cmp_probs(ptr(q), i64(q.stride()), ptr(kc), ptr(be), ptr(out), B, H, G, T, dk, nbp, float(scale),
                                dtype_code(q), stream_ptr(dev)), "nsa_cmp_probs")
    return out


def eq9_scores(p_cmp, l: int, d: int, l_prime: int):
    """[..., n_cmp] -> [..., ceil(n_cmp/(l'/d))] fp32."""
    dev = require_cuda(p_cmp)
    n_cmp = p_cmp.shape[-1]
    s_ = l_prime // d
    n_sel = (n_cmp + s_ - 1) // s_
    p = p_cmp.float().contiguous()
    out = torch.empty(*p.shape[:-1], n_sel, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(lib.nsa_eq9_scores(ptr(p), ptr(out), p.numel() // n_cmp, n_cmp, int(l), int(d), int(l_prime),
                                 stream_ptr(dev)), "nsa_eq9_scores")
    return out


def gate_mlp_fwd(x, w1, b1, w2, b2):
    """Branch-gate MLP through the C ABI: x [..., Dm] -> (logits [..., O] fp32, hidden [N, D2] for the backward)."""
    dev = require_cuda(x, w1, w2)
    Dm, D2, O = x.shape[-1], w1.shape[0], w2.shape[0]
    x2 = x.reshape(-1, Dm).contiguous()
    N = x2.shape[0]
    hidden = torch.empty(N, D2, device=dev, dtype=x.dtype)
    logits = torch.empty(*x.shape[:-1], O, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        check(lib.nsa_gate_mlp_fwd(ptr(x2), ptr(w1), ptr(b1), ptr(w2), ptr(b2), ptr(hidden), ptr(logits), N, Dm, D2, O, dtype_code(x),
                                   stream_ptr(dev)), "nsa_gate_mlp_fwd")
    return logits, hidden


def gate_mlp_bwd(x, w1, w2, hidden, dlogits, need_dx: bool):
    """-> (dx [..., Dm] in x's dtype or None, dw1, db1, dw2, db2 fp32)."""
    dev = require_cuda(x, w1, w2, hidden, dlogits)
    Dm, D2, O = x.shape[-1], w1.shape[0], w2.shape[0]
    x2 = x.reshape(-1, Dm).contiguous()
    N = x2.shape[0]
    dl = dlogits.reshape(N, O).float().contiguous()
    dx = torch.empty(N, Dm, device=dev, dtype=x.dtype) if need_dx else None
    f32 = lambda *s_: torch.empty(*s_, device=dev, dtype=torch.float32)
    dw1, db1, dw2, db2 = f32(D2, Dm), f32(D2), f32(O, D2), f32(O)
    nbytes = lib.nsa_gate_mlp_workspace_bytes(N, Dm, D2, O, dtype_code(x), 1)
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        check(lib.nsa_gate_mlp_bwd(ptr(x2), ptr(w1), ptr(w2), ptr(hidden), ptr(dl), ptr(dx), ptr(dw1), ptr(db1), ptr(dw2), ptr(db2), N,
                                   Dm, D2, O, dtype_code(x), ptr(ws), nbytes, stream_ptr(dev)), "nsa_gate_mlp_bwd")
    return (dx.view(x.shape) if need_dx else None), dw1, db1, dw2, db2


def gate_mix_fwd(logits, o_cmp, o_slc, o_win, gate_mode: str, token_major: bool = False):
    """logits [B,T,3H]; branch outputs [B,H,T,dv] -> out [B,H,T,dv] (token_major: backed by a [B,T,H,dv] buffer),
    gates [B,H,T,3] fp32."""
    dev = require_cuda(logits, o_cmp, o_slc, o_win)
    B, H, T, dv = o_cmp.shape
    lg = logits.float().contiguous()
    o_cmp, o_slc, o_win = o_cmp.contiguous(), o_slc.contiguous(), o_win.contiguous()
    out = _mixed_empty(o_cmp, token_major)
    gates = torch.empty(B, H, T, 3, device=dev, dtype=torch.float32)
    mode = _lib.GATE_SOFTMAX if gate_mode == "softmax" else _lib.GATE_SIGMOID
    with torch.cuda.device(dev):
        check(lib.nsa_gate_mix_fwd(ptr(lg), ptr(o_cmp), ptr(o_slc), ptr(o_win), ptr(out), ptr(gates), B, H, T, dv, mode,
                                   dtype_code(o_cmp), 1 if token_major else 0, stream_ptr(dev)), "nsa_gate_mix_fwd")
    return out, gates


def gate_mix_bwd(gates, o_cmp, o_slc, o_win, dout, gate_mode: str, want_delta: bool = False):
    """-> (do_cmp, do_slc, do_win, dlogits [B,T,3H] fp32)."""
    dev = require_cuda(gates, o_cmp, o_slc, o_win, dout)
    B, H, T, dv = o_cmp.shape
    # the upstream gradient is read as it lies when it is head-major or token-major ([B,T,H,dv] memory), copied otherwise
    dout_tm = (not dout.is_contiguous()) and dout.permute(0, 2, 1, 3).is_contiguous()
    if not dout_tm:
        dout = dout.contiguous()
    o_cmp, o_slc, o_win = o_cmp.contiguous(), o_slc.contiguous(), o_win.contiguous()
    d0, d1, d2 = torch.empty_like(o_cmp), torch.empty_like(o_cmp), torch.empty_like(o_cmp)
    dlogits = torch.empty(B, T, 3 * H, device=dev, dtype=torch.float32)
    mode = _lib.GATE_SOFTMAX if gate_mode == "softmax" else _lib.GATE_SIGMOID
    delta = torch.empty(3, B, H, T, device=dev, dtype=torch.float32) if want_delta else None
    with torch.cuda.device(dev):
        check(lib.nsa_gate_mix_bwd_delta(ptr(gates), ptr(o_cmp), ptr(o_slc), ptr(o_win), ptr(dout), ptr(d0), ptr(d1), ptr(d2),
                                         ptr(dlogits), ptr(delta), B, H, T, dv, mode, dtype_code(o_cmp), 1 if dout_tm else 0,
                                         stream_ptr(dev)),
              "nsa_gate_mix_bwd")
    return (d0, d1, d2, dlogits, delta) if want_delta else (d0, d1, d2, dlogits)


# ------------------------------------------------------------------------------------------------
# the whole layer through nsa_layer_fwd / nsa_layer_bwd
# ------------------------------------------------------------------------------------------------

def layer_desc(q, k, v, U: int, l: int, d: int, l_prime: int, n: int, n_fixed: int, window: int, gate_mode: str, scale: float,
               token_major: bool) -> "_lib.LayerDesc":
    B, H, T, dk = q.shape
    return _lib.LayerDesc(B=B, H=H, G=k.shape[1], T=T, dk=dk, dv=v.shape[-1], U=int(U), l=int(l), d=int(d), l_prime=int(l_prime),
                          n=int(n), n_fixed=int(n_fixed), window=int(window),
                          gate_mode=_lib.GATE_SOFTMAX if gate_mode == "softmax" else _lib.GATE_SIGMOID, dtype=dtype_code(q),
                          out_token_major=1 if token_major else 0, scale=float(scale))


def layer_ctx_views(desc, ctx: torch.Tensor):
    """Named tensors inside the layer's context buffer (views, no copies)."""
    import ctypes
    offs = (ctypes.c_size_t * (len(_lib.CTX_PIECES) + 1))()
    lib.nsa_layer_ctx_bytes(ctypes.byref(desc), offs)
    B, H, G, T, dk, dv, n = desc.B, desc.H, desc.G, desc.T, desc.dk, desc.dv, desc.n
    dt = torch.bfloat16 if desc.dtype == _lib.BF16 else torch.float32
    nb = (T - desc.l) // desc.d + 1 if T >= desc.l else 0
    nbp = _next_pow2(max(nb, 1))
    shapes = dict(o_cmp=((B, H, T, dv), dt), L_cmp=((B, H, T), torch.float32), M_cmp=((B, H, T), torch.float32),
                  o_slc=((B, H, T, dv), dt), L_slc=((B, H, T), torch.float32), M_slc=((B, H, T), torch.float32),
                  o_win=((B, H, T, dv), dt), L_win=((B, H, T), torch.float32), M_win=((B, H, T), torch.float32),
                  gates=((B, H, T, 3), torch.float32), indices=((B, G, T, n), torch.int32),
                  k_cmp=((B, G, dk, nbp), torch.float32), k_cmp_lp=((B, G, dk, nbp), dt), v_cmp=((B, G, nbp, dv), dt),
                  block_ends=((nbp,), torch.int32))
    out = {}
    for i, name in enumerate(_lib.CTX_PIECES):
        if name not in shapes:
            continue
        shape, dtype = shapes[name]
        numel = 1
        for s_ in shape:
            numel *= s_
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        out[name] = ctx[offs[i]:offs[i] + nbytes].view(dtype).view(shape)
    return out


def _mixed_out(desc, q):
    if desc.out_token_major:
        return torch.empty(desc.B, desc.T, desc.H, desc.dv, device=q.device, dtype=q.dtype).permute(0, 2, 1, 3)
    return torch.empty(desc.B, desc.H, desc.T, desc.dv, device=q.device, dtype=q.dtype)


def layer_fwd(desc, q, kv_slc, kv_cmp, kv_win, gate_logits, phi, indices=None):
    """-> (out [B,H,T,dv] (token-major memory when the descriptor says so), ctx).  kv_* = (k [B,G,dk,T], v [B,G,T,dv])."""
    import ctypes
    dev = require_cuda(q, gate_logits)
    ctx_bytes = lib.nsa_layer_ctx_bytes(ctypes.byref(desc), None)
    if ctx_bytes == 0:
        raise _lib.NSAKernelError(f"nsa_layer_ctx_bytes: {lib.nsa_last_error().decode()}")
    ctx = torch.empty(ctx_bytes, device=dev, dtype=torch.uint8)
    nbytes = lib.nsa_layer_workspace_bytes(ctypes.byref(desc), 0)
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    out = _mixed_out(desc, q)
    pos, w1, b1, w2, b2 = phi
    with torch.cuda.device(dev):
        check(lib.nsa_layer_fwd(ctypes.byref(desc), ptr(q), ptr(kv_slc[0]), ptr(kv_slc[1]), ptr(kv_cmp[0]), ptr(kv_cmp[1]), ptr(kv_win[0]),
                                ptr(kv_win[1]), ptr(gate_logits), ptr(pos), ptr(w1), ptr(b1), ptr(w2), ptr(b2), ptr(indices), ptr(out),
                                ptr(ctx), ctx_bytes, ptr(ws), nbytes, stream_ptr(dev)), "nsa_layer_fwd")
    return out, ctx


def layer_bwd(desc, q, kv_slc, kv_cmp, kv_win, phi, ctx, dout, shared_kv: bool):
    """-> dq, (dk, dv) per stream in the order selection, compression, window (time-major dK [B,G,T,dk]; with shared_kv
    the three are one pair of buffers), dlogits fp32, (dpos, dw1, db1, dw2, db2) fp32."""
    import ctypes
    dev = require_cuda(q, ctx, dout)
    B, H, G, T, dk, dv, U, l = desc.B, desc.H, desc.G, desc.T, desc.dk, desc.dv, desc.U, desc.l
    dq = torch.empty_like(q)
    mk = lambda: (torch.zeros(B, G, T, dk, device=dev, dtype=q.dtype), torch.zeros(B, G, T, dv, device=dev, dtype=q.dtype))
    g_slc = mk()
    g_cmp, g_win = (g_slc, g_slc) if shared_kv else (mk(), mk())
    f32 = lambda *s_: torch.empty(*s_, device=dev, dtype=torch.float32)
    dlogits = f32(B, T, 3 * H)
    dpos, dw1, db1, dw2, db2 = f32(l, l), f32(U, dk + l), f32(U), f32(dk, U), f32(dk)
    nbytes = lib.nsa_layer_workspace_bytes(ctypes.byref(desc), 1)
    ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
    pos, w1, b1, w2, b2 = phi
    with torch.cuda.device(dev):
        check(lib.nsa_layer_bwd(ctypes.byref(desc), ptr(q), ptr(kv_slc[0]), ptr(kv_slc[1]), ptr(kv_cmp[0]), ptr(kv_win[0]), ptr(kv_win[1]),
                                ptr(pos), ptr(w1), ptr(w2), ptr(ctx), ctx.numel(), ptr(dout), ptr(dq), ptr(g_slc[0]), ptr(g_slc[1]),
                                ptr(g_cmp[0]), ptr(g_cmp[1]), ptr(g_win[0]), ptr(g_win[1]), ptr(dlogits), ptr(dpos), ptr(dw1), ptr(db1),
                                ptr(dw2), ptr(db2), ptr(ws), nbytes, stream_ptr(dev)), "nsa_layer_bwd")
    return dq, g_slc, g_cmp, g_win, dlogits, (dpos, dw1, db1, dw2, db2)
