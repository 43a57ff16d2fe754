"""GPU parity tests: every CUDA entry point against the CPU oracle and the committed golden vectors.

All calls go through the C ABI (ctypes -> libnsa_b200.so).  Tolerances are those of the task:
1e-3 relative (max-abs over max-abs) for fp32 I/O, 2e-2 max-abs for bf16 I/O, indices bit-exact
outside the stated ambiguity set.
"""
import json
import math
import os

import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O
from tests.util import (INDEX_LOG, ambiguous_rows, check_layer_against_oracle, close, heads_mask, index_agreement, max_abs,
                        oracle_layer_with_grads, rel_err)

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
META = json.load(open(os.path.join(GOLD, "golden_meta.json")))
DEV = "cuda"


@pytest.fixture(scope="module")
def nsa_mod():
    import nsa
    import nsa.kernels
    return nsa


def _case(name):
    c = META["cases"][name]
    g = dict(np.load(os.path.join(GOLD, name + ".npz")))
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=c["seed"],
                        l_prime=c["l_prime"])
    return c, g, inp


def _cfg(nsa_mod, c, **kw):
    return nsa_mod.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"],
                             l_prime=c["l_prime"], n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"], **kw)


def _dev(t, dtype=torch.float32, grad=False):
    x = t.to(DEV, dtype).contiguous()
    return x.requires_grad_(True) if grad else x


# ---------------------------------------------------------------------------------------------
# branches: autograd wrappers vs golden vectors (reference outputs) and vs the oracle
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(META["cases"]))
@pytest.mark.parametrize("branch", ["win", "cmp", "slc"])
def test_branch_fp32_against_golden(nsa_mod, name, branch):
    from nsa.kernels import CompressionAttention, SelectionAttention, SlidingWindowAttention
    c, g, inp = _case(name)
    cfg = _cfg(nsa_mod, c)
    rows = torch.from_numpy(g["rows"])
    scale = c["dk"] ** -0.5
    q = _dev(inp["q"], grad=True)
    do = _dev(inp["do"])
    if branch == "cmp":
        k = _dev(torch.from_numpy(g["k_cmp"]), grad=True)
        v = _dev(torch.from_numpy(g["v_cmp"]), grad=True)
        o = CompressionAttention.apply(q, k, v, torch.from_numpy(g["block_ends"]).to(DEV), scale, cfg)
    else:
        k = _dev(inp["k"], grad=True)
        v = _dev(inp["v"], grad=True)
        if branch == "win":
            o = SlidingWindowAttention.apply(q, k, v, scale, c["w"], cfg)
        else:
            o = SelectionAttention.apply(q, k, v, torch.from_numpy(g["indices"]).long().to(DEV), scale, cfg)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    assert dk.shape == k.shape  # wrapper hands dK back in K's [B,G,dk,T] layout
    assert rel_err(o[:, :, rows], torch.from_numpy(g[branch + "_o"])) < 1e-3
    assert rel_err(dq[:, :, rows], torch.from_numpy(g[branch + "_dq"])) < 1e-3
    if branch == "cmp":
        assert rel_err(dk, torch.from_numpy(g["cmp_dk"])) < 1e-3
        assert rel_err(dv, torch.from_numpy(g["cmp_dv"])) < 1e-3
    else:
        assert rel_err(dk[..., rows], torch.from_numpy(g[branch + "_dk"])) < 1e-3
        assert rel_err(dv[:, :, rows], torch.from_numpy(g[branch + "_dv"])) < 1e-3


def _oracle_branch(branch, q, k, v, extra, c, scale):
    if branch == "win":
        return O.sliding_window_attention(q, k, v, c["w"], scale, return_stats=True)
    if branch == "cmp":
        return O.compression_attention(q, k, v, extra, scale, return_stats=True)
    return O.selection_attention(q, k, v, extra, c["l_prime"], scale, return_stats=True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("branch", ["win", "cmp", "slc"])
def test_branch_against_oracle_with_stats(nsa_mod, branch, dtype):
    """O, L, M and all gradients on a ragged shape (T not a multiple of anything, dk != dv)."""
    from nsa import ops
    B, H, G, T, dk, dv = 2, 6, 2, 333, 48, 80
    c = dict(w=70, l_prime=16)
    gen = torch.Generator().manual_seed(5)
    rnd = lambda *s: torch.randn(*s, generator=gen).to(dtype).float()
    q, do = rnd(B, H, T, dk), rnd(B, H, T, dv)
    scale = dk ** -0.5
    if branch == "cmp":
        NB = 40
        k, v = rnd(B, G, dk, NB), rnd(B, G, NB, dv)
        extra = (torch.arange(NB, dtype=torch.int32) * 8 + 15)
        extra[-3:] = 999999
    else:
        k, v = rnd(B, G, dk, T), rnd(B, G, T, dv)
        extra = None
        if branch == "slc":
            nblk = (T + 15) // 16
            extra = torch.randint(-1, nblk, (B, G, T, 6), generator=gen)
            extra[:, :, 5] = -1                      # an empty row
            extra[:, :, 40, :] = extra[:, :, 40, :1]  # a row of repeated ids
    qo, ko, vo = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_ref, M_ref, L_ref = _oracle_branch(branch, qo, ko, vo, extra, c, scale)
    g_ref = torch.autograd.grad(o_ref, (qo, ko, vo), do)
    qd, kd, vd, dod = _dev(q, dtype), _dev(k, dtype), _dev(v, dtype), _dev(do, dtype)
    if branch == "win":
        o, L, M = ops.sliding_fwd(qd, kd, vd, c["w"], scale)
        dq, dkey, dval = ops.sliding_bwd(qd, kd, vd, o, dod, L, M, c["w"], scale)
    elif branch == "cmp":
        be = extra.to(DEV)
        o, L, M = ops.cmp_attn_fwd(qd, kd, vd, be, scale)
        dq, dkey, dval = ops.cmp_attn_bwd(qd, kd, vd, be, o, dod, L, M, scale)
    else:
        idx = extra.to(DEV, torch.int32)
        o, L, M = ops.slc_fwd(qd, kd, vd, idx, c["l_prime"], scale)
        dq, dkey, dval = ops.slc_bwd(qd, kd, vd, idx, o, dod, L, M, c["l_prime"], scale)
    assert dkey.shape == (B, G, k.shape[-1], dk)  # time-major dK from the kernel
    finite = torch.isfinite(M_ref)
    assert torch.equal(torch.isfinite(M.cpu()), finite) and torch.equal(torch.isfinite(L.cpu()), finite)
    if dtype == torch.float32:
        assert rel_err(o, o_ref) < 1e-3
        assert max_abs(M.cpu()[finite], M_ref[finite]) < 1e-4 * (1 + M_ref[finite].abs().max().item())
        assert max_abs(L.cpu()[finite], L_ref[finite]) < 1e-4 * (1 + L_ref[finite].abs().max().item())
        assert rel_err(dq, g_ref[0]) < 1e-3
        assert rel_err(dkey.transpose(-1, -2), g_ref[1]) < 1e-3
        assert rel_err(dval, g_ref[2]) < 1e-3
    else:
        assert max_abs(o.float(), o_ref) < 2e-2
        # gradients of N(0,1) data are O(1..10): 2e-2 of the reference's largest magnitude
        assert max_abs(dq.float(), g_ref[0]) < 2e-2 * max(1.0, g_ref[0].abs().max().item())
        assert max_abs(dkey.float().transpose(-1, -2), g_ref[1]) < 2e-2 * max(1.0, g_ref[1].abs().max().item())
        assert max_abs(dval.float(), g_ref[2]) < 2e-2 * max(1.0, g_ref[2].abs().max().item())
    # rows that see nothing: O = 0, M = L = -inf
    assert (o.float().cpu()[~finite] == 0).all()


def test_backward_is_bit_reproducible(nsa_mod):
    from nsa import ops
    B, H, G, T, dk, dv = 1, 8, 2, 300, 64, 64
    gen = torch.Generator().manual_seed(9)
    q, k, v, do = (torch.randn(*s, generator=gen).to(DEV) for s in
                   [(B, H, T, dk), (B, G, dk, T), (B, G, T, dv), (B, H, T, dv)])
    idx = torch.randint(-1, (T + 31) // 32, (B, G, T, 8), generator=gen).to(DEV, torch.int32)
    o, L, M = ops.slc_fwd(q, k, v, idx, 32, 0.125)
    r1 = ops.slc_bwd(q, k, v, idx, o, do, L, M, 32, 0.125)
    r2 = ops.slc_bwd(q, k, v, idx, o, do, L, M, 32, 0.125)
    assert all(torch.equal(a, b) for a, b in zip(r1, r2))
    o, L, M = ops.sliding_fwd(q, k, v, 77, 0.125)
    r1 = ops.sliding_bwd(q, k, v, o, do, L, M, 77, 0.125)
    r2 = ops.sliding_bwd(q, k, v, o, do, L, M, 77, 0.125)
    assert all(torch.equal(a, b) for a, b in zip(r1, r2))


# ---------------------------------------------------------------------------------------------
# raw kernel-call contract through the launcher shims
# ---------------------------------------------------------------------------------------------

def _raw_sliding(nsa_mod, q, k, v, window, scale, kstrides):
    B, H, T, dk = q.shape
    G, dv = k.shape[1], v.shape[-1]
    out = torch.empty(B, H, T, dv, device=DEV, dtype=q.dtype)
    L = torch.empty(B, H, T, device=DEV, dtype=torch.float32)
    M = torch.empty_like(L)
    grid = lambda META: ((T + META["BLOCK_M"] - 1) // META["BLOCK_M"], B * H)
    nsa_mod._nsa_sliding_window_fwd_kernel[grid](
        q, k, v, out, scale, L, M, *q.stride(), *kstrides, *v.stride(), *out.stride(), *L.stride(), *M.stride(),
        Z=B, H=H, N_KV_GROUPS=G, N_CTX=T, WINDOW_SIZE=window, HEAD_DIM_QK=dk, HEAD_DIM_V=dv, BLOCK_M=32, BLOCK_N=32)
    return out, L, M


def test_raw_contract_sliding_and_stride_honouring(nsa_mod):
    """Shapes/seed of the reference's tests/test_accuracy.py:26-44 and the wrong-stride contract test
    (tests/test_kernel_contracts.py:68-90): un-swapped K strides must change the answer by > 0.1."""
    B, H, G, T, d, w = 2, 8, 2, 64, 32, 16
    torch.manual_seed(42)
    q = torch.randn(B, H, T, d, device=DEV) * 0.02
    k = torch.randn(B, G, d, T, device=DEV) * 0.02
    v = torch.randn(B, G, T, d, device=DEV) * 0.02
    scale = 1.0 / math.sqrt(d)
    good = [k.stride(0), k.stride(1), k.stride(3), k.stride(2)]
    out, L, M = _raw_sliding(nsa_mod, q, k, v, w, scale, good)
    ref = O.sliding_window_attention(q.cpu(), k.cpu(), v.cpu(), w, scale)
    assert rel_err(out, ref) < 1e-3
    # N(0,1) inputs as in the reference's contract test: un-swapped strides must not fault and must differ
    q1, k1, v1 = (torch.randn_like(t) for t in (q, k, v))
    good1, _, _ = _raw_sliding(nsa_mod, q1, k1, v1, w, scale, good)
    bad1, _, _ = _raw_sliding(nsa_mod, q1, k1, v1, w, scale, list(k1.stride()))
    assert torch.isfinite(bad1).all()
    assert ((good1 - bad1).abs() / (good1.abs() + 1e-8)).max() > 0.1 and rel_err(bad1, good1) > 0.1
    # backward through the raw contract: dK is [B,G,T,dk], zero-initialised by the caller, added into
    do = torch.randn_like(out)
    dq = torch.zeros_like(q)
    dk_ = torch.zeros(B, G, T, d, device=DEV)
    dv_ = torch.zeros_like(v)
    grid = lambda META: ((T + META["BLOCK_M"] - 1) // META["BLOCK_M"], B * H)
    args = (q, k, v, out, do, scale, L, M, *q.stride(), *good, *v.stride(), *out.stride(), *L.stride(), *M.stride(),
            dq, dk_, dv_, *dq.stride(), *dk_.stride(), *dv_.stride())
    kw = dict(Z=B, H=H, N_KV_GROUPS=G, N_CTX=T, WINDOW_SIZE=w, HEAD_DIM_QK=d, HEAD_DIM_V=d, BLOCK_M=32, BLOCK_N=32)
    nsa_mod._nsa_sliding_window_bwd_kernel[grid](*args, **kw)
    qc, kc, vc = (t.cpu().clone().requires_grad_(True) for t in (q, k, v))
    g = torch.autograd.grad(O.sliding_window_attention(qc, kc, vc, w, scale), (qc, kc, vc), do.cpu())
    assert rel_err(dq, g[0]) < 1e-3 and rel_err(dk_.transpose(-1, -2), g[1]) < 1e-3 and rel_err(dv_, g[2]) < 1e-3
    once = dk_.clone()
    nsa_mod._nsa_sliding_window_bwd_kernel[grid](*args, **kw)      # second launch adds into dK/dV, overwrites dQ
    assert rel_err(dk_, 2 * once) < 1e-5 and rel_err(dq, g[0]) < 1e-3
    # statistics matter: zeroed L/M must change the gradients (tests/test_kernel_contracts.py:253-289)
    dq2 = torch.zeros_like(q)
    args2 = list(args)
    args2[6], args2[7] = torch.zeros_like(L), torch.zeros_like(M)
    args2[-15] = dq2
    nsa_mod._nsa_sliding_window_bwd_kernel[grid](*args2, **kw)
    assert (dq2 - dq).abs().max() > 1e-4 * dq.abs().max()


def test_raw_contract_compression_and_selection(nsa_mod):
    """Shapes of the reference's tests/test_branches.py:232-252 (N_BLOCKS=8, block_ends=arange(7,64,8))
    and :459-492 (l'=32, n=4, ids [0, local-1, local, local+1] deduplicated, -1 padded)."""
    B, H, G, T, d = 2, 8, 2, 64, 32
    torch.manual_seed(42)
    q = torch.randn(B, H, T, d, device=DEV) * 0.02
    scale = 1.0 / math.sqrt(d)
    out = torch.empty(B, H, T, d, device=DEV)
    L = torch.empty(B, H, T, device=DEV)
    M = torch.empty_like(L)
    grid = lambda META: ((T + META["BLOCK_M"] - 1) // META["BLOCK_M"], B * H)
    NB = 8
    kc = torch.randn(B, G, d, NB, device=DEV) * 0.02
    vc = torch.randn(B, G, NB, d, device=DEV) * 0.02
    be = torch.arange(7, 64, 8, device=DEV, dtype=torch.int32)
    nsa_mod._nsa_compression_fwd_kernel[grid](
        q, kc, vc, be, out, scale, L, M, *q.stride(), kc.stride(0), kc.stride(1), kc.stride(3), kc.stride(2),
        *vc.stride(), *out.stride(), *L.stride(), *M.stride(),
        Z=B, H=H, N_KV_GROUPS=G, N_CTX_Q=T, N_BLOCKS=NB, HEAD_DIM_QK=d, HEAD_DIM_V=d, BLOCK_M=32, BLOCK_N=32)
    ref = O.compression_attention(q.cpu(), kc.cpu(), vc.cpu(), be.cpu(), scale)
    assert rel_err(out, ref) < 1e-3
    assert (out[:, :, :7] == 0).all()                # nothing visible before the first block end
    lp, n = 32, 4
    k = torch.randn(B, G, d, T, device=DEV) * 0.02
    v = torch.randn(B, G, T, d, device=DEV) * 0.02
    idx = torch.full((B, G, T, n), -1, dtype=torch.int32)
    for t in range(T):
        loc = t // lp
        ids = []
        for b_ in [0, loc - 1, loc, loc + 1]:
            if 0 <= b_ < T // lp and b_ not in ids:
                ids.append(b_)
        idx[:, :, t, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
    idx = idx.to(DEV)
    nsa_mod._nsa_sparse_selection_fwd_kernel[grid](
        q, k, v, idx, out, scale, L, M, *q.stride(), k.stride(0), k.stride(1), k.stride(3), k.stride(2), *v.stride(),
        *out.stride(), *idx.stride(), *L.stride(), *M.stride(),
        Z=B, H=H, N_KV_GROUPS=G, N_CTX_Q=T, N_CTX_KV=T, N_BLOCKS=n, BLOCK_SIZE_SELECTION=lp, IS_CAUSAL=True,
        HEAD_DIM_QK=d, HEAD_DIM_V=d, BLOCK_M=32, BLOCK_N=32)
    ref = O.selection_attention(q.cpu(), k.cpu(), v.cpu(), idx.cpu().long(), lp, scale)
    assert rel_err(out, ref) < 1e-3


# ---------------------------------------------------------------------------------------------
# phi, scoring + top-n, gate/mix
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", sorted(META["cases"]))
def test_phi_compress_against_golden_and_oracle_grads(nsa_mod, name):
    from nsa.kernels import _PhiCompress
    c, g, inp = _case(name)
    phi = inp["phi"]
    params = [_dev(p, grad=True) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2)]
    keys = _dev(inp["k"].transpose(-1, -2), grad=True)
    vals = _dev(inp["v"], grad=True)
    k_cmp, v_cmp = _PhiCompress.apply(keys, vals, *params, c["l"], c["d"])
    assert rel_err(k_cmp, torch.from_numpy(g["k_cmp"])) < 1e-4
    assert rel_err(v_cmp, torch.from_numpy(g["v_cmp"])) < 1e-4
    gen = torch.Generator().manual_seed(1)
    gk, gv = torch.randn(k_cmp.shape, generator=gen), torch.randn(v_cmp.shape, generator=gen)
    grads = torch.autograd.grad((k_cmp, v_cmp), [keys, vals] + params, (gk.to(DEV), gv.to(DEV)))
    ko = inp["k"].transpose(-1, -2).clone().requires_grad_(True)
    vo = inp["v"].clone().requires_grad_(True)
    po = [p.clone().requires_grad_(True) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2)]
    kc_o, vc_o, _, _ = O.compress_tokens(ko, vo, O.PhiParams(*po), c["l"], c["d"])
    ref = torch.autograd.grad((kc_o, vc_o), [ko, vo] + po, (gk, gv))
    for a, b in zip(grads, ref):
        assert rel_err(a, b) < 1e-3


@pytest.mark.parametrize("name", sorted(META["cases"]))
def test_score_topn_indices_bit_exact(nsa_mod, name):
    from nsa import ops
    c, g, inp = _case(name)
    scale = c["dk"] ** -0.5
    k_cmp = torch.from_numpy(g["k_cmp"])
    be = torch.from_numpy(g["block_ends"])
    idx = ops.score_topn(_dev(inp["q"]), _dev(k_cmp), be.to(DEV), c["l"], c["d"], c["l_prime"], c["n"], 3, scale).cpu()
    gold = torch.from_numpy(g["indices"])
    p = O.compression_probabilities(inp["q"], k_cmp, be, scale)
    sel = O.selection_scores_from_compression(p, c["l"], c["d"], c["l_prime"])
    agg = sel.view(c["B"], c["G"], c["H"] // c["G"], c["T"], -1).sum(2)
    amb = ambiguous_rows(agg, c["n"]) | (torch.from_numpy(g["indices_fp64"]) != gold).any(-1)
    mism = (idx != gold).any(-1)
    INDEX_LOG.append((f"score_topn fp32 {name}", mism.numel(), int(amb.sum()), int(mism.sum()), int((mism & ~amb).sum())))
    assert not (mism & ~amb).any(), f"{int((mism & ~amb).sum())} unambiguous rows differ"
    assert amb.float().mean() < 0.05
    # Eq. 9 / Eq. 10-11 on materialised tensors through the mirrored host functions
    cfg = _cfg(nsa_mod, c)
    from nsa.kernels import derive_selection_from_compression_per_timestep, select_top_k_blocks_per_query_with_gqa
    sel_gpu = derive_selection_from_compression_per_timestep(p.to(DEV), cfg)
    assert torch.equal(sel_gpu.cpu(), sel)                      # same adds in the same order
    idx2 = select_top_k_blocks_per_query_with_gqa(sel.to(DEV), cfg)
    assert idx2.dtype == torch.int64 and torch.equal(idx2.cpu(), gold.long())
    probs = ops.cmp_probs(_dev(inp["q"]), _dev(k_cmp), be.to(DEV), scale)
    assert rel_err(probs, p) < 1e-4


def test_top_n_known_answers_on_gpu(nsa_mod):
    """Literals of the reference's tests/test_whitepaper_spec.py:39-78 through the mirrored function."""
    from nsa.kernels import select_top_k_blocks_per_query_with_gqa as sel_fn
    s = torch.arange(5, dtype=torch.float32, device=DEV).view(1, 1, 1, 5).repeat(1, 2, 3, 1)
    cfg = nsa_mod.NSAConfig(l_prime=2, d=1, l=1, n=3, n_heads=2, n_kv_groups=1, include_fixed_in_selection=False)
    idx = sel_fn(s, cfg)
    assert all(idx[0, 0, t].tolist() == [4, 3, 2] for t in range(3))
    cfg = nsa_mod.NSAConfig(l_prime=2, d=1, l=1, n=3, n_heads=2, n_kv_groups=1, include_fixed_in_selection=True, n_fixed=3)
    idx = sel_fn(s, cfg)
    assert idx[0, 0, 0].tolist() == [0, 4, 3] and idx[0, 0, 2].tolist() == [0, 1, 4]
    cfg = nsa_mod.NSAConfig(l_prime=2, d=1, l=1, n=4, n_heads=2, n_kv_groups=1)
    idx = sel_fn(torch.zeros(1, 2, 2, 2, device=DEV), cfg)
    assert idx.shape[-1] == 4 and (idx[0, 0, 0, 2:] == -1).all()
    cfg = nsa_mod.NSAConfig(l_prime=2, d=1, l=1, n=4, n_heads=1, n_kv_groups=1, include_fixed_in_selection=False)
    t = torch.tensor([.5, .5, .1, .5, 0., 0.], device=DEV).view(1, 1, 1, 6)
    assert sel_fn(t, cfg)[0, 0, 0].tolist() == [0, 1, 3, 2]   # ties go to the lower block id


@pytest.mark.parametrize("mode", ["sigmoid", "softmax"])
@pytest.mark.parametrize("dtype,dv", [(torch.float32, 80), (torch.bfloat16, 80), (torch.bfloat16, 128)])
def test_gate_mix(nsa_mod, mode, dtype, dv):
    from nsa.kernels import _GateMix
    B, H, T = 2, 6, 37
    gen = torch.Generator().manual_seed(3)
    rnd = lambda *s: torch.randn(*s, generator=gen).to(dtype).float()
    lg, oc, os_, ow, do = rnd(B, T, 3 * H), rnd(B, H, T, dv), rnd(B, H, T, dv), rnd(B, H, T, dv), rnd(B, H, T, dv)
    ts = [t.clone().requires_grad_(True) for t in (lg, oc, os_, ow)]
    gt = ts[0].view(B, T, H, 3).permute(0, 2, 1, 3)
    gt = torch.softmax(gt, -1) if mode == "softmax" else torch.sigmoid(gt)
    ref = O.mix_branches(gt, *ts[1:])
    gref = torch.autograd.grad(ref, ts, do)
    td = [_dev(lg, torch.float32, True)] + [_dev(t, dtype, True) for t in (oc, os_, ow)]
    out, gates = _GateMix.apply(*td, mode)
    gg = torch.autograd.grad(out, td, _dev(do, dtype))
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert max_abs(gates, gt) < 1e-5
    assert max_abs(out.float(), ref) < tol * max(1.0, ref.abs().max().item())
    for a, b in zip(gg, gref):
        assert max_abs(a.float(), b) < tol * max(1.0, b.abs().max().item())


# ---------------------------------------------------------------------------------------------
# the whole layer (BASELINE config 1) and the module
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name,gate_mode", [("cfg1", "sigmoid"), ("small", "softmax")])
def test_layer_fp32_forward_backward(nsa_mod, name, gate_mode):
    c, g, inp = _case(name)
    info, mism, r = check_layer_against_oracle(f"layer fp32 {name}", nsa_mod, c, inp, torch.float32, gate_mode=gate_mode)
    assert not mism.any(), "fp32 I/O: selected block ids must equal the oracle's on these fixtures"


def test_layer_bf16_forward_backward(nsa_mod):
    c, g, inp = _case("cfg1")
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=c["seed"],
                        l_prime=c["l_prime"], dtype=torch.bfloat16)
    check_layer_against_oracle("layer bf16 cfg1", nsa_mod, c, inp, torch.bfloat16)


@pytest.mark.timeout(1200)
@pytest.mark.parametrize("B,T", [(1, 2048), (1, 4096), (2, 2048)])
def test_layer_bf16_at_the_benchmarked_head_configuration(nsa_mod, B, T):
    """H=64 query heads in G=4 groups, dk=192, dv=128, keys with per-block offsets (BASELINE configs 3-5), bf16, through the
    single autograd node the benchmark uses (dQ of the three branches summed in the selection backward, row sums handed
    over by the gate/mix backward): outputs and all twelve gradients against the oracle."""
    from nsa._lib import lib
    c = dict(B=B, H=64, G=4, T=T, dk=192, dv=128, d_model=512, l=32, d=16, l_prime=64, n=16, w=512)
    inp = O.make_inputs(c["B"], c["H"], c["G"], T, c["dk"], c["dv"], c["d_model"], c["l"], seed=23, block_offset_std=0.5,
                        l_prime=c["l_prime"], dtype=torch.bfloat16)
    O.LOW_MEMORY = True
    try:
        check_layer_against_oracle(f"layer bf16 B={B} H=64 G=4 dk=192 dv=128 T={T}", nsa_mod, c, inp, torch.bfloat16)
    finally:
        O.LOW_MEMORY = False
    assert lib.nsa_device_timeouts(0) == 0


def test_module_forward_matches_reference_module(nsa_mod):
    """NSAAttention with the reference's parameter names against the golden whole-module run."""
    c, g, inp = _case("small")
    cfg = _cfg(nsa_mod, c)
    model = nsa_mod.NSAAttention(cfg).to(DEV)
    phi, gp = inp["phi"], inp["gate"]
    proj = O.draw_projection_weights(c["seed"] + 11, c["d_model"], c["H"], c["G"], c["dk"], c["dv"])
    sd = {f"{n}.weight": w for n, w in proj.items()}
    sd.update({"pos_embed.weight": phi.pos_embed, "compress_mlp.0.weight": phi.w1, "compress_mlp.0.bias": phi.b1,
               "compress_mlp.2.weight": phi.w2, "compress_mlp.2.bias": phi.b2, "gate_mlp.0.weight": gp.w1,
               "gate_mlp.0.bias": gp.b1, "gate_mlp.2.weight": gp.w2, "gate_mlp.2.bias": gp.b2})
    model.load_state_dict(sd, strict=True)
    gen = torch.Generator().manual_seed(c["seed"] + 7)
    hidden = (torch.randn(c["B"], c["T"], c["d_model"], generator=gen) * 0.5).to(DEV)
    for training in (False, True):
        model.train(training)
        y, info = model(hidden, output_attentions=True)
        rows = g["rows"]
        assert info["gates"].shape == (c["B"], c["T"], c["H"], 3)
        assert info["selected_indices"].shape == (c["B"], c["G"], c["T"], c["n"])
        assert rel_err(info["compression_scores"][:, :, rows], torch.from_numpy(g["mod_p_cmp"])) < 1e-3
        assert rel_err(info["selection_scores"][:, :, rows], torch.from_numpy(g["mod_sel"])) < 1e-3
        assert rel_err(info["gates"][:, rows], torch.from_numpy(g["mod_gates"])) < 1e-3
        # the module's output row t mixes all heads of position t: compare the positions whose block ids agree in
        # every group (always, whether or not other rows differ), and require agreement outside near-ties
        gold_idx = torch.from_numpy(g["mod_indices"]).long()
        same = (info["selected_indices"].cpu() == gold_idx).all(-1).all(1)            # [B,T]
        INDEX_LOG.append((f"module small training={training}", same.numel(), -1, int((~same).sum()), -1))
        assert same.float().mean() > 0.98
        got, want = y[:, rows].detach().cpu(), torch.from_numpy(g["mod_y"])
        keep = same[:, rows]
        assert keep.any()
        assert ((got - want).abs()[keep].max() / want.abs().max()).item() < 1e-3
    y.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    k_cmp, v_cmp, be, nb = model.compress_tokens(torch.randn(1, c["G"], 24 * 4, c["dk"], device=DEV),
                                                 torch.randn(1, c["G"], 24 * 4, c["dv"], device=DEV))
    assert nb == (96 - c["l"]) // c["d"] + 1 and int(be[1]) == c["d"] + c["l"] - 1


def test_cpu_tensors_are_rejected(nsa_mod):
    from nsa import ops
    with pytest.raises(RuntimeError):
        ops.sliding_fwd(torch.zeros(1, 2, 4, 8), torch.zeros(1, 1, 8, 4), torch.zeros(1, 1, 4, 8), 2, 1.0)


@pytest.mark.parametrize("T,dk,dv,H,G,n,w,include_fixed,gate_mode", [
    (777, 96, 80, 6, 3, 5, 100, True, "sigmoid"),       # ragged T (padded-block n_sel), head dims off the tile sizes
    (333, 64, 64, 4, 2, 3, 50, False, "softmax"),       # no forced blocks, softmax gates
    (40, 32, 48, 2, 1, 16, 512, True, "sigmoid"),       # barely one compression block, window and n beyond T
    (20, 32, 32, 4, 2, 4, 8, True, "sigmoid"),          # shorter than one compression block: only the padding block exists
])
def test_layer_fp32_odd_shapes(nsa_mod, T, dk, dv, H, G, n, w, include_fixed, gate_mode):
    """The generic kernels on shapes off every tile size, against the oracle layer (fp32)."""
    c = dict(B=2, H=H, G=G, T=T, dk=dk, dv=dv, d_model=48, l=32, d=16, l_prime=64, n=n, w=w, seed=41)
    inp = O.make_inputs(c["B"], H, G, T, dk, dv, c["d_model"], c["l"], seed=c["seed"], block_offset_std=0.5)
    check_layer_against_oracle(f"layer fp32 odd T={T} dk={dk} dv={dv}", nsa_mod, c, inp, torch.float32, gate_mode=gate_mode,
                               include_fixed=include_fixed)


def test_module_dropout_and_state_dict_round_trip(nsa_mod):
    """dropout_p > 0 (the reference applies nn.Dropout to the projected output, nsa/kernels.py:2477): training-mode calls
    differ from one another and from eval, eval is deterministic and equals the dropout-free module; the token-major
    path into o_proj gives gradients for every parameter."""
    c = dict(d_model=64, dk=64, dv=64, H=4, G=2, T=256)
    mk = lambda p: nsa_mod.NSAAttention(nsa_mod.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], n_heads=c["H"],
                                                         n_kv_groups=c["G"], l=32, d=16, l_prime=64, n=4, w=64, dropout_p=p)).to(DEV)
    torch.manual_seed(3)
    plain, drop = mk(0.0), mk(0.5)
    drop.load_state_dict(plain.state_dict(), strict=True)
    x = torch.randn(2, c["T"], c["d_model"], device=DEV)
    plain.eval(); drop.eval()
    y0, _ = plain(x)
    y1, _ = drop(x)
    y2, _ = drop(x)
    assert torch.equal(y1, y2) and torch.equal(y0, y1)
    drop.train()
    a, _ = drop(x)
    b, _ = drop(x)
    assert not torch.equal(a, b) and (a == 0).float().mean() > 0.3
    a.sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in drop.parameters())
