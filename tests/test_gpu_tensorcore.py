"""Tensor-core (tcgen05) kernels against the CPU oracle at small sizes and against the stride-generic
CUDA kernels at sizes the oracle cannot reach.  bf16 I/O: 2e-2 max-abs on outputs."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.util import max_abs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _inputs(B, H, G, T, dk, dv, Tk=None, seed=0):
    gen = torch.Generator().manual_seed(seed)
    Tk = T if Tk is None else Tk
    rnd = lambda *s: torch.randn(*s, generator=gen).bfloat16()
    return rnd(B, H, T, dk), rnd(B, G, dk, Tk), rnd(B, G, Tk, dv), rnd(B, H, T, dv)


def _no_timeouts():
    from nsa._lib import lib
    assert lib.nsa_device_timeouts(1) == 0, "a tensor-core CTA gave up on a barrier wait"


def _check_stats(L, M, L_ref, M_ref):
    fin = torch.isfinite(M_ref)
    assert torch.equal(torch.isfinite(M.cpu()), fin) and torch.equal(torch.isfinite(L.cpu()), fin)
    lse, lse_ref = (M + L).cpu()[fin], (M_ref + L_ref)[fin]
    assert (lse - lse_ref).abs().max() < 2e-2
    assert (M.cpu()[fin] - M_ref[fin]).abs().max() < 2e-2 * (1 + M_ref[fin].abs().max())


@pytest.mark.parametrize("dk,dv,H,G,T,w", [(64, 64, 4, 2, 512, 200), (192, 128, 4, 1, 1024, 512),
                                           (128, 128, 2, 1, 384, 128), (192, 128, 2, 1, 256, 1000)])
def test_sliding_forward_tensorcore_vs_oracle(dk, dv, H, G, T, w):
    from nsa import ops
    q, k, v, _ = _inputs(2, H, G, T, dk, dv, seed=1)
    scale = dk ** -0.5
    o, L, M = ops.sliding_fwd(q.to(DEV), k.to(DEV), v.to(DEV), w, scale)
    torch.cuda.synchronize()
    _no_timeouts()
    o_ref, M_ref, L_ref = O.sliding_window_attention(q.float(), k.float(), v.float(), w, scale, return_stats=True)
    assert max_abs(o.float(), o_ref) < 2e-2
    _check_stats(L, M, L_ref, M_ref)


@pytest.mark.parametrize("dk,dv,H,G,T", [(64, 64, 4, 2, 2048), (192, 128, 2, 1, 4096 + 2048)])
def test_compression_forward_tensorcore_vs_oracle(dk, dv, H, G, T):
    from nsa import ops
    l, d = 32, 16
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    q, kc, vc, _ = _inputs(1, H, G, T, dk, dv, Tk=nbp, seed=2)
    kc[..., nb:] = 0
    vc[:, :, nb:] = 0
    be = torch.full((nbp,), 999999, dtype=torch.int32)
    be[:nb] = torch.arange(nb, dtype=torch.int32) * d + l - 1
    scale = dk ** -0.5
    o, L, M = ops.cmp_attn_fwd(q.to(DEV), kc.to(DEV), vc.to(DEV), be.to(DEV), scale, blocks=(l, d, nb))
    torch.cuda.synchronize()
    _no_timeouts()
    o_ref, M_ref, L_ref = O.compression_attention(q.float(), kc.float(), vc.float(), be, scale, return_stats=True)
    assert max_abs(o.float(), o_ref) < 2e-2
    assert (o[:, :, : l - 1] == 0).all()
    _check_stats(L, M, L_ref, M_ref)


def test_forward_tensorcore_vs_generic_at_scale():
    """Paper head dims at T=8192 (16 heads of one group): tensor-core vs stride-generic kernels."""
    from nsa import ops
    B, H, G, T, dk, dv = 1, 16, 1, 8192, 192, 128
    q, k, v, _ = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=3))
    scale = dk ** -0.5
    o, L, M = ops.sliding_fwd(q, k, v, 512, scale)
    og, Lg, Mg = ops.sliding_fwd(q, k, v, 512, scale, generic=True)
    assert max_abs(o.float(), og.float()) < 2e-2 and max_abs(M + L, Mg + Lg) < 2e-2
    l, d = 32, 16
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    kc = torch.zeros(B, G, dk, nbp, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros(B, G, nbp, dv, device=DEV, dtype=torch.bfloat16)
    kc[..., :nb] = torch.randn(B, G, dk, nb, device=DEV).bfloat16()
    vc[:, :, :nb] = torch.randn(B, G, nb, dv, device=DEV).bfloat16()
    be = torch.full((nbp,), 999999, dtype=torch.int32, device=DEV)
    be[:nb] = torch.arange(nb, dtype=torch.int32, device=DEV) * d + l - 1
    o, L, M = ops.cmp_attn_fwd(q, kc, vc, be, scale, blocks=(l, d, nb))
    og, Lg, Mg = ops.cmp_attn_fwd(q, kc, vc, be, scale, generic=True)
    torch.cuda.synchronize()
    _no_timeouts()
    assert max_abs(o.float(), og.float()) < 2e-2
    fin = torch.isfinite(Mg)
    assert torch.equal(torch.isfinite(M), fin) and max_abs((M + L)[fin], (Mg + Lg)[fin]) < 2e-2


def _grad_close(a, ref, what):
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    err = max_abs(a.float(), ref)
    assert err < tol, f"{what}: max-abs {err:.4g} > {tol:.4g}"


@pytest.mark.parametrize("dk,dv,H,G,T,w", [(64, 64, 4, 2, 512, 200), (192, 128, 4, 1, 1024, 512),
                                           (128, 128, 2, 1, 384, 128), (192, 128, 2, 1, 256, 1000)])
def test_sliding_backward_tensorcore_vs_oracle(dk, dv, H, G, T, w):
    from nsa import ops
    q, k, v, do = _inputs(2, H, G, T, dk, dv, seed=4)
    scale = dk ** -0.5
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    o, L, M = ops.sliding_fwd(qd, kd, vd, w, scale)
    dq, dkey, dval = ops.sliding_bwd(qd, kd, vd, o, dod, L, M, w, scale)
    dq2, dkey2, dval2 = ops.sliding_bwd(qd, kd, vd, o, dod, L, M, w, scale)
    # small-scratch variant: the dQ kernel recomputes S and dP instead of taking dS^T from the dK/dV kernel
    dq3, dkey3, dval3 = ops.sliding_bwd(qd, kd, vd, o, dod, L, M, w, scale, recompute=True)
    torch.cuda.synchronize()
    _no_timeouts()
    assert torch.equal(dq, dq2) and torch.equal(dkey, dkey2) and torch.equal(dval, dval2)   # fixed summation order
    assert torch.equal(dkey, dkey3) and torch.equal(dval, dval3)
    qo, ko, vo = (t.float().requires_grad_(True) for t in (q, k, v))
    g = torch.autograd.grad(O.sliding_window_attention(qo, ko, vo, w, scale), (qo, ko, vo), do.float())
    _grad_close(dq, g[0], "dq")
    _grad_close(dq3, g[0], "dq (recomputed S, dP)")
    _grad_close(dkey.transpose(-1, -2), g[1], "dk")
    _grad_close(dval, g[2], "dv")


@pytest.mark.parametrize("dk,dv,H,G,T", [(64, 64, 4, 2, 2048), (192, 128, 2, 1, 4096 + 2048)])
def test_compression_backward_tensorcore_vs_oracle(dk, dv, H, G, T):
    from nsa import ops
    l, d = 32, 16
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    q, kc, vc, do = _inputs(1, H, G, T, dk, dv, Tk=nbp, seed=5)
    kc[..., nb:] = 0
    vc[:, :, nb:] = 0
    be = torch.full((nbp,), 999999, dtype=torch.int32)
    be[:nb] = torch.arange(nb, dtype=torch.int32) * d + l - 1
    scale = dk ** -0.5
    qd, kd, vd, dod, bed = (t.to(DEV) for t in (q, kc, vc, do, be))
    o, L, M = ops.cmp_attn_fwd(qd, kd, vd, bed, scale, blocks=(l, d, nb))
    dq, dkc, dvc = ops.cmp_attn_bwd(qd, kd, vd, bed, o, dod, L, M, scale, blocks=(l, d, nb))
    dq3, dkc3, dvc3 = ops.cmp_attn_bwd(qd, kd, vd, bed, o, dod, L, M, scale, blocks=(l, d, nb), recompute=True)
    torch.cuda.synchronize()
    _no_timeouts()
    assert torch.equal(dkc, dkc3) and torch.equal(dvc, dvc3)
    qo, ko, vo = (t.float().requires_grad_(True) for t in (q, kc, vc))
    g = torch.autograd.grad(O.compression_attention(qo, ko, vo, be, scale), (qo, ko, vo), do.float())
    _grad_close(dq, g[0], "dq")
    _grad_close(dq3, g[0], "dq (recomputed S, dP)")
    _grad_close(dkc.transpose(-1, -2), g[1], "dk_cmp")
    _grad_close(dvc, g[2], "dv_cmp")
    assert (dkc[:, :, nb:] == 0).all() and (dvc[:, :, nb:] == 0).all()


def test_backward_tensorcore_vs_generic_at_scale():
    from nsa import ops
    B, H, G, T, dk, dv = 1, 16, 1, 4096, 192, 128
    q, k, v, do = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=6))
    scale = dk ** -0.5
    o, L, M = ops.sliding_fwd(q, k, v, 512, scale)
    tc = ops.sliding_bwd(q, k, v, o, do, L, M, 512, scale)
    gen = ops.sliding_bwd(q, k, v, o, do, L, M, 512, scale, generic=True)
    for a, b_, n in zip(tc, gen, ("dq", "dk", "dv")):
        _grad_close(a, b_.float().cpu(), "sliding " + n)
    l, d = 32, 16
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    kc = torch.zeros(B, G, dk, nbp, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros(B, G, nbp, dv, device=DEV, dtype=torch.bfloat16)
    kc[..., :nb] = torch.randn(B, G, dk, nb, device=DEV).bfloat16()
    vc[:, :, :nb] = torch.randn(B, G, nb, dv, device=DEV).bfloat16()
    be = torch.full((nbp,), 999999, dtype=torch.int32, device=DEV)
    be[:nb] = torch.arange(nb, dtype=torch.int32, device=DEV) * d + l - 1
    o, L, M = ops.cmp_attn_fwd(q, kc, vc, be, scale, blocks=(l, d, nb))
    tc = ops.cmp_attn_bwd(q, kc, vc, be, o, do, L, M, scale, blocks=(l, d, nb))
    gen = ops.cmp_attn_bwd(q, kc, vc, be, o, do, L, M, scale, generic=True)
    torch.cuda.synchronize()
    _no_timeouts()
    for a, b_, n in zip(tc, gen, ("dq", "dk", "dv")):
        _grad_close(a, b_.float().cpu(), "compression " + n)


def _random_indices(B, G, T, n, lp, gen, with_holes=True):
    """Per-query block ids like the layer produces (block 0, the local blocks, random earlier blocks),
    plus -1 slots, repeated ids and ids of future blocks when with_holes."""
    nblk = (T + lp - 1) // lp
    idx = torch.randint(0, nblk, (B, G, T, n), generator=gen)
    t = torch.arange(T)
    idx = torch.minimum(idx, (t // lp).view(1, 1, T, 1).expand_as(idx) + (1 if with_holes else 0))
    idx[..., 0] = 0
    idx[..., 1] = (t // lp).view(1, 1, T)
    if with_holes:
        idx[..., -1] = -1
        idx[:, :, 7::13, 2] = idx[:, :, 7::13, 3]      # repeated ids
        idx[:, :, 5] = -1                               # an empty row
    return idx.to(torch.int32)


@pytest.mark.parametrize("dk,dv,H,G,T,n", [(64, 64, 8, 2, 512, 6), (192, 128, 16, 1, 1024, 16), (128, 128, 32, 1, 256, 4)])
def test_selection_forward_tensorcore_vs_oracle(dk, dv, H, G, T, n):
    from nsa import ops
    gen = torch.Generator().manual_seed(7)
    q, k, v, _ = _inputs(2, H, G, T, dk, dv, seed=7)
    idx = _random_indices(2, G, T, n, 64, gen)
    scale = dk ** -0.5
    o, L, M = ops.slc_fwd(q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV), 64, scale)
    torch.cuda.synchronize()
    _no_timeouts()
    o_ref, M_ref, L_ref = O.selection_attention(q.float(), k.float(), v.float(), idx.long(), 64, scale, return_stats=True)
    assert max_abs(o.float(), o_ref) < 2e-2
    _check_stats(L, M, L_ref, M_ref)
    assert (o[:, :, 5] == 0).all()


def test_selection_forward_tensorcore_vs_generic_at_scale():
    from nsa import ops
    B, H, G, T, dk, dv, n = 1, 32, 2, 8192, 192, 128, 16
    gen = torch.Generator().manual_seed(8)
    q, k, v, _ = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=8))
    idx = _random_indices(B, G, T, n, 64, gen, with_holes=False).to(DEV)
    scale = dk ** -0.5
    o, L, M = ops.slc_fwd(q, k, v, idx, 64, scale)
    og, Lg, Mg = ops.slc_fwd(q, k, v, idx, 64, scale, generic=True)
    torch.cuda.synchronize()
    _no_timeouts()
    assert max_abs(o.float(), og.float()) < 2e-2 and max_abs(M + L, Mg + Lg) < 2e-2


@pytest.mark.parametrize("dk,dv,H,G,T,n", [(64, 64, 8, 2, 512, 6), (192, 128, 16, 1, 1024, 16), (128, 128, 32, 1, 256, 4)])
def test_selection_backward_tensorcore_vs_oracle(dk, dv, H, G, T, n):
    from nsa import ops
    gen = torch.Generator().manual_seed(9)
    q, k, v, do = _inputs(2, H, G, T, dk, dv, seed=9)
    idx = _random_indices(2, G, T, n, 64, gen)
    scale = dk ** -0.5
    qd, kd, vd, dod, idd = (t.to(DEV) for t in (q, k, v, do, idx))
    o, L, M = ops.slc_fwd(qd, kd, vd, idd, 64, scale)
    r1 = ops.slc_bwd(qd, kd, vd, idd, o, dod, L, M, 64, scale)
    r2 = ops.slc_bwd(qd, kd, vd, idd, o, dod, L, M, 64, scale)
    torch.cuda.synchronize()
    _no_timeouts()
    assert all(torch.equal(a, b_) for a, b_ in zip(r1, r2))          # fixed summation order
    qo, ko, vo = (t.float().requires_grad_(True) for t in (q, k, v))
    g = torch.autograd.grad(O.selection_attention(qo, ko, vo, idx.long(), 64, scale), (qo, ko, vo), do.float())
    _grad_close(r1[0], g[0], "dq")
    _grad_close(r1[1].transpose(-1, -2), g[1], "dk")
    _grad_close(r1[2], g[2], "dv")


def test_selection_backward_tensorcore_vs_generic_at_scale():
    from nsa import ops
    B, H, G, T, dk, dv, n = 1, 32, 2, 4096, 192, 128, 16
    gen = torch.Generator().manual_seed(10)
    q, k, v, do = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=10))
    idx = _random_indices(B, G, T, n, 64, gen, with_holes=False).to(DEV)
    scale = dk ** -0.5
    o, L, M = ops.slc_fwd(q, k, v, idx, 64, scale)
    tc = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale)
    gen_ = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale, generic=True)
    torch.cuda.synchronize()
    _no_timeouts()
    for a, b_, nme in zip(tc, gen_, ("dq", "dk", "dv")):
        _grad_close(a, b_.float().cpu(), "selection " + nme)


# the two long cases reach the 16- and 32-candidates-per-lane variants of the row top-n kernel (n_sel = 512, 1024)
@pytest.mark.timeout(600)
@pytest.mark.parametrize("dk,H,G,T", [(64, 8, 2, 2048), (192, 16, 1, 4096), (64, 4, 2, 32768), (64, 2, 1, 65536)])
def test_score_topn_tensorcore_bit_exact_outside_ambiguity(dk, H, G, T):
    """Fused Eq. 8-11 on tensor cores (bf16 hi + lo split of the fp32 keys) against the fp32 CPU oracle:
    identical block ids on every row whose ranking does not hinge on rounding, and identical to the
    stride-generic CUDA kernel under the same rule."""
    from nsa import ops
    from tests.util import ambiguous_rows
    l, d, lp, n = 32, 16, 64, 16
    inp = O.make_inputs(1, H, G, T, dk, 64, 64, l, seed=11, block_offset_std=0.5, dtype=torch.bfloat16)
    k_cmp, _, be, nb = O.compress_tokens(inp["k"].transpose(-1, -2), inp["v"], inp["phi"], l, d)
    scale = dk ** -0.5
    p = O.compression_probabilities(inp["q"], k_cmp, be, scale)
    sel = O.selection_scores_from_compression(p, l, d, lp)
    ref = O.select_top_n(sel, G, n, lp)
    agg = sel.view(1, G, H // G, T, -1).sum(2)
    amb = ambiguous_rows(agg, n)
    qd = inp["q"].bfloat16().to(DEV)
    tc = ops.score_topn(qd, k_cmp.to(DEV), be.to(DEV), l, d, lp, n, 3, scale, n_real_blocks=nb).cpu().long()
    gen = ops.score_topn(qd, k_cmp.to(DEV), be.to(DEV), l, d, lp, n, 3, scale, generic=True).cpu().long()
    torch.cuda.synchronize()
    _no_timeouts()
    bad_tc = (tc != ref).any(-1) & ~amb
    bad_gen = (gen != ref).any(-1) & ~amb
    from tests.util import INDEX_LOG
    INDEX_LOG.append((f"score_topn tensor-core dk={dk} H={H} G={G} T={T}", amb.numel(), int(amb.sum()), int((tc != ref).any(-1).sum()), int(bad_tc.sum())))
    INDEX_LOG.append((f"score_topn generic     dk={dk} H={H} G={G} T={T}", amb.numel(), int(amb.sum()), int((gen != ref).any(-1).sum()), int(bad_gen.sum())))
    assert not bad_gen.any(), f"generic kernel: {int(bad_gen.sum())} unambiguous rows differ"
    assert not bad_tc.any(), f"tensor-core kernel: {int(bad_tc.sum())} unambiguous rows differ, first {bad_tc.nonzero()[:3].tolist()}"
    # the ambiguity set is a property of the data (phi weights N(0,0.02) make the softmax over thousands of compressed
    # blocks nearly uniform: 14 % of the rows at T=2048, 19 % at 4096, 39 % at 32768 and 43 % at 65536 hold a pair of
    # adjacent top scores within 1e-5 relative); what must stay small is the number of rows that actually differ,
    # inside the set included (measured: at most 0.21 %)
    assert amb.float().mean() < 0.46
    assert (tc != ref).any(-1).float().mean() < 0.004 and (gen != ref).any(-1).float().mean() < 0.004
    # early rows: forced blocks first, never-visible blocks listed in id order, -1 padding only when blocks run out
    assert tc[0, 0, 0].tolist()[:3] == [0, 1, 2] and (tc >= -1).all() and (tc < (T + lp - 1) // lp).all()


def test_ragged_bf16_sequence_runs_on_padded_tiles():
    """A long bf16 sequence whose length is no multiple of the 128-row tile is padded inside nsa_layer and runs on the
    tensor-core kernels; rows, indices and gradients are those of the unpadded sequence (oracle, bf16 tolerance)."""
    import nsa
    from nsa.kernels import nsa_layer
    from nsa._lib import lib
    from tests.util import ambiguous_rows, oracle_layer_with_grads
    c = dict(B=1, H=4, G=2, T=2048 + 77, dk=64, dv=64, d_model=32, l=32, d=16, l_prime=64, n=16, w=512)
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=17,
                        block_offset_std=0.5, dtype=torch.bfloat16)
    cfg = nsa.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"],
                        l_prime=c["l_prime"], n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    q, k, v = (inp[x].bfloat16().to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    phi, gp = inp["phi"], inp["gate"]
    params = [p.to(DEV).requires_grad_(True) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2)]
    lin = torch.nn.functional.linear
    xg = inp["x"].to(DEV)
    logits = lin(torch.relu(lin(xg, gp.w1.to(DEV), gp.b1.to(DEV))), gp.w2.to(DEV), gp.b2.to(DEV))
    lib.nsa_profile_enable(1)
    out, info = nsa_layer(q, k, v, logits, tuple(params), cfg, return_info=True)
    grads = torch.autograd.grad(out, [q, k, v], inp["do"].bfloat16().to(DEV))
    import ctypes
    buf = ctypes.create_string_buffer(1 << 16)
    lib.nsa_profile_report(buf, 1 << 16)
    lib.nsa_profile_enable(0)
    launched = buf.value.decode()
    assert "slc_bwd_fused" in launched and "score_topn_tc" in launched, launched    # the tensor-core path ran
    _no_timeouts()
    T = c["T"]
    assert out.shape == (1, c["H"], T, c["dv"]) and info["indices"].shape[2] == T and grads[1].shape == k.shape
    nb = (T - c["l"]) // c["d"] + 1
    assert info["k_cmp"].shape[-1] == O.next_pow2(nb) and int(info["block_ends"][nb - 1]) == (nb - 1) * c["d"] + c["l"] - 1
    assert (info["block_ends"][nb:] == 999999).all()
    from tests.util import GRAD_NAMES, close, heads_mask, index_agreement
    r, gref = oracle_layer_with_grads(inp, c)
    where = "ragged bf16 T=2125 (padded tiles)"
    agg = r["sel_scores"].view(1, c["G"], c["H"] // c["G"], T, -1).sum(2)
    mism = index_agreement(where, info["indices"], r["indices"], agg, c["n"])
    ok = heads_mask(~mism, c["H"])
    close(where, "out[rows with equal ids]", out, r["out"], bf16=True, rows=ok)
    close(where, "dq[rows with equal ids]", grads[0], gref[0], bf16=True, grad=True, rows=ok)
    # the oracle's ids fed to the CUDA branches: every element of the outputs and of dQ, dK, dV
    q2, k2, v2 = (inp[x].bfloat16().to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
    out2 = nsa_layer(q2, k2, v2, logits, tuple(params), cfg, indices=r["indices"])
    grads2 = torch.autograd.grad(out2, [q2, k2, v2], inp["do"].bfloat16().to(DEV))
    close(where, "out[oracle ids]", out2, r["out"], bf16=True)
    for name, a_, b_ in zip(GRAD_NAMES, grads2, gref[:3]):
        close(where, name + "[oracle ids]", a_, b_, bf16=True, grad=True)


@pytest.mark.parametrize("dtype,T", [(torch.bfloat16, 1024), (torch.float32, 300)])
def test_selection_backward_adds_the_other_branches_dq(dtype, T):
    """dq_add0/dq_add1 of nsa_slc_bwd: dq = dq_selection + a + b, summed in fp32 and rounded once (tensor-core and generic paths)."""
    from nsa import ops
    B, H, G, dk, dv, n = 1, 16, 1, 64, 64, 8
    gen = torch.Generator().manual_seed(12)
    q, k, v, do = (t.to(DEV, dtype) for t in _inputs(B, H, G, T, dk, dv, seed=12))
    idx = _random_indices(B, G, T, n, 64, gen, with_holes=False).to(DEV)
    a, b_ = (torch.randn(B, H, T, dk, generator=gen).to(DEV, dtype) for _ in range(2))
    scale = dk ** -0.5
    o, L, M = ops.slc_fwd(q, k, v, idx, 64, scale)
    plain = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale)
    both = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale, dq_addends=(a, b_))
    one = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale, dq_addends=(a,))
    again = ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale)          # the addends served one call only
    torch.cuda.synchronize()
    _no_timeouts()
    assert torch.equal(again[0], plain[0]) and torch.equal(both[1], plain[1]) and torch.equal(both[2], plain[2])
    tol = 4e-2 if dtype == torch.bfloat16 else 1e-5
    want = plain[0].float() + a.float() + b_.float()
    assert max_abs(both[0].float(), want) < tol * max(1.0, want.abs().max().item())
    want1 = plain[0].float() + a.float()
    assert max_abs(one[0].float(), want1) < tol * max(1.0, want1.abs().max().item())


def test_backward_takes_the_row_sums_from_the_caller():
    """row_delta of the backward entry points: with the row sums dO.O handed in, the three tensor-core backward paths return what they return
    when they compute the sums themselves (same sums up to fp32 summation order), and a wrong delta changes the result,
    which shows that it is used; the hint serves one call."""
    from nsa import ops
    B, H, G, T, dk, dv, n = 1, 16, 1, 1024, 64, 64, 8
    gen = torch.Generator().manual_seed(14)
    q, k, v, do = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=14))
    scale = dk ** -0.5
    idx = _random_indices(B, G, T, n, 64, gen, with_holes=False).to(DEV)

    def check(fwd, bwd):
        o, L, M = fwd()
        delta = (o.float() * do.float()).sum(-1)
        plain = bwd(o, L, M)
        given = bwd(o, L, M, row_delta=delta)
        after = bwd(o, L, M)
        wrong = bwd(o, L, M, row_delta=delta + 1.0)
        torch.cuda.synchronize()
        _no_timeouts()
        for a, b_, c in zip(plain, given, after):
            assert torch.equal(a, c)
            assert max_abs(a.float(), b_.float()) < 2e-2 * max(1.0, a.float().abs().max().item())
        assert max_abs(plain[0].float(), wrong[0].float()) > 0.05

    check(lambda: ops.sliding_fwd(q, k, v, 512, scale), lambda o, L, M, **kw: ops.sliding_bwd(q, k, v, o, do, L, M, 512, scale, **kw))
    check(lambda: ops.slc_fwd(q, k, v, idx, 64, scale), lambda o, L, M, **kw: ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale, **kw))


@pytest.mark.parametrize("dtype,dk,dv,H,G,T,n", [(torch.bfloat16, 192, 128, 16, 1, 1024, 16), (torch.bfloat16, 64, 64, 8, 2, 512, 6),
                                                 (torch.bfloat16, 128, 128, 64, 1, 256, 4), (torch.float32, 48, 80, 6, 3, 333, 5)])
@pytest.mark.parametrize("mode", ["sigmoid", "softmax"])
def test_selection_forward_with_the_mix_epilogue(dtype, dk, dv, H, G, T, n, mode):
    """nsa_slc_fwd_mix: the gate + mix done by the kernel that merges the selection partials (tensor-core path: the
    bulk-copy merge, and the plain one when a group has more than 32 heads; stride-generic path: a separate pass inside
    the entry point) gives bit for bit what the stand-alone pass gives on the same branch outputs, in the head-major and
    in the token-major output layout; the gate/mix backward reads a token-major upstream gradient as it lies."""
    from nsa import ops
    gen = torch.Generator().manual_seed(15)
    B = 2
    rnd = lambda *s: torch.randn(*s, generator=gen).to(dtype).to(DEV)
    q, k, v = rnd(B, H, T, dk), rnd(B, G, dk, T), rnd(B, G, T, dv)
    oc, ow, do = rnd(B, H, T, dv), rnd(B, H, T, dv), rnd(B, H, T, dv)
    lg = torch.randn(B, T, 3 * H, generator=gen).to(DEV)
    lp = 64 if dtype == torch.bfloat16 else 16
    idx = torch.randint(-1, (T + lp - 1) // lp, (B, G, T, n), generator=gen).to(DEV, torch.int32)
    idx[:, :, 5] = -1
    scale = dk ** -0.5
    o_ref, L_ref, M_ref = ops.slc_fwd(q, k, v, idx, lp, scale)
    out_ref, gates_ref = ops.gate_mix_fwd(lg, oc, o_ref, ow, mode)
    for tm in (False, True):
        o, L, M, out, gates = ops.slc_fwd_mix(q, k, v, idx, lp, scale, lg, oc, ow, mode, token_major=tm)
        torch.cuda.synchronize()
        assert out.shape == out_ref.shape and out.permute(0, 2, 1, 3).is_contiguous() == tm
        assert torch.equal(o, o_ref) and torch.equal(L, L_ref) and torch.equal(M, M_ref)
        assert torch.equal(gates, gates_ref)
        assert torch.equal(out.contiguous(), out_ref)
        out2, _ = ops.gate_mix_fwd(lg, oc, o_ref, ow, mode, token_major=tm)
        assert torch.equal(out2.contiguous(), out_ref)
    plain = ops.gate_mix_bwd(gates_ref, oc, o_ref, ow, do, mode, want_delta=True)
    do_tm = do.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)       # same values, [B,T,H,dv] in memory
    assert not do_tm.is_contiguous()
    given = ops.gate_mix_bwd(gates_ref, oc, o_ref, ow, do_tm, mode, want_delta=True)
    torch.cuda.synchronize()
    _no_timeouts()
    assert all(torch.equal(a, b_) for a, b_ in zip(plain, given))


@pytest.mark.parametrize("shared_kv", [True, False])
def test_layer_entry_points_match_the_composed_branch_calls(shared_kv):
    """nsa_layer_fwd / nsa_layer_bwd (one C call each way) against the same layer composed from the branch entry points
    (what the long-context mode runs): identical kernels, so outputs, dQ and the gate gradient agree bit for bit; dK/dV
    are accumulated in one buffer per k/v pair inside the library (one bf16 rounding per branch) and agree within it."""
    import nsa
    import nsa.kernels as K
    c = dict(B=1, H=8, G=2, T=1024, dk=64, dv=64, d_model=32, l=32, d=16, l_prime=64, n=8, w=200)
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=19, block_offset_std=0.5,
                        dtype=torch.bfloat16)
    cfg = nsa.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"], l_prime=c["l_prime"],
                        n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    gen = torch.Generator().manual_seed(4)
    logits = torch.randn(1, c["T"], 3 * c["H"], generator=gen).to(DEV)
    extra = None
    if not shared_kv:
        mk = lambda: (torch.randn(1, c["G"], c["dk"], c["T"], generator=gen).bfloat16().to(DEV),
                      torch.randn(1, c["G"], c["T"], c["dv"], generator=gen).bfloat16().to(DEV))
        extra = (mk(), mk())

    def run(use_c):
        K._USE_C_LAYER = use_c
        try:
            q, k, v = (inp[x].bfloat16().to(DEV).requires_grad_(True) for x in ("q", "k", "v"))
            phi = [p.to(DEV).requires_grad_(True) for p in (inp["phi"].pos_embed, inp["phi"].w1, inp["phi"].b1, inp["phi"].w2, inp["phi"].b2)]
            lg = logits.clone().requires_grad_(True)
            kw = {}
            leaves = [q, k, v, lg] + phi
            if extra is not None:
                kv = [tuple(t.clone().requires_grad_(True) for t in pair) for pair in extra]
                kw = dict(kv_compress=kv[0], kv_sliding=kv[1])
                leaves += [kv[0][0], kv[0][1], kv[1][0], kv[1][1]]
            out, info = K.nsa_layer(q, k, v, lg, tuple(phi), cfg, return_info=True, **kw)
            grads = torch.autograd.grad(out, leaves, inp["do"].bfloat16().to(DEV))
            return out, info, grads
        finally:
            K._USE_C_LAYER = True

    out_c, info_c, g_c = run(True)
    out_p, info_p, g_p = run(False)
    torch.cuda.synchronize()
    _no_timeouts()
    assert torch.equal(info_c["indices"], info_p["indices"])
    for key in ("o_cmp", "o_slc", "o_win", "gates"):
        assert torch.equal(info_c[key], info_p[key]), key
    assert torch.equal(out_c, out_p)
    assert torch.equal(g_c[0], g_p[0]) and torch.equal(g_c[3], g_p[3])          # dq, dlogits
    for a, b_ in zip(g_c[1:3] + g_c[4:], g_p[1:3] + g_p[4:]):
        _grad_close(a, b_.float().cpu(), "dk / dv / phi gradient")


@pytest.mark.parametrize("dk,dv,H,G,T", [(64, 64, 4, 2, 2048), (192, 128, 4, 1, 4096 + 2048)])
def test_compression_forward_on_split_keys_and_its_lse_in_scoring(dk, dv, H, G, T):
    """fp32 compressed keys handed over as bf16 hi + lo halves: the output and statistics follow the oracle on the fp32
    keys (closer than the bf16-key form can), the log-sum-exp equals the oracle's, and the scoring kernel that takes
    that log-sum-exp selects exactly the blocks it selects when it computes the row statistics itself."""
    from nsa import ops
    l, d, lp, n = 32, 16, 64, 16
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    gen = torch.Generator().manual_seed(12)
    q = torch.randn(1, H, T, dk, generator=gen).bfloat16()
    kc = torch.zeros(1, G, dk, nbp)
    kc[..., :nb] = torch.randn(1, G, dk, nb, generator=gen)
    vc = torch.zeros(1, G, nbp, dv)
    vc[:, :, :nb] = torch.randn(1, G, nb, dv, generator=gen)
    vc = vc.bfloat16()
    be = torch.full((nbp,), 999999, dtype=torch.int32)
    be[:nb] = torch.arange(nb, dtype=torch.int32) * d + l - 1
    scale = dk ** -0.5
    qd, kd, vd, bed = q.to(DEV), kc.to(DEV), vc.to(DEV), be.to(DEV)
    assert ops.cmp_exact_supported(qd, kd, vd)
    hi, lo = ops.split_keys(kd)
    assert (hi.float() + lo.float() - kd).abs().max() <= kd.abs().max() * 2.0 ** -16
    o, L, M, lse2 = ops.cmp_attn_fwd(qd, hi, vd, bed, scale, blocks=(l, d, nb), k_lo=lo)
    torch.cuda.synchronize()
    _no_timeouts()
    o_ref, M_ref, L_ref = O.compression_attention(q.float(), kc, vc.float(), be, scale, return_stats=True)
    assert max_abs(o.float(), o_ref) < 2e-2
    _check_stats(L, M, L_ref, M_ref)
    fin = torch.isfinite(M_ref)
    lse_ref = (M_ref + L_ref)[fin] * 1.4426950408889634        # L is the log of the row sum
    assert torch.isinf(lse2.cpu()[~fin]).all() and (lse2.cpu()[~fin] > 0).all()
    assert (lse2.cpu()[fin] - lse_ref).abs().max() < 2e-3
    ids_own = ops.score_topn(qd, kd, bed, l, d, lp, n, 3, scale, n_real_blocks=nb)
    ids_lse = ops.score_topn(qd, kd, bed, l, d, lp, n, 3, scale, n_real_blocks=nb, cmp_lse2=lse2)
    torch.cuda.synchronize()
    _no_timeouts()
    differ = (ids_own != ids_lse).any(-1)
    # the two log-sum-exps differ by rounding (1e-6 relative), which can swap two blocks whose scores tie to that level
    assert differ.float().mean().item() < 2e-3, f"{int(differ.sum())} of {differ.numel()} rows select other blocks"
    sel = O.selection_scores_from_compression(O.compression_probabilities(q.float(), kc, be, scale), l, d, lp)
    ref = O.select_top_n(sel, G, n, lp)
    clear = ~O.ambiguous_rows(sel.view(1, G, H // G, T, -1).sum(2), n)
    assert clear.float().mean().item() > 0.9
    assert torch.equal(ids_lse.cpu().long()[clear], ref[clear]), "rows without a near-tie select other blocks than the oracle"


def test_sliding_window_alone_at_its_benchmark_configuration():
    """The sliding-window branch alone at the size the project's second benchmark configuration names (B=4, H=64, G=4,
    T=8192, dk=192, dv=128, window 512, bf16, forward + backward): output rows and statistics against the CPU oracle's
    per-row attention on sampled positions (first rows, around the window length, tile edges, last row), gradients
    against the stride-generic kernels (which the small cases above pin to the oracle)."""
    from nsa import ops
    B, H, G, T, dk, dv, w = 4, 64, 4, 8192, 192, 128, 512
    q, k, v, do = (t.to(DEV) for t in _inputs(B, H, G, T, dk, dv, seed=21))
    scale = dk ** -0.5
    o, L, M = ops.sliding_fwd(q, k, v, w, scale)
    dq, dkey, dval = ops.sliding_bwd(q, k, v, o, do, L, M, w, scale)
    gen = ops.sliding_bwd(q, k, v, o, do, L, M, w, scale, generic=True)
    torch.cuda.synchronize()
    _no_timeouts()
    hpg = H // G
    pos = sorted({0, 1, 63, 64, 127, 128, 510, 511, 512, 513, 1023, 1024, 4095, 4096, 4097, T - 129, T - 128, T - 1} |
                 {int(x) for x in torch.randint(0, T, (24,), generator=torch.Generator().manual_seed(3))})
    qc, kc, vc = q.float().cpu(), k.float().cpu(), v.float().cpu()
    worst_o, worst_lse = 0.0, 0.0
    for t in pos:
        lo = max(0, t - w + 1)
        for g in range(G):
            s = torch.einsum("bhd,bdn->bhn", qc[:, g * hpg:(g + 1) * hpg, t], kc[:, g, :, lo:t + 1]) * scale
            ref = torch.softmax(s, -1) @ vc[:, g, lo:t + 1]
            got = o[:, g * hpg:(g + 1) * hpg, t].float().cpu()
            worst_o = max(worst_o, (got - ref).abs().max().item())
            lse = (M + L)[:, g * hpg:(g + 1) * hpg, t].cpu()
            worst_lse = max(worst_lse, (lse - torch.logsumexp(s, -1)).abs().max().item())
    assert worst_o < 2e-2 and worst_lse < 2e-2, (worst_o, worst_lse)
    for a, b_, n in zip((dq, dkey, dval), gen, ("dq", "dk", "dv")):
        _grad_close(a, b_.float().cpu(), "sliding window at B=4 T=8192: " + n)
