"""The CPU oracle against golden vectors produced by the reference project's own code.

The vectors were written by tests/golden/make_golden.py, which ran nsa/reference.py and
nsa/kernels.py of the reference on the seeded inputs re-drawn here.  Tolerances: 2e-5 relative
(max-abs over max-abs) for floating point, exact for indices outside the rows where the reference's
own fp32 and fp64 runs disagree.
"""
import json
import os

import numpy as np
import pytest
import torch

from oracle import nsa_oracle as O

GOLD = os.path.join(os.path.dirname(__file__), "golden")
META = json.load(open(os.path.join(GOLD, "golden_meta.json")))


def rel(a, b):
    a = torch.as_tensor(a, dtype=torch.float64)
    b = torch.as_tensor(b, dtype=torch.float64)
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


@pytest.fixture(scope="module", params=sorted(META["cases"]))
def case(request):
    c = META["cases"][request.param]
    g = dict(np.load(os.path.join(GOLD, request.param + ".npz")))
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=c["seed"],
                        l_prime=c["l_prime"])
    return c, g, inp


def test_phi_and_block_ends(case):
    c, g, inp = case
    k_cmp, v_cmp, be, nb = O.compress_tokens(inp["k"].transpose(-1, -2), inp["v"], inp["phi"], c["l"], c["d"])
    assert nb == int(g["n_blocks"])
    assert np.array_equal(be.numpy(), g["block_ends"])
    assert k_cmp.shape == g["k_cmp"].shape and v_cmp.shape == g["v_cmp"].shape
    assert rel(k_cmp, g["k_cmp"]) < 2e-5
    assert rel(v_cmp, g["v_cmp"]) < 2e-5


def test_scores_and_indices(case):
    c, g, inp = case
    rows = g["rows"]
    scale = c["dk"] ** -0.5
    k_cmp, be = torch.from_numpy(g["k_cmp"]), torch.from_numpy(g["block_ends"])
    p = O.compression_probabilities(inp["q"], k_cmp, be, scale)
    sel = O.selection_scores_from_compression(p, c["l"], c["d"], c["l_prime"])
    assert np.array_equal(sel[:, :, rows].numpy(), g["sel_rows"])          # same adds, same order
    idx = O.select_top_n(sel, c["G"], c["n"], c["l_prime"])
    assert np.array_equal(idx.numpy(), g["indices"])


@pytest.mark.parametrize("branch", ["win", "cmp", "slc"])
def test_branch_forward_backward(case, branch):
    c, g, inp = case
    rows = torch.from_numpy(g["rows"])
    scale = c["dk"] ** -0.5
    q = inp["q"].clone().requires_grad_(True)
    if branch == "cmp":
        k = torch.from_numpy(g["k_cmp"]).requires_grad_(True)
        v = torch.from_numpy(g["v_cmp"]).requires_grad_(True)
        o = O.compression_attention(q, k, v, torch.from_numpy(g["block_ends"]), scale)
    else:
        k = inp["k"].clone().requires_grad_(True)
        v = inp["v"].clone().requires_grad_(True)
        if branch == "win":
            o = O.sliding_window_attention(q, k, v, c["w"], scale)
        else:
            idx = O.selection_fallback_indices(torch.from_numpy(g["indices"]).long(), c["l_prime"])
            o = O.selection_attention(q, k, v, idx, c["l_prime"], scale)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), inp["do"])
    assert rel(o.detach()[:, :, rows], g[branch + "_o"]) < 2e-5
    assert rel(dq[:, :, rows], g[branch + "_dq"]) < 2e-5
    if branch == "cmp":
        assert rel(dk, g["cmp_dk"]) < 2e-5 and rel(dv, g["cmp_dv"]) < 2e-5
    else:
        assert rel(dk[..., rows], g[branch + "_dk"]) < 2e-5
        assert rel(dv[:, :, rows], g[branch + "_dv"]) < 2e-5


def test_whole_module_against_reference_forward(case):
    """Projections -> layer -> o_proj against NSAAttention.forward (eval, CPU) of the reference."""
    c, g, inp = case
    rows = g["rows"]
    proj = O.draw_projection_weights(c["seed"] + 11, c["d_model"], c["H"], c["G"], c["dk"], c["dv"])
    gen = torch.Generator().manual_seed(c["seed"] + 7)
    hidden = torch.randn(c["B"], c["T"], c["d_model"], generator=gen) * 0.5
    y, r = O.nsa_module_forward(hidden, proj, inp["phi"], inp["gate"], H=c["H"], G=c["G"], dk=c["dk"], dv=c["dv"],
                                l=c["l"], d=c["d"], l_prime=c["l_prime"], n=c["n"], w=c["w"])
    assert rel(r["p_cmp"][:, :, rows], g["mod_p_cmp"]) < 2e-5
    assert rel(r["sel_scores"][:, :, rows], g["mod_sel"]) < 2e-5
    assert rel(r["gates"].permute(0, 2, 1, 3)[:, rows], g["mod_gates"]) < 2e-5
    bad = (r["indices"].numpy() != g["mod_indices"]).any(-1)
    assert bad.mean() < 0.01, f"{bad.sum()} index rows differ"
    if not bad.any():
        assert rel(y[:, rows], g["mod_y"]) < 5e-5


def test_top_n_known_answers():
    """Literal expectations of the reference's tests/test_whitepaper_spec.py:39-78."""
    s = torch.arange(5, dtype=torch.float32).view(1, 1, 1, 5).repeat(1, 2, 3, 1)
    idx = O.select_top_n(s, 1, 3, 2, include_fixed=False, n_fixed=0)
    assert all(idx[0, 0, t].tolist() == [4, 3, 2] for t in range(3))
    idx = O.select_top_n(s, 1, 3, 2, include_fixed=True, n_fixed=3)
    assert idx[0, 0, 0].tolist() == [0, 4, 3] and idx[0, 0, 2].tolist() == [0, 1, 4]
    idx = O.select_top_n(torch.zeros(1, 2, 2, 2), 1, 4, 2)
    assert idx.shape[-1] == 4 and (idx[0, 0, 0, 2:] == -1).all()
    # stable ties go to the lower block id
    t = torch.tensor([.5, .5, .1, .5, 0., 0.]).view(1, 1, 1, 6)
    assert O.select_top_n(t, 1, 4, 2, include_fixed=False, n_fixed=0)[0, 0, 0].tolist() == [0, 1, 3, 2]


def test_eq9_stencil():
    """l=32, d=16, l'=64 gives weights [1,2,2,2,1] on p[4j..4j+4] (nsa/kernels.py:1953-1960)."""
    p = torch.rand(1, 1, 2, 32)
    sel = O.selection_scores_from_compression(p, 32, 16, 64)
    assert sel.shape[-1] == 8
    pp = torch.cat([p, torch.zeros(1, 1, 2, 8)], -1)
    w = torch.tensor([1., 2., 2., 2., 1.])
    for j in range(8):
        assert torch.allclose(sel[..., j], (pp[..., 4 * j:4 * j + 5] * w).sum(-1), rtol=1e-6, atol=1e-7)


def test_row_functions_agree_with_the_dense_oracle():
    """The sampled-row forms (used where a sequence is too long for the dense functions) against the dense, golden-pinned
    ones on the rows they share."""
    c = dict(B=2, H=8, G=2, T=700, dk=32, dv=48, l=32, d=16, lp=64, n=6, w=100)
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], 32, c["l"], seed=5, block_offset_std=0.5)
    scale = c["dk"] ** -0.5
    r = O.nsa_layer(inp["q"], inp["k"], inp["v"], inp["x"], inp["phi"], inp["gate"], l=c["l"], d=c["d"], l_prime=c["lp"],
                    n=c["n"], w=c["w"])
    pos = torch.tensor([0, 5, 30, 31, 32, 63, 64, 99, 100, 101, 383, 384, 385, 500, 699])
    qr = inp["q"][:, :, pos]
    idx, agg = O.score_rows(qr, pos, r["k_cmp"], r["block_ends"], l=c["l"], d=c["d"], l_prime=c["lp"], n=c["n"], scale=scale)
    assert torch.equal(idx, r["indices"][:, :, pos])
    full_agg = r["sel_scores"].view(c["B"], c["G"], c["H"] // c["G"], c["T"], -1).sum(2)[:, :, pos]
    assert torch.allclose(agg, full_agg, rtol=1e-5, atol=1e-7)
    o_cmp, o_slc, o_win = O.branch_rows(qr, pos, inp["k"], inp["v"], r["k_cmp"], r["v_cmp"], r["block_ends"], idx, w=c["w"],
                                        l_prime=c["lp"], scale=scale)
    for got, name in ((o_cmp, "o_cmp"), (o_slc, "o_slc"), (o_win, "o_win")):
        want = r[name][:, :, pos]
        assert (got - want).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item()), name
    # forced ids replace the layer's own choice and nothing else
    forced = r["indices"].clone()
    forced[:, :, 200:, 3:] = -1
    r2 = O.nsa_layer(inp["q"], inp["k"], inp["v"], inp["x"], inp["phi"], inp["gate"], l=c["l"], d=c["d"], l_prime=c["lp"],
                     n=c["n"], w=c["w"], indices=forced)
    assert torch.equal(r2["indices_own"], r["indices"]) and torch.equal(r2["o_cmp"], r["o_cmp"])
    assert torch.equal(r2["o_slc"][:, :, :200], r["o_slc"][:, :, :200]) and not torch.equal(r2["o_slc"], r["o_slc"])
