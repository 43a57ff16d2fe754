"""Shared helpers of the GPU parity tests: seeded inputs, oracle runs, error metrics, the parity log."""
import math

import torch

from oracle import nsa_oracle as O

# One line per comparison made through `close()`: (where, tensor, achieved max-abs, largest |reference|, bound).
# tests/conftest.py prints it at the end of the run, so the achieved errors are on record, not only pass/fail.
PARITY_LOG = []
# Index agreement of the full-layer runs: (where, rows, ambiguous rows, rows that differ, of those outside the ambiguity set)
INDEX_LOG = []


def rel_err(a, b):
    """max|a-b| / (max|b| + 1e-8): the metric of the reference's compare_outputs (nsa/reference.py:341-342)."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-8)).item()


def max_abs(a, b):
    return (a.detach().double().cpu() - b.detach().double().cpu()).abs().max().item()


def close(where, name, got, ref, *, bf16, grad=False, rows=None, bound=None):
    """Assert one tensor against its reference and log the achieved error.

    fp32 I/O: max|a-b| / max|ref| < 1e-3.  bf16 I/O: outputs max-abs < 2e-2; gradients max-abs < 2e-2 * max(1, max|ref|)
    (gradients of N(0,1) data reach magnitudes of 10 and more, where one bf16 rounding of the result alone is 3e-2).
    ``rows``: boolean mask over the leading dims selecting the rows to compare; ``bound`` overrides the relative bound.
    """
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    if rows is not None:
        got, ref = got[rows], ref[rows]
    if ref.numel() == 0:
        return
    err = (got.double() - ref.double()).abs().max().item()
    ref_max = ref.abs().max().item()
    if bf16:
        tol = (bound if bound is not None else 2e-2) * (max(1.0, ref_max) if grad else 1.0)
    else:
        tol = (bound if bound is not None else 1e-3) * (ref_max + 1e-8)
    PARITY_LOG.append((where, name, err, ref_max, tol))
    assert err < tol, f"{where}: {name} max-abs {err:.4g} exceeds {tol:.4g} (largest reference magnitude {ref_max:.4g})"


ambiguous_rows = O.ambiguous_rows


def index_agreement(where, idx_gpu, idx_ref, agg_scores, n, extra_ambiguous=None):
    """Compare block ids; returns the mask [B,G,T] of rows that differ.  Rows may differ only inside the ambiguity
    set; the counts go to INDEX_LOG."""
    amb = ambiguous_rows(agg_scores, n)
    if extra_ambiguous is not None:
        amb = amb | extra_ambiguous
    mism = (idx_gpu.cpu().long() != idx_ref.long()).any(-1)
    outside = mism & ~amb
    INDEX_LOG.append((where, mism.numel(), int(amb.sum()), int(mism.sum()), int(outside.sum())))
    assert not outside.any(), f"{where}: {int(outside.sum())} rows outside the ambiguity set select other blocks, first {outside.nonzero()[:3].tolist()}"
    return mism


def heads_mask(rows_bgt, H):
    """[B,G,T] row mask -> [B,H,T]."""
    B, G, T = rows_bgt.shape
    return rows_bgt.unsqueeze(2).expand(B, G, H // G, T).reshape(B, H, T)


def oracle_layer_with_grads(inp, cfg, dtype=torch.float32, include_fixed=True):
    """Oracle forward + autograd backward of the whole layer on CPU fp32."""
    q = inp["q"].clone().requires_grad_(True)
    k = inp["k"].clone().requires_grad_(True)
    v = inp["v"].clone().requires_grad_(True)
    phi, gp = inp["phi"], inp["gate"]
    plist = [phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2, gp.w1, gp.b1, gp.w2, gp.b2]
    plist = [p.clone().requires_grad_(True) for p in plist]
    phi2 = O.PhiParams(*plist[:5])
    gp2 = O.GateParams(*plist[5:])
    r = O.nsa_layer(q, k, v, inp["x"], phi2, gp2, l=cfg["l"], d=cfg["d"], l_prime=cfg["l_prime"], n=cfg["n"], w=cfg["w"],
                    gate_mode=cfg.get("gate_mode", "sigmoid"), include_fixed=include_fixed)
    leaves = [q, k, v] + plist
    grads = torch.autograd.grad(r["out"], leaves, inp["do"], allow_unused=True)   # phi is unused when T < l
    return r, [torch.zeros_like(x) if g is None else g for g, x in zip(grads, leaves)]


GRAD_NAMES = ["dq", "dk", "dv", "dpos", "dw1", "db1", "dw2", "db2", "dgw1", "dgb1", "dgw2", "dgb2"]


def gpu_layer_with_grads(nsa_mod, c, inp, dtype, dev="cuda", gate_mode="sigmoid", include_fixed=True, indices=None):
    """The CUDA layer on the same inputs: returns (out, info, the 12 gradients in GRAD_NAMES order)."""
    from nsa.kernels import nsa_layer
    cfg = nsa_mod.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"],
                            l_prime=c["l_prime"], n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"], gate_mode=gate_mode,
                            include_fixed_in_selection=include_fixed)
    q, k, v = (inp[n_].to(dev, dtype).contiguous().requires_grad_(True) for n_ in ("q", "k", "v"))
    phi, gp = inp["phi"], inp["gate"]
    params = [p.to(dev).contiguous().requires_grad_(True)
              for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2, gp.w1, gp.b1, gp.w2, gp.b2)]
    lin = torch.nn.functional.linear
    logits = lin(torch.relu(lin(inp["x"].to(dev), params[5], params[6])), params[7], params[8])
    out, info = nsa_layer(q, k, v, logits, tuple(params[:5]), cfg, return_info=True, indices=indices)
    leaves = [q, k, v] + params
    grads = torch.autograd.grad(out, leaves, inp["do"].to(dev, dtype), allow_unused=True)
    return out, info, [torch.zeros_like(x) if g is None else g for g, x in zip(grads, leaves)]


def check_layer_against_oracle(where, nsa_mod, c, inp, dtype, *, gate_mode="sigmoid", include_fixed=True, dev="cuda"):
    """Full-layer parity, unconditional.

    Run 1 (the layer's own block choice): ids equal the oracle's outside the ambiguity set (counts logged);
    O_cmp and O_win on every row; O_slc, the mixed output and dQ on every row whose ids agree (rows are independent
    per query).  Run 2 (the oracle's ids fed to the CUDA branches, so that near-ties cannot matter): outputs and all
    twelve gradients, every element.  Returns (info of run 1, rows that differ)."""
    bf16 = dtype == torch.bfloat16
    cc = dict(c, gate_mode=gate_mode)
    r, gref = oracle_layer_with_grads(inp, cc, include_fixed=include_fixed)
    ref = dict(zip(GRAD_NAMES, gref))
    B, H, G, T = c["B"], c["H"], c["G"], c["T"]
    out, info, grads = gpu_layer_with_grads(nsa_mod, c, inp, dtype, dev, gate_mode, include_fixed)
    agg = r["sel_scores"].view(B, G, H // G, T, -1).sum(2)
    mism = index_agreement(where, info["indices"], r["indices"], agg, c["n"])
    ok = heads_mask(~mism, H)
    for key in ("o_cmp", "o_win"):
        close(where, key, info[key], r[key], bf16=bf16)
    close(where, "o_slc[rows with equal ids]", info["o_slc"], r["o_slc"], bf16=bf16, rows=ok)
    close(where, "out[rows with equal ids]", out, r["out"], bf16=bf16, rows=ok)
    close(where, "dq[rows with equal ids]", grads[0], ref["dq"], bf16=bf16, grad=True, rows=ok)
    out2, info2, grads2 = gpu_layer_with_grads(nsa_mod, c, inp, dtype, dev, gate_mode, include_fixed, indices=r["indices"])
    close(where, "o_slc[oracle ids]", info2["o_slc"], r["o_slc"], bf16=bf16)
    close(where, "out[oracle ids]", out2, r["out"], bf16=bf16)
    for name, a in zip(GRAD_NAMES, grads2):
        b = ref[name]
        if name in ("dq", "dk", "dv"):
            close(where, name + "[oracle ids]", a, b, bf16=bf16, grad=True)
        elif name == "db2":
            # a constant added to every compressed key leaves the softmax unchanged: the true gradient is zero and
            # both sides hold rounding noise (with bf16 I/O: the sum over all blocks of the bf16 roundings of dK_cmp,
            # which no weight scales down); compared on the scale of the weight gradient next to it
            err = max_abs(a, b)
            tol = (0.25 if bf16 else 1e-3) * ref["dw2"].abs().max().item() + 1e-12      # dw2 = 0 when no block is ever visible
            PARITY_LOG.append((where, "db2 (on the scale of dw2)", err, ref["dw2"].abs().max().item(), tol))
            assert err < tol, f"{where}: db2 {err} vs {tol}"
        else:
            # weight gradients are fp32 tensors on both sides; with bf16 activations they carry the activations' rounding
            err, scale_ = max_abs(a, b), b.abs().max().item() + 1e-12
            tol = (3e-2 if bf16 else 1e-3) * scale_
            PARITY_LOG.append((where, name + "[oracle ids]", err, scale_, tol))
            assert err <= tol, f"{where}: {name} max-abs {err:.4g} exceeds {tol:.4g}"
    return info, mism, r


sample_positions = O.sample_positions
