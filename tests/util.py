"""Shared helpers of the GPU parity tests: seeded inputs, oracle runs, error metrics."""
import math

import torch

from oracle import nsa_oracle as O


def rel_err(a, b):
    """max|a-b| / (max|b| + 1e-8): the metric of the reference's compare_outputs (nsa/reference.py:341-342)."""
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return ((a - b).abs().max() / (b.abs().max() + 1e-8)).item()


def max_abs(a, b):
    return (a.detach().double().cpu() - b.detach().double().cpu()).abs().max().item()


def ambiguous_rows(sel_scores_grouped, n, tau=1e-5):
    """Rows [B,G,T] whose top-(n+1) aggregated scores hold an adjacent pair closer than tau (relative):
    there the ranking depends on fp32 rounding order and no independent implementation can be
    expected to agree bit for bit."""
    k = min(n + 1, sel_scores_grouped.shape[-1])
    top = torch.sort(sel_scores_grouped.double(), dim=-1, descending=True).values[..., :k]
    gap = (top[..., :-1] - top[..., 1:]) / top[..., :-1].abs().clamp_min(1e-30)
    both_zero = (top[..., :-1] == 0) & (top[..., 1:] == 0)      # exact ties are decided by index: not ambiguous
    return ((gap < tau) & ~both_zero).any(dim=-1)


def oracle_layer_with_grads(inp, cfg, dtype=torch.float32):
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
                    gate_mode=cfg.get("gate_mode", "sigmoid"))
    grads = torch.autograd.grad(r["out"], [q, k, v] + plist, inp["do"])
    return r, grads
