#!/usr/bin/env python3
"""Generate the golden fixtures in this directory from the reference project itself.

Usage (needs a checkout of Noumena-Network/NSA-Test; CPU only, a minute or two):

    python tests/golden/make_golden.py --reference /path/to/NSA-Test

The reference's ``nsa`` package is loaded under the alias ``nsa_ref`` (so it cannot clash with this
repository's own ``nsa`` package) and its own functions are run on seeded inputs:

* ``nsa/reference.py``: sliding_window_attention, compression_attention,
  selection_attention_reference (forward, and backward through autograd);
* ``nsa/kernels.py``: NSAAttention.compress_tokens, derive_selection_from_compression_per_timestep,
  select_top_k_blocks_per_query_with_gqa, and the whole NSAAttention.forward in eval mode (the
  reference's CPU path) with output_attentions=True.

Outputs are stored sub-sampled (a fixed set of query rows / key tokens) to keep the files small;
inputs are not stored, they are re-drawn from the same seeds by ``oracle.nsa_oracle.make_inputs``.
``tests/test_oracle_golden.py`` re-checks the CPU oracle against these files on every run.
"""
import argparse
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import nsa_oracle as O  # noqa: E402


def load_reference(root):
    spec = importlib.util.spec_from_file_location(
        "nsa_ref", os.path.join(root, "nsa", "__init__.py"),
        submodule_search_locations=[os.path.join(root, "nsa")])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nsa_ref"] = mod
    spec.loader.exec_module(mod)
    import nsa_ref.kernels as K
    import nsa_ref.reference as R
    return K, R


CASES = {
    # BASELINE config 1 at full size
    "cfg1": dict(B=2, H=8, G=2, T=512, dk=64, dv=64, d_model=512, l=32, d=16, l_prime=64, n=16, w=256, seed=0),
    # small odd-sized case: non power-of-two T, rows before the first compressed block, n < blocks
    "small": dict(B=1, H=4, G=2, T=200, dk=32, dv=16, d_model=64, l=8, d=4, l_prime=16, n=4, w=24, seed=3),
}


def rows_for(T):
    base = [0, 1, 6, 7, 8, 15, 16, 23, 24, 30, 31, 32, 47, 63, 64, 65, 127, 128, 199, 255, 256, 257, 300, 383, 511]
    return sorted({t for t in base if t < T} | {T - 1})


def run_case(name, c, K, R):
    torch.manual_seed(0)
    inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=c["seed"],
                        l_prime=c["l_prime"])
    cfg = K.NSAConfig(d_model=c["d_model"], head_dim_qk=c["dk"], head_dim_v=c["dv"], l=c["l"], d=c["d"],
                      l_prime=c["l_prime"], n=c["n"], w=c["w"], n_heads=c["H"], n_kv_groups=c["G"])
    model = K.NSAAttention(cfg)
    phi, gp = inp["phi"], inp["gate"]
    with torch.no_grad():
        model.pos_embed.weight.copy_(phi.pos_embed)
        model.compress_mlp[0].weight.copy_(phi.w1); model.compress_mlp[0].bias.copy_(phi.b1)
        model.compress_mlp[2].weight.copy_(phi.w2); model.compress_mlp[2].bias.copy_(phi.b2)
        model.gate_mlp[0].weight.copy_(gp.w1); model.gate_mlp[0].bias.copy_(gp.b1)
        model.gate_mlp[2].weight.copy_(gp.w2); model.gate_mlp[2].bias.copy_(gp.b2)
    rows = rows_for(c["T"])
    out = {"rows": np.array(rows)}
    q = inp["q"].clone().requires_grad_(True)
    k = inp["k"].clone().requires_grad_(True)
    v = inp["v"].clone().requires_grad_(True)
    do = inp["do"]
    scale = 1.0 / c["dk"] ** 0.5

    def grads(o):
        gq, gk, gv = torch.autograd.grad(o, (q, k, v), do, allow_unused=True)
        return gq, gk, gv

    # ---- phi, Eq. 8 (restated from the module's forward), Eq. 9, Eq. 10/11: reference code ----
    with torch.no_grad():
        k_cmp, v_cmp, block_ends, nb = model.compress_tokens(inp["k"].transpose(-1, -2).contiguous(), inp["v"])
        p_cmp = O.compression_probabilities(inp["q"], k_cmp, block_ends, scale)   # pinned by the module run below
        sel = K.derive_selection_from_compression_per_timestep(p_cmp, cfg)
        idx = K.select_top_k_blocks_per_query_with_gqa(sel, cfg)
        idx64 = K.select_top_k_blocks_per_query_with_gqa(
            K.derive_selection_from_compression_per_timestep(
                O.compression_probabilities(inp["q"].double(), k_cmp.double(), block_ends, scale), cfg), cfg)
    out.update(k_cmp=k_cmp.numpy(), v_cmp=v_cmp.numpy(), block_ends=block_ends.numpy(), n_blocks=np.array(nb),
               sel_rows=sel[:, :, rows].numpy(), indices=idx.numpy().astype(np.int32),
               indices_fp64=idx64.numpy().astype(np.int32))

    # ---- the three branches: reference.py forward + autograd backward ----
    o = R.sliding_window_attention(q, k, v, c["w"], scale)
    gq, gk, gv = grads(o)
    out.update(win_o=o.detach()[:, :, rows].numpy(), win_dq=gq[:, :, rows].numpy(),
               win_dk=gk[..., rows].numpy(), win_dv=gv[:, :, rows].numpy())
    kc = k_cmp.clone().requires_grad_(True)
    vc = v_cmp.clone().requires_grad_(True)
    o = R.compression_attention(q, kc, vc, block_ends, scale)
    gq, gkc, gvc = torch.autograd.grad(o, (q, kc, vc), do)
    out.update(cmp_o=o.detach()[:, :, rows].numpy(), cmp_dq=gq[:, :, rows].numpy(),
               cmp_dk=gkc.numpy(), cmp_dv=gvc.numpy())
    idx_fb = O.selection_fallback_indices(idx, c["l_prime"])
    o = R.selection_attention_reference(q, k, v, idx_fb, c["l_prime"], scale)
    gq, gk, gv = grads(o)
    out.update(slc_o=o.detach()[:, :, rows].numpy(), slc_dq=gq[:, :, rows].numpy(),
               slc_dk=gk[..., rows].numpy(), slc_dv=gv[:, :, rows].numpy())

    # ---- whole module, eval mode = the reference's CPU path (float64 branches) ----
    model.eval()
    proj = O.draw_projection_weights(c["seed"] + 11, c["d_model"], c["H"], c["G"], c["dk"], c["dv"])
    with torch.no_grad():
        for pname, wt in proj.items():
            getattr(model, pname).weight.copy_(wt)
    g = torch.Generator().manual_seed(c["seed"] + 7)
    hidden = torch.randn(c["B"], c["T"], c["d_model"], generator=g) * 0.5
    with torch.no_grad():
        y, info = model(hidden, output_attentions=True)
    torch.use_deterministic_algorithms(False)
    out.update(mod_y=y[:, rows].numpy(), mod_indices=info["selected_indices"].numpy().astype(np.int32),
               mod_gates=info["gates"][:, rows].numpy(),
               mod_p_cmp=info["compression_scores"][:, :, rows].numpy(),
               mod_sel=info["selection_scores"][:, :, rows].numpy())
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    return {k_: list(np.asarray(v_).shape) for k_, v_ in out.items()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of the reference project (Noumena-Network/NSA-Test)")
    args = ap.parse_args()
    K, R = load_reference(args.reference)
    meta = {"torch": torch.__version__, "cases": CASES, "shapes": {}}
    for name, c in CASES.items():
        meta["shapes"][name] = run_case(name, c, K, R)
        print("wrote", name)
    with open(os.path.join(HERE, "golden_meta.json"), "w") as f:
        json.dump(meta, f, indent=1)


if __name__ == "__main__":
    main()
