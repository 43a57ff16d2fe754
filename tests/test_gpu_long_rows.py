"""Long sequences at the benchmarked head configuration (H=64, G=4, dk=192, dv=128, bf16, keys with per-block
offsets): the CUDA forward path against the oracle on sampled query rows.

The dense oracle functions cannot hold a [T,T] score matrix at T=32768 or 65536, so the oracle is evaluated row by
row (oracle.branch_rows / score_rows, which follow the reference's own per-token loops) on a sample of positions
that contains the boundary rows of every branch.  Compressed keys are compared in full; block ids on the sampled rows
(bit-exact outside the ambiguity set, counts logged); O_cmp and O_win on every sampled row; O_slc on every sampled
row too, the oracle attending the blocks the CUDA path selected (so a near-tie in the ranking cannot hide an error in
the attention).  BASELINE config 3 is the first case (B=2, T=32768), the benchmark's sequence the second.
"""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.util import close, index_agreement, rel_err, sample_positions

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.timeout(1500)
@pytest.mark.parametrize("B,T,rows", [(2, 32768, 256), (1, 65536, 256)])
def test_sampled_rows_of_long_sequences(B, T, rows):
    import nsa
    from nsa.kernels import nsa_layer
    from nsa._lib import lib
    H, G, dk, dv, l, d, lp, n, w = 64, 4, 192, 128, 32, 16, 64, 16, 512
    where = f"sampled rows B={B} T={T}"
    inp = O.make_inputs(B, H, G, T, dk, dv, 64, l, seed=3, block_offset_std=0.5, l_prime=lp, dtype=torch.bfloat16)
    cfg = nsa.NSAConfig(d_model=64, head_dim_qk=dk, head_dim_v=dv, l=l, d=d, l_prime=lp, n=n, w=w, n_heads=H, n_kv_groups=G)
    phi = inp["phi"]
    params = tuple(p.to(DEV) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2))
    logits = torch.zeros(B, T, 3 * H, device=DEV)
    with torch.no_grad():
        _, info = nsa_layer(inp["q"].bfloat16().to(DEV), inp["k"].bfloat16().to(DEV), inp["v"].bfloat16().to(DEV), logits,
                            params, cfg, return_info=True)
    torch.cuda.synchronize()
    assert lib.nsa_device_timeouts(0) == 0
    pos = sample_positions(T, rows, l, w, lp, n, seed=T)
    assert len(pos) >= 64
    got = {k_: info[k_][:, :, pos.to(DEV)].cpu() for k_ in ("indices", "o_cmp", "o_slc", "o_win")}
    k_cmp_gpu, v_cmp_gpu = info["k_cmp"].cpu(), info["v_cmp"].float().cpu()
    del info
    torch.cuda.empty_cache()

    scale = dk ** -0.5
    k_cmp, v_cmp, be, nb = O.compress_tokens(inp["k"].transpose(-1, -2), inp["v"], phi, l, d)
    assert rel_err(k_cmp_gpu, k_cmp) < 1e-4, "compressed keys (they decide the top-n) differ from the oracle's"
    assert rel_err(v_cmp_gpu, v_cmp) < 1e-2
    qr = inp["q"][:, :, pos]
    idx_ref, agg = O.score_rows(qr, pos, k_cmp, be, l=l, d=d, l_prime=lp, n=n, scale=scale)
    mism = index_agreement(where, got["indices"], idx_ref, agg, n)
    assert mism.float().mean() < 0.02
    # early rows list the forced blocks first, then never-visible blocks in id order
    assert got["indices"][0, 0, 0].tolist()[:3] == [0, 1, 2]
    o_cmp, o_slc, o_win = O.branch_rows(qr, pos, inp["k"], inp["v"], k_cmp, v_cmp, be, got["indices"].long(), w=w, l_prime=lp,
                                        scale=scale)
    close(where, "o_cmp", got["o_cmp"], o_cmp, bf16=True)
    close(where, "o_win", got["o_win"], o_win, bf16=True)
    close(where, "o_slc (oracle attends the blocks the CUDA path chose)", got["o_slc"], o_slc, bf16=True)
