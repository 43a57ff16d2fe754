"""Query-sharded long-context mode: a query slice at positions q_pos0 + [0, Tq) against keys from position 0 must
reproduce the corresponding rows of the unsharded layer, and the slices' K/V and weight gradients must add up to the
unsharded ones (what the all-gather / reduce-scatter of `nsa.sharding.query_sharded_layer` exchanges between ranks).
The ranks are emulated one after the other on one GPU."""
import pytest
import torch

from tests.util import max_abs

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _setup(H, G, T, dk, dv, d_model, seed):
    from oracle import nsa_oracle as O
    inp = O.make_inputs(1, H, G, T, dk, dv, d_model, 32, seed=seed, block_offset_std=0.5, dtype=torch.bfloat16)
    q, k, v = (inp[n].bfloat16().to(DEV) for n in ("q", "k", "v"))
    g = torch.Generator().manual_seed(seed + 1)
    logits = torch.randn(1, T, 3 * H, generator=g).to(DEV)
    do = torch.randn(1, H, T, dv, generator=g).bfloat16().to(DEV)
    phi = tuple(p.to(DEV).float().requires_grad_(True) for p in (inp["phi"].pos_embed, inp["phi"].w1, inp["phi"].b1,
                                                                  inp["phi"].w2, inp["phi"].b2))
    return q, k, v, logits, do, phi


@pytest.mark.parametrize("dk,dv,H,G,T,world,balanced", [(64, 64, 8, 2, 2048, 2, False), (192, 128, 16, 1, 4096, 4, False),
                                                        (192, 128, 16, 1, 4096, 3, True)])
def test_query_slices_match_the_unsharded_layer(dk, dv, H, G, T, world, balanced):
    import nsa
    from nsa.kernels import nsa_layer
    from nsa._lib import lib
    cfg = nsa.NSAConfig(d_model=64, head_dim_qk=dk, head_dim_v=dv, l=32, d=16, l_prime=64, n=16, w=512, n_heads=H, n_kv_groups=G)
    q, k, v, logits, do, phi = _setup(H, G, T, dk, dv, 64, seed=21)

    def run(q_, logits_, do_, q_pos0):
        ql = q_.detach().requires_grad_(True)
        kl, vl = k.detach().requires_grad_(True), v.detach().requires_grad_(True)
        out, info = nsa_layer(ql, kl, vl, logits_, phi, cfg, return_info=True, q_pos0=q_pos0)
        grads = torch.autograd.grad(out, [ql, kl, vl] + list(phi), do_)
        return out.detach(), info["indices"], [g_.detach().float() for g_ in grads]

    out_full, idx_full, g_full = run(q, logits, do, 0)
    if balanced:
        # the uneven, work-balanced slices of the long-context mode (early ranks get more positions)
        from nsa.sharding import balanced_query_bounds
        bounds = balanced_query_bounds(T, world, 512 + 16 * 64, 16)
        assert len(set(b - a for a, b in zip(bounds, bounds[1:]))) > 1
    else:
        bounds = [r * (T // world) for r in range(world + 1)]
    outs, idxs, dqs = [], [], []
    sums = [torch.zeros_like(g_) for g_ in g_full[1:]]
    for r in range(world):
        sl = slice(bounds[r], bounds[r + 1])
        o_r, i_r, g_r = run(q[:, :, sl].contiguous(), logits[:, sl].contiguous(), do[:, :, sl].contiguous(), bounds[r])
        outs.append(o_r); idxs.append(i_r); dqs.append(g_r[0])
        for acc, g_ in zip(sums, g_r[1:]):
            acc += g_
    torch.cuda.synchronize()
    assert lib.nsa_device_timeouts(0) == 0
    assert torch.equal(torch.cat(idxs, dim=2), idx_full), "selected blocks differ between sharded and unsharded runs"
    assert max_abs(torch.cat(outs, dim=2).float(), out_full.float()) < 2e-2          # bf16 I/O tolerance
    assert max_abs(torch.cat(dqs, dim=2), g_full[0]) < 2e-2
    names = ("dk", "dv", "dpos", "dw1", "db1", "dw2", "db2")
    ref = dict(zip(names, g_full[1:]))
    for name, a, b in zip(names, sums, g_full[1:]):
        # db2 is zero mathematically (a constant added to every compressed key leaves the softmax unchanged): both sides
        # hold rounding noise, compared on the scale of the weight gradient next to it
        scale = max(1.0, (ref["dw2"] if name == "db2" else b).abs().max().item())
        assert max_abs(a, b) < 3e-2 * scale, f"{name}: sharded sum differs by {max_abs(a, b)} (scale {scale})"


def test_generic_scoring_kernel_honours_the_query_offset():
    """fp32 tensors take the row-per-CTA scoring kernel: a query slice with its position offset selects the same blocks
    as the same rows of the whole sequence."""
    from nsa import ops
    from oracle import nsa_oracle as O
    B, H, G, T, dk, l, d, lp, n = 2, 6, 3, 600, 48, 32, 16, 64, 5
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(B, H, T, dk, generator=gen).to(DEV)
    nb = (T - l) // d + 1
    nbp = O.next_pow2(nb)
    kc = torch.zeros(B, G, dk, nbp)
    kc[..., :nb] = torch.randn(B, G, dk, nb, generator=gen)
    kc = kc.to(DEV)
    be = torch.full((nbp,), 999999, dtype=torch.int32)
    be[:nb] = torch.arange(nb, dtype=torch.int32) * d + l - 1
    be = be.to(DEV)
    full = ops.score_topn(q, kc, be, l, d, lp, n, 3, dk ** -0.5)
    for lo, hi in ((0, 100), (100, 357), (357, 600)):
        part = ops.score_topn(q[:, :, lo:hi].contiguous(), kc, be, l, d, lp, n, 3, dk ** -0.5, -1, lo)
        assert torch.equal(part, full[:, :, lo:hi]), f"rows {lo}:{hi}"
