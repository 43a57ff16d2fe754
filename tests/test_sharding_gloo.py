"""World-size-2 CPU (gloo) test of the multi-rank host logic: batch sharding + one all-reduce of the
compression-MLP / gate-MLP weight gradients reproduces the single-process gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nsa_oracle as O

CFG = dict(B=2, H=4, G=2, T=96, dk=16, dv=16, d_model=32, l=8, d=4, l_prime=16, n=4, w=24)


def _weight_grads(inp, b0, b1):
    c = CFG
    phi, gp = inp["phi"], inp["gate"]
    ws = [p.clone().requires_grad_(True) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2, gp.w1, gp.b1, gp.w2, gp.b2)]
    r = O.nsa_layer(inp["q"][b0:b1], inp["k"][b0:b1], inp["v"][b0:b1], inp["x"][b0:b1], O.PhiParams(*ws[:5]), O.GateParams(*ws[5:]),
                    l=c["l"], d=c["d"], l_prime=c["l_prime"], n=c["n"], w=c["w"])
    return torch.autograd.grad(r["out"], ws, inp["do"][b0:b1])


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nsa.sharding import allreduce_grads, batch_shard
        c = CFG
        inp = O.make_inputs(c["B"], c["H"], c["G"], c["T"], c["dk"], c["dv"], c["d_model"], c["l"], seed=5, l_prime=c["l_prime"])
        b0, b1 = batch_shard(c["B"], world, rank)
        summed = allreduce_grads(_weight_grads(inp, b0, b1))
        if rank == 0:
            full = _weight_grads(inp, 0, c["B"])
            # index 4 is the second phi bias, whose true gradient is zero (softmax is shift invariant): skip it
            ret["err"] = max(((a - b).abs().max() / (b.abs().max() + 1e-12)).item()
                             for i, (a, b) in enumerate(zip(summed, full)) if i != 4)
    finally:
        dist.destroy_process_group()


def test_batch_shard_bounds():
    from nsa.sharding import batch_shard
    assert [batch_shard(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert [batch_shard(5, 2, r) for r in range(2)] == [(0, 3), (3, 5)]
    assert batch_shard(1, 2, 1) == (1, 1)
    with pytest.raises(ValueError):
        batch_shard(4, 2, 2)


def test_two_rank_weight_gradient_allreduce():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["err"] < 1e-5


def _gather_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nsa.sharding import all_gather_seq, query_shard
        T, step = 512, 256
        g = torch.Generator().manual_seed(9)
        full = torch.randn(2, 3, T, generator=g)
        wgt = torch.randn(2, 3, T, generator=g) * (rank + 1)       # each rank's loss weighs the gathered tensor differently
        t0, t1 = query_shard(T, world, rank)
        x = full[..., t0:t1].clone().requires_grad_(True)
        y = all_gather_seq(x, -1)
        # uneven slices (work-balanced long-context split) travel padded
        bounds = [0, 384, 512]
        xu = full[..., bounds[rank]:bounds[rank + 1]].clone().requires_grad_(True)
        yu = all_gather_seq(xu, -1, None, [384, 128])
        (yu * wgt).sum().backward()
        (y * wgt).sum().backward()
        ok_fwd = torch.equal(y.detach(), full)
        g2 = torch.Generator().manual_seed(9)
        torch.randn(2, 3, T, generator=g2)
        base = torch.randn(2, 3, T, generator=g2)
        want = base * sum(r + 1 for r in range(world))              # gradient summed over the ranks' losses
        ok_fwd = ok_fwd and torch.equal(yu.detach(), full)
        err_u = (xu.grad - want[..., bounds[rank]:bounds[rank + 1]]).abs().max().item()
        # an upstream gradient whose last two dimensions are swapped in memory (how dK reaches the exchange: the transposed
        # view of a time-major buffer): the reduce-scatter works in that layout and hands back a view of the same kind
        xs = full[..., bounds[rank]:bounds[rank + 1]].clone().requires_grad_(True)
        ys = all_gather_seq(xs, -1, None, [384, 128])
        g_tm = (wgt.transpose(-1, -2).contiguous()).transpose(-1, -2)       # values of wgt, time-major memory
        assert not g_tm.is_contiguous() and g_tm.transpose(-1, -2).is_contiguous()
        torch.autograd.backward([ys], [g_tm])
        err_s = (xs.grad - want[..., bounds[rank]:bounds[rank + 1]]).abs().max().item()
        ret[rank] = (ok_fwd, max((x.grad - want[..., t0:t1]).abs().max().item(), err_u, err_s), (t1 - t0) == step)
    finally:
        dist.destroy_process_group()


def test_balanced_query_bounds():
    from nsa.sharding import balanced_query_bounds
    b = balanced_query_bounds(65536, 8, 512 + 16 * 64, 16)
    assert b[0] == 0 and b[-1] == 65536 and all(x % 128 == 0 for x in b) and all(y > x for x, y in zip(b, b[1:]))
    cost = lambda lo, hi: sum(1536 + t / 16 for t in range(lo, hi, 64)) * 64
    works = [cost(lo, hi) for lo, hi in zip(b, b[1:])]
    assert max(works) / min(works) < 1.05          # equal work within the tile rounding
    assert (b[1] - b[0]) > 2 * (b[-1] - b[-2])     # early slices are much longer than late ones
    with pytest.raises(ValueError):
        balanced_query_bounds(256, 4, 100.0, 16)


def test_query_shard_bounds():
    from nsa.sharding import query_shard
    assert [query_shard(1024, 4, r) for r in range(4)] == [(0, 256), (256, 512), (512, 768), (768, 1024)]
    with pytest.raises(ValueError):
        query_shard(1000, 4, 0)
    with pytest.raises(ValueError):
        query_shard(512, 8, 0)      # 64-row slices are not whole query tiles


def test_two_rank_sequence_all_gather_and_gradient_reduce_scatter():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_gather_worker, args=(2, port, ret), nprocs=2, join=True)
    for r in range(2):
        ok_fwd, err, ok_len = ret[r]
        assert ok_fwd and ok_len and err < 1e-5


def _compress_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nsa.sharding import all_gather_seq, owned_block_range, sharded_compress
        B, G, T, dk, dv, l, d = 1, 2, 256, 16, 8, 32, 16
        inp = O.make_inputs(B, 4, G, T, dk, dv, 32, l, seed=3)
        phi = inp["phi"]
        bounds = [0, 160, 256]                                  # uneven slices; 160 is a multiple of the stride
        sizes = [bounds[i + 1] - bounds[i] for i in range(world)]
        t0, t1 = bounds[rank], bounds[rank + 1]
        k_loc = inp["k"][..., t0:t1].clone().requires_grad_(True)
        v_loc = inp["v"][:, :, t0:t1].clone().requires_grad_(True)
        k_full = all_gather_seq(k_loc, -1, None, sizes)
        v_full = all_gather_seq(v_loc, 2, None, sizes)
        fn = lambda keys, values: O.compress_tokens(keys, values, phi, l, d)[:2]
        k_cmp, v_cmp = sharded_compress(k_full, v_full, fn, bounds, rank, l, d)
        nb = (T - l) // d + 1
        gen = torch.Generator().manual_seed(17)
        wk, wv = torch.randn(B, G, dk, nb, generator=gen), torch.randn(B, G, nb, dv, generator=gen)
        ((k_cmp * wk).sum() * (rank + 1) + (v_cmp * wv).sum() * (rank + 1)).backward()   # every rank's loss weighs differently
        # single-process reference of the summed losses
        kr, vr = inp["k"].clone().requires_grad_(True), inp["v"].clone().requires_grad_(True)
        kc_ref, vc_ref, _, nb_ref = O.compress_tokens(kr.transpose(-1, -2), vr, phi, l, d)
        tot = sum(r + 1 for r in range(world))
        ((kc_ref[..., :nb] * wk).sum() * tot + (vc_ref[:, :, :nb] * wv).sum() * tot).backward()
        ret[rank] = dict(
            shape=tuple(k_cmp.shape) == (B, G, dk, nb) and tuple(v_cmp.shape) == (B, G, nb, dv) and nb == nb_ref,
            fwd=max((k_cmp.detach() - kc_ref.detach()[..., :nb]).abs().max().item(), (v_cmp.detach() - vc_ref.detach()[:, :, :nb]).abs().max().item()),
            gk=(k_loc.grad - kr.grad[..., t0:t1]).abs().max().item() / kr.grad.abs().max().item(),
            gv=(v_loc.grad - vr.grad[:, :, t0:t1]).abs().max().item() / vr.grad.abs().max().item(),
            owned=owned_block_range(bounds, rank, l, d, T))
    finally:
        dist.destroy_process_group()


def test_two_rank_split_compression_matches_the_whole_sequence():
    """Long-context mode: every rank compresses the blocks that start in its slice (reaching l - d tokens into the next
    one), the compressed keys/values are all-gathered, and their gradients return through a reduce-scatter and the
    owners' phi backward into the gradient of the gathered K/V."""
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_compress_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0]["owned"] == (0, 10) and ret[1]["owned"] == (10, 15)
    for r in range(2):
        assert ret[r]["shape"] and ret[r]["fwd"] < 1e-6 and ret[r]["gk"] < 1e-5 and ret[r]["gv"] < 1e-5, dict(ret[r])


def test_owned_block_ranges_cover_every_block_once():
    from nsa.sharding import balanced_query_bounds, owned_block_range
    T, l, d = 65536, 32, 16
    b = balanced_query_bounds(T, 8, 512 + 16 * 64, d)
    r = [owned_block_range(b, i, l, d, T) for i in range(8)]
    assert r[0][0] == 0 and r[-1][1] == (T - l) // d + 1 and all(x[1] == y[0] for x, y in zip(r, r[1:]))
    with pytest.raises(ValueError):
        owned_block_range([0, 100, 256], 0, l, d, 256)
