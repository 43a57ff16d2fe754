"""Checks that stand in for a memory checker and a fault injector, which are not available where these kernels run:

* guard bands: every tensor and scratch buffer the wrappers allocate is placed between two 4 KiB bands of a known
  byte pattern, the kernels run, and the bands must come back untouched (an out-of-bounds WRITE of any kernel shows
  here instead of corrupting a neighbour);
* the bounded waits: a self-test kernel lets a wait run out (a barrier nothing arrives at, a limit of 2^16 clocks);
  the library must come back, count the time-out, refuse further work with an error status, and work again after
  the condition has been acknowledged.  Nothing here faults, traps or spins without a limit.
"""
import contextlib

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
HALO = 4096
PATTERN = 0xA5


class _GuardedTorch:
    """Stand-in for the ``torch`` module inside nsa.ops: allocations come with guard bands; the rest passes through."""

    def __init__(self):
        self.bands = []

    def __getattr__(self, name):
        return getattr(torch, name)

    def _alloc(self, shape, dtype, device):
        shape = tuple(int(s) for s in shape)
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        pad = (-nbytes) % 256
        raw = torch.full((HALO + nbytes + pad + HALO,), PATTERN, dtype=torch.uint8, device=device)
        self.bands.append((raw, nbytes))
        return raw[HALO:HALO + nbytes].view(dtype).view(shape)

    @staticmethod
    def _shape(args):
        return tuple(args[0]) if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)) else args

    def empty(self, *shape, device=None, dtype=torch.float32, **kw):
        return self._alloc(self._shape(shape), dtype, device)

    def zeros(self, *shape, device=None, dtype=torch.float32, **kw):
        return self._alloc(self._shape(shape), dtype, device).zero_()

    def empty_like(self, t, **kw):
        return self._alloc(t.shape, t.dtype, t.device)

    def check(self):
        torch.cuda.synchronize()
        for i, (raw, nbytes) in enumerate(self.bands):
            lo, hi = raw[:HALO], raw[HALO + nbytes:]
            assert bool((lo == PATTERN).all()), f"allocation {i} ({nbytes} bytes): bytes written BEFORE the buffer"
            assert bool((hi == PATTERN).all()), f"allocation {i} ({nbytes} bytes): bytes written AFTER the buffer"
        return len(self.bands)


@contextlib.contextmanager
def guard_bands():
    from nsa import ops
    g = _GuardedTorch()
    real = ops.torch
    ops.torch = g
    try:
        yield g
    finally:
        ops.torch = real


def _idx(B, G, T, n, gen):
    nblk = T // 64
    idx = torch.randint(0, nblk, (B, G, T, n), generator=gen)
    t = torch.arange(T)
    idx = torch.minimum(idx, (t // 64).view(1, 1, T, 1).expand_as(idx))
    idx[..., 0] = 0
    idx[..., 1] = (t // 64).view(1, 1, T)
    idx[..., -1] = -1
    return idx.to(torch.int32)


@pytest.mark.parametrize("dk,dv,H,G,T,n", [(192, 128, 16, 1, 1024, 16), (64, 64, 8, 2, 512, 6), (128, 128, 4, 1, 384, 4)])
def test_tensor_core_kernels_stay_inside_their_buffers(dk, dv, H, G, T, n):
    from nsa import ops
    from nsa._lib import lib
    gen = torch.Generator().manual_seed(31)
    B = 2
    rnd = lambda *s: torch.randn(*s, generator=gen).bfloat16().to(DEV)
    q, k, v, do = rnd(B, H, T, dk), rnd(B, G, dk, T), rnd(B, G, T, dv), rnd(B, H, T, dv)
    idx = _idx(B, G, T, n, gen).to(DEV)
    l, d = 32, 16
    nb = (T - l) // d + 1
    nbp = max(128, 1 << (nb - 1).bit_length())
    kc = torch.zeros(B, G, dk, nbp, device=DEV)
    kc[..., :nb] = torch.randn(B, G, dk, nb, generator=gen).to(DEV) * 0.1
    vc = torch.zeros(B, G, nbp, dv, device=DEV, dtype=torch.bfloat16)
    vc[:, :, :nb] = rnd(B, G, nb, dv)
    be = torch.full((nbp,), 999999, dtype=torch.int32, device=DEV)
    be[:nb] = torch.arange(nb, dtype=torch.int32, device=DEV) * d + l - 1
    scale = dk ** -0.5
    with guard_bands() as g:
        o, L, M = ops.sliding_fwd(q, k, v, 200, scale)
        ops.sliding_bwd(q, k, v, o, do, L, M, 200, scale)
        o, L, M = ops.cmp_attn_fwd(q, kc.bfloat16(), vc, be, scale, blocks=(l, d, nb))
        ops.cmp_attn_bwd(q, kc.bfloat16(), vc, be, o, do, L, M, scale, blocks=(l, d, nb))
        o, L, M = ops.slc_fwd(q, k, v, idx, 64, scale)
        ops.slc_bwd(q, k, v, idx, o, do, L, M, 64, scale, dq_addends=(torch.zeros_like(q), torch.zeros_like(q)))
        ops.score_topn(q, kc, be, l, d, 64, n, 3, scale, n_real_blocks=nb)
        lg = torch.randn(B, T, 3 * H, generator=gen).to(DEV)
        out, gates = ops.gate_mix_fwd(lg, o, o, o, "sigmoid")
        ops.gate_mix_bwd(gates, o, o, o, do, "sigmoid", want_delta=True)
        count = g.check()
    assert count >= 25
    assert lib.nsa_device_timeouts(0) == 0


def test_whole_layer_stays_inside_its_buffers():
    """The layer as the benchmark runs it (bf16, one autograd node for the three branches), every allocation of the
    wrappers guarded, including the stride-generic kernels on a second, ragged fp32 shape."""
    import nsa
    import nsa.kernels as K
    from nsa.kernels import nsa_layer
    from oracle import nsa_oracle as O
    # composed from the branch entry points (every tensor and scratch buffer is an allocation of its own, each guarded),
    # then as the single library call each way (context and workspace guarded as wholes)
    for use_c, (T, dk, dv, H, G, dtype) in [(u, s_) for u in (False, True)
                                            for s_ in [(1024, 192, 128, 16, 1, torch.bfloat16), (333, 48, 80, 6, 3, torch.float32)]]:
        K._USE_C_LAYER = use_c
        inp = O.make_inputs(1, H, G, T, dk, dv, 32, 32, seed=7, block_offset_std=0.5, dtype=dtype)
        cfg = nsa.NSAConfig(d_model=32, head_dim_qk=dk, head_dim_v=dv, l=32, d=16, l_prime=64, n=16, w=100, n_heads=H, n_kv_groups=G)
        q, k, v = (inp[x].to(DEV, dtype).requires_grad_(True) for x in ("q", "k", "v"))
        phi = inp["phi"]
        params = tuple(p.to(DEV).requires_grad_(True) for p in (phi.pos_embed, phi.w1, phi.b1, phi.w2, phi.b2))
        logits = torch.randn(1, T, 3 * H, device=DEV, requires_grad=True)
        try:
            with guard_bands() as g:
                out = nsa_layer(q, k, v, logits, params, cfg)
                torch.autograd.grad(out, [q, k, v, logits] + list(params), inp["do"].to(DEV, dtype))
                assert g.check() >= (8 if use_c else 30)
        finally:
            K._USE_C_LAYER = True


def test_a_wait_that_runs_out_is_reported_and_refused_until_acknowledged():
    from nsa import ops
    from nsa._lib import NSAKernelError, lib
    import ctypes
    gen = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(*s, generator=gen).bfloat16().to(DEV) for s in [(1, 4, 256, 64), (1, 2, 64, 256), (1, 2, 256, 64)])
    good, _, _ = ops.sliding_fwd(q, k, v, 100, 0.125)           # healthy call; sets up this device's time-out record
    torch.cuda.synchronize()
    assert lib.nsa_device_timeouts(1) == 0
    try:
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert lib.nsa_selftest_wait_timeout(1 << 16, st) == 0, lib.nsa_last_error().decode()   # returns: the wait gave up
        assert lib.nsa_device_timeouts(0) == 1
        with pytest.raises(NSAKernelError, match="time-out"):
            ops.sliding_fwd(q, k, v, 100, 0.125)                # refused with an error status, not silently skipped
        with pytest.raises(NSAKernelError, match="time-out"):
            ops.score_topn(q, torch.zeros(1, 2, 64, 128, device=DEV), torch.zeros(128, dtype=torch.int32, device=DEV), 32, 16, 64,
                           4, 3, 0.125)
    finally:
        assert lib.nsa_device_timeouts(1) >= 0                  # acknowledge: clears counter and flag
    assert lib.nsa_device_timeouts(0) == 0
    again, _, _ = ops.sliding_fwd(q, k, v, 100, 0.125)
    torch.cuda.synchronize()
    assert torch.equal(again, good)
    assert lib.nsa_selftest_wait_timeout(0, None) == -1 and lib.nsa_selftest_wait_timeout(1 << 30, None) == -1
