"""The workspace-free sliding-window backward (nsa_sliding_bwd_noalloc) against the regular entry point.

Some callers of the library cannot allocate device memory when they need a backward pass (inside a graph
capture, under a runtime that owns all memory, in a loop that must stay off the allocator); for them the
library carries its own fixed scratch array.  This test calls the entry point straight through the C ABI,
twice in a row (all calls share the one array and it keeps the previous call's contents), and expects the
gradients of nsa_sliding_bwd bit for bit: both run the same kernels.  It lives in the file pytest collects
last, so a run that stops at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _call_noalloc(lib, q, k, v, o, do, L, M, window, scale):
    B, H, T, dk = q.shape
    G, dv = k.shape[1], v.shape[-1]
    dq = torch.empty_like(q)
    dkey = torch.zeros(B, G, T, dk, device=DEV, dtype=q.dtype)
    dval = torch.zeros(B, G, T, dv, device=DEV, dtype=q.dtype)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.nsa_sliding_bwd_noalloc(p(q), p(k), p(v), p(o), p(do), p(L), p(M), p(dq), p(dkey), p(dval), B, H, G, T, dk, dv,
                                     window, scale, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, (dq, dkey, dval)


def test_noalloc_sliding_backward_matches_workspace_version():
    from nsa import ops
    from nsa._lib import lib
    gen = torch.Generator().manual_seed(21)
    outs = []
    for (B, H, G, T, dk, dv, w) in [(2, 4, 2, 512, 64, 64, 200), (1, 4, 1, 1024, 192, 128, 512)]:   # two calls in a row
        q, k, v, do = (torch.randn(*s, generator=gen).bfloat16().to(DEV) for s in
                       [(B, H, T, dk), (B, G, dk, T), (B, G, T, dv), (B, H, T, dv)])
        scale = dk ** -0.5
        o, L, M = ops.sliding_fwd(q, k, v, w, scale)
        ref = ops.sliding_bwd(q, k, v, o, do, L, M, w, scale)
        rc, got = _call_noalloc(lib, q, k, v, o, do, L, M, w, scale)
        assert rc == 0, lib.nsa_last_error().decode()
        torch.cuda.synchronize()
        for a, b_, name in zip(got, ref, ("dq", "dk", "dv")):
            assert torch.isfinite(a.float()).all(), name
            assert (a.float() - b_.float()).abs().max().item() <= 2e-2 * max(1.0, b_.float().abs().max().item()), name
            assert torch.equal(a, b_), f"{name}: same kernels, expected identical bits"
        outs.append(got)
    assert lib.nsa_device_timeouts(0) == 0


def test_noalloc_rejects_what_it_cannot_hold():
    from nsa._lib import lib
    z = torch.zeros(16, device=DEV, dtype=torch.bfloat16)
    f = torch.zeros(16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 64 heads x 32768 queries = 2,097,152 rows: twice the built-in scratch -> refused before any launch
    rc = lib.nsa_sliding_bwd_noalloc(p(z), p(z), p(z), p(z), p(z), p(f), p(f), p(z), p(z), p(z), 1, 64, 4, 32768, 192, 128, 512, 0.07, st)
    assert rc == -4 and b"exceed" in lib.nsa_last_error()
    # a shape outside the tensor-core kernels (T not a multiple of 128) is pointed to the regular entry point
    rc = lib.nsa_sliding_bwd_noalloc(p(z), p(z), p(z), p(z), p(z), p(f), p(f), p(z), p(z), p(z), 1, 4, 2, 100, 64, 64, 16, 0.1, st)
    assert rc == -4 and b"nsa_sliding_bwd" in lib.nsa_last_error()


@pytest.mark.timeout(600)
def test_noalloc_at_the_limit_and_after_it():
    """Exactly 2^20 rows fill the built-in scratch to its last element; a smaller call right after it finds the large
    call's values in the array and must not be affected by them; one tile more per head is refused."""
    from nsa import ops
    from nsa._lib import lib
    gen = torch.Generator(device=DEV).manual_seed(22)

    def case(B, H, G, T, dk, dv, w):
        q, k, v, do = (torch.randn(*s, generator=gen, device=DEV).bfloat16() for s in
                       [(B, H, T, dk), (B, G, dk, T), (B, G, T, dv), (B, H, T, dv)])
        scale = dk ** -0.5
        o, L, M = ops.sliding_fwd(q, k, v, w, scale)
        ref = ops.sliding_bwd(q, k, v, o, do, L, M, w, scale)
        rc, got = _call_noalloc(lib, q, k, v, o, do, L, M, w, scale)
        assert rc == 0, lib.nsa_last_error().decode()
        torch.cuda.synchronize()
        for a, b_, name in zip(got, ref, ("dq", "dk", "dv")):
            assert torch.equal(a, b_), f"{name} at B*H*T = {B * H * T}"

    case(1, 16, 8, 65536, 64, 64, 512)            # 16 * 65536 = 1,048,576 rows: the limit itself
    case(2, 4, 2, 512, 64, 64, 200)               # stale scratch from the large call is harmless
    z = torch.zeros(16, device=DEV, dtype=torch.bfloat16)
    f = torch.zeros(16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.nsa_sliding_bwd_noalloc(p(z), p(z), p(z), p(z), p(z), p(f), p(f), p(z), p(z), p(z), 1, 16, 8, 65536 + 128, 64, 64, 512,
                                     0.125, st)
    assert rc == -4 and b"exceed" in lib.nsa_last_error()
    assert lib.nsa_device_timeouts(0) == 0
