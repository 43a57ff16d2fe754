"""CPU-side checks: the C-ABI library loads and exports what the header declares, the configuration
validates like the reference's, the launcher shims carry the reference's parameter order."""
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    import nsa._lib as L
    header = open(os.path.join(ROOT, "include", "nsa_b200.h")).read()
    declared = set(re.findall(r"NSA_API\s+[\w\s\*]+?\b(nsa_\w+)\s*\(", header))
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(L.lib, name), f"{name} declared in the header but not exported"
    assert declared == set(L.PROTOTYPES), "ctypes prototypes out of sync with the header"
    assert b"sm_100a" in L.lib.nsa_version()


def test_argument_errors_without_a_gpu():
    """Bad arguments are rejected before any CUDA call, with a message."""
    import nsa._lib as L
    rc = L.lib.nsa_sliding_fwd(None, None, None, None, None, None, None, 1, 3, 2, 8, 8, 8, 4, 1.0, 0, 0, None)
    assert rc == -1 and b"H/G" in L.lib.nsa_last_error()
    rc = L.lib.nsa_sliding_fwd(None, None, None, None, None, None, None, 1, 4, 2, 8, 8, 8, 4, 1.0, 0, 0, None)
    assert rc == -1 and b"null" in L.lib.nsa_last_error()
    rc = L.lib.nsa_topn_from_scores(None, None, 1, 4, 2, 8, 8, 2, 100, 0, None)
    assert rc == -1
    assert L.lib.nsa_slc_bwd_workspace_bytes(1, 64, 4, 65536, 65536, 192, 128, 16, 64, 1, 0) > 4 * 65536 * 16 * 4
    # the stride-generic family only needs the inverse index
    assert L.lib.nsa_slc_bwd_workspace_bytes(1, 64, 4, 65536, 65536, 192, 128, 16, 64, 1, L.FLAG_GENERIC) < (1 << 28)


def test_config_defaults_and_validation():
    """Defaults of the paper configuration (nsa/kernels.py:516-591) and the rejected settings."""
    from nsa import NSAConfig
    c = NSAConfig()
    assert (c.d_model, c.head_dim_qk, c.head_dim_v, c.l, c.d, c.l_prime, c.n, c.w) == (2560, 192, 128, 32, 16, 64, 16, 512)
    assert (c.n_heads, c.n_kv_groups, c.n_fixed, c.n_dynamic, c.gate_mode) == (64, 4, 3, 13, "sigmoid")
    assert c.heads_per_group == 16 and c.head_dim_qk_padded == 256 and c.head_dim_v_padded == 128
    c = NSAConfig(include_fixed_in_selection=False)
    assert c.n_fixed == 0 and c.n_dynamic == 16
    for bad in (dict(l=0), dict(l_prime=0), dict(d=0), dict(n=0), dict(w=0), dict(gate_mode="tanh"),
                dict(n_heads=6, n_kv_groups=4), dict(l=24, d=16)):
        with pytest.raises((AssertionError, ValueError)):
            NSAConfig(**bad)


def test_package_surface():
    import nsa
    import nsa.kernels as K
    assert nsa.__version__ == "1.0.0"
    assert set(nsa.__all__) == {"NSAConfig", "NSAAttention", "_nsa_sliding_window_fwd_kernel",
                                "_nsa_sliding_window_bwd_kernel", "_nsa_compression_fwd_kernel",
                                "_nsa_compression_bwd_kernel", "_nsa_sparse_selection_fwd_kernel",
                                "_nsa_sparse_selection_bwd_kernel"}
    for n in ("CompressionAttention", "SelectionAttention", "SlidingWindowAttention",
              "derive_selection_from_compression_per_timestep", "select_top_k_blocks_per_query_with_gqa"):
        assert hasattr(K, n)
    # positional parameter counts of the six reference kernels (nsa/kernels.py:595, 837, 1152, 1304, 1534, 1691)
    counts = {"_nsa_sparse_selection_fwd_kernel": 34, "_nsa_sparse_selection_bwd_kernel": 50,
              "_nsa_sliding_window_fwd_kernel": 29, "_nsa_sliding_window_bwd_kernel": 45,
              "_nsa_compression_fwd_kernel": 30, "_nsa_compression_bwd_kernel": 46}
    for n, cnt in counts.items():
        assert len(getattr(nsa, n).positional) == cnt, n
    assert nsa._nsa_sliding_window_fwd_kernel.positional[:9] == ["Q", "K", "V", "Out", "sm_scale", "L", "M", "stride_qz", "stride_qh"]
    assert nsa._nsa_sliding_window_fwd_kernel.positional[11:15] == ["stride_kz", "stride_kg", "stride_kn", "stride_kk"]


def test_module_parameter_names_match_reference_state_dict():
    from nsa import NSAAttention, NSAConfig
    m = NSAAttention(NSAConfig(d_model=64, head_dim_qk=16, head_dim_v=16, n_heads=4, n_kv_groups=2, l=8, d=4, l_prime=8, n=4, w=8))
    names = set(m.state_dict())
    expect = {f"{p}.weight" for p in ("q_proj", "k_compress", "v_compress", "k_select", "v_select", "k_sliding", "v_sliding",
                                      "pos_embed", "compress_mlp.0", "compress_mlp.2", "gate_mlp.0", "gate_mlp.2", "o_proj")}
    expect |= {f"{p}.bias" for p in ("compress_mlp.0", "compress_mlp.2", "gate_mlp.0", "gate_mlp.2")}
    assert names == expect
    with pytest.raises(RuntimeError):      # no CPU path
        m(torch.zeros(1, 16, 64))


def test_reference_helpers():
    from nsa.reference import compare_outputs, create_block_ends
    assert create_block_ends(64, 8, 8, device="cpu").tolist() == list(range(7, 64, 8))
    assert create_block_ends(20, 8, 4, device="cpu").tolist() == [7, 11, 15, 19]
    ok, _ = compare_outputs(torch.ones(3), torch.ones(3))
    assert ok


def test_library_keeps_no_call_pairing_state():
    """Query offset, row sums and dQ addends travel in the argument lists: no setter is exported."""
    import nsa._lib as L
    for gone in ("nsa_set_query_offset", "nsa_set_row_delta", "nsa_set_dq_addends", "nsa_set_kernel_family"):
        assert not hasattr(L.lib, gone), gone


def test_launcher_checks_every_tensor_before_launching():
    """The launcher shims refuse, before any launch, strides that would make a kernel write past a tensor, negative
    strides, and serve over-reaching read-only tensors from a padded copy."""
    from nsa.kernels import _Launcher
    t = torch.zeros(2, 3, 8, 4)
    assert _Launcher._extent("t", t.stride(), t.shape) == t.numel()
    assert _Launcher._fits("t", t, t.stride(), t.shape) is t
    with pytest.raises(ValueError, match="storage holds"):
        _Launcher._fits("dK", t, (192, 64, 8, 1), (2, 3, 8, 8))         # strides of a tensor twice as wide
    with pytest.raises(ValueError, match="negative"):
        _Launcher._fits("Out", t, (96, 32, -4, 1), t.shape)
    wide = _Launcher._safe("K", t, (192, 64, 8, 1), (2, 3, 8, 8))       # read-only: padded copy, original values first
    assert wide.numel() >= _Launcher._extent("K", (192, 64, 8, 1), (2, 3, 8, 8)) and wide is not t
    assert _Launcher._fits("K^T", t, (96, 32, 1, 4), (2, 3, 4, 8)) is t   # a transposed view stays inside the storage
    assert _Launcher._safe("K", t, t.stride(), t.shape) is t
    view = t[:, :, 2:]                                                   # storage offset counts against the room left
    with pytest.raises(ValueError):
        _Launcher._fits("dQ", view, t.stride(), t.shape)
