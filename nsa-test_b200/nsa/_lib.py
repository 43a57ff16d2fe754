"""ctypes binding of libnsa_b200.so, the C-ABI library of the sm_100a kernels (include/nsa_b200.h).

There is no fallback of any kind: if the shared library is missing, importing this module raises,
and every wrapper raises on tensors that are not on a CUDA device.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p, POINTER

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnsa_b200.so")

F32, BF16 = 0, 1
GATE_SIGMOID, GATE_SOFTMAX = 0, 1
FLAG_GENERIC, FLAG_RECOMPUTE = 1, 2

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first (python nsa-test_b200/build.py, or "
        "__graft_entry__.build()).  This package has no CPU or PyTorch fallback."
    )

lib = ctypes.CDLL(LIB_PATH)

_P = c_void_p
_I64P = POINTER(c_int64)

class LayerDesc(ctypes.Structure):
    """nsa_layer_desc of include/nsa_b200.h."""
    _fields_ = [(n_, c_int) for n_ in ("B", "H", "G", "T", "dk", "dv", "U", "l", "d", "l_prime", "n", "n_fixed", "window",
                                       "gate_mode", "dtype", "out_token_major")] + [("scale", c_float)]


# pieces of the layer's context buffer, in the order of enum nsa_layer_ctx_piece
CTX_PIECES = ("o_cmp", "L_cmp", "M_cmp", "o_slc", "L_slc", "M_slc", "o_win", "L_win", "M_win", "gates", "indices", "k_cmp",
              "k_cmp_lp", "v_cmp", "block_ends", "k_cmp_lo", "lse2_cmp", "phi_saved")
_DESCP = POINTER(LayerDesc)

# name -> (restype, argtypes); mirrors include/nsa_b200.h declaration by declaration
PROTOTYPES = {
    "nsa_last_error": (c_char_p, []),
    "nsa_version": (c_char_p, []),
    "nsa_selftest_wait_timeout": (c_int, [ctypes.c_longlong, _P]),
    "nsa_profile_enable": (c_int, [c_int]),
    "nsa_profile_report": (c_int, [ctypes.c_char_p, c_size_t]),
    "nsa_device_timeouts": (c_int, [c_int]),
    "nsa_sliding_fwd": (c_int, [_P] * 6 + [_I64P] + [c_int] * 7 + [c_float, c_int, c_int, _P]),
    "nsa_attn_bwd_workspace_bytes": (c_size_t, [c_int] * 10),
    "nsa_sliding_bwd": (c_int, [_P] * 10 + [_I64P] + [c_int] * 7 + [c_float, c_int, _P, c_int, _P, c_size_t, _P]),
    "nsa_sliding_bwd_noalloc": (c_int, [_P] * 10 + [c_int] * 7 + [c_float, _P]),
    "nsa_cmp_attn_fwd": (c_int, [_P] * 7 + [_I64P] + [c_int] * 7 + [c_float] + [c_int] * 6 + [_P, _P, _P]),
    "nsa_cmp_attn_exact_supported": (c_int, [c_int] * 8),
    "nsa_split_keys_hi_lo": (c_int, [_P, _P, _P, c_int64, _P]),
    "nsa_cmp_attn_bwd": (c_int, [_P] * 11 + [_I64P] + [c_int] * 7 + [c_float] + [c_int] * 5 + [_P, c_int, _P, c_size_t, _P]),
    "nsa_slc_fwd_workspace_bytes": (c_size_t, [c_int] * 11),
    "nsa_slc_fwd": (c_int, [_P] * 7 + [_I64P] + [c_int] * 9 + [c_float, c_int, c_int, c_int, _P, c_size_t, _P]),
    "nsa_slc_bwd_workspace_bytes": (c_size_t, [c_int] * 11),
    "nsa_slc_bwd": (c_int, [_P] * 11 + [_I64P] + [c_int] * 9 + [c_float, c_int, c_int, _P, _P, _P, c_int, _P, c_size_t, _P]),
    "nsa_cmp_phi_saved_bytes": (c_size_t, [c_int] * 6),
    "nsa_cmp_phi_workspace_bytes": (c_size_t, [c_int] * 11),
    "nsa_cmp_phi_fwd": (c_int, [_P] * 10 + [c_int] * 10 + [_P, c_size_t, _P, c_size_t, _P]),
    "nsa_cmp_phi_bwd": (c_int, [_P] * 7 + [c_size_t] + [_P] * 7 + [c_int] * 10 + [_P, c_size_t, _P]),
    "nsa_gate_mlp_workspace_bytes": (c_size_t, [c_int64, c_int, c_int, c_int, c_int, c_int]),
    "nsa_gate_mlp_fwd": (c_int, [_P] * 7 + [c_int64, c_int, c_int, c_int, c_int, _P]),
    "nsa_gate_mlp_bwd": (c_int, [_P] * 10 + [c_int64, c_int, c_int, c_int, c_int, _P, c_size_t, _P]),
    "nsa_layer_ctx_bytes": (c_size_t, [_DESCP, POINTER(c_size_t)]),
    "nsa_layer_workspace_bytes": (c_size_t, [_DESCP, c_int]),
    "nsa_layer_fwd": (c_int, [_DESCP] + [_P] * 16 + [c_size_t, _P, c_size_t, _P]),
    "nsa_layer_bwd": (c_int, [_DESCP] + [_P] * 10 + [c_size_t] + [_P] * 14 + [_P, c_size_t, _P]),
    "nsa_phi_pool_fwd": (c_int, [_P, _P, _P, _I64P, _P, _P] + [c_int] * 10 + [_P]),
    "nsa_phi_pool_bwd": (c_int, [_P] * 7 + [c_int] * 9 + [_P]),
    "nsa_score_topn_workspace_bytes": (c_size_t, [c_int] * 12),
    "nsa_score_topn": (c_int, [_P, _I64P, _P, _P, _P] + [c_int] * 11 + [c_float, c_int, c_int, c_int, c_int, _P, _P, c_size_t, _P]),
    "nsa_topn_from_scores": (c_int, [_P, _P] + [c_int] * 8 + [_P]),
    "nsa_cmp_probs": (c_int, [_P, _I64P, _P, _P, _P] + [c_int] * 6 + [c_float, c_int, _P]),
    "nsa_eq9_scores": (c_int, [_P, _P, c_int64] + [c_int] * 4 + [_P]),
    "nsa_gate_mix_fwd": (c_int, [_P] * 6 + [c_int] * 7 + [_P]),
    "nsa_gate_mix_bwd": (c_int, [_P] * 9 + [c_int] * 7 + [_P]),
    "nsa_gate_mix_bwd_delta": (c_int, [_P] * 10 + [c_int] * 7 + [_P]),
    "nsa_slc_fwd_mix": (c_int, [_P] * 7 + [_I64P] + [c_int] * 9 + [c_float, c_int, c_int, c_int] + [_P] * 5 + [c_int, c_int, _P, c_size_t, _P]),
}

for _name, (_res, _args) in PROTOTYPES.items():
    _fn = getattr(lib, _name)  # AttributeError here = library and header out of sync
    _fn.restype = _res
    _fn.argtypes = _args


class NSAKernelError(RuntimeError):
    """A C-ABI entry point returned a non-zero status."""


def check(status: int, what: str) -> None:
    if status != 0:
        raise NSAKernelError(f"{what} failed with status {status}: {lib.nsa_last_error().decode()}")


def dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"NSA kernels take float32 or bfloat16 tensors, got {t.dtype}")


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("NSA kernels run on CUDA tensors only; this package has no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise RuntimeError("no tensor given")
    return dev


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def i64(vals):
    return (c_int64 * len(vals))(*[int(v) for v in vals])


def stream_ptr(dev: torch.device):
    return c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def profile_kernels(fn):
    """Run fn() with per-kernel event timing on; returns {kernel family: (launches, total_ms)}."""
    lib.nsa_profile_enable(1)
    try:
        fn()
        buf = ctypes.create_string_buffer(1 << 16)
        check(lib.nsa_profile_report(buf, len(buf)), "nsa_profile_report")
    finally:
        lib.nsa_profile_enable(0)
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out
