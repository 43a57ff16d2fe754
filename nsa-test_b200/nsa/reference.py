"""Test helpers under the reference project's ``nsa.reference`` names.

The reference ships slow loop-based PyTorch implementations of the three branches in this module
(nsa/reference.py:13-254) and its tests import them from here.  This package does not carry a second
implementation of the attention math: the attention functions below forward to a checkout of the
reference project when the environment variable ``NSA_REFERENCE_PATH`` points at one, and raise
otherwise.  The small tensor helpers (block ends, seeded inputs, error metric) are provided directly.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from typing import Tuple

import torch


def _upstream():
    root = os.environ.get("NSA_REFERENCE_PATH")
    if not root or not os.path.exists(os.path.join(root, "nsa", "reference.py")):
        raise RuntimeError("this function lives in the reference project; set NSA_REFERENCE_PATH to a checkout of it")
    name = "_nsa_upstream_reference"
    if name not in sys.modules:
        spec = importlib.util.spec_from_file_location(name, os.path.join(root, "nsa", "reference.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name]


def sliding_window_attention(*args, **kwargs):
    return _upstream().sliding_window_attention(*args, **kwargs)


def compression_attention(*args, **kwargs):
    return _upstream().compression_attention(*args, **kwargs)


def selection_attention_reference(*args, **kwargs):
    return _upstream().selection_attention_reference(*args, **kwargs)


def dense_attention_reference(*args, **kwargs):
    return _upstream().dense_attention_reference(*args, **kwargs)


def compress_kv_simple(*args, **kwargs):
    return _upstream().compress_kv_simple(*args, **kwargs)


def create_block_ends(T: int, block_size: int, stride: int, device="cuda") -> torch.Tensor:
    """Block end positions min(start + block_size, T) - 1 for starts 0, stride, ... up to the block that
    reaches the end of the sequence; int32 [N_BLOCKS]."""
    ends = []
    start = 0
    while start < T:
        end = min(start + block_size, T) - 1
        ends.append(end)
        if end >= T - 1:
            break
        start += stride
    return torch.tensor(ends, device=device, dtype=torch.int32)


def compare_outputs(output_kernel: torch.Tensor, output_ref: torch.Tensor, tolerance: float = 1e-3,
                    name: str = "Output") -> Tuple[bool, float]:
    """max|a-b| / (max|b| + 1e-8) against a tolerance; returns (passed, relative error)."""
    diff = (output_kernel - output_ref).abs()
    rel = diff.max() / (output_ref.abs().max() + 1e-8)
    print(f"{name} relative error: {rel:.6f}")
    return bool(rel < tolerance), rel


def generate_test_tensors(B: int = 2, H: int = 8, G: int = 2, T: int = 64, dk: int = 32, dv: int = 32,
                          device: str = "cuda", dtype: torch.dtype = torch.float32, seed: int = 42):
    """Seeded q [B,H,T,dk], k [B,G,dk,T] (head dim before time), v [B,G,T,dv], scaled by 0.02,
    requiring grad."""
    torch.manual_seed(seed)
    q = torch.randn(B, H, T, dk, device=device, dtype=dtype) * 0.02
    k = torch.randn(B, G, dk, T, device=device, dtype=dtype) * 0.02
    v = torch.randn(B, G, T, dv, device=device, dtype=dtype) * 0.02
    for t in (q, k, v):
        t.requires_grad_(True)
    return q, k, v
