"""nsa - Native Sparse Attention for NVIDIA B200 (sm_100a).

Drop-in for the Python surface of Noumena-Network/NSA-Test's ``nsa`` package (nsa/__init__.py:13-37):
the same eight exported names, backed by hand-written CUDA kernels behind a C ABI
(include/nsa_b200.h).  There is no Triton, no CPU path and no PyTorch fallback: importing the package
without the built shared library raises.
"""
from .kernels import (
    NSAConfig,
    NSAAttention,
    _nsa_sliding_window_fwd_kernel,
    _nsa_sliding_window_bwd_kernel,
    _nsa_compression_fwd_kernel,
    _nsa_compression_bwd_kernel,
    _nsa_sparse_selection_fwd_kernel,
    _nsa_sparse_selection_bwd_kernel,
)

__version__ = "1.0.0"

__all__ = [
    "NSAConfig",
    "NSAAttention",
    "_nsa_sliding_window_fwd_kernel",
    "_nsa_sliding_window_bwd_kernel",
    "_nsa_compression_fwd_kernel",
    "_nsa_compression_bwd_kernel",
    "_nsa_sparse_selection_fwd_kernel",
    "_nsa_sparse_selection_bwd_kernel",
]
