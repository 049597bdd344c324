"""fused_compress_mse / fused_compress_ip (reference triton_kernels/compress.py:210-303)."""

from __future__ import annotations

import torch

from .. import ops

HAS_TRITON = False


def _bits_from(n_tables: int) -> int:
    bits = int(n_tables).bit_length() - 1
    if (1 << bits) != n_tables or not 1 <= bits <= 4:
        raise ValueError(f"expected 2**b - 1 boundaries / 2**b centroids with b in 1..4, got {n_tables}")
    return bits


def fused_compress_mse(x: torch.Tensor, Pi: torch.Tensor, boundaries: torch.Tensor):
    """x (..., d) -> (codes uint8 (..., d), norms fp32 (...))."""
    return ops.compress_mse(x, Pi, boundaries, _bits_from(boundaries.numel() + 1), packed=False)


def fused_compress_ip(x: torch.Tensor, Pi: torch.Tensor, boundaries: torch.Tensor, S: torch.Tensor,
                      centroids: torch.Tensor):
    """x (..., d) -> (codes, sign bits, norms)."""
    return ops.compress_ip(x, Pi, boundaries, centroids, S, _bits_from(centroids.numel()), packed=False)
