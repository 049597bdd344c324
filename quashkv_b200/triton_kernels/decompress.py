"""fused_decompress_mse / fused_decompress_ip (reference triton_kernels/decompress.py:194-285)."""

from __future__ import annotations

import torch

from .. import ops
from .compress import _bits_from

HAS_TRITON = False


def fused_decompress_mse(indices: torch.Tensor, norms: torch.Tensor, Pi: torch.Tensor,
                         centroids: torch.Tensor) -> torch.Tensor:
    return ops.decompress(indices, norms, Pi, centroids, _bits_from(centroids.numel()))


def fused_decompress_ip(mse_indices: torch.Tensor, qjl_signs: torch.Tensor, norms: torch.Tensor,
                        Pi: torch.Tensor, centroids: torch.Tensor, S: torch.Tensor, qjl_scale: float) -> torch.Tensor:
    return ops.decompress(mse_indices, norms, Pi, centroids, _bits_from(centroids.numel()),
                          signs=qjl_signs, S=S, qjl_scale=qjl_scale)
