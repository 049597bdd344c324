"""Bit packing of code tensors (drop-in for the reference's quashkv/packing.py).

Layout: the last axis becomes an LSB-first stream of ``bits``-wide fields
(1-bit 8 per byte, 2-bit 4 per byte, 3-bit 8 values per 3 bytes, 4-bit low nibble
first).  The work is done by the ``qkv_pack`` / ``qkv_unpack`` kernels.
"""

from __future__ import annotations

import torch

from . import ops


def pack_bits(indices: torch.Tensor, bits: int) -> torch.Tensor:
    """(..., d) uint8 codes in [0, 2**bits) -> (..., packed bytes) uint8; bits == 8 passes through."""
    return ops.pack(indices, bits)


def unpack_bits(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    """Inverse of :func:`pack_bits`; ``d`` is the unpacked last dimension."""
    return ops.unpack(packed, bits, d)


def packed_size(d: int, bits: int) -> int:
    """ceil(d*bits/8), the reference's formula (quashkv/packing.py:162-165)."""
    return (d * bits + 7) // 8
