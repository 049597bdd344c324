"""fused_quantized_attention over a list of unpacked blocks
(reference triton_kernels/attention.py:307-394).

The kernel reads packed planes, so the blocks' one-byte-per-coordinate tensors are
packed into planes first (two small kernels per block); callers that already hold
an engine should call ``QuashKVEngine.attention``, which skips this step.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from .compress import _bits_from

HAS_TRITON = False


@dataclass
class CompressedBlock:
    mse_indices: torch.Tensor   # (B, H, S, D) uint8
    qjl_signs: torch.Tensor     # (B, H, S, D) uint8
    key_norms: torch.Tensor     # (B, H, S) float32
    val_indices: torch.Tensor   # (B, H, S, D) uint8
    val_norms: torch.Tensor     # (B, H, S) float32
    seq_len: int


def fused_quantized_attention(queries: torch.Tensor, blocks: list, Pi: torch.Tensor,
                              key_centroids: torch.Tensor, val_centroids: torch.Tensor, S: torch.Tensor,
                              qjl_scale: float, scale: Optional[float] = None, causal: bool = False,
                              total_kv_tokens: int = 0) -> torch.Tensor:
    """With ``causal``, query row i sits at position ``total_kv_tokens - Q + i`` and sees keys at positions up to
    its own (reference attention.py:119-123).  ``total_kv_tokens = 0`` (the default, for which the reference masks
    every key and returns NaN) is read as "the number of tokens in ``blocks``"."""
    B, H, Q, D = queries.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    kb, vb = _bits_from(key_centroids.numel()), _bits_from(val_centroids.numel())
    cat = lambda name: torch.cat([getattr(b, name) for b in blocks], dim=2)  # noqa: E731
    Hkv = blocks[0].key_norms.shape[1]
    kv = sum(b.seq_len for b in blocks)
    seg = B * Hkv
    k_codes = ops.pack(cat("mse_indices"), kb).reshape(seg, kv, -1)
    k_signs = ops.pack(cat("qjl_signs"), 1).reshape(seg, kv, -1)
    v_codes = ops.pack(cat("val_indices"), vb).reshape(seg, kv, -1)
    k_norms = cat("key_norms").float().reshape(seg, kv).contiguous()
    v_norms = cat("val_norms").float().reshape(seg, kv).contiguous()

    def run(q, n_keys, is_causal):
        return ops.attention(q, k_codes, k_signs, k_norms, v_codes, v_norms, n_keys, Hkv, kb + 1, vb, Pi,
                             key_centroids, val_centroids, S, float(qjl_scale), float(scale), is_causal)

    total = int(total_kv_tokens) if total_kv_tokens else kv
    if not causal or total == kv:
        return run(queries, kv, bool(causal))
    if total < kv:
        # the queries sit before the end of the blocks: keys at positions >= total are hidden from all of them
        if total < Q:
            raise ValueError(f"causal attention: total_kv_tokens = {total} puts query rows before position 0")
        return run(queries, total, True)
    # the queries sit past the end of the blocks: the last rows see every key, the first
    # Q - (total - kv) rows are the causal tail of the stored keys
    n_causal = Q - (total - kv)
    if n_causal <= 0:
        return run(queries, kv, False)
    if n_causal > kv:
        raise ValueError(f"causal attention: total_kv_tokens = {total} puts query rows before position 0")
    head = run(queries[:, :, :n_causal], kv, True)
    tail = run(queries[:, :, n_causal:], kv, False)
    return torch.cat([head, tail], dim=2)
