"""QuashKVCache: one compressed engine per decoder layer, HuggingFace ``Cache.update`` shape.

Interface of the reference's quashkv/integrations/hf_cache.py (:19-203).  ``update``
compresses the new tokens into the layer's packed planes and returns the whole
history decompressed by one kernel launch per tensor; keys come back from the code
centroids only (the sign bits serve the fused attention path, reference :96-121).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..engine import QuashKVEngine


@dataclass
class QuashKVCacheConfig:
    key_bits: int = 3
    value_bits: int = 3
    seed: int = 42


class QuashKVCache:
    def __init__(self, num_layers: int, head_dim: int, config: Optional[QuashKVCacheConfig] = None,
                 device="cpu"):
        self.config = config or QuashKVCacheConfig()
        self.num_layers, self.head_dim = num_layers, head_dim
        self.device = torch.device(device)
        self.engines = [
            QuashKVEngine(head_dim=head_dim, key_bits=self.config.key_bits, value_bits=self.config.value_bits,
                          seed=self.config.seed + layer, device=device)
            for layer in range(num_layers)
        ]

    @classmethod
    def from_model(cls, model, config: Optional[QuashKVCacheConfig] = None, device=None) -> "QuashKVCache":
        mc = model.config
        num_layers = getattr(mc, "num_hidden_layers", None)
        if num_layers is None:
            raise ValueError("Cannot detect num_hidden_layers from model config")
        head_dim = getattr(mc, "head_dim", None)
        if head_dim is None:
            head_dim = mc.hidden_size // mc.num_attention_heads
        if device is None:
            device = next(model.parameters()).device
        return cls(num_layers=num_layers, head_dim=head_dim, config=config, device=device)

    def _decompress_engine(self, engine: QuashKVEngine, out_dtype=torch.float32):
        return engine.decompress_all(with_signs=False, out_dtype=out_dtype)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict] = None):
        """Append (batch, kv_heads, new_seq, head_dim) states; return the full decompressed K, V."""
        engine = self.engines[layer_idx]
        engine.append(key_states, value_states)
        return self._decompress_engine(engine)

    def attention(self, queries: torch.Tensor, layer_idx: int, scale: Optional[float] = None,
                  causal: bool = False) -> torch.Tensor:
        """Attention straight over the layer's packed cache (no decompression); query heads may be a
        multiple of the KV heads."""
        return self.engines[layer_idx].attention(queries, scale=scale, causal=causal)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.engines[layer_idx].total_tokens

    def get_max_cache_length(self) -> Optional[int]:
        return None

    def __getitem__(self, layer_idx: int):
        engine = self.engines[layer_idx]
        if engine.num_blocks == 0:
            return (torch.empty(0), torch.empty(0))
        return self._decompress_engine(engine)

    def __len__(self) -> int:
        return self.num_layers

    def __iter__(self):
        for i in range(self.num_layers):
            yield self[i]

    def reset(self) -> None:
        for engine in self.engines:
            engine.clear()

    def compression_stats(self) -> dict:
        original = compressed = 0
        tokens = []
        for e in self.engines:
            tokens.append(e.total_tokens)
            if e.total_tokens > 0:
                d = e.head_dim
                original += e.total_tokens * 2 * d * 16
                compressed += e.total_tokens * (e.key_bits * d + 32 + e.value_bits * d + 32)
        return {
            "num_layers": self.num_layers,
            "tokens_per_layer": tokens,
            "total_original_bits": original,
            "total_compressed_bits": compressed,
            "overall_compression_ratio": original / compressed if compressed > 0 else 0,
        }
