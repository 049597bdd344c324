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


# ---------------------------------------------------------------------------------------------------
# The cache as a `transformers.Cache`, with the fused decode route
# ---------------------------------------------------------------------------------------------------
# The reference's generation loop (benchmarks/generation_demo.py:222-344) decompresses every layer's whole
# history for every generated token and rebuilds a DynamicCache from it (hf_cache.py:96-152): its attention never
# reads the compressed form.  Here the model's attention layers call the packed-cache attention kernel
# directly: `update` only appends the new tokens, and an attention function registered with transformers'
# attention interface reads the layer's engine.  Nothing is decompressed in the decode loop.

FUSED_ATTENTION_NAME = "quashkv_fused"


def _hf():
    try:
        from transformers import AttentionInterface
        from transformers.cache_utils import Cache, CacheLayerMixin
        return Cache, CacheLayerMixin, AttentionInterface
    except ImportError as e:            # transformers is optional for the rest of the package
        raise ImportError("the HuggingFace cache interface needs the `transformers` package") from e


def quashkv_fused_attention(module, query, key, value, attention_mask=None, dropout=0.0, scaling=None, **kwargs):
    """Attention function for transformers' attention interface: the layer's keys and values have already been
    appended to its engine by `QuashKVHFCache.update`; `key` / `value` (the new tokens only) and the mask are not
    read.  Rows of a multi-token call are causal among themselves (prefill); a single-token call sees the whole
    cache (decode).  Padding masks are not supported: every sequence of the batch has the cache's length."""
    cache = getattr(module, "quashkv_cache", None)
    if cache is None:
        raise RuntimeError("quashkv_fused attention: no QuashKVHFCache attached to this layer (call cache.attach(model))")
    engine = cache.engines[module.layer_idx]
    out = engine.attention(query, scale=scaling, causal=query.shape[2] > 1)          # (B, Hq, Q, D) fp32
    return out.to(query.dtype).transpose(1, 2).contiguous(), None


def make_hf_cache(quash_cache: "QuashKVCache", fused: bool = True):
    """A `transformers.Cache` over the engines of ``quash_cache``.

    fused=True   `update` appends the new tokens and hands them straight back; attention must then run through
                 `quashkv_fused_attention` (see `attach`), which reads the packed cache.
    fused=False  `update` returns the whole history decompressed, keys from the code centroids only, as the
                 reference's cache does (hf_cache.py:96-152); any attention implementation works on it."""
    Cache, CacheLayerMixin, AttentionInterface = _hf()

    class _Layer(CacheLayerMixin):
        is_compileable = False
        is_sliding = False

        def __init__(self, engine):
            super().__init__()
            self.engine = engine

        def lazy_initialization(self, key_states, value_states):
            self.is_initialized = True

        def update(self, key_states, value_states, *args, **kwargs):
            self.is_initialized = True
            self.engine.append(key_states, value_states)
            if fused:
                return key_states, value_states
            keys, values = self.engine.decompress_all(with_signs=False)
            return keys.to(key_states.dtype), values.to(value_states.dtype)

        def get_seq_length(self) -> int:
            return self.engine.total_tokens

        def get_mask_sizes(self, query_length: int):
            return self.engine.total_tokens + query_length, 0

        def get_max_cache_shape(self) -> int:
            return -1

        def reset(self) -> None:
            self.engine.clear()

    class QuashKVHFCache(Cache):
        def __init__(self):
            super().__init__(layers=[_Layer(e) for e in quash_cache.engines])
            self.engines = quash_cache.engines
            self.fused = fused

        def attach(self, model):
            """Point every attention layer of ``model`` at this cache and, for the fused route, switch the model to
            the packed-cache attention function.  Returns the model's previous attention implementation."""
            previous = model.config._attn_implementation
            if fused:
                from transformers import AttentionMaskInterface
                from transformers.masking_utils import sdpa_mask
                AttentionInterface.register(FUSED_ATTENTION_NAME, quashkv_fused_attention)
                AttentionMaskInterface.register(FUSED_ATTENTION_NAME, sdpa_mask)
                model.config._attn_implementation = FUSED_ATTENTION_NAME
            for module in model.modules():
                if hasattr(module, "layer_idx") and hasattr(module, "q_proj"):
                    module.quashkv_cache = self
            return previous

        def detach(self, model, previous: str) -> None:
            model.config._attn_implementation = previous
            for module in model.modules():
                if getattr(module, "quashkv_cache", None) is self:
                    del module.quashkv_cache

    return QuashKVHFCache()
