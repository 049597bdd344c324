"""Serving-engine integration: compressed KV pages and block-table attention.

Mirrors the reference module ``quashkv/integrations/vllm_backend.py``:

* ``QuashKVPageConfig`` (reference :73-79), ``QuashKVPageManager`` (:82-195),
  ``quashkv_attention_forward`` (:202-231), ``QuashKVModelManager`` (:237-308) and
  ``register_quashkv_backend`` (:315-341) keep their names, arguments and error behaviour.  The
  page manager of the reference is a thin wrapper around one ``QuashKVEngine`` per layer and
  attends over that engine's contiguous blocks; so does this one, through the packed-cache
  attention kernel instead of unpacking every block.
* ``QuashKVPagedCache`` goes one step further than the reference, which stops at
  ``NotImplementedError`` before real paging: a pool of ``block_size``-token pages shared by many
  sequences of different lengths, a block table per sequence, appends that scatter the packed
  rows into the pages, and attention that reads the pages through the block table
  (``qkv_attention_paged``).  A serving engine that already owns block tables can call
  ``attention_with_tables`` with its own tensors.

Only CUDA tensors are accepted; there is no CPU implementation.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..engine import QuashKVEngine
from ..triton_kernels.attention import CompressedBlock

try:                                     # the reference probes for vLLM the same way (:58-67)
    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl  # noqa: F401
    HAS_VLLM = True
except Exception:                        # not installed, or not importable without a GPU
    HAS_VLLM = False


@dataclass
class QuashKVPageConfig:
    """Configuration for compressed KV pages (reference :73-79)."""
    key_bits: int = 3       # 2-bit MSE + 1-bit QJL
    value_bits: int = 3     # 3-bit MSE
    block_size: int = 16    # tokens per page block
    seed: int = 42


class QuashKVPageManager:
    """Compressed KV storage of one attention layer, backed by one engine (reference :82-195)."""

    def __init__(self, num_kv_heads: int, head_size: int, config: QuashKVPageConfig,
                 device: torch.device, layer_idx: int = 0):
        self.num_kv_heads = num_kv_heads
        self.head_size = head_size
        self.config = config
        self.device = device
        self.engine = QuashKVEngine(head_dim=head_size, key_bits=config.key_bits, value_bits=config.value_bits,
                                    seed=config.seed + layer_idx, device=device)

    def compress_and_store(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys, values (batch, num_kv_heads, seq_len, head_size): compress and append."""
        self.engine.append(keys, values)

    def get_compressed_blocks(self) -> list:
        """The cache as unpacked ``CompressedBlock`` records, one per append (reference :135-148)."""
        blocks = []
        for blk in self.engine._cache:
            mse, qjl, val = self.engine._unpack_block(blk)
            blocks.append(CompressedBlock(mse_indices=mse, qjl_signs=qjl, key_norms=blk.key_norms,
                                          val_indices=val, val_norms=blk.val_norms, seq_len=blk.seq_len))
        return blocks

    def attention(self, queries: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        """queries (batch, heads, q_len, head_size) over the whole stored history (reference :150-186).

        The reference unpacks every block and hands the list to ``fused_quantized_attention``; the result is
        the same when the engine attends over its packed planes, which is what runs here."""
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_size)
        if self.engine.num_blocks == 0:
            raise ValueError("No compressed KV blocks stored yet")
        return self.engine.attention(queries, scale=scale)

    @property
    def total_tokens(self) -> int:
        return self.engine.total_tokens

    def clear(self) -> None:
        self.engine.clear()

    def compression_ratio(self) -> float:
        return self.engine.compression_ratio()


def quashkv_attention_forward(queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                              page_manager: QuashKVPageManager, scale: Optional[float] = None) -> torch.Tensor:
    """Compress-and-attend of one layer step (reference :202-231)."""
    page_manager.compress_and_store(keys, values)
    return page_manager.attention(queries, scale=scale)


class QuashKVModelManager:
    """One page manager per layer (reference :237-308)."""

    def __init__(self, num_layers: int, num_kv_heads: int, head_size: int,
                 config: Optional[QuashKVPageConfig] = None, device="cuda"):
        self.num_layers = num_layers
        self.config = config or QuashKVPageConfig()
        self.device = torch.device(device)
        self.layers = [QuashKVPageManager(num_kv_heads=num_kv_heads, head_size=head_size, config=self.config,
                                          device=self.device, layer_idx=i) for i in range(num_layers)]

    def forward_layer(self, layer_idx: int, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor,
                      scale: Optional[float] = None) -> torch.Tensor:
        return quashkv_attention_forward(queries, keys, values, self.layers[layer_idx], scale)

    def clear(self) -> None:
        for layer in self.layers:
            layer.clear()

    def stats(self) -> dict:
        return {
            "num_layers": self.num_layers,
            "tokens_per_layer": [layer.total_tokens for layer in self.layers],
            "compression_ratios": [layer.compression_ratio() for layer in self.layers],
            "config": {"key_bits": self.config.key_bits, "value_bits": self.config.value_bits,
                       "block_size": self.config.block_size},
        }

    def total_compressed_bytes(self) -> int:
        return sum(layer.engine.actual_memory_bytes() for layer in self.layers)


def register_quashkv_backend() -> None:
    """Same contract as the reference (:315-341): ImportError without vLLM, else NotImplementedError."""
    if not HAS_VLLM:
        raise ImportError("vLLM is not installed. Install it with: pip install vllm>=0.6")
    raise NotImplementedError(
        "Registration as a vLLM attention backend is not wired up. Use QuashKVPagedCache "
        "(block tables, per-sequence lengths) or QuashKVModelManager directly.")


# ---------------------------------------------------------------------------------------------------
# Real pages: a shared pool, block tables, per-sequence lengths
# ---------------------------------------------------------------------------------------------------
class QuashKVPagedCache:
    """A pool of compressed KV pages shared by many sequences of one attention layer.

    A sequence owns a list of pages and a token count.  For head size 128 at 3/3 bits with ``block_size`` a
    multiple of 16 the pool is ``records [num_blocks, num_kv_heads, block_size / 16, 1664]``: 16-token tile
    records, the layout the tensor-core attention kernel streams (a 16-token page is exactly one record per
    head).  Otherwise the pool is the five row-major planes ``[num_blocks, num_kv_heads, block_size, row
    bytes]`` (codes, sign bits) and ``[num_blocks, num_kv_heads, block_size]`` (norms) of the generic kernel.
    """

    def __init__(self, num_blocks: int, num_kv_heads: int, head_size: int,
                 config: Optional[QuashKVPageConfig] = None, device="cuda", layer_idx: int = 0):
        self.config = config or QuashKVPageConfig()
        if num_blocks < 1 or self.config.block_size < 1:
            raise ValueError("num_blocks and block_size must be positive")
        self.num_blocks = num_blocks
        self.num_kv_heads = num_kv_heads
        self.head_size = head_size
        self.block_size = self.config.block_size
        self.device = torch.device(device)
        self.engine = QuashKVEngine(head_dim=head_size, key_bits=self.config.key_bits,
                                    value_bits=self.config.value_bits, seed=self.config.seed + layer_idx,
                                    device=self.device)
        pk, ps, pv = self.engine._row_bytes()
        shape = (num_blocks, num_kv_heads, self.block_size)
        u8 = dict(dtype=torch.uint8, device=self.device)
        f32 = dict(dtype=torch.float32, device=self.device)
        self.tiled = self.engine._tiled and self.block_size % ops.TILE_TOKENS == 0
        if self.tiled:
            self.planes = {"records": torch.zeros((num_blocks, num_kv_heads, self.block_size // ops.TILE_TOKENS,
                                                   ops.TILE_BYTES), **u8)}
        else:
            self.planes = {
                "k_codes": torch.zeros((*shape, pk), **u8), "k_signs": torch.zeros((*shape, ps), **u8),
                "k_norms": torch.zeros(shape, **f32),
                "v_codes": torch.zeros((*shape, pv), **u8), "v_norms": torch.zeros(shape, **f32),
            }
        self._free = list(range(num_blocks - 1, -1, -1))      # pop() hands out block 0 first
        self._blocks: dict = {}                                # sequence id -> list of block ids
        self._lens: dict = {}                                  # sequence id -> tokens stored

    # ---- bookkeeping (host) ---------------------------------------------------------------------
    @property
    def free_blocks(self) -> int:
        return len(self._free)

    def seq_len(self, seq_id) -> int:
        return self._lens.get(seq_id, 0)

    def blocks_of(self, seq_id) -> list:
        return list(self._blocks.get(seq_id, []))

    def free(self, seq_id) -> None:
        """Return a sequence's pages to the pool."""
        self._free.extend(reversed(self._blocks.pop(seq_id, [])))
        self._lens.pop(seq_id, None)

    def clear(self) -> None:
        for seq_id in list(self._blocks):
            self.free(seq_id)

    def _grow(self, seq_id, new_tokens: int) -> None:
        blocks = self._blocks.setdefault(seq_id, [])
        need = -(-(self._lens.get(seq_id, 0) + new_tokens) // self.block_size) - len(blocks)
        if need > len(self._free):
            raise RuntimeError(f"KV page pool exhausted: sequence {seq_id!r} needs {need} more pages, "
                               f"{len(self._free)} free")
        for _ in range(need):
            blocks.append(self._free.pop())

    def block_table(self, seq_ids: Sequence) -> tuple:
        """(block_table (n, max_blocks) int32, seq_lens (n) int32, max length) for a batch of sequences."""
        width = max(1, max(len(self._blocks.get(s, [])) for s in seq_ids))
        table = np.zeros((len(seq_ids), width), dtype=np.int32)
        for i, s in enumerate(seq_ids):
            b = self._blocks.get(s, [])
            table[i, :len(b)] = b
        lens = np.asarray([self._lens.get(s, 0) for s in seq_ids], dtype=np.int32)
        return (torch.from_numpy(table).to(self.device), torch.from_numpy(lens).to(self.device),
                int(lens.max()) if len(lens) else 0)

    # ---- data path --------------------------------------------------------------------------------
    def append(self, seq_ids: Sequence, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys, values (n_seq, num_kv_heads, new_tokens, head_size): the next ``new_tokens`` positions of
        every listed sequence (new sequences start at position 0)."""
        ops._need_cuda(keys, "QuashKVPagedCache.append")
        n, H, T, D = keys.shape
        if n != len(seq_ids) or H != self.num_kv_heads or D != self.head_size or values.shape != keys.shape:
            raise ValueError(f"Expected keys and values of shape ({len(seq_ids)}, {self.num_kv_heads}, T, "
                             f"{self.head_size})")
        if T == 0:
            return
        bs = self.block_size
        slots = np.empty((n, H, T), dtype=np.int64)
        for i, s in enumerate(seq_ids):
            self._grow(s, T)
            pos = self._lens.get(s, 0) + np.arange(T)
            blk = np.asarray(self._blocks[s], dtype=np.int64)[pos // bs]
            slots[i] = (blk[None, :] * H + np.arange(H)[:, None]) * bs + (pos % bs)[None, :]
            self._lens[s] = self._lens.get(s, 0) + T
        self._store(keys, values, torch.from_numpy(slots.reshape(-1)).to(self.device))

    def append_with_tables(self, keys: torch.Tensor, values: torch.Tensor, block_table: torch.Tensor,
                           start_lens: torch.Tensor) -> None:
        """The same store for a caller that owns the page allocation (a serving engine): ``block_table`` (n_seq,
        max_blocks) int32 and ``start_lens`` (n_seq) int32 live on the device, the new tokens of sequence i go to
        positions start_lens[i] .. start_lens[i] + new_tokens - 1 of its pages.  The slots are computed on the
        device: no host loop and no host-to-device copy per decode step.  The pool's own bookkeeping
        (``seq_len``, ``free``) is not involved."""
        ops._need_cuda(keys, "QuashKVPagedCache.append_with_tables")
        n, H, T, D = keys.shape
        if H != self.num_kv_heads or D != self.head_size or values.shape != keys.shape or \
                block_table.shape[0] != n or start_lens.numel() != n:
            raise ValueError(f"Expected keys and values of shape (n_seq, {self.num_kv_heads}, T, {self.head_size}) with "
                             "a block table and start lengths for n_seq sequences")
        if T == 0:
            return
        bs = self.block_size
        dev = keys.device
        pos = start_lens.to(torch.int64).reshape(n, 1) + torch.arange(T, device=dev, dtype=torch.int64).reshape(1, T)
        blk = torch.gather(block_table.to(torch.int64), 1, torch.div(pos, bs, rounding_mode="floor"))       # (n, T)
        heads = torch.arange(H, device=dev, dtype=torch.int64).reshape(1, H, 1)
        slots = (blk.reshape(n, 1, T) * H + heads) * bs + (pos % bs).reshape(n, 1, T)
        self._store(keys, values, slots.reshape(-1).contiguous())

    def _store(self, keys: torch.Tensor, values: torch.Tensor, slots_d: torch.Tensor) -> None:
        """Compress (n_seq, heads, T, d) keys and values and file every token at its slot
        ((block * heads + head) * block_size + offset)."""
        n, H, T, D = keys.shape
        kq, vq = self.engine.key_quantizer, self.engine.value_quantizer
        Pi, k_bounds, k_cents, Sgn = kq._on(keys.device)
        _, v_bounds, _ = vq._on(keys.device)
        codes, signs, k_norms = ops.compress_ip(keys, Pi, k_bounds, k_cents, Sgn, kq.mse_bits, packed=True)
        v_codes, v_norms = ops.compress_mse(values, Pi, v_bounds, self.config.value_bits, packed=True)
        p = self.planes
        if self.tiled:
            flat = lambda t: t.reshape(n * H * T, -1).contiguous()      # noqa: E731
            ops.tile_rows(flat(codes), flat(signs), k_norms.reshape(-1).contiguous(), flat(v_codes),
                          v_norms.reshape(-1).contiguous(), p["records"], 1, 0, 0, slots_d)
            return
        for src, name in ((codes, "k_codes"), (signs, "k_signs"), (k_norms, "k_norms"),
                          (v_codes, "v_codes"), (v_norms, "v_norms")):
            ops.scatter_rows(src.contiguous(), p[name], slots_d)

    def rows_of(self, seq_id) -> dict:
        """The stored tokens of one sequence as the five packed planes ``[num_kv_heads, tokens, ...]`` in the
        reference's row layout (exact copies; for inspection and tests)."""
        n, H, bs = self._lens.get(seq_id, 0), self.num_kv_heads, self.block_size
        pos = torch.arange(n, device=self.device)
        blk = torch.tensor(self._blocks.get(seq_id, []), dtype=torch.int64, device=self.device)[pos // bs]
        slots = ((blk[None, :] * H + torch.arange(H, device=self.device)[:, None]) * bs + (pos % bs)[None, :]).reshape(-1)
        names = ("k_codes", "k_signs", "k_norms", "v_codes", "v_norms")
        if self.tiled:
            rows = ops.untile_rows(self.planes["records"], H * n, 1, 0, 0, slots.contiguous())
        else:
            rows = [self.planes[name].reshape(self.num_blocks * H * bs, -1)[slots] for name in names]
        return {name: r.reshape(H, n, -1) if r.dim() == 2 and name.endswith(("codes", "signs")) else r.reshape(H, n)
                for name, r in zip(names, rows)}

    def attention_with_tables(self, queries: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                              max_kv_len: int, scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
        """queries (n_seq, q_heads, q_len, head_size); block_table (n_seq, max_blocks) int32 and seq_lens
        (n_seq) int32 on the device; ``max_kv_len`` an upper bound of seq_lens known on the host."""
        ops._need_cuda(queries, "QuashKVPagedCache.attention")
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_size)
        n, Hq, Q, D = queries.shape
        if D != self.head_size or Hq % self.num_kv_heads != 0 or block_table.shape[0] != n or seq_lens.numel() != n:
            raise ValueError(f"queries {tuple(queries.shape)} do not match {self.num_kv_heads} KV heads of size "
                             f"{self.head_size} and a block table for {block_table.shape[0]} sequences")
        if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
            raise ValueError("block_table and seq_lens must be int32")
        kq, vq = self.engine.key_quantizer, self.engine.value_quantizer
        Pi, _, k_cents, Sgn = kq._on(queries.device)
        _, _, v_cents = vq._on(queries.device)
        p = self.planes
        if self.tiled:
            return ops.attention_tiled(queries, p["records"], 0, int(max_kv_len), self.num_kv_heads,
                                       block_table.contiguous(), seq_lens.contiguous(), self.block_size, Pi,
                                       k_cents, v_cents, Sgn, kq.qjl_scale, float(scale), bool(causal))
        return ops.attention_paged(queries, p["k_codes"], p["k_signs"], p["k_norms"], p["v_codes"], p["v_norms"],
                                   block_table.contiguous(), seq_lens.contiguous(), int(max_kv_len),
                                   self.config.key_bits, self.config.value_bits, Pi, k_cents, v_cents, Sgn,
                                   kq.qjl_scale, float(scale), bool(causal))

    def attention(self, seq_ids: Sequence, queries: torch.Tensor, scale: Optional[float] = None,
                  causal: bool = False) -> torch.Tensor:
        """Attention of every listed sequence over its own pages; with ``causal`` the q_len query rows are the
        last q_len positions of each sequence."""
        table, lens, longest = self.block_table(seq_ids)
        if longest == 0:
            raise ValueError("No compressed KV blocks stored yet")
        return self.attention_with_tables(queries, table, lens, longest, scale=scale, causal=causal)
