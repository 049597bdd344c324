"""QuashKVEngine: compressed KV storage and attention over it.

Same constructor, methods and error texts as the reference's engine
(quashkv/engine.py:54-360).  What differs is underneath:

* storage is always the packed form, kept in five pre-allocated planes
  ``[batch*heads, capacity, bytes]`` that grow geometrically; ``append`` compresses
  straight into the tail of the planes (no per-call block tensors, no
  concatenation);
* ``attention`` is one call of the packed-cache attention kernel (online softmax,
  split over the KV length, values accumulated in the rotated domain);
* ``_cache`` is a list of per-append block *views* built on demand: packed views of
  the planes when ``pack_storage=True``, unpacked copies when ``False`` (what the
  reference stores), so code that inspects blocks keeps working.

Query heads may outnumber KV heads (grouped-query attention, query head h reads KV
head h // group); the reference requires equal counts.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional

import torch

from . import ops
from .constants import DEFAULT_SEED, DEFAULT_TOTAL_BITS
from .quantizer import InnerProductQuantizer, MSEQuantizer


@dataclass
class CompressedKVBlock:
    """One appended block (field meaning as in reference engine.py:30-51)."""
    mse_indices: torch.Tensor
    qjl_signs: torch.Tensor
    key_norms: torch.Tensor
    val_indices: torch.Tensor
    val_norms: torch.Tensor
    seq_len: int
    packed: bool = False


class QuashKVEngine:
    def __init__(self, head_dim: int = 128, key_bits: int = DEFAULT_TOTAL_BITS,
                 value_bits: int = DEFAULT_TOTAL_BITS, seed: int = DEFAULT_SEED,
                 device="cpu", pack_storage: bool = False):
        self.head_dim, self.key_bits, self.value_bits, self.seed = head_dim, key_bits, value_bits, seed
        self.device = torch.device(device)
        self.pack_storage = pack_storage
        self.key_quantizer = InnerProductQuantizer(d=head_dim, total_bits=key_bits, seed=seed, device=device)
        self.value_quantizer = MSEQuantizer(d=head_dim, bits=value_bits, seed=seed, device=device)
        # Storage: 16-token tile records when the tensor-core decode kernel covers the configuration (head_dim
        # 128, 3-bit keys and values, a value table with c[7-i] = -c[i], a key table with c0 + c3 = c1 + c2), else
        # the five row-major planes.  QUASHKV_B200_ROW_STORAGE=1 keeps the row-major planes everywhere (for A/B
        # checks).
        self._tiled = ops.tiled_layout_ok(head_dim, key_bits, value_bits) and \
            ops.tiled_tables_ok(self.key_quantizer.mse_quantizer.codebook.centroids,
                                self.value_quantizer.codebook.centroids) and \
            os.environ.get("QUASHKV_B200_ROW_STORAGE") != "1"
        self._planes = None          # dict: {"records"} or the five planes
        self._shape = None           # (batch, heads)
        self._capacity = 0
        self._total_tokens = 0
        self._block_lens: list[int] = []
        self._block_cache = None
        self._tiled_call = None      # prepared attention call of the decode loop (ops.TiledAttentionCall)
        self._row_call = None        # ... over row-major planes (ops.RowAttentionCall)
        self._append_call = None     # prepared compression of new tokens (ops.AppendCall)

    # ---- compression ------------------------------------------------------------------------
    def compress_keys(self, keys: torch.Tensor):
        return self.key_quantizer.compress(keys)

    def compress_values(self, values: torch.Tensor):
        return self.value_quantizer.compress(values)

    # ---- storage ----------------------------------------------------------------------------
    def _row_bytes(self):
        d = self.head_dim
        return (ops.packed_row_bytes(d, self.key_bits - 1), ops.packed_row_bytes(d, 1),
                ops.packed_row_bytes(d, self.value_bits))

    def _allocate(self, segments: int, capacity: int, device) -> dict:
        u8 = dict(dtype=torch.uint8, device=device)
        if self._tiled:          # 16-token tile records, the layout the tensor-core decode kernel streams
            return {"records": torch.zeros((segments, capacity // ops.TILE_TOKENS, ops.TILE_BYTES), **u8)}
        pk, ps, pv = self._row_bytes()
        f32 = dict(dtype=torch.float32, device=device)
        return {
            "k_codes": torch.zeros((segments, capacity, pk), **u8),
            "k_signs": torch.zeros((segments, capacity, ps), **u8),
            "k_norms": torch.zeros((segments, capacity), **f32),
            "v_codes": torch.zeros((segments, capacity, pv), **u8),
            "v_norms": torch.zeros((segments, capacity), **f32),
        }

    def reserve(self, batch: int, heads: int, capacity: int, device=None) -> None:
        """Pre-size the storage (optional; ``append`` grows it as needed)."""
        device = torch.device(device) if device is not None else self.device
        capacity = -(-capacity // 64) * 64      # whole 64-row groups: 16-byte aligned plane rows, whole tiles
        if self._planes is None:
            self._shape = (batch, heads)
            self._planes = self._allocate(batch * heads, capacity, device)
            self._capacity = capacity
        elif capacity > self._capacity:
            grown = self._allocate(self._shape[0] * self._shape[1], capacity, self._device())
            used = -(-self._total_tokens // ops.TILE_TOKENS) if self._tiled else self._total_tokens
            for name, plane in self._planes.items():
                grown[name][:, :used] = plane[:, :used]
            self._planes, self._capacity = grown, capacity
            self._block_cache = None

    def _device(self):
        return next(iter(self._planes.values())).device

    def _write(self, keys: torch.Tensor, values: torch.Tensor, seg0: int, offset: int) -> None:
        """Compress (b, H, S, d) keys / values into segments seg0.. at token offset ``offset``."""
        kq, vq = self.key_quantizer, self.value_quantizer
        Pi, k_bounds, k_cents, Sgn = kq._on(keys.device)
        _, v_bounds, _ = vq._on(keys.device)
        b, H, S, _ = keys.shape
        p = self._planes
        if seg0 == 0 and (b, H) == self._shape:
            # the usual append over all segments: the prepared call (no op dispatcher, kept staging planes)
            call = self._append_call
            if call is None or call.device != keys.device or call.consts[0].data_ptr() != Pi.data_ptr():
                call = self._append_call = ops.AppendCall(Pi, k_bounds, k_cents, Sgn, kq.mse_bits, v_bounds,
                                                          self.value_bits)
            with torch.cuda.device(keys.device):
                if self._tiled:
                    call.into_records(keys, values, p["records"], self._row_bytes(), self._capacity, offset)
                else:
                    call.into_planes(keys, values, p, offset)
            return
        if not self._tiled:
            sl = slice(seg0, seg0 + b * H)
            ops.append_kv(keys, values, Pi, k_bounds, k_cents, Sgn, kq.mse_bits, v_bounds, self.value_bits,
                          p["k_codes"][sl], p["k_signs"][sl], p["k_norms"][sl], p["v_codes"][sl], p["v_norms"][sl],
                          offset)
            return
        # tiled storage: the compress kernels write the reference's packed rows into a dense staging area, an
        # exact integer kernel files every token into its record
        pk, ps, pv = self._row_bytes()
        n = b * H * S
        u8 = dict(dtype=torch.uint8, device=keys.device)
        st = (torch.empty((b * H, S, pk), **u8), torch.empty((b * H, S, ps), **u8),
              torch.empty((b * H, S), dtype=torch.float32, device=keys.device),
              torch.empty((b * H, S, pv), **u8), torch.empty((b * H, S), dtype=torch.float32, device=keys.device))
        ops.append_kv(keys, values, Pi, k_bounds, k_cents, Sgn, kq.mse_bits, v_bounds, self.value_bits, *st, 0)
        assert st[2].numel() == n
        ops.tile_rows(*st, p["records"][seg0:seg0 + b * H], S, self._capacity, offset, None)

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """Compress (batch, heads, seq, head_dim) keys and values and add them to the cache."""
        ops._need_cuda(keys, "QuashKVEngine.append")
        B, H, S, D = keys.shape
        if D != self.head_dim or values.shape != keys.shape:
            raise ValueError(f"Expected keys and values of shape (B, H, S, {self.head_dim})")
        if self._planes is not None and self._total_tokens == 0 and \
                ((B, H) != self._shape or self._device() != keys.device):
            self._planes = None          # an emptied cache takes any shape next, like the reference's clear()
        if self._planes is None:
            self.reserve(B, H, max(64, S), keys.device)
        elif (B, H) != self._shape:
            raise ValueError(f"Cache holds (batch, heads) = {self._shape}, got {(B, H)}")
        need = self._total_tokens + S
        if need > self._capacity:
            self.reserve(B, H, max(need, 2 * self._capacity))
        if S > 0:
            self._write(keys, values, 0, self._total_tokens)
        self._block_lens.append(S)
        self._total_tokens = need
        self._block_cache = None

    def clear(self) -> None:
        """Empty the cache (reference engine.py:174-177).  The storage is kept for the next sequence of the
        same (batch, heads); ``append`` re-allocates when the next one differs."""
        self._total_tokens = 0
        self._block_lens = []
        self._block_cache = None

    @property
    def total_tokens(self) -> int:
        return self._total_tokens

    @property
    def num_blocks(self) -> int:
        return len(self._block_lens)

    def row_planes(self, start: int = 0, stop: Optional[int] = None) -> dict:
        """The five packed planes ``[batch*heads, stop - start, ...]`` in the reference's row layout
        (packing.py:22-94): views of the storage, or exact untiled copies when the storage is tile records."""
        stop = self._total_tokens if stop is None else stop
        n = max(stop - start, 0)
        p = self._planes
        if not self._tiled:
            return {name: plane[:, start:stop] for name, plane in p.items()}
        segs = self._shape[0] * self._shape[1]
        kc, ks, kn, vc, vn = ops.untile_rows(p["records"], segs * n, max(n, 1), self._capacity, start, None)
        return {"k_codes": kc.reshape(segs, n, -1), "k_signs": ks.reshape(segs, n, -1), "k_norms": kn.reshape(segs, n),
                "v_codes": vc.reshape(segs, n, -1), "v_norms": vn.reshape(segs, n)}

    @property
    def _cache(self) -> list:
        """Per-append blocks, (B, H, seq, ...) tensors like the reference keeps."""
        if self._block_cache is None:
            blocks, off = [], 0
            B, H = self._shape if self._shape else (0, 0)
            p = self.row_planes() if self._block_lens else {}
            for n in self._block_lens:
                view = lambda t: t[:, off:off + n].reshape(B, H, n, *t.shape[2:])  # noqa: E731
                mse, sgn, val = view(p["k_codes"]), view(p["k_signs"]), view(p["v_codes"])
                if not self.pack_storage:
                    d = self.head_dim
                    mse = ops.unpack(mse, self.key_bits - 1, d)
                    sgn = ops.unpack(sgn, 1, d)
                    val = ops.unpack(val, self.value_bits, d)
                blocks.append(CompressedKVBlock(mse, sgn, view(p["k_norms"]), val, view(p["v_norms"]), n,
                                                self.pack_storage))
                off += n
            self._block_cache = blocks
        return self._block_cache

    def _unpack_block(self, block: CompressedKVBlock):
        """(mse_indices, qjl_signs, val_indices) as one uint8 per coordinate."""
        if not block.packed:
            return block.mse_indices, block.qjl_signs, block.val_indices
        d = self.head_dim
        return (ops.unpack(block.mse_indices, self.key_bits - 1, d), ops.unpack(block.qjl_signs, 1, d),
                ops.unpack(block.val_indices, self.value_bits, d))

    # ---- attention --------------------------------------------------------------------------
    def attention(self, queries: torch.Tensor, scale: Optional[float] = None, causal: bool = False) -> torch.Tensor:
        """queries (batch, q_heads, q_len, head_dim) -> (batch, q_heads, q_len, head_dim) fp32.

        With ``causal`` the q_len queries are the last q_len positions of the cache."""
        if not self._block_lens:
            raise ValueError("No compressed KV blocks in cache. Call append() first.")
        ops._need_cuda(queries, "QuashKVEngine.attention")
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_dim)
        B, Hq, Q, D = queries.shape
        Bc, Hkv = self._shape
        if B != Bc or D != self.head_dim or Hq % Hkv != 0:
            raise ValueError(f"queries {tuple(queries.shape)} do not match a cache of batch {Bc}, "
                             f"{Hkv} KV heads, head_dim {self.head_dim}")
        kq, vq = self.key_quantizer, self.value_quantizer
        Pi, _, k_cents, Sgn = kq._on(queries.device)
        _, _, v_cents = vq._on(queries.device)
        p = self._planes
        if self._tiled:
            call = self._tiled_call
            if call is None or call.device != queries.device or call.consts[0].data_ptr() != Pi.data_ptr():
                call = self._tiled_call = ops.TiledAttentionCall(Pi, k_cents, v_cents, Sgn, kq.qjl_scale)
            with torch.cuda.device(queries.device):
                return call(queries.detach(), p["records"], self._capacity, self._total_tokens, Hkv, float(scale),
                            bool(causal))
        call = self._row_call
        if call is None or call.device != queries.device or call.consts[0].data_ptr() != Pi.data_ptr():
            call = self._row_call = ops.RowAttentionCall(Pi, k_cents, v_cents, Sgn, kq.qjl_scale, self.key_bits,
                                                         self.value_bits)
        with torch.cuda.device(queries.device):
            return call(queries.detach(), p, self._total_tokens, Hkv, float(scale), bool(causal))

    def attention_from_host(self, queries_host: torch.Tensor, out_host: torch.Tensor,
                            scale: Optional[float] = None, causal: bool = False) -> torch.cuda.Event:
        """Attention for a query that lives in pinned host memory, with the result written to a pinned host
        buffer: ``out_host`` (batch, q_heads, q_len, head_dim) fp32 holds the output once the returned event
        has completed.  The two transfers run on side streams with two device buffers in rotation, so that
        back-to-back calls (decode steps of different requests, layers of a pipeline) overlap their copies
        with each other's kernels; ``queries_host`` must stay unchanged until the event completes.  The
        reference has no counterpart: its tensors are wherever the caller put them."""
        if not (queries_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("attention_from_host expects pinned host tensors")
        if out_host.dtype != torch.float32 or out_host.shape != queries_host.shape:
            raise ValueError("out_host must be fp32 with the shape of the queries")
        dev = self._device() if self._planes is not None else None
        if dev is None:
            raise ValueError("No compressed KV blocks in cache. Call append() first.")
        if self._tiled and os.environ.get("QUASHKV_B200_HOST_IO") != "torch":
            return self._attention_from_host_lean(queries_host, out_host, dev, scale, causal)
        io = getattr(self, "_host_io", None)
        if io is None or io["device"] != dev:
            io = self._host_io = {"device": dev, "h2d": torch.cuda.Stream(dev), "d2h": torch.cuda.Stream(dev),
                                  "slots": [{"q": None, "free": None} for _ in range(2)], "n": 0}
        slot = io["slots"][io["n"] % 2]
        io["n"] += 1
        compute = torch.cuda.current_stream(dev)
        if slot["q"] is None or slot["q"].shape != queries_host.shape or slot["q"].dtype != queries_host.dtype:
            slot["q"] = torch.empty(queries_host.shape, dtype=queries_host.dtype, device=dev)
            slot["free"] = None
        with torch.cuda.stream(io["h2d"]):
            if slot["free"] is not None:
                io["h2d"].wait_event(slot["free"])          # the kernels that read this buffer two calls ago
            slot["q"].copy_(queries_host, non_blocking=True)
            arrived = io["h2d"].record_event()
        compute.wait_event(arrived)
        out = self.attention(slot["q"], scale=scale, causal=causal)
        slot["free"] = compute.record_event()
        with torch.cuda.stream(io["d2h"]):
            io["d2h"].wait_event(slot["free"])
            out_host.copy_(out, non_blocking=True)
            out.record_stream(io["d2h"])                    # the allocator must not reuse it before the copy ran
            return io["d2h"].record_event()

    def _attention_from_host_lean(self, queries_host, out_host, dev, scale, causal) -> torch.cuda.Event:
        """The same three-stream pipeline for a tiled cache with the host work cut down: device buffers for the
        queries and the outputs are kept per slot, the copies and the ordering between the streams go through the
        CUDA runtime directly (raw stream and event handles), and the attention call writes into the slot's
        output buffer.  A decode step over one KV head of a sharded cache lasts about 55 us on the device; the
        generic path spends more than that on the host."""
        rt = ops.cudart()
        io = getattr(self, "_host_io_lean", None)
        if io is None or io["device"] != dev:
            with torch.cuda.device(dev):
                io = self._host_io_lean = {
                    "device": dev, "h2d": torch.cuda.Stream(dev), "d2h": torch.cuda.Stream(dev), "n": 0,
                    "slots": [{"q": None, "out": None, "arrived": torch.cuda.Event(), "computed": torch.cuda.Event(),
                               "copied": torch.cuda.Event()} for _ in range(2)]}
                for sl in io["slots"]:                    # an event has a handle once it has been recorded
                    for name in ("arrived", "computed", "copied"):
                        sl[name].record(io["h2d"])
        slot = io["slots"][io["n"] % 2]
        io["n"] += 1
        if slot["q"] is None or slot["q"].shape != queries_host.shape or slot["q"].dtype != queries_host.dtype:
            torch.cuda.synchronize(dev)                   # (re)allocation: nothing may still use the old buffers
            slot["q"] = torch.empty(queries_host.shape, dtype=queries_host.dtype, device=dev)
            slot["out"] = torch.empty(queries_host.shape, dtype=torch.float32, device=dev)
        compute = torch.cuda.current_stream(dev).cuda_stream
        h2d, d2h = io["h2d"].cuda_stream, io["d2h"].cuda_stream
        arrived, computed, copied = (slot[k].cuda_event for k in ("arrived", "computed", "copied"))
        kq, vq = self.key_quantizer, self.value_quantizer
        Pi, _, k_cents, Sgn = kq._on(dev)
        _, _, v_cents = vq._on(dev)
        call = self._tiled_call
        if call is None or call.device != dev or call.consts[0].data_ptr() != Pi.data_ptr():
            call = self._tiled_call = ops.TiledAttentionCall(Pi, k_cents, v_cents, Sgn, kq.qjl_scale)
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_dim)
        B, Hq = queries_host.shape[0], queries_host.shape[1]
        Hkv = self._shape[1]
        if B != self._shape[0] or Hq % Hkv != 0 or queries_host.shape[-1] != self.head_dim:
            raise ValueError(f"queries {tuple(queries_host.shape)} do not match a cache of {self._shape[0]} x {Hkv} heads")
        ok = 0
        # the slot's query buffer is free once the kernels of two calls ago have read it (computed), its output
        # buffer once that call's copy back has read it (copied)
        ok |= rt.cudaStreamWaitEvent(h2d, computed, 0)
        ok |= rt.cudaMemcpyAsync(slot["q"].data_ptr(), queries_host.data_ptr(),
                                 queries_host.numel() * queries_host.element_size(), 1, h2d)
        ok |= rt.cudaEventRecord(arrived, h2d)
        ok |= rt.cudaStreamWaitEvent(compute, arrived, 0)
        ok |= rt.cudaStreamWaitEvent(compute, copied, 0)
        with torch.cuda.device(dev):
            call(slot["q"], self._planes["records"], self._capacity, self._total_tokens, Hkv, float(scale),
                 bool(causal), out=slot["out"], stream=compute)
        ok |= rt.cudaEventRecord(computed, compute)
        ok |= rt.cudaStreamWaitEvent(d2h, computed, 0)
        ok |= rt.cudaMemcpyAsync(out_host.data_ptr(), slot["out"].data_ptr(), out_host.numel() * 4, 2, d2h)
        ok |= rt.cudaEventRecord(copied, d2h)
        if ok != 0:
            raise RuntimeError("quashkv_b200: a CUDA runtime call of the host-buffer path failed")
        done = torch.cuda.Event()
        done.record(io["d2h"])
        return done

    # ---- decompression of the whole cache (used by the HF-style cache) ----------------------------
    def decompress_all(self, with_signs: bool = False, out_dtype=torch.float32):
        """(keys, values) of shape (batch, heads, total_tokens, head_dim).  Keys use the code
        centroids only unless ``with_signs`` adds the sign term."""
        B, H = self._shape
        n, d = self._total_tokens, self.head_dim
        p = self.row_planes()
        stride = p["k_norms"].stride(0)          # rows between segments: n for untiled copies, the capacity for views
        kq, vq = self.key_quantizer, self.value_quantizer
        dev = self._device()
        Pi, _, k_cents, Sgn = kq._on(dev)
        _, _, v_cents = vq._on(dev)
        keys = ops.decompress_rows(p["k_codes"], p["k_norms"], Pi, k_cents, kq.mse_bits, d, B * H, n,
                                   stride, 0, signs=p["k_signs"] if with_signs else None,
                                   S=Sgn if with_signs else None, qjl_scale=kq.qjl_scale, out_dtype=out_dtype)
        vals = ops.decompress_rows(p["v_codes"], p["v_norms"], Pi, v_cents, self.value_bits, d, B * H, n,
                                   stride, 0, out_dtype=out_dtype)
        return keys.reshape(B, H, n, d), vals.reshape(B, H, n, d)

    # ---- statistics (formulas of reference engine.py:305-337) -------------------------------------
    def compression_ratio(self, original_dtype: torch.dtype = torch.float16) -> float:
        if not self._block_lens:
            return 1.0
        orig_bits = torch.finfo(original_dtype).bits
        per_token = 2 * self.head_dim * orig_bits
        compressed = self.key_bits * self.head_dim + 32 + self.value_bits * self.head_dim + 32
        return per_token / compressed

    def actual_memory_bytes(self) -> int:
        """Bytes of the stored blocks: packed rows, or one byte per coordinate when
        ``pack_storage=False`` (what the reference would hold), plus fp32 norms."""
        if not self._block_lens:
            return 0
        B, H = self._shape
        d = self.head_dim
        pk, ps, pv = self._row_bytes() if self.pack_storage else (d, d, d)
        return B * H * self._total_tokens * (pk + ps + pv + 8)

    def to(self, device) -> "QuashKVEngine":
        self.device = torch.device(device)
        self.key_quantizer.to(device)
        self.value_quantizer.to(device)
        if self._planes is not None:
            self._planes = {k: v.to(device) for k, v in self._planes.items()}
            self._block_cache = None
        return self

    def __repr__(self) -> str:
        return (f"QuashKVEngine(head_dim={self.head_dim}, key_bits={self.key_bits}, "
                f"value_bits={self.value_bits}, cached_tokens={self._total_tokens}, "
                f"blocks={len(self._block_lens)}, device={self.device})")
