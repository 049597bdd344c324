"""ctypes binding of ``libquashkv_b200.so`` (the C ABI declared in include/quashkv_b200.h).

The library is the product: there is no Python or CPU implementation behind it.
``lib()`` raises if the shared object is missing, and every wrapper turns a
non-zero status into ``RuntimeError`` with the library's own message.
"""

from __future__ import annotations

import ctypes as C
import os

from ._build import LIB_PATH

F32, BF16, F16 = 0, 1, 2
INDEX_MAX_K = 128

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t


class Rows(C.Structure):
    """qkv_rows_t: vector n lives at row (n // seg_len) * seg_stride + seg_off + n % seg_len."""
    _fields_ = [("seg_len", _i64), ("seg_stride", _i64), ("seg_off", _i64)]


class Cache(C.Structure):
    """qkv_cache_t: the five packed planes of a [segments, capacity, ...] cache."""
    _fields_ = [("k_codes", _vp), ("k_signs", _vp), ("k_norms", _vp), ("v_codes", _vp),
                ("v_norms", _vp), ("capacity", _i64)]


class PagedCache(C.Structure):
    """qkv_paged_cache_t: the five packed planes of a [blocks, kv heads, block_size, ...] pool, the
    (B, max_blocks) int32 block table and the (B) int32 token counts."""
    _fields_ = [("k_codes", _vp), ("k_signs", _vp), ("k_norms", _vp), ("v_codes", _vp), ("v_norms", _vp),
                ("block_table", _vp), ("seq_lens", _vp), ("max_blocks", _i), ("block_size", _i)]


class TiledCache(C.Structure):
    """qkv_tiled_cache_t: 16-token tile records, contiguous per (batch, kv head) or paged through a block table."""
    _fields_ = [("records", _vp), ("capacity", _i64), ("block_table", _vp), ("seq_lens", _vp),
                ("max_blocks", _i), ("block_size", _i)]


TILE_TOKENS, TILE_BYTES = 16, 1664

# symbol -> (restype, argtypes); every symbol include/quashkv_b200.h declares is listed here
SIGNATURES = {
    "qkv_abi_version": (_i, []),
    "qkv_strerror": (C.c_char_p, [_i]),
    "qkv_pack": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "qkv_unpack": (_i, [_vp, _vp, _i64, _i, _i, _vp]),
    "qkv_compress_mse": (_i, [_vp, _i, _i64, _i64, _i, _vp, _vp, _i, _vp, _i, _vp, Rows, _vp]),
    "qkv_compress_ip": (_i, [_vp, _i, _i64, _i64, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _vp, Rows, _vp]),
    "qkv_compress_mixed": (_i, [_vp, _i, _i64, _i64, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _vp, Rows, _vp]),
    "qkv_compress_mixed_ip": (_i, [_vp, _i, _i64, _i64, _i, _vp, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _vp, _vp, _i,
                                   _vp, Rows, _vp]),
    "qkv_mixed_row_bytes": (_i64, [_i, _i, _i, _i]),
    "qkv_decompress": (_i, [_vp, _vp, _i, _vp, Rows, _i64, _i, _vp, _vp, _i, _vp, _f, _vp, _i, _i64, _vp]),
    "qkv_decompress_mixed": (_i, [_vp, _i, _vp, Rows, _i64, _i, _vp, _vp, _vp, _i, _vp, _i, _vp, _i, _i64, _vp]),
    "qkv_attention_workspace_bytes": (_sz, [_i, _i, _i, _i, _i64, _i]),
    "qkv_attention": (_i, [_vp, _i, Cache, _i, _i, _i, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _f, _i,
                           _vp, _vp, _sz, _vp]),
    "qkv_attention_static_scratch": (_i, [_vp, _i, Cache, _i, _i, _i, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp,
                                          _f, _f, _i, _vp, _vp]),
    "qkv_attention_paged": (_i, [_vp, _i, PagedCache, _i, _i, _i, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _f,
                                 _i, _vp, _vp, _sz, _vp]),
    "qkv_tile_rows": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _vp, Rows, _vp, _vp]),
    "qkv_untile_rows": (_i, [_vp, Rows, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp]),
    "qkv_attention_tiled": (_i, [_vp, _i, TiledCache, _i, _i, _i, _i, _i64, _i, _i, _i, _vp, _vp, _vp, _vp, _f, _f,
                                 _i, _vp, _vp, _sz, _vp]),
    "qkv_scatter_rows": (_i, [_vp, _vp, _vp, _i64, _i, _vp]),
    "qkv_index_workspace_bytes": (_sz, [_i64, _i, _i, _i]),
    "qkv_index_scan_topk": (_i, [_vp, _i, _i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _f, _i, _i64, _vp, _vp,
                                 _vp, _sz, _vp]),
    "qkv_index_scores": (_i, [_vp, _i, _i, _vp, _vp, _vp, _i64, _i, _vp, _vp, _vp, _f, _vp, _vp, _sz, _vp]),
    "qkv_topk_merge": (_i, [_vp, _vp, _i, _i64, _i, _vp, _vp, _vp]),
    "qkv_tensor_core_timeouts": (_i64, []),
}

_LIB = None


def lib() -> C.CDLL:
    """Load the shared object once; fail loudly if it has not been built."""
    global _LIB
    if _LIB is None:
        path = os.environ.get("QUASHKV_B200_LIB", LIB_PATH)
        if not os.path.exists(path):
            raise RuntimeError(
                f"quashkv_b200: {path} not found. Build it with `python -m quashkv_b200._build` "
                "(needs nvcc); there is no fallback implementation.")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError if the library lacks a declared symbol
            fn.restype, fn.argtypes = res, args
        if handle.qkv_abi_version() != 1:
            raise RuntimeError("quashkv_b200: ABI version mismatch between header and library")
        _LIB = handle
    return _LIB


def check(code: int, what: str) -> None:
    if code != 0:
        msg = lib().qkv_strerror(code).decode()
        raise RuntimeError(f"quashkv_b200: {what} failed: {msg} (code {code})")
