"""PyTorch custom ops (namespace ``quashkv_b200``) over the C ABI of libquashkv_b200.so.

Each op allocates its outputs and workspace with torch, passes raw device
pointers and the current CUDA stream to one ``extern "C"`` entry point, and
returns.  Only a CUDA implementation is registered: calling an op on CPU
tensors raises from the dispatcher, there is no fallback.

Plain Python wrappers of the same names (``ops.compress_mse(...)``) are what the
host classes call; they normalise shapes and dtypes and then invoke the
registered op.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import Cache, Rows, TILE_BYTES, TILE_TOKENS, TiledCache

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def packed_row_bytes(d: int, bits: int) -> int:
    """Bytes of one packed row: 3-bit rows are whole 8-field groups (3 bytes each), like the
    reference's pack_bits (quashkv/packing.py:61-81); otherwise ceil(d*bits/8)."""
    if bits == 8:
        return d
    return 3 * ((d + 7) // 8) if bits == 3 else (d * bits + 7) // 8


def _p(t: Optional[torch.Tensor]):
    """Device pointer of a tensor for the C call.  A host pointer must never reach a kernel: anything that is
    not a CUDA tensor is refused here."""
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError(f"quashkv_b200: expected a CUDA tensor, got one on {t.device}")
    return C.c_void_p(t.data_ptr())


def _same_device(device: torch.device, *tensors: Optional[torch.Tensor]) -> None:
    """Data tensors (codes, norms, records, tables of indices) are not moved for the caller: they have to be on
    the device the call runs on."""
    for t in tensors:
        if t is not None and t.device != device:
            raise ValueError(f"quashkv_b200: tensors of one call on different devices ({t.device} and {device})")


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _f32(t: torch.Tensor, device: Optional[torch.device] = None) -> torch.Tensor:
    """fp32, contiguous, and on `device` when one is given (small constants such as Pi, tables and S follow the
    data; the quantizer classes keep per-device copies, the functional entry points convert per call)."""
    t = t.detach()
    return t.to(device=t.device if device is None else device, dtype=torch.float32).contiguous()


class _Keep:
    """Device pointers of converted arguments, with the converted tensors held until the C call has
    returned: a pointer taken from a temporary would otherwise outlive its storage, and the next allocation
    on the stream could hand that storage out again before the kernel has read it."""

    def __init__(self, device: torch.device):
        self.held = []
        self.device = device

    def f32(self, t: Optional[torch.Tensor]):
        if t is None:
            return None
        t = _f32(t, self.device)
        self.held.append(t)
        return _p(t)

    def u8(self, t: torch.Tensor):
        t = t.detach().to(device=self.device, dtype=torch.uint8).contiguous()
        self.held.append(t)
        return _p(t)


def _flat(x: torch.Tensor):
    d = x.shape[-1]
    if x.dtype not in _DT:
        x = x.float()
    return x.detach().reshape(-1, d).contiguous(), d


def _dense(n: int) -> Rows:
    return Rows(max(n, 1), 0, 0)


# ---------------------------------------------------------------------------------------------
# op implementations (CUDA only)
# ---------------------------------------------------------------------------------------------

@torch.library.custom_op("quashkv_b200::pack", mutates_args=(), device_types="cuda")
def _pack(codes: torch.Tensor, bits: int) -> torch.Tensor:
    d = codes.shape[-1]
    flat = codes.reshape(-1, d).contiguous()
    out = torch.empty((flat.shape[0], packed_row_bytes(d, bits)), dtype=torch.uint8, device=codes.device)
    A = _Keep(codes.device)
    with torch.cuda.device(codes.device):
        _lib.check(_lib.lib().qkv_pack(_p(flat), _p(out), flat.shape[0], d, bits, _stream(codes)), "pack")
    return out.reshape(*codes.shape[:-1], out.shape[1])


@_pack.register_fake
def _(codes, bits):
    return codes.new_empty((*codes.shape[:-1], packed_row_bytes(codes.shape[-1], bits)))


@torch.library.custom_op("quashkv_b200::unpack", mutates_args=(), device_types="cuda")
def _unpack(packed: torch.Tensor, bits: int, d: int) -> torch.Tensor:
    flat = packed.reshape(-1, packed.shape[-1])
    need = packed_row_bytes(d, bits)
    if flat.shape[1] < need:
        raise ValueError(f"packed rows of {flat.shape[1]} bytes cannot hold {d} fields of {bits} bits")
    flat = flat[:, :need].contiguous()
    out = torch.empty((flat.shape[0], d), dtype=torch.uint8, device=packed.device)
    A = _Keep(packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().qkv_unpack(_p(flat), _p(out), flat.shape[0], d, bits, _stream(packed)), "unpack")
    return out.reshape(*packed.shape[:-1], d)


@_unpack.register_fake
def _(packed, bits, d):
    return packed.new_empty((*packed.shape[:-1], d))


@torch.library.custom_op("quashkv_b200::compress_mse", mutates_args=(), device_types="cuda")
def _compress_mse(x: torch.Tensor, Pi: torch.Tensor, boundaries: torch.Tensor, bits: int,
                  packed: bool) -> tuple[torch.Tensor, torch.Tensor]:
    flat, d = _flat(x)
    n = flat.shape[0]
    width = packed_row_bytes(d, bits) if packed else d
    codes = torch.empty((n, width), dtype=torch.uint8, device=x.device)
    norms = torch.empty((n,), dtype=torch.float32, device=x.device)
    A = _Keep(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().qkv_compress_mse(
            _p(flat), _DT[flat.dtype], d, n, d, A.f32(Pi), A.f32(boundaries), bits,
            _p(codes), int(packed), _p(norms), _dense(n), _stream(x)), "compress_mse")
    return codes.reshape(*x.shape[:-1], width), norms.reshape(x.shape[:-1])


@_compress_mse.register_fake
def _(x, Pi, boundaries, bits, packed):
    d = x.shape[-1]
    width = packed_row_bytes(d, bits) if packed else d
    return (x.new_empty((*x.shape[:-1], width), dtype=torch.uint8),
            x.new_empty(x.shape[:-1], dtype=torch.float32))


@torch.library.custom_op("quashkv_b200::compress_ip", mutates_args=(), device_types="cuda")
def _compress_ip(x: torch.Tensor, Pi: torch.Tensor, boundaries: torch.Tensor, centroids: torch.Tensor,
                 S: torch.Tensor, mse_bits: int, packed: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    flat, d = _flat(x)
    n = flat.shape[0]
    cw = packed_row_bytes(d, mse_bits) if packed else d
    sw = packed_row_bytes(d, 1) if packed else d
    codes = torch.empty((n, cw), dtype=torch.uint8, device=x.device)
    signs = torch.empty((n, sw), dtype=torch.uint8, device=x.device)
    norms = torch.empty((n,), dtype=torch.float32, device=x.device)
    A = _Keep(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().qkv_compress_ip(
            _p(flat), _DT[flat.dtype], d, n, d, A.f32(Pi), A.f32(boundaries), A.f32(centroids),
            mse_bits, A.f32(S), _p(codes), _p(signs), int(packed), _p(norms), _dense(n), _stream(x)),
            "compress_ip")
    lead = x.shape[:-1]
    return codes.reshape(*lead, cw), signs.reshape(*lead, sw), norms.reshape(lead)


@_compress_ip.register_fake
def _(x, Pi, boundaries, centroids, S, mse_bits, packed):
    d = x.shape[-1]
    cw = packed_row_bytes(d, mse_bits) if packed else d
    sw = packed_row_bytes(d, 1) if packed else d
    return (x.new_empty((*x.shape[:-1], cw), dtype=torch.uint8),
            x.new_empty((*x.shape[:-1], sw), dtype=torch.uint8),
            x.new_empty(x.shape[:-1], dtype=torch.float32))


@torch.library.custom_op("quashkv_b200::append_kv", mutates_args=("k_codes", "k_signs", "k_norms", "v_codes", "v_norms"),
                         device_types="cuda")
def _append_kv(keys: torch.Tensor, values: torch.Tensor, Pi: torch.Tensor,
               k_bounds: torch.Tensor, k_cents: torch.Tensor, S: torch.Tensor, mse_bits: int,
               v_bounds: torch.Tensor, val_bits: int,
               k_codes: torch.Tensor, k_signs: torch.Tensor, k_norms: torch.Tensor,
               v_codes: torch.Tensor, v_norms: torch.Tensor, offset: int) -> None:
    """Compress (B,H,S,d) keys and values straight into the packed cache planes
    [B*H, capacity, ...] at rows offset..offset+S of every (batch, head) segment."""
    kf, d = _flat(keys)
    vf, _ = _flat(values)
    s_new = keys.shape[-2]
    cap = k_norms.shape[-1]
    rows = Rows(s_new, cap, offset)
    _same_device(keys.device, values, k_codes, k_signs, k_norms, v_codes, v_norms)
    Pi32 = _f32(Pi, keys.device)
    A = _Keep(keys.device)
    with torch.cuda.device(keys.device):
        L = _lib.lib()
        _lib.check(L.qkv_compress_ip(
            _p(kf), _DT[kf.dtype], d, kf.shape[0], d, _p(Pi32), A.f32(k_bounds), A.f32(k_cents), mse_bits,
            A.f32(S), _p(k_codes), _p(k_signs), 1, _p(k_norms), rows, _stream(keys)), "append keys")
        _lib.check(L.qkv_compress_mse(
            _p(vf), _DT[vf.dtype], d, vf.shape[0], d, _p(Pi32), A.f32(v_bounds), val_bits,
            _p(v_codes), 1, _p(v_norms), rows, _stream(keys)), "append values")


@torch.library.custom_op("quashkv_b200::compress_ip_into", mutates_args=("codes", "signs", "norms"),
                         device_types="cuda")
def _compress_ip_into(x: torch.Tensor, Pi: torch.Tensor, boundaries: torch.Tensor, centroids: torch.Tensor,
                      S: torch.Tensor, mse_bits: int, codes: torch.Tensor, signs: torch.Tensor,
                      norms: torch.Tensor, offset: int) -> None:
    """Compress (N,d) vectors into packed planes [capacity, bytes] at rows offset..offset+N."""
    flat, d = _flat(x)
    n = flat.shape[0]
    A = _Keep(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().qkv_compress_ip(
            _p(flat), _DT[flat.dtype], d, n, d, A.f32(Pi), A.f32(boundaries), A.f32(centroids),
            mse_bits, A.f32(S), _p(codes), _p(signs), 1, _p(norms), Rows(max(n, 1), 0, offset),
            _stream(x)), "compress_ip_into")


@torch.library.custom_op("quashkv_b200::compress_mixed", mutates_args=(), device_types="cuda")
def _compress_mixed(x: torch.Tensor, Pi: torch.Tensor, is_outlier: torch.Tensor,
                    bounds_out: torch.Tensor, bits_out: int, bounds_reg: torch.Tensor, bits_reg: int,
                    packed: bool, n_out: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``n_out`` = number of marked channels of ``is_outlier`` (known on the host, so that the packed row width
    needs no device read)."""
    flat, d = _flat(x)
    n = flat.shape[0]
    width = int(_lib.lib().qkv_mixed_row_bytes(d, n_out, bits_out, bits_reg)) if packed else d
    codes = torch.empty((n, width), dtype=torch.uint8, device=x.device)
    norms = torch.empty((n,), dtype=torch.float32, device=x.device)
    A = _Keep(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().qkv_compress_mixed(
            _p(flat), _DT[flat.dtype], d, n, d, A.f32(Pi), A.u8(is_outlier), A.f32(bounds_out), bits_out,
            A.f32(bounds_reg), bits_reg, _p(codes), int(packed), _p(norms), _dense(n), _stream(x)),
            "compress_mixed")
    return codes.reshape(*x.shape[:-1], width), norms.reshape(x.shape[:-1])


@_compress_mixed.register_fake
def _(x, Pi, is_outlier, bounds_out, bits_out, bounds_reg, bits_reg, packed, n_out):
    d = x.shape[-1]
    width = (n_out * bits_out + 7) // 8 + ((d - n_out) * bits_reg + 7) // 8 if packed else d
    return (x.new_empty((*x.shape[:-1], width), dtype=torch.uint8),
            x.new_empty(x.shape[:-1], dtype=torch.float32))


@torch.library.custom_op("quashkv_b200::compress_mixed_ip", mutates_args=(), device_types="cuda")
def _compress_mixed_ip(x: torch.Tensor, Pi: torch.Tensor, is_outlier: torch.Tensor,
                       bounds_out: torch.Tensor, cents_out: torch.Tensor, bits_out: int,
                       bounds_reg: torch.Tensor, cents_reg: torch.Tensor, bits_reg: int,
                       S: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Mixed-precision codes and residual sign bits, one uint8 per coordinate each, and the norms."""
    flat, d = _flat(x)
    n = flat.shape[0]
    codes = torch.empty((n, d), dtype=torch.uint8, device=x.device)
    signs = torch.empty((n, d), dtype=torch.uint8, device=x.device)
    norms = torch.empty((n,), dtype=torch.float32, device=x.device)
    A = _Keep(x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().qkv_compress_mixed_ip(
            _p(flat), _DT[flat.dtype], d, n, d, A.f32(Pi), A.u8(is_outlier), A.f32(bounds_out), A.f32(cents_out),
            bits_out, A.f32(bounds_reg), A.f32(cents_reg), bits_reg, A.f32(S), _p(codes), _p(signs), 0, _p(norms),
            _dense(n), _stream(x)), "compress_mixed_ip")
    lead = x.shape[:-1]
    return codes.reshape(*lead, d), signs.reshape(*lead, d), norms.reshape(lead)


@_compress_mixed_ip.register_fake
def _(x, Pi, is_outlier, bounds_out, cents_out, bits_out, bounds_reg, cents_reg, bits_reg, S):
    return (x.new_empty(x.shape, dtype=torch.uint8), x.new_empty(x.shape, dtype=torch.uint8),
            x.new_empty(x.shape[:-1], dtype=torch.float32))


@torch.library.custom_op("quashkv_b200::decompress", mutates_args=(), device_types="cuda")
def _decompress(codes: torch.Tensor, signs: Optional[torch.Tensor], norms: torch.Tensor, Pi: torch.Tensor,
                centroids: torch.Tensor, bits: int, S: Optional[torch.Tensor], qjl_scale: float,
                packed: bool, d: int, seg_len: int, seg_stride: int, seg_off: int, n_vec: int,
                out_dtype: torch.dtype) -> torch.Tensor:
    """Rows of the code/norm planes are addressed with (seg_len, seg_stride, seg_off); the
    output is dense (n_vec, d)."""
    out = torch.empty((n_vec, d), dtype=out_dtype, device=codes.device)
    _same_device(codes.device, codes, signs, norms)
    A = _Keep(codes.device)
    with torch.cuda.device(codes.device):
        _lib.check(_lib.lib().qkv_decompress(
            _p(codes), _p(signs), int(packed), _p(norms), Rows(seg_len, seg_stride, seg_off), n_vec, d,
            A.f32(Pi), A.f32(centroids), bits, A.f32(S), float(qjl_scale),
            _p(out), _DT[out_dtype], d, _stream(codes)), "decompress")
    return out


@_decompress.register_fake
def _(codes, signs, norms, Pi, centroids, bits, S, qjl_scale, packed, d, seg_len, seg_stride, seg_off,
      n_vec, out_dtype):
    return codes.new_empty((n_vec, d), dtype=out_dtype)


@torch.library.custom_op("quashkv_b200::decompress_mixed", mutates_args=(), device_types="cuda")
def _decompress_mixed(codes: torch.Tensor, norms: torch.Tensor, Pi: torch.Tensor, is_outlier: torch.Tensor,
                      cents_out: torch.Tensor, bits_out: int, cents_reg: torch.Tensor, bits_reg: int,
                      packed: bool, d: int) -> torch.Tensor:
    flat = codes.reshape(-1, codes.shape[-1]).contiguous()
    n = flat.shape[0]
    out = torch.empty((n, d), dtype=torch.float32, device=codes.device)
    _same_device(codes.device, codes, norms)
    A = _Keep(codes.device)
    with torch.cuda.device(codes.device):
        _lib.check(_lib.lib().qkv_decompress_mixed(
            _p(flat), int(packed), A.f32(norms.reshape(-1)), _dense(n), n, d, A.f32(Pi),
            A.u8(is_outlier), A.f32(cents_out), bits_out,
            A.f32(cents_reg), bits_reg, _p(out), _lib.F32, d, _stream(codes)), "decompress_mixed")
    return out.reshape(*codes.shape[:-1], d)


@_decompress_mixed.register_fake
def _(codes, norms, Pi, is_outlier, cents_out, bits_out, cents_reg, bits_reg, packed, d):
    return codes.new_empty((*codes.shape[:-1], d), dtype=torch.float32)


@torch.library.custom_op("quashkv_b200::attention", mutates_args=(), device_types="cuda")
def _attention(q: torch.Tensor, k_codes: torch.Tensor, k_signs: torch.Tensor, k_norms: torch.Tensor,
               v_codes: torch.Tensor, v_norms: torch.Tensor, kv_len: int, n_kv_heads: int,
               key_bits: int, val_bits: int, Pi: torch.Tensor, key_centroids: torch.Tensor,
               val_centroids: torch.Tensor, S: torch.Tensor, qjl_scale: float, scale: float,
               causal: bool) -> torch.Tensor:
    """q (B,Hq,Q,d); planes [B*Hkv, capacity, bytes] packed; returns (B,Hq,Q,d) fp32."""
    B, Hq, Q, d = q.shape
    if q.dtype not in _DT:
        q = q.float()
    qc = q.detach().contiguous()
    cap = k_norms.shape[-1]
    out = torch.empty((B, Hq, Q, d), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    ws_bytes = L.qkv_attention_workspace_bytes(B, Hq, n_kv_heads, Q, kv_len, d)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=q.device)
    _same_device(q.device, k_codes, k_signs, k_norms, v_codes, v_norms)
    _p(k_codes)                                        # refuses anything that is not device memory
    cache = Cache(k_codes.data_ptr(), k_signs.data_ptr(), k_norms.data_ptr(), v_codes.data_ptr(),
                  v_norms.data_ptr(), cap)
    A = _Keep(q.device)
    with torch.cuda.device(q.device):
        _lib.check(L.qkv_attention(
            _p(qc), _DT[qc.dtype], cache, B, Hq, n_kv_heads, Q, kv_len, d, key_bits, val_bits,
            A.f32(Pi), A.f32(key_centroids), A.f32(val_centroids), A.f32(S),
            float(qjl_scale), float(scale), int(causal), _p(out), _p(ws), ws_bytes, _stream(q)), "attention")
    return out


@_attention.register_fake
def _(q, k_codes, k_signs, k_norms, v_codes, v_norms, kv_len, n_kv_heads, key_bits, val_bits, Pi,
      key_centroids, val_centroids, S, qjl_scale, scale, causal):
    return q.new_empty(q.shape, dtype=torch.float32)


@torch.library.custom_op("quashkv_b200::attention_paged", mutates_args=(), device_types="cuda")
def _attention_paged(q: torch.Tensor, k_codes: torch.Tensor, k_signs: torch.Tensor, k_norms: torch.Tensor,
                     v_codes: torch.Tensor, v_norms: torch.Tensor, block_table: torch.Tensor,
                     seq_lens: torch.Tensor, max_kv_len: int, key_bits: int, val_bits: int, Pi: torch.Tensor,
                     key_centroids: torch.Tensor, val_centroids: torch.Tensor, S: torch.Tensor,
                     qjl_scale: float, scale: float, causal: bool) -> torch.Tensor:
    """q (B,Hq,Q,d); pool planes [blocks, Hkv, block_size, bytes] packed; block_table (B, max_blocks) int32;
    seq_lens (B) int32; max_kv_len an upper bound of seq_lens known on the host.  Returns (B,Hq,Q,d) fp32."""
    B, Hq, Q, d = q.shape
    if q.dtype not in _DT:
        q = q.float()
    qc = q.detach().contiguous()
    n_kv_heads, block_size = k_norms.shape[1], k_norms.shape[2]
    out = torch.empty((B, Hq, Q, d), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    ws_bytes = L.qkv_attention_workspace_bytes(B, Hq, n_kv_heads, Q, max_kv_len, d)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=q.device)
    _same_device(q.device, k_codes, k_signs, k_norms, v_codes, v_norms, block_table, seq_lens)
    _p(k_codes)
    pool = _lib.PagedCache(k_codes.data_ptr(), k_signs.data_ptr(), k_norms.data_ptr(), v_codes.data_ptr(),
                           v_norms.data_ptr(), block_table.data_ptr(), seq_lens.data_ptr(),
                           block_table.shape[1], block_size)
    A = _Keep(q.device)
    with torch.cuda.device(q.device):
        _lib.check(L.qkv_attention_paged(
            _p(qc), _DT[qc.dtype], pool, B, Hq, n_kv_heads, Q, max_kv_len, d, key_bits, val_bits,
            A.f32(Pi), A.f32(key_centroids), A.f32(val_centroids), A.f32(S),
            float(qjl_scale), float(scale), int(causal), _p(out), _p(ws), ws_bytes, _stream(q)), "attention_paged")
    return out


@_attention_paged.register_fake
def _(q, k_codes, k_signs, k_norms, v_codes, v_norms, block_table, seq_lens, max_kv_len, key_bits, val_bits, Pi,
      key_centroids, val_centroids, S, qjl_scale, scale, causal):
    return q.new_empty(q.shape, dtype=torch.float32)


@torch.library.custom_op("quashkv_b200::scatter_rows", mutates_args=("dst",), device_types="cuda")
def _scatter_rows(src: torch.Tensor, dst: torch.Tensor, slots: torch.Tensor) -> None:
    """Row i of src (n, ...) goes to row slots[i] of dst (rows, ...); rows are whole trailing slices."""
    n = slots.numel()
    row_bytes = (src.numel() // max(n, 1)) * src.element_size()
    _same_device(src.device, src, dst, slots)
    A = _Keep(src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().qkv_scatter_rows(_p(src), _p(dst), _p(slots), n, row_bytes, _stream(src)),
                   "scatter_rows")


# ---- tile records (the cache layout of the tensor-core decode kernel) ---------------------------------

def tiled_layout_ok(d: int, key_bits: int, val_bits: int) -> bool:
    """Tile records exist for head_dim 128 with 3-bit keys and 3-bit values."""
    return d == 128 and key_bits == 3 and val_bits == 3


def tiled_tables_ok(key_centroids: torch.Tensor, value_centroids: torch.Tensor) -> bool:
    """What the tile records and their decode kernel presume of the tables (the kernel writes NaN otherwise):
    a symmetric 8-entry value table and a 4-entry key table that is affine in the two bits of its code."""
    kc, vc = key_centroids.detach().float().cpu(), value_centroids.detach().float().cpu()
    if kc.numel() != 4 or vc.numel() != 8:
        return False
    sym = float((vc + vc.flip(0)).abs().max()) <= 1e-6 * float(vc.abs().max())
    aff = abs(float((kc[3] - kc[2]) - (kc[1] - kc[0]))) <= 1e-6 * float(kc.abs().max())
    return sym and aff


@torch.library.custom_op("quashkv_b200::tile_rows", mutates_args=("records",), device_types="cuda")
def _tile_rows(k_codes: torch.Tensor, k_signs: torch.Tensor, k_norms: torch.Tensor, v_codes: torch.Tensor,
               v_norms: torch.Tensor, records: torch.Tensor, seg_len: int, seg_stride: int, seg_off: int,
               slots: Optional[torch.Tensor]) -> None:
    """File dense packed rows (n, 32 / 16 / 48 bytes, fp32 norms) into 16-token tile records.  Row i goes to
    token slot slots[i], or (i // seg_len) * seg_stride + seg_off + i % seg_len when slots is None."""
    n = k_norms.numel()
    _same_device(records.device, records, k_codes, k_signs, k_norms, v_codes, v_norms, slots)
    A = _Keep(records.device)
    with torch.cuda.device(records.device):
        _lib.check(_lib.lib().qkv_tile_rows(
            _p(k_codes), _p(k_signs), _p(k_norms), _p(v_codes), _p(v_norms), n, _p(records),
            Rows(max(seg_len, 1), seg_stride, seg_off), _p(slots), _stream(records)), "tile_rows")


@torch.library.custom_op("quashkv_b200::untile_rows", mutates_args=(), device_types="cuda")
def _untile_rows(records: torch.Tensor, n_rows: int, seg_len: int, seg_stride: int, seg_off: int,
                 slots: Optional[torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The reference's packed rows of n_rows token slots of a tiled cache: (k_codes (n,32), k_signs (n,16),
    k_norms (n), v_codes (n,48), v_norms (n))."""
    dev = records.device
    kc = torch.empty((n_rows, 32), dtype=torch.uint8, device=dev)
    ks = torch.empty((n_rows, 16), dtype=torch.uint8, device=dev)
    kn = torch.empty((n_rows,), dtype=torch.float32, device=dev)
    vc = torch.empty((n_rows, 48), dtype=torch.uint8, device=dev)
    vn = torch.empty((n_rows,), dtype=torch.float32, device=dev)
    _same_device(dev, records, slots)
    A = _Keep(dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().qkv_untile_rows(
            _p(records), Rows(max(seg_len, 1), seg_stride, seg_off), _p(slots), n_rows, _p(kc), _p(ks), _p(kn),
            _p(vc), _p(vn), _stream(records)), "untile_rows")
    return kc, ks, kn, vc, vn


@_untile_rows.register_fake
def _(records, n_rows, seg_len, seg_stride, seg_off, slots):
    u8 = lambda w: records.new_empty((n_rows, w), dtype=torch.uint8)      # noqa: E731
    f32 = lambda: records.new_empty((n_rows,), dtype=torch.float32)       # noqa: E731
    return u8(32), u8(16), f32(), u8(48), f32()


@torch.library.custom_op("quashkv_b200::attention_tiled", mutates_args=(), device_types="cuda")
def _attention_tiled(q: torch.Tensor, records: torch.Tensor, capacity: int, kv_len: int, n_kv_heads: int,
                     block_table: Optional[torch.Tensor], seq_lens: Optional[torch.Tensor], block_size: int,
                     Pi: torch.Tensor, key_centroids: torch.Tensor, val_centroids: torch.Tensor, S: torch.Tensor,
                     qjl_scale: float, scale: float, causal: bool) -> torch.Tensor:
    """q (B,Hq,Q,128); records [B*Hkv, capacity/16, 1664] (contiguous) or [blocks, Hkv, block_size/16, 1664] with a
    (B, max_blocks) int32 block table and (B) int32 lengths (paged; kv_len is then their host-known upper
    bound).  Returns (B,Hq,Q,128) fp32.  Pi, centroids and S must be contiguous fp32."""
    B, Hq, Q, d = q.shape
    if q.dtype not in _DT:
        q = q.float()
    qc = q.detach().contiguous()
    out = torch.empty((B, Hq, Q, d), dtype=torch.float32, device=q.device)
    L = _lib.lib()
    ws_bytes = L.qkv_attention_workspace_bytes(B, Hq, n_kv_heads, Q, kv_len, d)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=q.device)
    paged = block_table is not None
    _same_device(q.device, records, block_table, seq_lens)
    _p(records)
    cache = TiledCache(records.data_ptr(), capacity, block_table.data_ptr() if paged else None,
                       seq_lens.data_ptr() if paged else None, block_table.shape[1] if paged else 0, block_size)
    Pi32, kc32, vc32, S32 = (_f32(t, q.device) for t in (Pi, key_centroids, val_centroids, S))   # held until the call returns
    A = _Keep(q.device)
    with torch.cuda.device(q.device):
        _lib.check(L.qkv_attention_tiled(
            _p(qc), _DT[qc.dtype], cache, B, Hq, n_kv_heads, Q, kv_len, d, 3, 3, _p(Pi32), _p(kc32), _p(vc32),
            _p(S32), float(qjl_scale), float(scale), int(causal), _p(out), _p(ws), ws_bytes, _stream(q)),
            "attention_tiled")
    return out


class RowAttentionCall:
    """The C call of the ``attention`` op (row-major packed planes; ``QuashKVEngine.attention``, reference
    engine.py:204-299), prepared once for an engine's decode loop:
    constants converted once, the workspace kept and grown when needed, no op dispatcher.  A decode step over a
    short cache is a few tens of microseconds of device work; the generic op spends more than that on the
    host.  One instance serves one stream at a time (the workspace is shared by its calls)."""

    def __init__(self, Pi, key_centroids, val_centroids, S, qjl_scale: float, key_bits: int, val_bits: int):
        self.consts = tuple(_f32(t) for t in (Pi, key_centroids, val_centroids, S))
        self.ptrs = tuple(_p(t) for t in self.consts)
        self.qjl_scale, self.key_bits, self.val_bits = float(qjl_scale), int(key_bits), int(val_bits)
        self.device = self.consts[0].device
        self.ws = None
        self.lib = _lib.lib()
        self.fn = self.lib.qkv_attention

    def __call__(self, q: torch.Tensor, planes: dict, kv_len: int, n_kv_heads: int, scale: float,
                 causal: bool) -> torch.Tensor:
        B, Hq, Q, d = q.shape
        if q.dtype not in _DT:
            q = q.float()
        qc = q if q.is_contiguous() else q.contiguous()
        kn = planes["k_norms"]
        if qc.device != self.device or kn.device != self.device:
            raise ValueError(f"quashkv_b200: queries on {qc.device}, planes on {kn.device}, constants on {self.device}")
        out = torch.empty((B, Hq, Q, d), dtype=torch.float32, device=q.device)
        need = self.lib.qkv_attention_workspace_bytes(B, Hq, n_kv_heads, Q, kv_len, d)
        if self.ws is None or self.ws.numel() < need:
            self.ws = torch.empty((max(need + need // 4, 1 << 16),), dtype=torch.uint8, device=q.device)
        cache = Cache(planes["k_codes"].data_ptr(), planes["k_signs"].data_ptr(), kn.data_ptr(),
                      planes["v_codes"].data_ptr(), planes["v_norms"].data_ptr(), kn.shape[-1])
        rc = self.fn(qc.data_ptr(), _DT[qc.dtype], cache, B, Hq, n_kv_heads, Q, kv_len, d, self.key_bits,
                     self.val_bits, *self.ptrs, self.qjl_scale, scale, int(causal), out.data_ptr(),
                     self.ws.data_ptr(), self.ws.numel(), torch.cuda.current_stream(q.device).cuda_stream)
        if rc:
            _lib.check(rc, "attention")
        return out


class AppendCall:
    """Compression of new keys and values into an engine's storage (``QuashKVEngine.append``, reference
    engine.py:145-172), prepared once: constants converted once,
    the staging planes of a tiled cache kept between calls, the library called directly.  The generic ops cost
    80-120 us of host time per one-token append (dispatcher, conversions, five allocations)."""

    def __init__(self, Pi, k_bounds, k_cents, S, mse_bits: int, v_bounds, val_bits: int):
        self.consts = tuple(_f32(t) for t in (Pi, k_bounds, k_cents, S, v_bounds))
        self.Pi, self.kb, self.kc, self.S, self.vb = (_p(t) for t in self.consts)
        self.mse_bits, self.val_bits = int(mse_bits), int(val_bits)
        self.device = self.consts[0].device
        self.lib = _lib.lib()
        self.stage = None           # tiled: (k_codes, k_signs, k_norms, v_codes, v_norms) for up to stage_rows rows
        self.stage_rows = 0
        self.stage_stream = None    # the staging planes belong to the stream they were last used on

    def _compress(self, keys, values, ptrs, rows: "Rows", stream) -> None:
        kf, d = _flat(keys)
        vf, _ = _flat(values)
        if kf.device != self.device or vf.device != self.device:
            raise ValueError(f"quashkv_b200: keys on {kf.device}, constants on {self.device}")
        L = self.lib
        rc = L.qkv_compress_ip(kf.data_ptr(), _DT[kf.dtype], d, kf.shape[0], d, self.Pi, self.kb, self.kc,
                               self.mse_bits, self.S, ptrs[0], ptrs[1], 1, ptrs[2], rows, stream)
        if rc:
            _lib.check(rc, "append keys")
        rc = L.qkv_compress_mse(vf.data_ptr(), _DT[vf.dtype], d, vf.shape[0], d, self.Pi, self.vb, self.val_bits,
                                ptrs[3], 1, ptrs[4], rows, stream)
        if rc:
            _lib.check(rc, "append values")

    def into_planes(self, keys: torch.Tensor, values: torch.Tensor, planes: dict, offset: int) -> None:
        """(B,H,S,d) keys / values into row-major planes [B*H, capacity, ...] at rows offset..offset+S."""
        kn = planes["k_norms"]
        if kn.device != self.device:
            raise ValueError(f"quashkv_b200: planes on {kn.device}, constants on {self.device}")
        ptrs = tuple(C.c_void_p(planes[n].data_ptr()) for n in ("k_codes", "k_signs", "k_norms", "v_codes", "v_norms"))
        self._compress(keys, values, ptrs, Rows(keys.shape[-2], kn.shape[-1], offset),
                       C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))

    def into_records(self, keys: torch.Tensor, values: torch.Tensor, records: torch.Tensor, row_bytes: tuple,
                     capacity: int, offset: int) -> None:
        """(B,H,S,d) keys / values into tile records [B*H, capacity/16, 1664] at tokens offset..offset+S."""
        if records.device != self.device:
            raise ValueError(f"quashkv_b200: records on {records.device}, constants on {self.device}")
        b, H, S, _ = keys.shape
        n = b * H * S
        stream_handle = torch.cuda.current_stream(self.device).cuda_stream
        if self.stage is None or self.stage_rows < n or self.stage_stream != stream_handle:
            pk, ps, pv = row_bytes
            u8 = dict(dtype=torch.uint8, device=self.device)
            f32 = dict(dtype=torch.float32, device=self.device)
            self.stage = (torch.empty((n, pk), **u8), torch.empty((n, ps), **u8), torch.empty((n,), **f32),
                          torch.empty((n, pv), **u8), torch.empty((n,), **f32))
            self.stage_rows = n
            self.stage_stream = stream_handle
        ptrs = tuple(C.c_void_p(t.data_ptr()) for t in self.stage)
        stream = C.c_void_p(stream_handle)
        self._compress(keys, values, ptrs, _dense(n), stream)
        rc = self.lib.qkv_tile_rows(*ptrs, n, C.c_void_p(records.data_ptr()), Rows(max(S, 1), capacity, offset), None,
                                    stream)
        if rc:
            _lib.check(rc, "tile_rows")


_CUDART = None


def cudart():
    """The CUDA runtime that torch has loaded, through ctypes: raw asynchronous copies and event calls for the
    host-buffer path, where the stream context managers of torch cost more than the device work of a short
    decode step."""
    global _CUDART
    if _CUDART is None:
        rt = C.CDLL("libcudart.so.12")
        rt.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        rt.cudaMemcpyAsync.restype = C.c_int
        rt.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
        rt.cudaEventRecord.restype = C.c_int
        rt.cudaStreamWaitEvent.argtypes = [C.c_void_p, C.c_void_p, C.c_uint]
        rt.cudaStreamWaitEvent.restype = C.c_int
        _CUDART = rt
    return _CUDART


class TiledAttentionCall:
    """The same C call as the ``attention_tiled`` op (``QuashKVEngine.attention``, reference engine.py:204-299,
    over a cache kept as tile records), prepared once for an engine's decode loop: constants are
    converted and kept, the workspace is kept between calls and grows when a longer cache needs more, and the
    call goes to the library without passing through the op dispatcher.  A decode step over one KV head of a
    sharded cache lasts tens of microseconds on the device; the per-call host work of the generic op (four
    tensor conversions, a workspace allocation, the dispatcher) is as long.  One instance serves one stream at
    a time (the workspace is shared by its calls)."""

    def __init__(self, Pi, key_centroids, val_centroids, S, qjl_scale: float):
        self.consts = tuple(_f32(t) for t in (Pi, key_centroids, val_centroids, S))
        self.ptrs = tuple(_p(t) for t in self.consts)
        self.qjl_scale = float(qjl_scale)
        self.device = self.consts[0].device
        self.ws = None
        self.lib = _lib.lib()
        self.fn = self.lib.qkv_attention_tiled

    def __call__(self, q: torch.Tensor, records: torch.Tensor, capacity: int, kv_len: int, n_kv_heads: int,
                 scale: float, causal: bool, out: Optional[torch.Tensor] = None,
                 stream: Optional[int] = None) -> torch.Tensor:
        """``out`` (fp32, contiguous, shape of q) is written when given; ``stream`` is a raw stream handle
        (default: the current stream of q's device)."""
        B, Hq, Q, d = q.shape
        if q.dtype not in _DT:
            q = q.float()
        qc = q if q.is_contiguous() else q.contiguous()
        if qc.device != self.device or records.device != self.device:
            raise ValueError(f"quashkv_b200: queries on {qc.device}, records on {records.device}, constants on {self.device}")
        if out is None:
            out = torch.empty((B, Hq, Q, d), dtype=torch.float32, device=q.device)
        elif out.dtype != torch.float32 or out.shape != q.shape or not out.is_contiguous() or out.device != self.device:
            raise ValueError("quashkv_b200: out must be a contiguous fp32 tensor of the queries' shape on their device")
        need = self.lib.qkv_attention_workspace_bytes(B, Hq, n_kv_heads, Q, kv_len, d)
        if self.ws is None or self.ws.numel() < need:
            self.ws = torch.empty((max(need + need // 4, 1 << 16),), dtype=torch.uint8, device=q.device)
        cache = TiledCache(records.data_ptr(), capacity, None, None, 0, 0)
        rc = self.fn(qc.data_ptr(), _DT[qc.dtype], cache, B, Hq, n_kv_heads, Q, kv_len, d, 3, 3, *self.ptrs,
                     self.qjl_scale, scale, int(causal), out.data_ptr(), self.ws.data_ptr(), self.ws.numel(),
                     torch.cuda.current_stream(q.device).cuda_stream if stream is None else stream)
        if rc:
            _lib.check(rc, "attention_tiled")
        return out


@_attention_tiled.register_fake
def _(q, records, capacity, kv_len, n_kv_heads, block_table, seq_lens, block_size, Pi, key_centroids,
      val_centroids, S, qjl_scale, scale, causal):
    return q.new_empty(q.shape, dtype=torch.float32)


@torch.library.custom_op("quashkv_b200::index_scan_topk", mutates_args=(), device_types="cuda")
def _index_scan_topk(queries: torch.Tensor, db_codes: torch.Tensor, db_signs: torch.Tensor,
                     db_norms: torch.Tensor, n_vectors: int, bits: int, Pi: torch.Tensor,
                     centroids: torch.Tensor, S: torch.Tensor, qjl_scale: float, k: int,
                     id_base: int) -> tuple[torch.Tensor, torch.Tensor]:
    qf = _f32(queries)
    M, d = qf.shape
    scores = torch.empty((M, k), dtype=torch.float32, device=qf.device)
    ids = torch.empty((M, k), dtype=torch.int64, device=qf.device)
    L = _lib.lib()
    ws_bytes = L.qkv_index_workspace_bytes(n_vectors, M, d, k)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=qf.device)
    _same_device(qf.device, qf, db_codes, db_signs, db_norms)
    A = _Keep(qf.device)
    with torch.cuda.device(qf.device):
        _lib.check(L.qkv_index_scan_topk(
            _p(qf), M, d, _p(db_codes), _p(db_signs), _p(db_norms), n_vectors, bits, A.f32(Pi),
            A.f32(centroids), A.f32(S), float(qjl_scale), k, id_base, _p(scores), _p(ids),
            _p(ws), ws_bytes, _stream(qf)), "index_scan_topk")
    return scores, ids


@_index_scan_topk.register_fake
def _(queries, db_codes, db_signs, db_norms, n_vectors, bits, Pi, centroids, S, qjl_scale, k, id_base):
    M = queries.shape[0]
    return queries.new_empty((M, k), dtype=torch.float32), queries.new_empty((M, k), dtype=torch.int64)


@torch.library.custom_op("quashkv_b200::index_scores", mutates_args=(), device_types="cuda")
def _index_scores(queries: torch.Tensor, db_codes: torch.Tensor, db_signs: torch.Tensor,
                  db_norms: torch.Tensor, n_vectors: int, bits: int, Pi: torch.Tensor,
                  centroids: torch.Tensor, S: torch.Tensor, qjl_scale: float) -> torch.Tensor:
    qf = _f32(queries)
    M, d = qf.shape
    out = torch.empty((M, n_vectors), dtype=torch.float32, device=qf.device)
    L = _lib.lib()
    ws_bytes = L.qkv_index_workspace_bytes(n_vectors, M, d, 1)
    ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=qf.device)
    _same_device(qf.device, qf, db_codes, db_signs, db_norms)
    A = _Keep(qf.device)
    with torch.cuda.device(qf.device):
        _lib.check(L.qkv_index_scores(
            _p(qf), M, d, _p(db_codes), _p(db_signs), _p(db_norms), n_vectors, bits, A.f32(Pi),
            A.f32(centroids), A.f32(S), float(qjl_scale), _p(out), _p(ws), ws_bytes, _stream(qf)),
            "index_scores")
    return out


@_index_scores.register_fake
def _(queries, db_codes, db_signs, db_norms, n_vectors, bits, Pi, centroids, S, qjl_scale):
    return queries.new_empty((queries.shape[0], n_vectors), dtype=torch.float32)


@torch.library.custom_op("quashkv_b200::topk_merge", mutates_args=(), device_types="cuda")
def _topk_merge(scores: torch.Tensor, ids: torch.Tensor, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    s = _f32(scores)
    i = ids.to(torch.int64).contiguous()
    M, n_cand = s.shape
    out_s = torch.empty((M, k), dtype=torch.float32, device=s.device)
    out_i = torch.empty((M, k), dtype=torch.int64, device=s.device)
    _same_device(s.device, s, i)
    A = _Keep(s.device)
    with torch.cuda.device(s.device):
        _lib.check(_lib.lib().qkv_topk_merge(_p(s), _p(i), M, n_cand, k, _p(out_s), _p(out_i), _stream(s)),
                   "topk_merge")
    return out_s, out_i


@_topk_merge.register_fake
def _(scores, ids, k):
    M = scores.shape[0]
    return scores.new_empty((M, k), dtype=torch.float32), ids.new_empty((M, k), dtype=torch.int64)


# ---------------------------------------------------------------------------------------------
# public wrappers
# ---------------------------------------------------------------------------------------------

def _need_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"quashkv_b200.{what}: expected a CUDA tensor, got device '{t.device}'. The hot path runs "
            "only as sm_100a kernels; there is no CPU implementation.")


def pack(codes, bits):
    if bits == 8:
        return codes
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bits: {bits}")
    _need_cuda(codes, "pack")
    return _pack(codes, bits)


def unpack(packed, bits, d):
    if bits == 8:
        return packed
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bits: {bits}")
    _need_cuda(packed, "unpack")
    return _unpack(packed, bits, d)


def compress_mse(x, Pi, boundaries, bits, packed=False):
    _need_cuda(x, "compress_mse")
    return _compress_mse(x, Pi, boundaries, bits, packed)


def compress_ip(x, Pi, boundaries, centroids, S, mse_bits, packed=False):
    _need_cuda(x, "compress_ip")
    return _compress_ip(x, Pi, boundaries, centroids, S, mse_bits, packed)


def compress_mixed(x, Pi, is_outlier, bounds_out, bits_out, bounds_reg, bits_reg, packed=False, n_out=None):
    """``n_out``: how many channels ``is_outlier`` marks; counted here (one device read) when not given."""
    _need_cuda(x, "compress_mixed")
    if n_out is None:
        n_out = int(is_outlier.sum().item()) if packed else 0
    return _compress_mixed(x, Pi, is_outlier, bounds_out, bits_out, bounds_reg, bits_reg, packed, int(n_out))


def compress_mixed_ip(x, Pi, is_outlier, bounds_out, cents_out, bits_out, bounds_reg, cents_reg, bits_reg, S):
    _need_cuda(x, "compress_mixed_ip")
    return _compress_mixed_ip(x, Pi, is_outlier, bounds_out, cents_out, bits_out, bounds_reg, cents_reg, bits_reg, S)


def decompress(codes, norms, Pi, centroids, bits, *, signs=None, S=None, qjl_scale=0.0, packed=False,
               d=None, out_dtype=torch.float32):
    """Dense planes: codes (..., d) or (..., packed bytes), norms (...)."""
    _need_cuda(codes, "decompress")
    if d is None:
        d = codes.shape[-1]
    lead = codes.shape[:-1]
    flat = codes.reshape(-1, codes.shape[-1]).contiguous()
    sflat = None if signs is None else signs.reshape(-1, signs.shape[-1]).contiguous()
    n = flat.shape[0]
    out = _decompress(flat, sflat, _f32(norms).reshape(-1), Pi, centroids, bits, S, qjl_scale, packed, d,
                      max(n, 1), 0, 0, n, out_dtype)
    return out.reshape(*lead, d)


def decompress_rows(codes, norms, Pi, centroids, bits, d, n_seg, seg_len, seg_stride, seg_off, *,
                    signs=None, S=None, qjl_scale=0.0, out_dtype=torch.float32):
    """Packed cache planes [n_seg, capacity, bytes]: rows seg_off..seg_off+seg_len of each segment."""
    _need_cuda(codes, "decompress_rows")
    return _decompress(codes, signs, norms, Pi, centroids, bits, S, qjl_scale, True, d,
                       seg_len, seg_stride, seg_off, n_seg * seg_len, out_dtype)


def decompress_mixed(codes, norms, Pi, is_outlier, cents_out, bits_out, cents_reg, bits_reg, packed=False,
                     d=None):
    _need_cuda(codes, "decompress_mixed")
    return _decompress_mixed(codes, norms, Pi, is_outlier, cents_out, bits_out, cents_reg, bits_reg, packed,
                             codes.shape[-1] if d is None else d)


append_kv = _append_kv
compress_ip_into = _compress_ip_into
attention = _attention
attention_paged = _attention_paged
scatter_rows = _scatter_rows
tile_rows = _tile_rows
untile_rows = _untile_rows
attention_tiled = _attention_tiled
index_scan_topk = _index_scan_topk
index_scores = _index_scores
topk_merge = _topk_merge
INDEX_MAX_K = _lib.INDEX_MAX_K
