"""Shared checks for the parity tests."""

import numpy as np
import torch


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp(min=1e-30))


def ulp_diff(a: torch.Tensor, b: torch.Tensor) -> int:
    """Largest distance in units of fp32 representable steps."""
    ia = a.cpu().contiguous().view(torch.int32).long()
    ib = b.cpu().contiguous().view(torch.int32).long()
    return int((ia - ib).abs().max()) if ia.numel() else 0


def code_ties(x, Pi, tables, got, want, kind="code", centroids=None, S=None, codes_for_resid=None):
    """Explain every mismatch between two code tensors as a tie.

    For 'code' mismatches the fp64 rotated coordinate must lie within ``tol`` of a decision
    boundary; for 'sign' mismatches the fp64 residual must be within ``tol`` of zero.
    Returns (n_mismatch, n_total, max_distance)."""
    got, want = got.cpu(), want.cpu()
    bad = (got != want)
    n_bad = int(bad.sum())
    if n_bad == 0:
        return 0, got.numel(), 0.0
    x64 = x.double().cpu()
    rot = (x64 / x64.norm(dim=-1, keepdim=True).clamp(min=1e-8)) @ Pi.double().cpu().T
    if kind == "code":
        dist = (rot.unsqueeze(-1) - tables.double().cpu()).abs().min(dim=-1).values
    else:
        dist = (rot - centroids.double().cpu()[codes_for_resid.cpu().long()]).abs()
    return n_bad, got.numel(), float(dist[bad].max())


def tile_records_reference(k_codes, k_signs, k_norms, v_codes, v_norms):
    """Tile records of whole 16-token groups, written from the format's definition with numpy (the CUDA
    tiling kernel is checked against this): inputs are the reference's packed rows of n = 16 * R tokens,
    (n,32) (n,16) (n,) (n,48) (n,); returns (R, 1664) uint8.

    Lane L = 4 g + t.  [0,512) key codes: 16 B per lane = bytes 8t..8t+7 of tokens g and g+8.  [512,1024) value
    magnitudes: 16 B per lane = words m = 0..3, byte b of a word for token 2t + (b&1) + 8 (b>>1), 2-bit field f
    for coordinate 16 g + 4 m + f.  [1024,1536) sign bits: 16 B per lane = bytes 4t..4t+3 of the key sign rows of
    tokens g, g+8, then the 16-bit value-sign pieces of tokens 2t, 2t+1, 2t+8, 2t+9, bit p for coordinate 16 g + p.  [1536,1664) per g: key norms of tokens g, g+8, value norms of tokens g, g+8.  A 3-bit value
    code u is stored as negative = (u < 4) and magnitude index u - 4 (u >= 4) or 3 - u."""
    k_codes, k_signs, v_codes = (np.asarray(a, dtype=np.uint8) for a in (k_codes, k_signs, v_codes))
    k_norms, v_norms = np.asarray(k_norms, dtype=np.float32), np.asarray(v_norms, dtype=np.float32)
    n = k_codes.shape[0]
    assert n % 16 == 0
    R = n // 16
    bits = np.unpackbits(v_codes, axis=1, bitorder="little").reshape(n, 128, 3)
    u = bits[:, :, 0] + 2 * bits[:, :, 1] + 4 * bits[:, :, 2]                   # (n,128) codes 0..7
    neg = (u < 4).astype(np.uint32)
    mag = np.where(u >= 4, u - 4, 3 - u).astype(np.uint32)
    rec = np.zeros((R, 1664), dtype=np.uint8)
    kc = k_codes.reshape(R, 16, 32)
    ks = k_signs.reshape(R, 16, 16)
    mag = mag.reshape(R, 16, 128)
    neg = neg.reshape(R, 16, 128)
    kn, vn = k_norms.reshape(R, 16), v_norms.reshape(R, 16)
    for g in range(8):
        for t_ in range(4):
            L = 4 * g + t_
            rec[:, 16 * L:16 * L + 8] = kc[:, g, 8 * t_:8 * t_ + 8]
            rec[:, 16 * L + 8:16 * L + 16] = kc[:, g + 8, 8 * t_:8 * t_ + 8]
            rec[:, 1024 + 16 * L:1024 + 16 * L + 4] = ks[:, g, 4 * t_:4 * t_ + 4]
            rec[:, 1024 + 16 * L + 4:1024 + 16 * L + 8] = ks[:, g + 8, 4 * t_:4 * t_ + 4]
            for b in range(4):
                tok = 2 * t_ + (b & 1) + 8 * (b >> 1)
                for m in range(4):
                    byte = sum(mag[:, tok, 16 * g + 4 * m + f] << (2 * f) for f in range(4))
                    rec[:, 512 + 16 * L + 4 * m + b] = byte.astype(np.uint8)
                piece = sum(neg[:, tok, 16 * g + p_] << p_ for p_ in range(16)).astype(np.uint16)
                off = 1024 + 16 * L + 8 + 4 * (b >> 1) + 2 * (b & 1)
                rec[:, off] = (piece & 0xFF).astype(np.uint8)
                rec[:, off + 1] = (piece >> 8).astype(np.uint8)
        nrm = np.stack([kn[:, g], kn[:, g + 8], vn[:, g], vn[:, g + 8]], axis=1).astype(np.float32)
        rec[:, 1536 + 16 * g:1536 + 16 * g + 16] = nrm.view(np.uint8).reshape(R, 16)
    return rec
