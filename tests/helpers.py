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

    Lane L = 4 g + t.  [0,512) key codes: 16 B per lane = bytes 8t..8t+7 of tokens g and g+8.  [512,768) key signs:
    8 B per lane = bytes 4t..4t+3 of tokens g, g+8.  Values: 24 B per lane = two 96-bit groups, group h for the
    token pair (2t+8h, 2t+8h+1), field f (bits 6f..6f+5) for coordinate 16 g + f, first token in the low three
    bits; a 3-bit value code u is stored as (u < 4) << 2 | (u - 4 if u >= 4 else 3 - u).  Words 0..3 of a lane in
    [768,1280) (16 B per lane), words 4, 5 in [1280,1536) (8 B per lane).  [1536,1664) per g: key norms of tokens
    g, g+8, value norms of tokens g, g+8."""
    k_codes, k_signs, v_codes = (np.asarray(a, dtype=np.uint8) for a in (k_codes, k_signs, v_codes))
    k_norms, v_norms = np.asarray(k_norms, dtype=np.float32), np.asarray(v_norms, dtype=np.float32)
    n = k_codes.shape[0]
    assert n % 16 == 0
    R = n // 16
    bits = np.unpackbits(v_codes, axis=1, bitorder="little").reshape(n, 128, 3)
    u = (bits[:, :, 0] + 2 * bits[:, :, 1] + 4 * bits[:, :, 2]).astype(np.int64)     # (n,128) codes 0..7
    stored = np.where(u >= 4, u - 4, 4 + (3 - u)).reshape(R, 16, 128)
    rec = np.zeros((R, 1664), dtype=np.uint8)
    kc = k_codes.reshape(R, 16, 32)
    ks = k_signs.reshape(R, 16, 16)
    kn, vn = k_norms.reshape(R, 16), v_norms.reshape(R, 16)
    for g in range(8):
        for t_ in range(4):
            L = 4 * g + t_
            rec[:, 16 * L:16 * L + 8] = kc[:, g, 8 * t_:8 * t_ + 8]
            rec[:, 16 * L + 8:16 * L + 16] = kc[:, g + 8, 8 * t_:8 * t_ + 8]
            rec[:, 512 + 8 * L:512 + 8 * L + 4] = ks[:, g, 4 * t_:4 * t_ + 4]
            rec[:, 512 + 8 * L + 4:512 + 8 * L + 8] = ks[:, g + 8, 4 * t_:4 * t_ + 4]
            words = []
            for h in range(2):
                ta, tb = 2 * t_ + 8 * h, 2 * t_ + 8 * h + 1
                group = np.zeros(R, dtype=object)                      # 96-bit integers
                for f in range(16):
                    field = stored[:, ta, 16 * g + f] | (stored[:, tb, 16 * g + f] << 3)
                    group = group + (field.astype(object) << (6 * f))
                words += [np.array([(int(x) >> (32 * w)) & 0xFFFFFFFF for x in group], dtype=np.uint32) for w in range(3)]
            six = np.stack(words, axis=1)                              # (R, 6) words of the lane
            rec[:, 768 + 16 * L:768 + 16 * L + 16] = six[:, :4].copy().view(np.uint8).reshape(R, 16)
            rec[:, 1280 + 8 * L:1280 + 8 * L + 8] = six[:, 4:].copy().view(np.uint8).reshape(R, 8)
        nrm = np.stack([kn[:, g], kn[:, g + 8], vn[:, g], vn[:, g + 8]], axis=1).astype(np.float32)
        rec[:, 1536 + 16 * g:1536 + 16 * g + 16] = nrm.view(np.uint8).reshape(R, 16)
    return rec
