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
