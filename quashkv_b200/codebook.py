"""Lloyd-Max scalar codebook for one coordinate of a randomly rotated unit vector.

Host-side, init-time only (a few dozen floats); the kernels receive the resulting
``centroids`` / ``boundaries`` tensors.  Same construction and interface as the
reference's ``LloydMaxCodebook`` (quashkv/codebook.py:63-139 solver, :181-275 class):
the values must equal the reference's bit for bit because they define the codes.
"""

from __future__ import annotations

import math
from functools import lru_cache

import torch

from .constants import LLOYD_MAX_ITER, LLOYD_MAX_RANGE_SIGMAS, LLOYD_MAX_TOL, SUPPORTED_BITS


def _coordinate_pdf(d: int, use_exact_pdf: bool):
    """Density of one coordinate and its support: N(0, 1/d), or the exact Beta-type law
    Gamma(d/2) / (sqrt(pi) Gamma((d-1)/2)) (1 - x^2)^((d-3)/2) on [-1, 1]."""
    sigma = 1.0 / math.sqrt(d)
    if not use_exact_pdf:
        norm = 1.0 / (math.sqrt(2 * math.pi) * sigma)
        return (lambda t: norm * math.exp(-t * t / (2 * sigma * sigma)),
                -LLOYD_MAX_RANGE_SIGMAS * sigma, LLOYD_MAX_RANGE_SIGMAS * sigma)
    from scipy import special
    log_c = special.gammaln(d / 2.0) - 0.5 * math.log(math.pi) - special.gammaln((d - 1) / 2.0)
    expo = (d - 3) / 2.0

    def beta(t):
        if abs(t) >= 1.0:
            return 0.0
        return math.exp(log_c) if expo == 0 else math.exp(log_c + expo * math.log(1.0 - t * t))
    return beta, -1.0, 1.0


def solve_lloyd_max(d: int, bits: int, *, use_exact_pdf: bool = False,
                    max_iter: int = LLOYD_MAX_ITER, tol: float = LLOYD_MAX_TOL):
    """Continuous 1-D k-means against the coordinate density: returns (centroids, boundaries)
    as Python float lists of length 2**bits and 2**bits - 1."""
    if bits not in SUPPORTED_BITS:
        raise ValueError(f"bits must be in {SUPPORTED_BITS}, got {bits}")
    from scipy import integrate
    pdf, lo, hi = _coordinate_pdf(d, use_exact_pdf)
    n = 1 << bits
    cents = [lo + (hi - lo) * (i + 0.5) / n for i in range(n)]

    def midpoints(c):
        return [(c[i] + c[i + 1]) / 2.0 for i in range(n - 1)]

    for _ in range(max_iter):
        edges = [lo * 5] + midpoints(cents) + [hi * 5]
        moved = []
        for i in range(n):
            mass_x, _ = integrate.quad(lambda t: t * pdf(t), edges[i], edges[i + 1], limit=100)
            mass, _ = integrate.quad(pdf, edges[i], edges[i + 1], limit=100)
            moved.append(mass_x / mass if mass > 1e-15 else cents[i])
        shift = max(abs(a - b) for a, b in zip(moved, cents))
        cents = moved
        if shift < tol:
            break
    return cents, midpoints(cents)


def compute_mse_cost(d: int, bits: int, *, use_exact_pdf: bool = False) -> float:
    """d * C(f_X, b): expected squared error of a unit vector under the optimal quantiser."""
    from scipy import integrate
    cents, bounds = solve_lloyd_max(d, bits, use_exact_pdf=use_exact_pdf)
    pdf, lo, hi = _coordinate_pdf(d, use_exact_pdf)
    edges = [lo * 5] + bounds + [hi * 5]
    total = 0.0
    for i, c in enumerate(cents):
        part, _ = integrate.quad(lambda t: (t - c) ** 2 * pdf(t), edges[i], edges[i + 1], limit=100)
        total += part
    return d * total


class LloydMaxCodebook:
    """Pre-solved codebook: ``centroids`` (2**bits,) and ``boundaries`` (2**bits-1,) fp32."""

    def __init__(self, d: int, bits: int, *, use_exact_pdf: bool = False):
        self.d, self.bits, self.n_levels = d, bits, 1 << bits
        cents, bounds = _solved(d, bits, use_exact_pdf)
        self.centroids = torch.tensor(cents, dtype=torch.float32)
        self.boundaries = torch.tensor(bounds, dtype=torch.float32)

    # The three methods below are small element-wise helpers kept for interface parity; the
    # compress / decompress kernels implement the same rules in fused form.
    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        """Index of the nearest centroid."""
        return (x.unsqueeze(-1) - self.centroids.to(x.device)).abs().argmin(dim=-1).to(torch.uint8)

    def dequantize(self, indices: torch.Tensor) -> torch.Tensor:
        return self.centroids.to(indices.device)[indices.long()]

    def quantize_boundary(self, x: torch.Tensor) -> torch.Tensor:
        """Number of boundaries strictly below each value."""
        return torch.bucketize(x, self.boundaries.to(x.device)).to(torch.uint8)

    def mse_cost(self) -> float:
        return compute_mse_cost(self.d, self.bits)

    def to(self, device) -> "LloydMaxCodebook":
        self.centroids = self.centroids.to(device)
        self.boundaries = self.boundaries.to(device)
        return self

    def __repr__(self) -> str:
        vals = ", ".join(f"{c:.6f}" for c in self.centroids.tolist())
        return f"LloydMaxCodebook(d={self.d}, bits={self.bits}, levels={self.n_levels}, centroids=[{vals}])"


@lru_cache(maxsize=64)
def _solved(d: int, bits: int, use_exact_pdf: bool):
    cents, bounds = solve_lloyd_max(d, bits, use_exact_pdf=use_exact_pdf)
    return tuple(cents), tuple(bounds)


@lru_cache(maxsize=32)
def get_codebook(d: int, bits: int) -> LloydMaxCodebook:
    return LloydMaxCodebook(d, bits)
