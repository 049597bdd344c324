"""Mixed-precision quantisers: more bits on the highest-variance rotated channels.

Interface of the reference's quashkv/mixed_precision.py (:25-197 MSE variant,
:200-322 IP variant).  Calibration (a variance top-k) stays torch on the data's
device; compress / decompress run as CUDA kernels that take the channel mask.
"""

from __future__ import annotations

from typing import Optional

import torch

from . import ops
from .codebook import LloydMaxCodebook
from .constants import DEFAULT_SEED, QJL_COEFF
from .quantizer import _DeviceConstants, _random_orthogonal, _random_signs


class MixedPrecisionMSEQuantizer:
    def __init__(self, d: int, outlier_bits: int = 3, regular_bits: int = 2, n_outliers: int = 32,
                 seed: int = DEFAULT_SEED, device="cpu"):
        if n_outliers < 0 or n_outliers > d:
            raise ValueError(f"n_outliers must be in [0, {d}], got {n_outliers}")
        if outlier_bits < regular_bits:
            raise ValueError("outlier_bits should be >= regular_bits")
        self.d, self.outlier_bits, self.regular_bits, self.n_outliers = d, outlier_bits, regular_bits, n_outliers
        self.seed = seed
        self.device = torch.device(device)
        self.Pi = _random_orthogonal(d, seed, self.device)
        self.outlier_codebook = LloydMaxCodebook(d, outlier_bits).to(self.device)
        self.regular_codebook = LloydMaxCodebook(d, regular_bits).to(self.device)
        self._outlier_indices: Optional[torch.Tensor] = None
        self._outlier_mask: Optional[torch.Tensor] = None
        self._mask_u8 = torch.zeros(d, dtype=torch.uint8, device=self.device)   # what the kernels read
        self._n_marked = 0
        self._consts = _DeviceConstants()

    @property
    def effective_bits(self) -> float:
        return (self.n_outliers * self.outlier_bits + (self.d - self.n_outliers) * self.regular_bits) / self.d

    @property
    def calibrated(self) -> bool:
        return self._outlier_mask is not None

    def calibrate(self, data: torch.Tensor) -> None:
        """Mark the n_outliers rotated channels of largest variance over unit-normalised ``data``."""
        if data.dim() != 2 or data.shape[1] != self.d:
            raise ValueError(f"Expected (N, {self.d}) calibration data")
        data = data.float()
        norms = data.norm(dim=-1, keepdim=True).clamp(min=1e-8)
        x_rot = (data / norms) @ self.Pi.to(data.device).T
        _, top = x_rot.var(dim=0).topk(self.n_outliers)
        self.set_outlier_channels(top)

    def set_outlier_channels(self, indices: torch.Tensor) -> None:
        self._outlier_indices = indices.sort().values.to(self.device)
        mask = torch.zeros(self.d, dtype=torch.bool, device=self.device)
        mask[self._outlier_indices] = True
        self._outlier_mask = mask
        self._mask_u8 = mask.to(torch.uint8)
        self._n_marked = int(torch.unique(self._outlier_indices).numel())    # host-side count, once per calibration
        self._consts.clear()

    def rotate(self, x):
        return x @ self.Pi.to(x.device).T

    def unrotate(self, x_rot):
        return x_rot @ self.Pi.to(x_rot.device)

    def _tables(self, device):
        c = self._consts       # uncalibrated: the all-zero mask puts the regular codebook on every channel
        return (c.get("Pi", self.Pi, device), c.get("m", self._mask_u8, device),
                c.get("ob", self.outlier_codebook.boundaries, device),
                c.get("rb", self.regular_codebook.boundaries, device),
                c.get("oc", self.outlier_codebook.centroids, device),
                c.get("rc", self.regular_codebook.centroids, device))

    def compress(self, x: torch.Tensor, packed: bool = False):
        """(..., d) -> (codes uint8, norms).  ``packed=True`` returns the packed mixed row
        (outlier channels at outlier_bits, then regular channels at regular_bits)."""
        Pi, mask, ob, rb, _, _ = self._tables(x.device)
        return ops.compress_mixed(x, Pi, mask, ob, self.outlier_bits, rb, self.regular_bits, packed,
                                  n_out=self._n_marked)

    def decompress(self, indices: torch.Tensor, norms: torch.Tensor, packed: bool = False) -> torch.Tensor:
        Pi, mask, _, _, oc, rc = self._tables(indices.device)
        return ops.decompress_mixed(indices, norms, Pi, mask, oc, self.outlier_bits, rc, self.regular_bits,
                                    packed, self.d)

    def to(self, device) -> "MixedPrecisionMSEQuantizer":
        self.device = torch.device(device)
        self.Pi = self.Pi.to(self.device)
        self.outlier_codebook.to(self.device)
        self.regular_codebook.to(self.device)
        if self._outlier_mask is not None:
            self._outlier_mask = self._outlier_mask.to(self.device)
            self._outlier_indices = self._outlier_indices.to(self.device)
        self._mask_u8 = self._mask_u8.to(self.device)
        self._consts.clear()
        return self


class MixedPrecisionIPQuantizer:
    """Mixed-precision codes at (bits - 1) plus one sign bit of the rotated residual on every channel
    (reference mixed_precision.py:200-322).  Both stages run in one kernel: the residual is taken against
    the centroid of the channel's own codebook while the rotated coordinate is still in a register."""

    def __init__(self, d: int, outlier_bits: int = 3, regular_bits: int = 2, n_outliers: int = 32,
                 seed: int = DEFAULT_SEED, device="cpu"):
        if regular_bits < 2:
            raise ValueError("IP quantizer needs at least 2 total bits")
        self.d, self.outlier_bits, self.regular_bits, self.n_outliers = d, outlier_bits, regular_bits, n_outliers
        self.seed = seed
        self.device = torch.device(device)
        self.mse_quantizer = MixedPrecisionMSEQuantizer(d, outlier_bits - 1, regular_bits - 1, n_outliers,
                                                        seed, device)
        self.S = _random_signs(d, seed, self.device)
        self.qjl_scale = QJL_COEFF / d
        self._consts = _DeviceConstants()

    @property
    def effective_bits(self) -> float:
        return self.mse_quantizer.effective_bits + 1.0

    @property
    def calibrated(self) -> bool:
        return self.mse_quantizer.calibrated

    def calibrate(self, data):
        self.mse_quantizer.calibrate(data)

    def set_outlier_channels(self, indices):
        self.mse_quantizer.set_outlier_channels(indices)

    def compress(self, x: torch.Tensor):
        """(..., d) -> (codes uint8 (..., d), signs uint8 in {0,1} (..., d), norms (...))."""
        mq = self.mse_quantizer
        Pi, mask, ob, rb, oc, rc = mq._tables(x.device)
        S = self._consts.get("S", self.S, x.device)
        return ops.compress_mixed_ip(x, Pi, mask, ob, oc, mq.outlier_bits, rb, rc, mq.regular_bits, S)

    def to(self, device):
        self.device = torch.device(device)
        self.mse_quantizer.to(device)
        self.S = self.S.to(device)
        self._consts.clear()
        return self
