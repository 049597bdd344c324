"""MSEQuantizer and InnerProductQuantizer with the reference's interface
(quashkv/quantizer.py:62-285); compress / decompress run as CUDA kernels.

The rotation matrix, sign vector and codebook are produced on the host with the
same torch calls as the reference, so a given (d, bits, seed) yields the same
constants and therefore the same codes.
"""

from __future__ import annotations

import torch

from . import ops
from .codebook import LloydMaxCodebook
from .constants import DEFAULT_SEED, DEFAULT_TOTAL_BITS, QJL_COEFF


def _random_orthogonal(d: int, seed: int, device) -> torch.Tensor:
    """Q of the QR factorisation of a seeded Gaussian matrix, columns signed by diag(R)
    (reference quantizer.py:32-44)."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    gauss = torch.randn(d, d, generator=gen, dtype=torch.float32, device="cpu")
    q, r = torch.linalg.qr(gauss)
    # the QR factor comes back column-major; the kernels read Pi row-major, so make it so once, here
    return (q * torch.sign(torch.diag(r)).unsqueeze(0)).contiguous().to(device)


def _random_signs(d: int, seed: int, device) -> torch.Tensor:
    """+-1 vector drawn from seed + 1_000_000 (reference quantizer.py:51-59)."""
    gen = torch.Generator(device="cpu").manual_seed(seed + 1_000_000)
    return torch.randint(0, 2, (d,), generator=gen, dtype=torch.float32, device="cpu").mul_(2).sub_(1).to(device)


class _DeviceConstants:
    """Copies of small constant tensors per device, so an object built with the default
    ``device="cpu"`` can still serve CUDA inputs.  A copy is tied to the very tensor object it was made
    from (held here, so its address cannot be recycled) and to that tensor's version counter: replacing or
    modifying the source tensor makes the next ``get`` copy again."""

    def __init__(self):
        self._copies = {}

    def get(self, name: str, tensor: torch.Tensor, device: torch.device) -> torch.Tensor:
        if tensor.device == device and tensor.is_contiguous():
            return tensor
        ent = self._copies.get((name, device))
        if ent is None or ent[0] is not tensor or ent[1] != tensor._version:
            ent = (tensor, tensor._version, tensor.to(device).contiguous())
            self._copies[(name, device)] = ent
        return ent[2]

    def clear(self) -> None:
        self._copies.clear()


class MSEQuantizer:
    """Rotate by Pi, then Lloyd-Max scalar quantisation of every coordinate."""

    def __init__(self, d: int, bits: int = 3, seed: int = DEFAULT_SEED, device="cpu",
                 use_exact_pdf: bool = False):
        self.d, self.bits, self.seed = d, bits, seed
        self.device = torch.device(device)
        self.Pi = _random_orthogonal(d, seed, self.device)
        self.codebook = LloydMaxCodebook(d, bits, use_exact_pdf=use_exact_pdf)
        self.codebook.to(self.device)
        self._consts = _DeviceConstants()

    def _on(self, device):
        c = self._consts
        return (c.get("Pi", self.Pi, device), c.get("b", self.codebook.boundaries, device),
                c.get("c", self.codebook.centroids, device))

    def rotate(self, x: torch.Tensor) -> torch.Tensor:
        return x @ self.Pi.to(x.device).T

    def unrotate(self, x_rot: torch.Tensor) -> torch.Tensor:
        return x_rot @ self.Pi.to(x_rot.device)

    def compress(self, x: torch.Tensor):
        """(..., d) -> (codes uint8 (..., d), norms fp32 (...))."""
        Pi, bounds, _ = self._on(x.device)
        return ops.compress_mse(x, Pi, bounds, self.bits, packed=False)

    def compress_packed(self, x: torch.Tensor):
        """Same, with codes already bit-packed (..., packed bytes)."""
        Pi, bounds, _ = self._on(x.device)
        return ops.compress_mse(x, Pi, bounds, self.bits, packed=True)

    def decompress(self, indices: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        Pi, _, cents = self._on(indices.device)
        return ops.decompress(indices, norms, Pi, cents, self.bits)

    def decompress_packed(self, packed: torch.Tensor, norms: torch.Tensor, out_dtype=torch.float32):
        Pi, _, cents = self._on(packed.device)
        return ops.decompress(packed, norms, Pi, cents, self.bits, packed=True, d=self.d, out_dtype=out_dtype)

    def to(self, device) -> "MSEQuantizer":
        self.device = torch.device(device)
        self.Pi = self.Pi.to(self.device)
        self.codebook.to(self.device)
        return self


class InnerProductQuantizer:
    """Keys: (b-1)-bit codes plus the sign bit of the rotated residual times S."""

    def __init__(self, d: int, total_bits: int = DEFAULT_TOTAL_BITS, seed: int = DEFAULT_SEED,
                 device="cpu", use_exact_pdf: bool = False):
        if total_bits < 2:
            raise ValueError("InnerProductQuantizer needs at least 2 total bits")
        self.d, self.total_bits, self.mse_bits, self.seed = d, total_bits, total_bits - 1, seed
        self.device = torch.device(device)
        self.mse_quantizer = MSEQuantizer(d, bits=self.mse_bits, seed=seed, device=device,
                                          use_exact_pdf=use_exact_pdf)
        self.S = _random_signs(d, seed, self.device)
        self.qjl_scale = QJL_COEFF / d
        self._consts = _DeviceConstants()

    def _on(self, device):
        Pi, bounds, cents = self.mse_quantizer._on(device)
        return Pi, bounds, cents, self._consts.get("S", self.S, device)

    def compress(self, x: torch.Tensor):
        """(..., d) -> (codes uint8 (..., d), signs uint8 in {0,1} (..., d), norms (...))."""
        Pi, bounds, cents, S = self._on(x.device)
        return ops.compress_ip(x, Pi, bounds, cents, S, self.mse_bits, packed=False)

    def compress_packed(self, x: torch.Tensor):
        Pi, bounds, cents, S = self._on(x.device)
        return ops.compress_ip(x, Pi, bounds, cents, S, self.mse_bits, packed=True)

    def decompress_for_dot(self, mse_indices, qjl_signs, norms, q_rot):
        """norm * (<q_rot, c[codes]> + qjl_scale * sum(|q_rot| * (2 sign - 1) * S)) for one rotated
        query per key row (reference quantizer.py:244-279).  A small broadcasting helper; bulk
        scoring goes through the attention and index-scan kernels."""
        _, _, cents, S = self._on(mse_indices.device)
        dots = (q_rot * cents[mse_indices.long()]).sum(dim=-1)
        corr = self.qjl_scale * (q_rot.abs() * (qjl_signs.float() * 2.0 - 1.0) * S).sum(dim=-1)
        return norms * (dots + corr)

    def to(self, device) -> "InnerProductQuantizer":
        self.device = torch.device(device)
        self.mse_quantizer.to(device)
        self.S = self.S.to(self.device)
        return self
