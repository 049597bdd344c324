"""QuashIndex: maximum inner-product search over compressed vectors.

Interface of the reference's quashkv/nn_search/index.py (:21-258).  Storage is
three packed planes that grow geometrically (no re-concatenation per ``add``);
``search`` streams the packed rows once per tile of 16 queries in the scan kernel
with a fused top-k.  Ties in score are broken by the lower id.
"""

from __future__ import annotations

import torch

from .. import ops
from ..quantizer import InnerProductQuantizer


class QuashIndex:
    def __init__(self, dim: int, bits: int = 3, seed: int = 42, device="cpu", pack_storage: bool = False):
        self.dim, self.bits, self.seed = dim, bits, seed
        self.device = torch.device(device)
        self.pack_storage = pack_storage
        self.quantizer = InnerProductQuantizer(d=dim, total_bits=bits, seed=seed, device=device)
        self._codes = self._signs = self._norm_plane = None
        self._capacity = 0
        self._n_vectors = 0
        self._unpacked = None

    @property
    def n_vectors(self) -> int:
        return self._n_vectors

    def __len__(self) -> int:
        return self._n_vectors

    # ---- storage views with the reference's attribute names -----------------------------------
    def _views(self):
        n = self._n_vectors
        return self._codes[:n], self._signs[:n], self._norm_plane[:n]

    def _get_unpacked(self):
        """(mse_indices, qjl_signs) as (N, dim) uint8."""
        if self._unpacked is None:
            codes, signs, _ = self._views()
            self._unpacked = (ops.unpack(codes, self.bits - 1, self.dim), ops.unpack(signs, 1, self.dim))
        return self._unpacked

    @property
    def _mse_indices(self):
        if self._n_vectors == 0:
            return None
        return self._views()[0] if self.pack_storage else self._get_unpacked()[0]

    @property
    def _qjl_signs(self):
        if self._n_vectors == 0:
            return None
        return self._views()[1] if self.pack_storage else self._get_unpacked()[1]

    @property
    def _norms(self):
        return None if self._n_vectors == 0 else self._views()[2]

    # ---- add ------------------------------------------------------------------------------------
    def _reserve(self, capacity: int, device) -> None:
        if capacity <= self._capacity:
            return
        pk = ops.packed_row_bytes(self.dim, self.bits - 1)
        ps = ops.packed_row_bytes(self.dim, 1)
        codes = torch.zeros((capacity, pk), dtype=torch.uint8, device=device)
        signs = torch.zeros((capacity, ps), dtype=torch.uint8, device=device)
        norms = torch.zeros((capacity,), dtype=torch.float32, device=device)
        n = self._n_vectors
        if n:
            codes[:n], signs[:n], norms[:n] = self._views()
        self._codes, self._signs, self._norm_plane, self._capacity = codes, signs, norms, capacity

    def add(self, vectors: torch.Tensor) -> None:
        """Compress (N, dim) vectors into the index."""
        if vectors.dim() != 2 or vectors.shape[1] != self.dim:
            raise ValueError(f"Expected (N, {self.dim}) tensor, got shape {tuple(vectors.shape)}")
        ops._need_cuda(vectors, "QuashIndex.add")
        n_new = vectors.shape[0]
        need = self._n_vectors + n_new
        if need > self._capacity:
            self._reserve(max(need, 2 * self._capacity), vectors.device)
        Pi, bounds, cents, S = self.quantizer._on(vectors.device)
        ops.compress_ip_into(vectors, Pi, bounds, cents, S, self.bits - 1, self._codes, self._signs,
                             self._norm_plane, self._n_vectors)
        self._n_vectors = need
        self._unpacked = None

    # ---- persistence ----------------------------------------------------------------------------
    # The reference keeps the index in memory only and rebuilds its tensors on every add
    # (nn_search/index.py:100-104); here the three packed planes are the native form, so they are also the
    # file form: one torch archive with the planes cut to n_vectors rows and the constructor arguments.
    FILE_FORMAT = 1

    def save(self, path) -> None:
        """Write the packed planes and the constructor arguments; the rotation, codebook and sign vector are
        regenerated from (dim, bits, seed) on load, as the constructor does."""
        if self._n_vectors:
            codes, signs, norms = (t.cpu() for t in self._views())
        else:
            codes = signs = norms = None
        torch.save({"format": self.FILE_FORMAT, "dim": self.dim, "bits": self.bits, "seed": self.seed,
                    "pack_storage": self.pack_storage, "n_vectors": self._n_vectors,
                    "codes": codes, "signs": signs, "norms": norms}, path)

    @classmethod
    def load(cls, path, device="cuda") -> "QuashIndex":
        """Rebuild an index from ``save``'s file on ``device``; more vectors can be added afterwards."""
        blob = torch.load(path, map_location="cpu", weights_only=True)
        if not isinstance(blob, dict) or blob.get("format") != cls.FILE_FORMAT:
            raise ValueError(f"{path}: not a QuashIndex file of format {cls.FILE_FORMAT}")
        index = cls(blob["dim"], blob["bits"], blob["seed"], device=device, pack_storage=blob["pack_storage"])
        n = blob["n_vectors"]
        if n:
            pk = ops.packed_row_bytes(index.dim, index.bits - 1)
            ps = ops.packed_row_bytes(index.dim, 1)
            if (tuple(blob["codes"].shape) != (n, pk) or tuple(blob["signs"].shape) != (n, ps)
                    or tuple(blob["norms"].shape) != (n,)):
                raise ValueError(f"{path}: plane shapes do not match {n} vectors of dim {index.dim} at "
                                 f"{index.bits} bits")
            index._reserve(n, index.device)
            index._codes[:n] = blob["codes"].to(index.device)
            index._signs[:n] = blob["signs"].to(index.device)
            index._norm_plane[:n] = blob["norms"].to(index.device)
            index._n_vectors = n
        return index

    # ---- search ---------------------------------------------------------------------------------
    def search(self, queries: torch.Tensor, k: int = 10, id_base: int = 0):
        """(M, dim) queries -> (scores (M,k) descending, indices (M,k) int64)."""
        if self._n_vectors == 0:
            raise ValueError("Index is empty. Call add() first.")
        k = min(k, self._n_vectors)
        ops._need_cuda(queries, "QuashIndex.search")
        codes, signs, norms = self._views()
        Pi, _, cents, S = self.quantizer._on(queries.device)
        q = queries.float()
        if k <= ops.INDEX_MAX_K:
            return ops.index_scan_topk(q, codes, signs, norms, self._n_vectors, self.bits, Pi, cents, S,
                                       self.quantizer.qjl_scale, k, id_base)
        # k above the fused selection's limit: dense scores from the scan kernel, then a sort
        scores = ops.index_scores(q, codes, signs, norms, self._n_vectors, self.bits, Pi, cents, S,
                                  self.quantizer.qjl_scale)
        top_s, top_i = torch.topk(scores, k, dim=1)
        return top_s, top_i + id_base

    # ---- evaluation helpers (plain torch, as in the reference) --------------------------------------
    @staticmethod
    def brute_force(queries: torch.Tensor, database: torch.Tensor, k: int = 10):
        k = min(k, database.shape[0])
        return torch.topk(queries @ database.T, k, dim=1)

    def recall_at_k(self, queries: torch.Tensor, database: torch.Tensor, k: int = 10) -> float:
        _, approx = self.search(queries, k)
        _, exact = self.brute_force(queries, database.to(queries.device), k)
        hits = (approx.unsqueeze(2) == exact.unsqueeze(1)).any(dim=2).sum().item()
        return hits / (queries.shape[0] * approx.shape[1])

    def memory_bytes(self) -> int:
        if self._n_vectors == 0:
            return 0
        d = self.dim
        pk, ps = (ops.packed_row_bytes(d, self.bits - 1), ops.packed_row_bytes(d, 1)) if self.pack_storage else (d, d)
        return self._n_vectors * (pk + ps + 4)

    def compression_ratio(self, original_dtype: torch.dtype = torch.float32) -> float:
        if self._n_vectors == 0:
            return 1.0
        original = self._n_vectors * self.dim * (torch.finfo(original_dtype).bits // 8)
        compressed = self.memory_bytes()
        return original / compressed if compressed > 0 else float("inf")

    def reset(self) -> None:
        self._n_vectors = 0
        self._unpacked = None

    def __repr__(self) -> str:
        return (f"QuashIndex(dim={self.dim}, bits={self.bits}, n_vectors={self._n_vectors}, "
                f"pack_storage={self.pack_storage}, device={self.device})")
