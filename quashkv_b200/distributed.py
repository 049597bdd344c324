"""Multi-GPU partitioning of the hot path: one process per GPU, ``torch.distributed``.

* Attention shards by KV head: every rank owns ``heads_for_rank`` of the cache planes and the
  query heads that read them; there is no exchange inside the path (the output stays
  sharded by head, optionally all-gathered).
* Index search shards by database rows: every rank scans its contiguous row range for all
  queries, the per-rank top-k lists (scores + global ids) are all-gathered (a few MB) and
  each rank merges them with the merge kernel.  The reference has neither; the merge rule is
  the search's own order (higher score first, then lower id).

The collective layer is independent of the device: ``ShardedIndex`` takes the local scan and
the merge as callables, so the exchange logic also runs on CPU ranks (gloo) in the tests.
"""

from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.distributed as dist


def row_range(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced row range of ``rank`` (the first n_rows % world ranks get one more)."""
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def heads_for_rank(n_kv_heads: int, world: int, rank: int) -> tuple[int, int]:
    """KV-head range of ``rank``; world must divide the head count (each rank then also owns the
    query heads group*start .. group*end)."""
    if n_kv_heads % world != 0:
        raise ValueError(f"{n_kv_heads} KV heads do not divide over {world} ranks")
    per = n_kv_heads // world
    return rank * per, (rank + 1) * per


def all_gather_topk(scores: torch.Tensor, ids: torch.Tensor, k: int, group=None):
    """Pad a rank's (M, k_local) list to k columns, all-gather, return (M, world*k) candidates.

    Raises on every rank if the ranks disagree on M or k (checked with a small all-gather
    before the payload so that a mismatch cannot leave a rank waiting in the collective)."""
    world = dist.get_world_size(group)
    meta = torch.tensor([scores.shape[0], k], dtype=torch.int64, device=scores.device)
    metas = [torch.empty_like(meta) for _ in range(world)]
    dist.all_gather(metas, meta, group=group)
    if any(not torch.equal(m, meta) for m in metas):
        raise RuntimeError(f"sharded search: ranks disagree on (queries, k): {[m.tolist() for m in metas]}")
    pad = k - scores.shape[1]
    if pad > 0:
        scores = torch.cat([scores, scores.new_full((scores.shape[0], pad), -math.inf)], dim=1)
        ids = torch.cat([ids, ids.new_full((ids.shape[0], pad), -1)], dim=1)
    scores, ids = scores.contiguous(), ids.contiguous()
    gs = [torch.empty_like(scores) for _ in range(world)]
    gi = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(gs, scores, group=group)
    dist.all_gather(gi, ids, group=group)
    return torch.cat(gs, dim=1), torch.cat(gi, dim=1)


class ShardedIndex:
    """Database-sharded search.  ``local_search(queries, k_local, id_base) -> (scores, ids)`` scans
    this rank's rows; ``merge(scores, ids, k) -> (scores, ids)`` reduces candidate lists."""

    def __init__(self, n_total: int, local_search: Callable, merge: Callable, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_total = n_total
        self.start, self.end = row_range(n_total, self.world, self.rank)
        self._search, self._merge = local_search, merge

    def search(self, queries: torch.Tensor, k: int = 10):
        k = min(k, self.n_total)
        n_local = self.end - self.start
        if n_local > 0:
            s, i = self._search(queries, min(k, n_local), self.start)
        else:   # an empty shard contributes no candidates
            s = queries.new_zeros((queries.shape[0], 0), dtype=torch.float32)
            i = torch.zeros((queries.shape[0], 0), dtype=torch.int64, device=queries.device)
        cs, ci = all_gather_topk(s, i, k, self.group)
        return self._merge(cs, ci, k)


def sharded_quash_index(database: torch.Tensor, dim: int, bits: int = 3, seed: int = 42, group=None):
    """Build this rank's QuashIndex over its row range of ``database`` (any rank may pass the full
    tensor or only its own rows via ``database[start:end]``) and wrap it for sharded search."""
    from . import ops
    from .nn_search import QuashIndex
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    start, end = row_range(database.shape[0], world, rank)
    index = QuashIndex(dim, bits, seed=seed, device=database.device, pack_storage=True)
    if end > start:
        index.add(database[start:end])
    return ShardedIndex(database.shape[0], lambda q, k, base: index.search(q, k, id_base=base),
                        ops.topk_merge, group)


def gather_heads(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather per-rank attention outputs (B, Hq/world, Q, d) along the head axis."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)
