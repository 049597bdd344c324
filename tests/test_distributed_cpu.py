"""The sharded-search exchange on two CPU ranks (gloo): row ranges, global ids, padding of
short shards, the all-gather layout and the merge rule, with the oracle as the local scan.
Failure handling is exercised on the host: ranks that disagree on k raise on every rank."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from quashkv_b200.distributed import ShardedIndex, heads_for_rank, row_range
from oracle import quashkv_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, case, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d, m, k = 64, 6, 10
        g = torch.Generator().manual_seed(99)
        db = torch.randn(n, d, generator=g)
        qs = torch.randn(m, d, generator=g)
        Pi, S = orc.rotation_matrix(d, 42), orc.sign_vector(d, 42)
        cent, bnd = orc.lloyd_max_tables(d, 2)
        mse, sg, nrm = orc.compress_ip(db, Pi, bnd, cent, S)
        scale = orc.QJL_COEFF / d

        def local(q, kk, base):
            a, b = row_range(n, world, rank)
            s, i = orc.index_search(q, mse[a:b], sg[a:b], nrm[a:b], Pi, cent, S, scale, kk)
            return s, i + base

        if case == "mismatch":
            idx = ShardedIndex(n, local, orc.merge_topk)
            try:
                idx.search(qs, k + rank)          # ranks disagree on k
                out[rank] = "no error"
            except RuntimeError as e:
                out[rank] = "raised" if "disagree" in str(e) else repr(e)
            return
        idx = ShardedIndex(n, local, orc.merge_topk)
        s, i = idx.search(qs, k)
        ws, wi = orc.index_search(qs, mse, sg, nrm, Pi, cent, S, scale, k)
        ok = torch.equal(i, wi) and torch.allclose(s, ws, atol=1e-5)
        out[rank] = "ok" if ok else f"ids differ: {i.tolist()} vs {wi.tolist()}"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n,case", [(1000, "search"), (13, "search"), (1, "search"), (500, "mismatch")])
def test_sharded_search_two_cpu_ranks(n, case):
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, n, case, out), nprocs=world, join=True)
        want = "raised" if case == "mismatch" else "ok"
        assert dict(out) == {0: want, 1: want}


def test_partition_helpers():
    assert [row_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert [row_range(2, 4, r) for r in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 2)]
    covered = np.concatenate([np.arange(*row_range(10_000_000, 8, r)) for r in range(8)])
    assert covered.size == 10_000_000 and np.array_equal(covered, np.arange(10_000_000))
    assert [heads_for_rank(8, w, w - 1) for w in (1, 2, 4, 8)] == [(0, 8), (4, 8), (6, 8), (7, 8)]
    with pytest.raises(ValueError):
        heads_for_rank(8, 3, 0)
