"""Multi-GPU runs of the sharded paths (NCCL, one process per GPU).  Skipped with fewer than two GPUs.

Index: every rank builds the index over its row range, searches all queries, all-gathers the
per-rank top-k and merges; the result must equal the single-index search on rank 0's GPU.
Attention: KV heads are split over the ranks; gathered outputs must equal the unsharded call.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import quashkv_b200 as qk
        from quashkv_b200.distributed import gather_heads, heads_for_rank, sharded_quash_index
        g = torch.Generator().manual_seed(5)
        db = torch.randn(50_001, 128, generator=g).to(dev)
        qs = torch.randn(33, 128, generator=g).to(dev)
        sharded = sharded_quash_index(db, 128, bits=3, seed=42)
        s, i = sharded.search(qs, 10)
        whole = qk.QuashIndex(128, 3, seed=42, device=dev, pack_storage=True)
        whole.add(db)
        ws, wi = whole.search(qs, 10)
        ok_index = torch.equal(i, wi) and torch.equal(s, ws)

        B, Hkv, G, S, D = 2, 4, 4, 3000, 128
        K, V = torch.randn(B, Hkv, S, D, generator=g).to(dev), torch.randn(B, Hkv, S, D, generator=g).to(dev)
        Q = torch.randn(B, Hkv * G, 1, D, generator=g).to(dev)
        full = qk.QuashKVEngine(D, 3, 3, seed=42, pack_storage=True)
        full.append(K, V)
        want = full.attention(Q)
        h0, h1 = heads_for_rank(Hkv, world, rank)
        mine = qk.QuashKVEngine(D, 3, 3, seed=42, pack_storage=True)
        mine.append(K[:, h0:h1].contiguous(), V[:, h0:h1].contiguous())
        got = gather_heads(mine.attention(Q[:, h0 * G:h1 * G].contiguous()))
        # another head count gives another split plan: equal up to the rounding of the fp16 softmax weights
        ok_attn = float((got - want).norm() / want.norm()) < 1e-4
        out[rank] = "ok" if ok_index and ok_attn else f"index {ok_index} attention {ok_attn}"
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_index_and_head_sharded_attention_on_two_gpus():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
        assert dict(out) == {0: "ok", 1: "ok"}
