#!/usr/bin/env python
"""Benchmark of the compressed-KV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the decode-attention configuration of the reference's benchmark list): one bf16
query token per step against a packed cache of batch 32 x 8 KV heads x 32768 tokens,
head_dim 128, 4 query heads per KV head, 3-bit keys (2-bit codes + sign bit) and 3-bit
values; K/V drawn N(0,1) with 4 channels per head scaled x8.  A step is one attention call
over the whole cache.  With N > 1 every rank holds such a cache for its own 8 KV heads (KV
heads are independent units: no collective in the path; weak scaling).

Printed JSON line (rank 0):
  value     packed cache bytes read per second, all ranks, inputs resident in HBM
  e2e       same through the public API with the query copied from pinned host memory and the
            output copied back, inside the timed region
  roofline  value of one rank against the measured HBM copy bandwidth
  cpu_baseline  the reference's CPU algorithm (oracle port, torch on all host cores) on one
            batch element of the same workload
  extra     compress / decompress / index-scan throughput on the other configurations

``--impl reference`` times the CPU port alone, on the same metric.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, HQ, HKV, S, D, G = 32, 32, 8, 32768, 128, 4
KEY_BITS, VAL_BITS = 3, 3
BYTES_PER_TOKEN_HEAD = 32 + 16 + 4 + 48 + 4        # codes, signs, norm, value codes, norm
WORKLOAD = "decode_attention_b32_kv8x32768_d128_gqa4_k3v3_bf16"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def outlier_kv(batch, heads, seq, dim, seed, device, dtype):
    g = torch.Generator(device=device).manual_seed(seed)
    K = torch.randn(batch, heads, seq, dim, generator=g, device=device)
    V = torch.randn(batch, heads, seq, dim, generator=g, device=device)
    for h in range(heads):
        ch = torch.randperm(dim, generator=torch.Generator().manual_seed(seed + h))[:4].to(device)
        K[:, h, :, ch] *= 8
        V[:, h, :, ch] *= 8
    return K.to(dtype), V.to(dtype)


class ClockSampler:
    """nvidia-smi clock / throttle samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        mhz, mx, reasons = [], None, set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7 or not f[1].isdigit():
                continue
            mhz.append(int(f[1]))
            mx = int(f[2]) if f[2].isdigit() else mx
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if mhz:
            self.summary = {"sm_mhz": statistics.median(mhz), "sm_max_mhz": mx, "reasons": sorted(reasons)}


def cpu_reference_step(sample, threads):
    """One pass of the reference's CPU attention over the sample (one batch element)."""
    from oracle import quashkv_oracle as orc
    q, planes, consts = sample
    return orc.attention_gqa(q, *planes, *consts, n_kv_heads=HKV)


def make_cpu_sample(seed=2):
    from oracle import quashkv_oracle as orc
    K, V = outlier_kv(1, HKV, S, D, seed, "cpu", torch.bfloat16)
    Pi, Sg = orc.rotation_matrix(D, 42), orc.sign_vector(D, 42)
    kc, kb = orc.lloyd_max_tables(D, KEY_BITS - 1)
    vc, vb = orc.lloyd_max_tables(D, VAL_BITS)
    mse, sg, kn = orc.compress_ip(K.float(), Pi, kb, kc, Sg)
    vi, vn = orc.compress_mse(V.float(), Pi, vb)
    q = torch.randn(1, HQ, 1, D, generator=torch.Generator().manual_seed(1000)).to(torch.bfloat16).float()
    return q, (mse, sg, kn, vi, vn), (Pi, kc, vc, Sg, orc.QJL_COEFF / D)


def time_cpu(steps, warmup):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    sample = make_cpu_sample()
    for _ in range(warmup):
        cpu_reference_step(sample, threads)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_reference_step(sample, threads)
        times.append(time.perf_counter() - t0)
    sample_bytes = HKV * S * BYTES_PER_TOKEN_HEAD
    sec = sum(times) / len(times)
    return sample_bytes / sec / 1e9, sec, threads


def cpu_extras():
    """The oracle port of the secondary paths on the host cores, on bounded samples (a few seconds in all):
    the CPU figures that stand beside the `extra` block of the GPU arm."""
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from oracle import quashkv_oracle as orc
    out = {}
    g = torch.Generator().manual_seed(3)
    n = 1 << 16
    x = torch.randn(n, D, generator=g).to(torch.bfloat16)
    Pi, Sg = orc.rotation_matrix(D, 42), orc.sign_vector(D, 42)
    for bits in (2, 3):
        cent, bnd = orc.lloyd_max_tables(D, bits)
        t0 = time.perf_counter()
        codes, norms = orc.compress_mse(x, Pi, bnd)
        orc.pack_bits(codes, bits)
        out[f"compress_mse_{bits}bit_Mvec_s"] = n / (time.perf_counter() - t0) / 1e6
        t0 = time.perf_counter()
        orc.decompress_mse(codes, norms, Pi, cent)
        out[f"decompress_mse_{bits}bit_Mvec_s"] = n / (time.perf_counter() - t0) / 1e6
    cent2, bnd2 = orc.lloyd_max_tables(D, 2)
    n_db, m = 100_000, 16
    db = torch.randn(n_db, D, generator=g)
    mse, sg, nrm = orc.compress_ip(db, Pi, bnd2, cent2, Sg)
    qs = torch.randn(m, D, generator=g)
    qjl = math.sqrt(math.pi / 2.0) / D
    t0 = time.perf_counter()
    orc.index_search(qs, mse, sg, nrm, Pi, cent2, Sg, qjl, 10)
    sec = time.perf_counter() - t0
    out["index_search_1M_x1024_queries_s"] = m / (sec * (1_000_000 / n_db))     # scaled to the 1M-row shard
    out["sample"] = "65,536 vectors (compress / decompress incl. packing); 100,000 rows x 16 queries scaled to 1M rows"
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(args.steps, 10)
    gbs, sec, threads = time_cpu(steps, min(args.warmup, 2))
    sample = "one batch element (8 KV heads x 32768 tokens, 32 query heads) of the 32-element workload per step"
    print(json.dumps({
        "impl": "reference", "metric": "packed_kv_decode_attention_hbm_gbps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": 32, "kv_heads_per_gpu": HKV, "query_heads_per_gpu": HQ,
                   "kv_len": S, "head_dim": D, "key_bits": KEY_BITS, "value_bits": VAL_BITS, "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extra": {} if args.no_extras else cpu_extras(),
    }))


def extras(device):
    """Secondary throughputs (not part of the timed headline): compress / decompress on the bulk
    prefill shape and the index scan on a 1M-vector shard."""
    import quashkv_b200 as qk
    out = {}

    def timed(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps / 1e3

    x = torch.randn(16 * 8 * 8192, D, device=device, generator=torch.Generator(device=device).manual_seed(3))
    heavy = torch.randperm(D, generator=torch.Generator().manual_seed(3))[:32].to(device)
    x[:, heavy] = torch.distributions.StudentT(3.0).sample((x.shape[0], 32)).to(device) * 4
    x = x.to(torch.bfloat16)
    n = x.shape[0]
    for bits in (2, 3, 4):
        q = qk.MSEQuantizer(D, bits, seed=42)
        sec = timed(lambda: q.compress_packed(x))
        codes, norms = q.compress_packed(x)
        out[f"compress_mse_{bits}bit_Mvec_s"] = n / sec / 1e6
        sec = timed(lambda: q.decompress_packed(codes, norms))
        out[f"decompress_mse_{bits}bit_Mvec_s"] = n / sec / 1e6
        if bits == 3:
            sec = timed(lambda: q.decompress_packed(codes, norms, out_dtype=torch.bfloat16))
            out["decompress_mse_3bit_bf16_out_Mvec_s"] = n / sec / 1e6
    ipq = qk.InnerProductQuantizer(D, 3, seed=42)
    out["compress_ip_3bit_Mvec_s"] = n / timed(lambda: ipq.compress_packed(x)) / 1e6
    mp = qk.MixedPrecisionMSEQuantizer(D, 3, 2, 32, seed=42)
    mp.calibrate(x[:4096].float())
    out["compress_mixed_2p5bit_Mvec_s"] = n / timed(lambda: mp.compress(x, packed=True)) / 1e6
    mcodes, mnorms = mp.compress(x, packed=True)
    out["decompress_mixed_2p5bit_Mvec_s"] = n / timed(lambda: mp.decompress(mcodes, mnorms, packed=True)) / 1e6
    del x
    # causal prefill attention over the packed cache: 2 x 8 KV heads x 4096 tokens, 32 query heads, all rows
    eng = qk.QuashKVEngine(D, 3, 3, seed=42, pack_storage=True)
    gk = torch.Generator(device=device).manual_seed(11)
    Kp = torch.randn(2, 8, 4096, D, device=device, generator=gk).to(torch.bfloat16)
    Vp = torch.randn(2, 8, 4096, D, device=device, generator=gk).to(torch.bfloat16)
    Qp = torch.randn(2, 32, 4096, D, device=device, generator=gk).to(torch.bfloat16)
    eng.append(Kp, Vp)
    out["prefill_causal_4096_ms"] = timed(lambda: eng.attention(Qp, causal=True), reps=2) * 1e3
    del eng, Kp, Vp, Qp
    # decode attention through a block table: the headline shape (32 sequences x 8 KV heads x 32768 tokens, 32
    # query heads) as 16-token pages handed out in random order, then the same pool with ragged lengths
    from quashkv_b200.integrations.vllm_backend import QuashKVPagedCache
    n_seq, per_seq = 32, 32768 // 16
    pool = QuashKVPagedCache(n_seq * per_seq, 8, D, device=device)
    gp = torch.Generator(device=device).manual_seed(12)
    for name, plane in pool.planes.items():
        if plane.dtype == torch.uint8:
            plane.copy_(torch.randint(0, 256, plane.shape, device=device, dtype=torch.uint8, generator=gp))
        else:
            plane.copy_(torch.rand(plane.shape, device=device, generator=gp) + 0.5)
    table = torch.randperm(n_seq * per_seq, device=device, generator=gp).to(torch.int32).reshape(n_seq, per_seq)
    Qd = torch.randn(n_seq, 32, 1, D, device=device, generator=gp).to(torch.bfloat16)
    row_bytes = 8 * (32 + 16 + 48 + 8)          # packed bytes of one token over the 8 KV heads
    full = torch.full((n_seq,), 32768, dtype=torch.int32, device=device)
    sec = timed(lambda: pool.attention_with_tables(Qd, table, full, 32768), reps=20)
    out["paged_decode_32x32768_GB_s"] = n_seq * 32768 * row_bytes / sec / 1e9
    ragged = torch.randint(1024, 32769, (n_seq,), device=device, generator=gp).to(torch.int32)
    sec = timed(lambda: pool.attention_with_tables(Qd, table, ragged, 32768), reps=20)
    out["paged_decode_ragged_1k_32k_GB_s"] = int(ragged.sum()) * row_bytes / sec / 1e9
    del pool, table, Qd
    g = torch.Generator(device=device).manual_seed(6)
    n_db, m = 1_000_000, 1024
    db = torch.randn(n_db, D, device=device, generator=g)
    db = db / db.norm(dim=1, keepdim=True) * (torch.rand(n_db, 1, device=device, generator=g) * 1.5 + 0.5)
    qs = torch.randn(m, D, device=device, generator=torch.Generator(device=device).manual_seed(7))
    index = qk.QuashIndex(D, 3, seed=42, pack_storage=True)
    index.add(db)
    sec = timed(lambda: index.search(qs, 10), reps=2)
    out["index_search_1M_x1024_queries_s"] = m / sec
    out["index_recall_at_10"] = index.recall_at_k(qs[:256], db, 10)
    return out


def run_ours(args):
    import torch.distributed as dist
    import quashkv_b200 as qk
    from quashkv_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU implementation")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _lib.lib()   # fail before any timing if the CUDA library is missing

    # ---- build the cache: bf16 K/V -> packed planes, batch row by batch row ----------------------
    eng = qk.QuashKVEngine(D, KEY_BITS, VAL_BITS, seed=42, device=device, pack_storage=True)
    B = args.batch
    eng.reserve(B, HKV, S, device)
    kq, vq = eng.key_quantizer, eng.value_quantizer
    from quashkv_b200 import ops
    Pi, kb, kc, Sg = kq._on(device)
    _, vb, _ = vq._on(device)
    p = eng._planes
    for b in range(B):
        K, V = outlier_kv(1, HKV, S, D, 2 + 31 * b + 1000 * rank, device, torch.bfloat16)
        sl = slice(b * HKV, (b + 1) * HKV)
        ops.append_kv(K, V, Pi, kb, kc, Sg, KEY_BITS - 1, vb, VAL_BITS, p["k_codes"][sl], p["k_signs"][sl],
                      p["k_norms"][sl], p["v_codes"][sl], p["v_norms"][sl], 0)
    eng._block_lens, eng._total_tokens = [S], S
    del K, V
    step_bytes = eng.actual_memory_bytes()
    assert step_bytes == B * HKV * S * BYTES_PER_TOKEN_HEAD

    q_host = [torch.randn(B, HQ, 1, D, generator=torch.Generator().manual_seed(1000 + s)).to(torch.bfloat16).pin_memory()
              for s in range(4)]
    q_dev = [q.to(device) for q in q_host]
    out_host = [torch.empty(B, HQ, 1, D, dtype=torch.float32).pin_memory() for _ in range(2)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    stream = torch.cuda.current_stream()
    # ---- device-resident timing -------------------------------------------------------------------
    for s in range(args.warmup):
        eng.attention(q_dev[s % 4])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        e0.record(stream)
        for s in range(args.steps):
            eng.attention(q_dev[s % 4])
        e1.record(stream)
        barrier()
    ms_dev = max_over_ranks(e0.elapsed_time(e1))

    # ---- end to end: pinned host query in, output back to pinned host, every step ----------------
    # (the engine's host entry point: copies on side streams, two buffers in rotation, so that a step's transfers
    # overlap the neighbouring steps' kernels; every step's query goes in and every step's output comes back)
    for s in range(args.warmup):
        eng.attention_from_host(q_host[s % 4], out_host[s % 2])
    barrier()
    e0.record(stream)
    for s in range(args.steps):
        landed = eng.attention_from_host(q_host[s % 4], out_host[s % 2])
    stream.wait_event(landed)              # the last output is in host memory when the clock stops
    e1.record(stream)
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    per_step = ms_dev / args.steps
    value = world * step_bytes / (per_step * 1e-3) / 1e9
    e2e = world * step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    peak, which = peaks()
    achieved = step_bytes / (per_step * 1e-3) / 1e9
    line = {
        "metric": "packed_kv_decode_attention_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": B, "kv_heads_per_gpu": HKV, "query_heads_per_gpu": HQ,
                   "kv_len": S, "head_dim": D, "key_bits": KEY_BITS, "value_bits": VAL_BITS,
                   "bytes_per_step_per_gpu": step_bytes, "l2": "inputs (872 MB per GPU) exceed the 126 MB L2"},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": q_host[0].numel() * 2,
                "d2h_bytes_per_step": out_host[0].numel() * 4},
        "gpu_launches": 2 * args.steps,   # query rotation (+ table prep), split scan with fused merge
        "clocks": clocks.summary,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": which,
                     "note": "per-GPU packed bytes / whole attention call (query rotation + split scan + merge)"},
    }
    # dram__bytes_read + write of one attend_decode_mma_kernel launch from the ncu capture summarised
    # in profiles/attend_decode_mma_decode_batch8.md (223.2 MB at batch 8, traffic grows with the
    # token-heads processed: x4 at the benchmark's batch 32)
    if B == 32:
        line["roofline"]["traffic"] = 4 * 223.2e6
    if B != 32:
        line["config"]["workload"] = WORKLOAD + f"_REDUCED_batch{B}"
    if world == 1 and not args.no_cpu:
        gbs, sec, threads = time_cpu(3, 1)
        line["cpu_baseline"] = {
            "value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "one batch element (8 KV heads x 32768 tokens, 32 query heads) per pass, mean of 3 passes"}
    if world == 1 and not args.no_extras:
        line["extra"] = extras(device)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--batch", type=int, default=B,
                    help="batch elements in the cache (default 32 = the benchmark workload; smaller for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--extras-only", action="store_true",
                    help="run only the secondary compress / decompress / index measurements (for profiler captures)")
    args = ap.parse_args()
    if args.batch == B:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    else:   # a reduced case for profiling: not a benchmark number
        args.no_extras = True
    if args.extras_only:
        torch.cuda.set_device(0)
        print(json.dumps({"extra": extras(torch.device("cuda", 0))}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
