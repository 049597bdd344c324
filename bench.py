#!/usr/bin/env python
"""Benchmark of the compressed-KV hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the decode-attention configuration of the reference's benchmark list): one bf16 query token per
step against a packed cache of batch 32 x 8 KV heads x 32768 tokens, head_dim 128, 4 query heads per KV
head, 3-bit keys (2-bit codes + sign bit) and 3-bit values; K/V drawn N(0,1) with 4 channels per head scaled
x8.  A step is one attention call over the whole cache.  With N > 1 the SAME cache is sharded by KV head:
rank r owns 8/N KV heads and the 32/N query heads that read them (KV heads are independent units: no
collective in the path; strong scaling, 872 MB / N per rank and step).

Timing: W warm-up steps, then blocks of exactly K steps, each bracketed by a barrier and a device
synchronisation and timed with CUDA events (max over ranks); blocks are repeated until half a second has
been timed and the MEDIAN block is reported, so that a block of a few milliseconds is not at the mercy of one
disturbance.  `ms_per_step` = median block / K.

Printed JSON line (rank 0):
  value     packed cache bytes read per second, all ranks, inputs resident in HBM
  e2e       same through the public API with the query copied from pinned host memory and the output copied
            back, inside the timed region
  roofline  one rank's bytes per second against the measured HBM copy bandwidth
  parity    relative L2 error of the timed configuration's output against the CPU oracle on a sampled head
  cpu_baseline  the reference's CPU algorithm (oracle port, torch on all host cores) on one batch element
  extra     compress / decompress / prefill / paged / index-search throughput on the other configurations

``--impl reference`` times the CPU port alone, on the same metric and configuration.
"""

from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import re
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
METRIC = "packed_kv_decode_attention_hbm_gbps"
MIN_TIMED_S = 0.5


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops_sustained", 1395.3)), "measured"
    return 6650.0, 1400.0, "fallback"


def workload_config(world: int, batch: int = B) -> dict:
    """The configuration both arms print: the whole job and one GPU's share of it."""
    return {"workload": WORKLOAD if batch == B else WORKLOAD + f"_REDUCED_batch{batch}",
            "batch": batch, "kv_heads": HKV, "query_heads": HQ, "kv_heads_per_gpu": HKV // world,
            "query_heads_per_gpu": HQ // world, "kv_len": S, "head_dim": D, "key_bits": KEY_BITS,
            "value_bits": VAL_BITS, "bytes_per_step": batch * HKV * S * BYTES_PER_TOKEN_HEAD,
            "bytes_per_step_per_gpu": batch * (HKV // world) * S * BYTES_PER_TOKEN_HEAD,
            "l2": "the cache (872 MB over all GPUs) is re-read every step; where a rank's share is below 256 MB "
                  "(8 GPUs: 109 MB, under the 126 MB L2) 1 GB is written between timed blocks"}


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
    """nvidia-smi clock / throttle samples of one GPU, every 100 ms from `start()` to `stop()`; the summary
    uses the samples whose time stamps fall inside the timed windows handed to `stop()`."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.gpu_id, self.proc = gpu_id, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", self.gpu_id], stdout=subprocess.PIPE, text=True)
        except OSError:
            self.proc = None
        return self

    def stop(self, windows):
        summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return summary
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
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                continue
            if not any(lo - 0.05 <= ts <= hi + 0.05 for lo, hi in windows):
                continue
            mhz.append(int(f[1]))
            mx = int(f[2]) if f[2].isdigit() else mx
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if mhz:
            summary = {"sm_mhz": statistics.median(mhz), "sm_max_mhz": mx, "reasons": sorted(reasons),
                       "samples": len(mhz)}
        return summary


# ---------------------------------------------------------------------------------------------------------
# CPU legs (the oracle port of the reference's algorithm, the only place this file runs anything of oracle/)
# ---------------------------------------------------------------------------------------------------------

CPU_SAMPLE = "one batch element (8 KV heads x 32768 tokens, 32 query heads) of the 32-element workload per step"


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
    """`steps` passes of the reference's CPU attention over the sample, after `warmup` passes."""
    from oracle import quashkv_oracle as orc
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, planes, consts = make_cpu_sample()
    for _ in range(warmup):
        orc.attention_gqa(q, *planes, *consts, n_kv_heads=HKV)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        orc.attention_gqa(q, *planes, *consts, n_kv_heads=HKV)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return HKV * S * BYTES_PER_TOKEN_HEAD / sec / 1e9, sec, threads


def cpu_extras():
    """The oracle port of the secondary paths on the host cores, on bounded samples (a few seconds in all):
    the CPU figures that stand beside the `extra` block of the GPU arm."""
    from oracle import quashkv_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
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
    out["index_search_10M_x10k_queries_s"] = m / (sec * (10_000_000 / n_db))    # and to the 10M-row database
    out["cores"] = os.cpu_count() or 1
    out["sample"] = ("65,536 vectors (compress / decompress incl. packing); 100,000 rows x 16 queries scaled "
                     "linearly in the rows to 1M and 10M rows")
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    gbs, sec, threads = time_cpu(args.steps, args.warmup)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(max(world, 1), args.batch),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": CPU_SAMPLE},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extra": {} if args.no_extras else cpu_extras(),
    }))


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------

def timed(fn, reps=10):
    """Seconds per call of fn on the current stream (two untimed calls first)."""
    fn()
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps / 1e3


def c3_tensor(device, rows=16 * 8 * 8192):
    """The bulk-prefill tensor: bf16 N(0,1) rows with 32 heavy-tail channels (Student-t, nu = 3, x4)."""
    x = torch.randn(rows, D, device=device, generator=torch.Generator(device=device).manual_seed(3))
    heavy = torch.randperm(D, generator=torch.Generator().manual_seed(3))[:32].to(device)
    x[:, heavy] = torch.distributions.StudentT(3.0).sample((rows, 32)).to(device) * 4
    return x.to(torch.bfloat16)


def compress_roofline(mvec_s, bits, hbm_gbs, tf_sustained, in_bytes=2 * D):
    """Compress of one bf16 vector reads 2 d bytes and writes the packed row and a norm; the rotation is 3 bf16
    products of 2 d^2 flops on the tensor cores (exact 3-term split of Pi).  The lower of the two bounds."""
    out_bytes = (D * bits + 7) // 8 + 4
    hbm_bound = hbm_gbs * 1e9 / (in_bytes + out_bytes) / 1e6
    tensor_bound = tf_sustained * 1e12 / (3 * 2 * D * D) / 1e6
    bound, peak = ("hbm", hbm_bound) if hbm_bound < tensor_bound else ("tensor", tensor_bound)
    return {"bound": bound, "achieved": mvec_s, "peak": peak, "unit": "Mvec/s", "frac": mvec_s / peak,
            "hbm_bound_Mvec_s": hbm_bound, "tensor_bound_Mvec_s": tensor_bound}


def config5(device, n_db=10_000_000, m=10_000, k=10, rows=None):
    """QuashIndex over (a shard of) the 10M x 128 database, 10k queries, k = 10: build in chunks, search, and
    recall@10 against exact fp32 inner products on 1024 of the queries (full database only)."""
    import quashkv_b200 as qk
    lo, hi = rows if rows is not None else (0, n_db)
    index = qk.QuashIndex(D, 3, seed=42, device=device, pack_storage=True)
    chunk = 1_000_000
    exact_s = exact_i = None
    qs = torch.randn(m, D, device=device, generator=torch.Generator(device=device).manual_seed(7))
    want_recall = rows is None
    for c0 in range(0, n_db, chunk):            # the database is generated chunk by chunk from per-chunk seeds
        c1 = min(c0 + chunk, n_db)
        if c1 <= lo or c0 >= hi:
            continue
        g = torch.Generator(device=device).manual_seed(6 + c0 // chunk)
        db = torch.randn(c1 - c0, D, device=device, generator=g)
        db = db / db.norm(dim=1, keepdim=True) * (torch.rand(c1 - c0, 1, device=device, generator=g) * 1.5 + 0.5)
        index.add(db[max(lo, c0) - c0:min(hi, c1) - c0])
        if want_recall:
            s, i = (qs[:1024] @ db.T).topk(k, dim=1)
            i = i + c0
            if exact_s is None:
                exact_s, exact_i = s, i
            else:
                s, j = torch.cat([exact_s, s], 1).topk(k, dim=1)
                exact_s, exact_i = s, torch.cat([exact_i, i], 1).gather(1, j)
        del db
    sec = timed(lambda: index.search(qs, k, id_base=lo), reps=2)
    out = {"rows": hi - lo, "queries": m, "k": k, "queries_s": m / sec, "search_ms": sec * 1e3}
    if want_recall:
        _, ids = index.search(qs[:1024], k)
        hits = (ids.unsqueeze(2) == exact_i.unsqueeze(1)).any(dim=2).float().sum(dim=1)
        out["recall_at_10"] = float(hits.mean() / k)
        out["recall_queries"] = 1024
        # dense contraction with one operand decoded on the fly: 2 * 2d flops per (query, row) pair
        out["tensor_TFLOP_s"] = 2 * 2 * D * float(hi - lo) * m / sec / 1e12
    return index, qs, out


def config4(device, with_cpu=True, new_tokens=256):
    """QuashKVCache inside a random-init Llama-architecture decoder (22 layers, hidden 2048, 32 query / 4 KV heads,
    head_dim 64, MLP 5632, vocab 32000, weights N(0, 0.02) from seed 4, bf16): a 1024-token prompt of random ids
    (seed 5), batch 8, 256 greedy tokens.  The compressed cache is attached as a transformers Cache whose
    attention runs on the packed cache (no decompression in the loop); tokens/s at 2 / 3 / 4 bits beside an
    uncompressed DynamicCache, and the cosine of every layer's attention output at the first decode step."""
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM
    from quashkv_b200.integrations.hf_cache import QuashKVCache, QuashKVCacheConfig, make_hf_cache
    cfg = LlamaConfig(num_hidden_layers=22, hidden_size=2048, num_attention_heads=32, num_key_value_heads=4,
                      head_dim=64, intermediate_size=5632, vocab_size=32000, max_position_embeddings=2048,
                      eos_token_id=None, bos_token_id=None, pad_token_id=None)
    torch.manual_seed(4)
    with torch.device(device):
        model = LlamaForCausalLM(cfg)
    model = model.to(torch.bfloat16).eval()
    prompt = torch.randint(0, 32000, (8, 1024), generator=torch.Generator().manual_seed(5)).to(device)
    layers = [m for m in model.modules() if hasattr(m, "layer_idx") and hasattr(m, "q_proj")]

    @torch.no_grad()
    def generate(cache, capture=None):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = model(input_ids=prompt, past_key_values=cache, use_cache=True)
        nxt = out.logits[:, -1].argmax(-1, keepdim=True)
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        hooks = []
        if capture is not None:             # attention outputs of the first decode step
            hooks = [m.register_forward_hook(lambda mod, a, o, i=i: capture.__setitem__(i, o[0].float())) for i, m in enumerate(layers)]
        for step in range(new_tokens):
            out = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            nxt = out.logits[:, -1].argmax(-1, keepdim=True)
            if step == 0:
                for h in hooks:
                    h.remove()
        torch.cuda.synchronize()
        t2 = time.perf_counter()
        return {"decode_tokens_s": prompt.shape[0] * new_tokens / (t2 - t1), "prefill_s": t1 - t0}

    out = {"model": "llama-architecture 22 x 2048, 32/4 heads, head_dim 64, random init (seed 4), bf16",
           "batch": 8, "prompt_tokens": 1024, "new_tokens": new_tokens}
    generate(DynamicCache(config=cfg))                       # warm-up of the model's kernels
    ref_attn = {}
    out["dynamic_cache"] = generate(DynamicCache(config=cfg), capture=ref_attn)
    for bits in (2, 3, 4):
        qc = QuashKVCache(cfg.num_hidden_layers, 64, QuashKVCacheConfig(key_bits=bits, value_bits=bits, seed=42), device=device)
        cache = make_hf_cache(qc, fused=True)
        previous = cache.attach(model)
        got = {}
        try:
            res = generate(cache, capture=got)
        finally:
            cache.detach(model, previous)
        cos = [float(torch.nn.functional.cosine_similarity(got[i].flatten(1), ref_attn[i].flatten(1), dim=1).mean())
               for i in range(len(layers))]
        res["attention_output_cosine_first_layer"] = cos[0]
        res["attention_output_cosine_mean"] = sum(cos) / len(cos)
        res["attention_output_cosine_min"] = min(cos)
        res["compression_ratio"] = qc.compression_stats()["overall_compression_ratio"]
        out[f"quashkv_{bits}bit"] = res
        del qc, cache
    if with_cpu:
        # The reference's loop on the host cores: per generated token and layer it decompresses the whole history
        # (keys and values) and attends over it.  One layer at the final length, scaled to 22 layers.
        from oracle import quashkv_oracle as orc
        torch.set_num_threads(os.cpu_count() or 1)
        Pi = orc.rotation_matrix(64, 42)
        cent, bnd = orc.lloyd_max_tables(64, 3)
        g = torch.Generator().manual_seed(5)
        codes, norms = orc.compress_mse(torch.randn(8, 4, 1280, 64, generator=g), Pi, bnd)
        q = torch.randn(8, 32, 1, 64, generator=g)
        t0 = time.perf_counter()
        for _ in range(3):
            k = orc.decompress_mse(codes, norms, Pi, cent)
            v = orc.decompress_mse(codes, norms, Pi, cent)
            torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(8, 1), v.repeat_interleave(8, 1))
        per_layer = (time.perf_counter() - t0) / 3
        out["cpu_reference_loop"] = {"decode_tokens_s": 8 / (22 * per_layer), "cores": os.cpu_count() or 1,
                                     "sample": "cache work of one layer at 1280 tokens (decompress K and V, attend), "
                                               "x 22 layers per token; the model's own matmuls not counted"}
    del model
    torch.cuda.empty_cache()
    return out


def extras(device, hbm_gbs, tf_sustained, with_cpu=True):
    """Secondary throughputs (not part of the timed headline): compress / decompress on the bulk prefill shape,
    causal prefill, the paged cache, and the index scan."""
    import quashkv_b200 as qk
    out = {}
    x = c3_tensor(device)
    n = x.shape[0]
    for bits in (2, 3, 4):
        q = qk.MSEQuantizer(D, bits, seed=42)
        sec = timed(lambda: q.compress_packed(x))
        codes, norms = q.compress_packed(x)
        out[f"compress_mse_{bits}bit_Mvec_s"] = n / sec / 1e6
        out[f"compress_mse_{bits}bit"] = {"value": n / sec / 1e6, "unit": "Mvec/s",
                                          "roofline": compress_roofline(n / sec / 1e6, bits, hbm_gbs, tf_sustained)}
        sec = timed(lambda: q.decompress_packed(codes, norms))
        out[f"decompress_mse_{bits}bit_Mvec_s"] = n / sec / 1e6
        if bits == 3:
            per_vec = (D * bits + 7) // 8 + 4 + 4 * D
            gbs = n * per_vec / sec / 1e9
            out["decompress_mse_3bit"] = {"value": n / sec / 1e6, "unit": "Mvec/s",
                                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_gbs, "unit": "GB/s",
                                                       "frac": gbs / hbm_gbs}}
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
    rec = pool.planes["records"]                    # random codes and sign bits, norms in [0.5, 1.5)
    rec.copy_(torch.randint(0, 256, rec.shape, device=device, dtype=torch.uint8, generator=gp))
    norms = torch.rand((*rec.shape[:-1], 32), device=device, generator=gp) + 0.5
    rec[..., 1536:] = norms.view(torch.uint8).reshape(*rec.shape[:-1], 128)
    table = torch.randperm(n_seq * per_seq, device=device, generator=gp).to(torch.int32).reshape(n_seq, per_seq)
    Qd = torch.randn(n_seq, 32, 1, D, device=device, generator=gp).to(torch.bfloat16)
    row_bytes = 8 * BYTES_PER_TOKEN_HEAD          # packed bytes of one token over the 8 KV heads
    full = torch.full((n_seq,), 32768, dtype=torch.int32, device=device)
    sec = timed(lambda: pool.attention_with_tables(Qd, table, full, 32768), reps=20)
    out["paged_decode_32x32768_GB_s"] = n_seq * 32768 * row_bytes / sec / 1e9
    ragged = torch.randint(1024, 32769, (n_seq,), device=device, generator=gp).to(torch.int32)
    sec = timed(lambda: pool.attention_with_tables(Qd, table, ragged, 32768), reps=20)
    out["paged_decode_ragged_1k_32k_GB_s"] = int(ragged.sum()) * row_bytes / sec / 1e9
    del pool, table, Qd, rec, norms
    # index: the 10M x 128 database with 10k queries (build in chunks, recall on 1024 queries), then 1024
    # queries over its first million rows
    index, qs, c5 = config5(device)
    out["config5_index_10M_x10k"] = c5
    small = qk.QuashIndex(D, 3, seed=42, device=device, pack_storage=True)
    small._codes, small._signs, small._norm_plane = (index._codes[:1_000_000], index._signs[:1_000_000],
                                                     index._norm_plane[:1_000_000])
    small._capacity = small._n_vectors = 1_000_000
    sec = timed(lambda: small.search(qs[:1024], 10), reps=2)
    out["index_search_1M_x1024_queries_s"] = 1024 / sec
    del index, small, qs
    torch.cuda.empty_cache()
    out["config4_llama_generation"] = config4(device, with_cpu=with_cpu)
    return out


def sharded_extras(device, world, rank, barrier, max_over_ranks):
    """At N > 1: compress over contiguous row ranges (no exchange) and the database-sharded index search with
    its all-gather and merge inside the timed call."""
    import quashkv_b200 as qk
    from quashkv_b200 import distributed as qd, ops
    out = {}
    # compress: the two bulk-prefill tensors (2 x 1,048,576 vectors) split by rows
    total = 2 * 16 * 8 * 8192
    lo, hi = qd.row_range(total, world, rank)
    x = c3_tensor(device, hi - lo)
    q = qk.MSEQuantizer(D, 3, seed=42)
    q.compress_packed(x)
    barrier()
    sec = max_over_ranks(timed(lambda: q.compress_packed(x)) * 1e3) / 1e3
    out["compress_mse_3bit_sharded_Mvec_s"] = total / sec / 1e6
    del x
    # index: 10M rows sharded, 10k queries on every rank, all-gather of (scores, ids), merge
    n_db = 10_000_000
    lo, hi = qd.row_range(n_db, world, rank)
    index, qs, local = config5(device, rows=(lo, hi))
    sharded = qd.ShardedIndex(n_db, lambda qq, k, base: index.search(qq, k, id_base=base), ops.topk_merge)
    sharded.search(qs, 10)
    barrier()
    sec = max_over_ranks(timed(lambda: sharded.search(qs, 10), reps=2) * 1e3) / 1e3
    s_loc, i_loc = index.search(qs, 10, id_base=lo)
    gather_sec = timed(lambda: qd.all_gather_topk(s_loc, i_loc, 10), reps=3)
    out["index_sharded_10M_x10k"] = {"queries_s": qs.shape[0] / sec, "search_ms": sec * 1e3,
                                      "rows_per_rank": hi - lo, "local_scan_ms": local["search_ms"],
                                      "all_gather_ms": gather_sec * 1e3, "all_gather_share": gather_sec / sec}
    del index
    return out


def run_ours(args):
    import torch.distributed as dist
    import quashkv_b200 as qk
    from quashkv_b200 import _lib
    from quashkv_b200.distributed import heads_for_rank

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
    hbm_gbs, tf_sustained, which = peaks()

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

    def all_ranks(ms):
        if world == 1:
            return [ms]
        t = torch.tensor([ms], device=device)
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        return [float(p) for p in parts]

    # ---- build this rank's share of the cache: bf16 K/V -> tile records, batch row by batch row -------------
    Bn = args.batch
    h0, h1 = heads_for_rank(HKV, world, rank)
    hkv, hq = h1 - h0, (h1 - h0) * G

    def build_cache(head_lo, head_hi):
        cache = qk.QuashKVEngine(D, KEY_BITS, VAL_BITS, seed=42, device=device, pack_storage=True)
        n_heads = head_hi - head_lo
        cache.reserve(Bn, n_heads, S, device)
        for b in range(Bn):     # the same global tensor at every N: all 8 heads are drawn, the rank keeps its own
            K, V = outlier_kv(1, HKV, S, D, 2 + 31 * b, device, torch.bfloat16)
            cache._write(K[:, head_lo:head_hi].contiguous(), V[:, head_lo:head_hi].contiguous(), b * n_heads, 0)
        cache._block_lens, cache._total_tokens = [S], S
        return cache

    eng = build_cache(h0, h1)
    step_bytes = eng.actual_memory_bytes()
    assert step_bytes == Bn * hkv * S * BYTES_PER_TOKEN_HEAD
    q_full = [torch.randn(Bn, HQ, 1, D, generator=torch.Generator().manual_seed(1000 + s)).to(torch.bfloat16)
              for s in range(4)]
    q_host = [q[:, h0 * G:h1 * G].contiguous().pin_memory() for q in q_full]
    q_dev = [q.to(device) for q in q_host]
    out_host = [torch.empty(Bn, hq, 1, D, dtype=torch.float32).pin_memory() for _ in range(2)]
    flush = torch.empty(1 << 30, dtype=torch.uint8, device=device) if step_bytes < (256 << 20) else None

    stream = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    windows = []

    def run_blocks(step, finish=None):
        """Blocks of args.steps steps until MIN_TIMED_S is timed (3 to 400 blocks); (median block ms as max over
        ranks, that block's per-rank ms, number of blocks)."""
        blocks, spent = [], 0.0
        while len(blocks) < min(3, args.max_blocks) or (spent < MIN_TIMED_S and len(blocks) < args.max_blocks):
            if flush is not None:
                flush.fill_(len(blocks) & 0xFF)         # a rank's share fits in L2: evict it between blocks
            barrier()
            t0 = time.time()
            e0.record(stream)
            for s in range(args.steps):
                step(s)
            if finish is not None:
                finish()
            e1.record(stream)
            barrier()
            windows.append((t0, time.time()))
            per_rank = all_ranks(e0.elapsed_time(e1))
            blocks.append((max(per_rank), per_rank))
            spent += max(per_rank) / 1e3
        blocks.sort(key=lambda blk: blk[0])
        mid = blocks[len(blocks) // 2]
        return mid[0], mid[1], len(blocks)

    sampler = None
    if rank == 0:
        try:
            gpu_id = "GPU-" + str(torch.cuda.get_device_properties(local).uuid)
        except Exception:
            gpu_id = str(local)
        sampler = ClockSampler(gpu_id).start()
    # ---- device-resident timing -------------------------------------------------------------------
    t_start = time.time()
    for s in range(args.warmup):
        eng.attention(q_dev[s % 4])
    barrier()
    while args.max_blocks > 1 and time.time() - t_start < 1.0:      # the clock sampler runs for a second before the first timed block
        eng.attention(q_dev[0])
        torch.cuda.synchronize()
    ms_dev, ranks_dev, n_blocks = run_blocks(lambda s: eng.attention(q_dev[s % 4]))

    # ---- end to end: pinned host query in, output back to pinned host, every step ----------------
    # (the engine's host entry point: copies on side streams, two buffers in rotation, so that a step's transfers
    # overlap the neighbouring steps' kernels; every step's query goes in and every step's output comes back)
    for s in range(args.warmup):
        eng.attention_from_host(q_host[s % 4], out_host[s % 2])
    landed = [None]

    def e2e_step(s):
        landed[0] = eng.attention_from_host(q_host[s % 4], out_host[s % 2])

    # the clock stops when the last output of the block is in host memory
    ms_e2e, ranks_e2e, _ = run_blocks(e2e_step, finish=lambda: stream.wait_event(landed[0]))
    clocks = sampler.stop(windows) if sampler is not None else None

    # host time of one call with the device idle (allocations, argument marshalling, two launches)
    torch.cuda.synchronize()
    n_host = 50 if args.max_blocks > 1 else 1
    t0 = time.perf_counter()
    for s in range(n_host):
        eng.attention(q_dev[s % 4])
    host_us = (time.perf_counter() - t0) / n_host * 1e6
    torch.cuda.synchronize()
    parity = parity_of_timed_config(eng, q_dev[0], h0) if rank == 0 else None

    extra = {}
    if world > 1 and not args.no_extras:
        # the same step with all 8 KV heads on every rank (weak scaling of the same kernel), for comparison
        del eng
        weak = build_cache(0, HKV)
        qw = [q.to(device) for q in q_full]
        for s in range(args.warmup):
            weak.attention(qw[s % 4])
        flush = None
        ms_weak, _, _ = run_blocks(lambda s: weak.attention(qw[s % 4]))
        extra["weak_scaling_8_kv_heads_per_gpu_GB_s"] = \
            world * weak.actual_memory_bytes() / (ms_weak / args.steps * 1e-3) / 1e9
        del weak, qw
        extra.update(sharded_extras(device, world, rank, barrier, max_over_ranks))
        eng = None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    per_step = ms_dev / args.steps
    total_bytes = world * step_bytes
    value = total_bytes / (per_step * 1e-3) / 1e9
    e2e = total_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
    achieved = step_bytes / (per_step * 1e-3) / 1e9          # one rank's bytes over the slowest rank's time
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "f16",
        "dtype_note": "fp16 tensor-core operands (decoded codes, query, softmax weights), fp32 accumulation",
        "data": "synthetic",
        "config": workload_config(world, Bn),
        "timing": {"blocks": n_blocks, "block_steps": args.steps, "reported": "median block, max over ranks",
                   "per_rank_ms_per_step": [m / args.steps for m in ranks_dev],
                   "per_rank_ms_per_step_e2e": [m / args.steps for m in ranks_e2e],
                   "host_us_per_call": host_us},
        "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": q_host[0].numel() * 2,
                "d2h_bytes_per_step": out_host[0].numel() * 4},
        "gpu_launches": 2 * args.steps,   # per block: query rotation (+ table prep), record scan with fused merge
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "traffic": None, "peak_source": which,
                     "note": "one GPU's packed bytes / its whole attention call (query rotation + record scan + merge)"},
        "parity": parity,
    }
    # dram bytes per token-head of one attend_tiled_kernel launch, from the ncu capture summarised in profiles/
    # (taken at batch 8; traffic grows in proportion to the token-heads a launch processes)
    prof = os.path.join(ROOT, "profiles", "attend_tiled_decode_batch8.md")
    if os.path.exists(prof):
        with open(prof) as f:
            m = re.search(r"dram_bytes_per_token_head:\s*([0-9.]+)", f.read())
        if m:
            line["roofline"]["traffic"] = float(m.group(1)) * Bn * hkv * S
    if world == 1 and not args.no_cpu:
        gbs, sec, threads = time_cpu(3, 1)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": CPU_SAMPLE + ", mean of 3 passes"}
    if world == 1 and not args.no_extras:
        del eng
        extra.update(extras(device, hbm_gbs, tf_sustained, with_cpu=not args.no_cpu))
        if not args.no_cpu:
            extra["cpu"] = cpu_extras()
    if extra:
        line["extra"] = extra
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def parity_of_timed_config(eng, q, head0):
    """Output of the timed engine for batch element 0, its first KV head, against the CPU oracle on the same
    tokens (a check of what was timed, not a timed quantity)."""
    from oracle import quashkv_oracle as orc
    out = eng.attention(q)[:1, :G].float().cpu()
    K, V = outlier_kv(1, HKV, S, D, 2, q.device, torch.bfloat16)
    Kh, Vh = K[:, head0:head0 + 1].float().cpu(), V[:, head0:head0 + 1].float().cpu()
    Pi, Sg = orc.rotation_matrix(D, 42), orc.sign_vector(D, 42)
    kc, kb = orc.lloyd_max_tables(D, KEY_BITS - 1)
    vc, vb = orc.lloyd_max_tables(D, VAL_BITS)
    mse, sg, kn = orc.compress_ip(Kh, Pi, kb, kc, Sg)
    vi, vn = orc.compress_mse(Vh, Pi, vb)
    want = orc.attention_gqa(q[:1, :G].float().cpu(), mse, sg, kn, vi, vn, Pi, kc, vc, Sg, orc.QJL_COEFF / D,
                             n_kv_heads=1)
    err = float((out - want).norm() / want.norm())
    return {"rel_l2_vs_oracle": err, "bar": 1e-3,
            "checked": "batch element 0, first KV head of rank 0 (4 query heads, 32768 tokens)"}


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
    ap.add_argument("--max-blocks", type=int, default=400,
                    help="upper limit of timed blocks per measurement (1 for profiler captures)")
    ap.add_argument("--extras-only", action="store_true",
                    help="run only the secondary compress / decompress / index measurements (for profiler captures)")
    args = ap.parse_args()
    if args.batch == B:
        args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    else:   # a reduced case for profiling: not a benchmark number
        args.no_extras = True
    if args.extras_only:
        torch.cuda.set_device(0)
        hbm, tf, _ = peaks()
        print(json.dumps({"extra": extras(torch.device("cuda", 0), hbm, tf)}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
