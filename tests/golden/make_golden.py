"""Generate the golden vectors under tests/golden/ from the reference implementation.

Run in a container where the reference project is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py [--ref /path/to/reference]

It imports the reference's own classes (read-only), runs them on seeded inputs,
asserts that the CPU oracle (oracle/quashkv_oracle.py) reproduces every output
bit for bit, and writes small ``.npz`` fixtures.  The tests read only the
fixtures; the reference is not needed to run them.

Inputs are drawn from ``torch.Generator`` seeds and are stored in the fixture
too (the generator's stream is not guaranteed across torch builds).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import quashkv_oracle as orc  # noqa: E402


def npy(t):
    return t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)


def same(a, b, what):
    a, b = npy(a), npy(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    assert np.array_equal(a, b), f"oracle != reference for {what}"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", required=True, help="checkout of the reference project (the directory that holds quashkv/)")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    sys.dont_write_bytecode = True
    import quashkv as ref
    from quashkv.triton_kernels.decompress import _decompress_ip_pytorch
    from quashkv.triton_kernels.attention import _fused_attention_pytorch, CompressedBlock
    from quashkv.integrations.hf_cache import QuashKVCache

    torch.set_num_threads(max(1, os.cpu_count() or 1))

    # ---- constants: codebooks, rotations, sign vectors ------------------------------
    consts = {}
    for d in (64, 96, 128):
        for bits in (1, 2, 3, 4):
            cb = ref.LloydMaxCodebook(d, bits)
            c, b = orc.lloyd_max_tables(d, bits)
            same(c, cb.centroids, f"centroids d={d} b={bits}")
            same(b, cb.boundaries, f"boundaries d={d} b={bits}")
            consts[f"cent_d{d}_b{bits}"] = npy(cb.centroids)
            consts[f"bnd_d{d}_b{bits}"] = npy(cb.boundaries)
    cbx = ref.LloydMaxCodebook(64, 2, use_exact_pdf=True)
    cx, bx = orc.lloyd_max_tables(64, 2, exact_pdf=True)
    same(cx, cbx.centroids, "exact-pdf centroids")
    consts["cent_exact_d64_b2"], consts["bnd_exact_d64_b2"] = npy(cx), npy(bx)
    for d, seed in ((128, 0), (128, 42), (64, 42), (96, 42), (64, 43)):
        q = ref.InnerProductQuantizer(d, 3, seed=seed)
        same(orc.rotation_matrix(d, seed), q.mse_quantizer.Pi, f"Pi d={d} seed={seed}")
        same(orc.sign_vector(d, seed), q.S, f"S d={d} seed={seed}")
        consts[f"Pi_d{d}_s{seed}"] = npy(q.mse_quantizer.Pi)
        consts[f"S_d{d}_s{seed}"] = npy(q.S)
    np.savez_compressed(os.path.join(HERE, "constants.npz"), **consts)

    # ---- packing known answers and round trips --------------------------------------
    pk = {}
    for bits in (1, 2, 3, 4):
        for d in (128, 64, 63, 65, 100, 127, 129, 8, 1):
            g = torch.Generator().manual_seed(100 * bits + d)
            codes = torch.randint(0, 1 << bits, (3, 5, d), generator=g, dtype=torch.uint8)
            p = ref.pack_bits(codes, bits)
            same(orc.pack_bits(codes, bits), p, f"pack b={bits} d={d}")
            same(orc.unpack_bits(p, bits, d), ref.unpack_bits(p, bits, d), f"unpack b={bits} d={d}")
            same(ref.unpack_bits(p, bits, d), codes, "round trip")
            pk[f"codes_b{bits}_d{d}"] = npy(codes)
            pk[f"packed_b{bits}_d{d}"] = npy(p)
    pk["ka_pack3_0to7"] = npy(ref.pack_bits(torch.arange(8, dtype=torch.uint8)[None], 3))
    pk["ka_pack2_0123"] = npy(ref.pack_bits(torch.tensor([[0, 1, 2, 3]], dtype=torch.uint8), 2))
    pk["ka_pack4_12"] = npy(ref.pack_bits(torch.tensor([[1, 2]], dtype=torch.uint8), 4))
    pk["ka_pack1_10000001"] = npy(ref.pack_bits(torch.tensor([[1, 0, 0, 0, 0, 0, 0, 1]], dtype=torch.uint8), 1))
    np.savez_compressed(os.path.join(HERE, "packing.npz"), **pk)

    # ---- configuration 1: engine(128, 3, 3, seed=0), (1,8,512,128) fp32 -------------
    g = torch.Generator().manual_seed(1234)
    K = torch.randn(1, 8, 512, 128, generator=g)
    V = torch.randn(1, 8, 512, 128, generator=g)
    Q = torch.randn(1, 8, 1, 128, generator=g)
    eng = ref.QuashKVEngine(128, 3, 3, seed=0, pack_storage=True)
    eng.append(K, V)
    out = eng.attention(Q)
    blk = eng._cache[0]
    kq, vq = eng.key_quantizer, eng.value_quantizer
    Pi, S = kq.mse_quantizer.Pi, kq.S
    kc, kb = kq.mse_quantizer.codebook.centroids, kq.mse_quantizer.codebook.boundaries
    vc, vb = vq.codebook.centroids, vq.codebook.boundaries
    mse, sg, kn = orc.compress_ip(K, Pi, kb, kc, S)
    vi, vn = orc.compress_mse(V, Pi, vb)
    same(orc.pack_bits(mse, 2), blk.mse_indices, "C1 mse plane")
    same(orc.pack_bits(sg, 1), blk.qjl_signs, "C1 qjl plane")
    same(orc.pack_bits(vi, 3), blk.val_indices, "C1 val plane")
    same(kn, blk.key_norms, "C1 key norms")
    same(vn, blk.val_norms, "C1 val norms")
    o = orc.attention(Q, mse, sg, kn, vi, vn, Pi, kc, vc, S, kq.qjl_scale)
    same(o, out, "C1 attention")
    # the value reconstruction and both key reconstructions
    vrec = vq.decompress(vi, vn)
    same(orc.decompress_mse(vi, vn, Pi, vc), vrec, "C1 value decompress")
    krec_ip = _decompress_ip_pytorch(mse, sg, kn, Pi, kc, S, kq.qjl_scale)
    same(orc.decompress_ip(mse, sg, kn, Pi, kc, S, kq.qjl_scale), krec_ip, "C1 key decompress (ip)")
    # grouped-query decode on the same cache: 32 query heads on 8 KV heads
    Qg = torch.randn(1, 32, 1, 128, generator=g)
    og = eng.attention(Qg.reshape(1, 8, 4, 128)).reshape(1, 32, 1, 128)
    same(orc.attention_gqa(Qg, mse, sg, kn, vi, vn, Pi, kc, vc, S, kq.qjl_scale, n_kv_heads=8), og, "C1 gqa")
    np.savez_compressed(
        os.path.join(HERE, "config1.npz"),
        K=npy(K), V=npy(V), Q=npy(Q), Qg=npy(Qg),
        mse_plane=npy(blk.mse_indices), qjl_plane=npy(blk.qjl_signs), val_plane=npy(blk.val_indices),
        key_norms=npy(blk.key_norms), val_norms=npy(blk.val_norms),
        out=npy(out), out_gqa=npy(og),
        vrec_head0=npy(vrec[0, 0, :64]), krec_ip_head0=npy(krec_ip[0, 0, :64]),
    )

    # ---- multi-block engines, causal, other head dims and bit widths ----------------
    eg = {}
    case = 0
    for (D, kbits, vbits, seed, blocks, qlen, causal) in (
        (64, 3, 3, 42, (32,), 4, False),
        (64, 3, 3, 42, (16, 8), 4, False),
        (64, 3, 3, 42, (16, 1, 1, 1, 5), 5, True),
        (96, 3, 3, 42, (17,), 3, True),
        (128, 4, 4, 42, (33, 15), 2, True),
        (128, 2, 2, 42, (40,), 1, False),
        (128, 3, 4, 7, (129,), 7, True),
        (64, 4, 2, 42, (1,), 1, False),
    ):
        g = torch.Generator().manual_seed(500 + case)
        e = ref.QuashKVEngine(D, kbits, vbits, seed=seed, pack_storage=bool(case % 2))
        ks, vs = [], []
        for n in blocks:
            k = torch.randn(2, 3, n, D, generator=g)
            v = torch.randn(2, 3, n, D, generator=g) * 1.7
            e.append(k, v)
            ks.append(k)
            vs.append(v)
        q = torch.randn(2, 3, qlen, D, generator=g)
        o = e.attention(q, causal=causal)
        kq, vq = e.key_quantizer, e.value_quantizer
        Pi, S = kq.mse_quantizer.Pi, kq.S
        kc, kb = kq.mse_quantizer.codebook.centroids, kq.mse_quantizer.codebook.boundaries
        Kc, Vc = torch.cat(ks, 2), torch.cat(vs, 2)
        mse, sg, kn = orc.compress_ip(Kc, Pi, kb, kc, S)
        vi, vn = orc.compress_mse(Vc, Pi, vq.codebook.boundaries)
        un = [e._unpack_block(b) for b in e._cache]
        same(mse, torch.cat([u[0] for u in un], 2), f"eng{case} mse")
        same(sg, torch.cat([u[1] for u in un], 2), f"eng{case} qjl")
        same(vi, torch.cat([u[2] for u in un], 2), f"eng{case} val")
        oo = orc.attention(q, mse, sg, kn, vi, vn, Pi, kc, vq.codebook.centroids, S, kq.qjl_scale,
                           causal=causal, total_tokens=e.total_tokens)
        # softmax over one concatenated score row: identical op order, so exact
        same(oo, o, f"eng{case} attention")
        # the reference's own online-softmax twin agrees to rounding only
        blocks_c = [CompressedBlock(u[0], u[1], b.key_norms, u[2], b.val_norms, b.seq_len)
                    for u, b in zip(un, e._cache)]
        o2 = _fused_attention_pytorch(q, blocks_c, Pi, kc, vq.codebook.centroids, S, kq.qjl_scale,
                                      1.0 / D ** 0.5, causal, e.total_tokens)
        assert torch.allclose(o2, o, atol=1e-5)
        eg[f"e{case}_meta"] = np.array([D, kbits, vbits, seed, qlen, int(causal), e.total_tokens])
        eg[f"e{case}_K"], eg[f"e{case}_V"], eg[f"e{case}_Q"] = npy(Kc), npy(Vc), npy(q)
        eg[f"e{case}_Pi"] = npy(Pi)
        eg[f"e{case}_mse"], eg[f"e{case}_qjl"], eg[f"e{case}_val"] = npy(mse), npy(sg), npy(vi)
        eg[f"e{case}_kn"], eg[f"e{case}_vn"], eg[f"e{case}_out"] = npy(kn), npy(vn), npy(o)
        case += 1
    eg["n_cases"] = np.array(case)
    np.savez_compressed(os.path.join(HERE, "engine_cases.npz"), **eg)

    # ---- quantiser classes at several widths, zero and tiny vectors -----------------
    qz = {}
    g = torch.Generator().manual_seed(77)
    for d in (64, 128):
        x = torch.randn(300, d, generator=g) * 3.0
        x[0] = 0.0
        x[1] = 1e-12
        x[2, 1:] = 0.0
        qz[f"x_d{d}"] = npy(x)
        for bits in (1, 2, 3, 4):
            m = ref.MSEQuantizer(d, bits, seed=42)
            idx, nrm = m.compress(x)
            i2, n2 = orc.compress_mse(x, m.Pi, m.codebook.boundaries)
            same(i2, idx, f"mse compress d={d} b={bits}")
            same(n2, nrm, "norms")
            rec = m.decompress(idx, nrm)
            same(orc.decompress_mse(idx, nrm, m.Pi, m.codebook.centroids), rec, "mse decompress")
            qz[f"mse_idx_d{d}_b{bits}"], qz[f"mse_norm_d{d}_b{bits}"] = npy(idx), npy(nrm)
            qz[f"mse_rec_d{d}_b{bits}"] = npy(rec)
        for bits in (2, 3, 4):
            ipq = ref.InnerProductQuantizer(d, bits, seed=42)
            a, b, c = ipq.compress(x)
            a2, b2, c2 = orc.compress_ip(x, ipq.mse_quantizer.Pi, ipq.mse_quantizer.codebook.boundaries,
                                         ipq.mse_quantizer.codebook.centroids, ipq.S)
            same(a2, a, "ip mse"), same(b2, b, "ip qjl"), same(c2, c, "ip norms")
            qz[f"ip_mse_d{d}_b{bits}"], qz[f"ip_qjl_d{d}_b{bits}"], qz[f"ip_norm_d{d}_b{bits}"] = npy(a), npy(b), npy(c)
            rec = _decompress_ip_pytorch(a, b, c, ipq.mse_quantizer.Pi, ipq.mse_quantizer.codebook.centroids,
                                         ipq.S, ipq.qjl_scale)
            qz[f"ip_rec_d{d}_b{bits}"] = npy(rec)
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **qz)

    # ---- mixed precision -------------------------------------------------------------
    g = torch.Generator().manual_seed(3)
    d = 128
    x = torch.randn(1536, d, generator=g)
    heavy = torch.randperm(d, generator=g)[:32]
    t = torch.distributions.StudentT(3.0)
    torch.manual_seed(33)
    x[:, heavy] = t.sample((1536, 32)) * 4.0
    mp = ref.MixedPrecisionMSEQuantizer(d, 3, 2, 32, seed=42)
    i_un, n_un = mp.compress(x[:64])
    same(orc.compress_mixed(x[:64], mp.Pi, None, mp.outlier_codebook.boundaries,
                            mp.regular_codebook.boundaries)[0], i_un, "mixed uncalibrated")
    mp.calibrate(x[:1024])
    ch = orc.outlier_channels(x[:1024], mp.Pi, 32)
    same(ch, mp._outlier_indices, "outlier channels")
    idx, nrm = mp.compress(x[1024:])
    i2, n2 = orc.compress_mixed(x[1024:], mp.Pi, mp._outlier_mask, mp.outlier_codebook.boundaries,
                                mp.regular_codebook.boundaries)
    same(i2, idx, "mixed codes"), same(n2, nrm, "mixed norms")
    rec = mp.decompress(idx, nrm)
    same(orc.decompress_mixed(idx, nrm, mp.Pi, mp._outlier_mask, mp.outlier_codebook.centroids,
                              mp.regular_codebook.centroids), rec, "mixed decompress")
    # two-stage variant: codes at (bits - 1) per channel group plus one residual sign bit on every channel
    mip = ref.MixedPrecisionIPQuantizer(d, 3, 2, 32, seed=42)
    u_codes, u_signs, u_norms = mip.compress(x[:64])              # uncalibrated: regular codebook everywhere
    mq = mip.mse_quantizer
    o_codes, o_signs, o_norms = orc.compress_mixed_ip(x[:64], mq.Pi, None, mq.outlier_codebook.boundaries,
                                                      mq.outlier_codebook.centroids, mq.regular_codebook.boundaries,
                                                      mq.regular_codebook.centroids, mip.S)
    same(o_codes, u_codes, "mixed ip uncalibrated codes"), same(o_signs, u_signs, "mixed ip uncalibrated signs")
    mip.calibrate(x[:1024])
    ip_codes, ip_signs, ip_norms = mip.compress(x[1024:])
    o_codes, o_signs, o_norms = orc.compress_mixed_ip(x[1024:], mq.Pi, mq._outlier_mask,
                                                      mq.outlier_codebook.boundaries, mq.outlier_codebook.centroids,
                                                      mq.regular_codebook.boundaries, mq.regular_codebook.centroids,
                                                      mip.S)
    same(o_codes, ip_codes, "mixed ip codes"), same(o_signs, ip_signs, "mixed ip signs")
    same(o_norms, ip_norms, "mixed ip norms")
    np.savez_compressed(os.path.join(HERE, "mixed.npz"), x=npy(x), channels=npy(ch), codes=npy(idx),
                        norms=npy(nrm), rec=npy(rec), codes_uncal=npy(i_un),
                        ip_channels=npy(mq._outlier_indices), ip_codes=npy(ip_codes), ip_signs=npy(ip_signs),
                        ip_norms=npy(ip_norms), ip_codes_uncal=npy(u_codes), ip_signs_uncal=npy(u_signs))

    # ---- index search ------------------------------------------------------------------
    ix = {}
    for tag, (d, n, m, k, bits) in {"a": (64, 1000, 10, 10, 3), "b": (128, 3000, 7, 10, 3),
                                     "c": (128, 500, 5, 600, 4), "d": (64, 257, 3, 1, 2)}.items():
        torch.set_num_threads(1)   # the (M,N) products here are small: keep them reproducible
        g = torch.Generator().manual_seed(900 + d + n)
        db = torch.randn(n, d, generator=g)
        db = db / db.norm(dim=1, keepdim=True) * (torch.rand(n, 1, generator=g) * 1.5 + 0.5)
        qs = torch.randn(m, d, generator=g)
        index = ref.QuashIndex(d, bits, seed=42, pack_storage=True)
        index.add(db[: n // 2])
        index.add(db[n // 2:])
        sc, ids = index.search(qs, k)
        qq = index.quantizer
        mse, sg = index._get_unpacked()
        s2, i2 = orc.index_search(qs, mse, sg, index._norms, qq.mse_quantizer.Pi,
                                  qq.mse_quantizer.codebook.centroids, qq.S, qq.qjl_scale, k)
        same(s2, sc, f"index scores {tag}"), same(i2, ids, f"index ids {tag}")
        full = orc.index_scores(qs, mse, sg, index._norms, qq.mse_quantizer.Pi,
                                qq.mse_quantizer.codebook.centroids, qq.S, qq.qjl_scale)
        ix[f"{tag}_meta"] = np.array([d, n, m, k, bits])
        ix[f"{tag}_db"], ix[f"{tag}_q"] = npy(db), npy(qs)
        ix[f"{tag}_mse_plane"], ix[f"{tag}_qjl_plane"] = npy(index._mse_indices), npy(index._qjl_signs)
        ix[f"{tag}_norms"], ix[f"{tag}_scores"], ix[f"{tag}_ids"] = npy(index._norms), npy(sc), npy(ids)
        ix[f"{tag}_all_scores"] = npy(full)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    np.savez_compressed(os.path.join(HERE, "index.npz"), **ix)

    # ---- HF-style cache: keys come back without the sign term -----------------------
    g = torch.Generator().manual_seed(11)
    cache = QuashKVCache(num_layers=2, head_dim=64)
    k1, v1 = torch.randn(2, 4, 9, 64, generator=g), torch.randn(2, 4, 9, 64, generator=g)
    k2, v2 = torch.randn(2, 4, 1, 64, generator=g), torch.randn(2, 4, 1, 64, generator=g)
    cache.update(k1, v1, 1)
    fk, fv = cache.update(k2, v2, 1)
    e = cache.engines[1]
    Pi = e.key_quantizer.mse_quantizer.Pi
    Kc, Vc = torch.cat([k1, k2], 2), torch.cat([v1, v2], 2)
    mse, sg, kn = orc.compress_ip(Kc, Pi, e.key_quantizer.mse_quantizer.codebook.boundaries,
                                  e.key_quantizer.mse_quantizer.codebook.centroids, e.key_quantizer.S)
    # per-block matmuls in the reference vs one matmul here: equal to rounding
    assert torch.allclose(orc.decompress_mse(mse, kn, Pi, e.key_quantizer.mse_quantizer.codebook.centroids),
                          fk, atol=1e-6)
    np.savez_compressed(os.path.join(HERE, "hf_cache.npz"), k1=npy(k1), v1=npy(v1), k2=npy(k2), v2=npy(v2),
                        full_k=npy(fk), full_v=npy(fv), seed=np.array(e.seed))

    total = sum(os.path.getsize(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith(".npz"))
    print(f"golden vectors written: {total / 1e6:.2f} MB")


if __name__ == "__main__":
    main()
