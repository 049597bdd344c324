"""The CPU oracle against the vectors generated from the reference implementation
(tests/golden/make_golden.py).  Runs without a GPU."""

import numpy as np
import torch

from oracle import quashkv_oracle as orc
from helpers import t


def exact(a, b):
    """Integer / layout results: bit for bit."""
    a = a.numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    assert a.shape == b.shape and np.array_equal(a, b)


def same(a, b):
    """Results downstream of a float matmul.  The golden vectors were produced by the
    reference's BLAS on one host; another host's BLAS may round differently, so codes may
    differ at decision-boundary ties (rate far below 1e-4) and floats in the last digits."""
    a = a.numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    assert a.shape == b.shape and a.dtype == b.dtype
    if a.dtype == np.uint8 or a.dtype == np.int64:
        assert (a != b).sum() <= max(8, 1e-4 * a.size)
    else:
        assert (~np.isclose(a, b, rtol=2e-5, atol=2e-5)).sum() <= max(8, 1e-4 * a.size)


def test_codebooks_rotation_signs(golden):
    g = golden("constants")
    for d in (64, 96, 128):
        for bits in (1, 2, 3, 4):
            c, b = orc.lloyd_max_tables(d, bits)
            exact(c, g[f"cent_d{d}_b{bits}"])
            exact(b, g[f"bnd_d{d}_b{bits}"])
    c, b = orc.lloyd_max_tables(64, 2, exact_pdf=True)
    same(c, g["cent_exact_d64_b2"])
    for d, seed in ((128, 0), (128, 42), (64, 42), (96, 42), (64, 43)):
        same(orc.rotation_matrix(d, seed), g[f"Pi_d{d}_s{seed}"])
        exact(orc.sign_vector(d, seed), g[f"S_d{d}_s{seed}"])


def test_packing_known_answers(golden):
    g = golden("packing")
    assert g["ka_pack3_0to7"].tolist() == [[0x88, 0xC6, 0xFA]]
    assert g["ka_pack2_0123"].tolist() == [[0xE4]]
    assert g["ka_pack4_12"].tolist() == [[0x21]]
    assert g["ka_pack1_10000001"].tolist() == [[0x81]]
    exact(orc.pack_bits(np.arange(8, dtype=np.uint8)[None], 3), g["ka_pack3_0to7"])
    for bits in (1, 2, 3, 4):
        for d in (128, 64, 63, 65, 100, 127, 129, 8, 1):
            codes, packed = g[f"codes_b{bits}_d{d}"], g[f"packed_b{bits}_d{d}"]
            exact(orc.pack_bits(codes, bits), packed)
            exact(orc.unpack_bits(packed, bits, d), codes)


def _c1_constants(golden):
    g = golden("constants")
    return (t(g["Pi_d128_s0"]), t(g["S_d128_s0"]), t(g["cent_d128_b2"]), t(g["bnd_d128_b2"]),
            t(g["cent_d128_b3"]), t(g["bnd_d128_b3"]))


def test_config1(golden):
    g = golden("config1")
    Pi, S, kc, kb, vc, vb = _c1_constants(golden)
    K, V, Q = t(g["K"]), t(g["V"]), t(g["Q"])
    mse, sg, kn = orc.compress_ip(K, Pi, kb, kc, S)
    vi, vn = orc.compress_mse(V, Pi, vb)
    same(orc.pack_bits(mse, 2), g["mse_plane"])
    same(orc.pack_bits(sg, 1), g["qjl_plane"])
    same(orc.pack_bits(vi, 3), g["val_plane"])
    same(kn, g["key_norms"])
    same(vn, g["val_norms"])
    qs = orc.QJL_COEFF / 128
    same(orc.attention(Q, mse, sg, kn, vi, vn, Pi, kc, vc, S, qs), g["out"])
    same(orc.attention_gqa(t(g["Qg"]), mse, sg, kn, vi, vn, Pi, kc, vc, S, qs, n_kv_heads=8), g["out_gqa"])
    same(orc.decompress_mse(vi, vn, Pi, vc)[0, 0, :64], g["vrec_head0"])
    same(orc.decompress_ip(mse, sg, kn, Pi, kc, S, qs)[0, 0, :64], g["krec_ip_head0"])


def test_engine_cases(golden):
    g, c = golden("engine_cases"), golden("constants")
    for i in range(int(g["n_cases"])):
        D, kbits, vbits, seed, qlen, causal, total = (int(v) for v in g[f"e{i}_meta"])
        Pi, S = t(g[f"e{i}_Pi"]), orc.sign_vector(D, seed)
        kc, kb = t(c[f"cent_d{D}_b{kbits - 1}"]), t(c[f"bnd_d{D}_b{kbits - 1}"])
        vc, vb = t(c[f"cent_d{D}_b{vbits}"]), t(c[f"bnd_d{D}_b{vbits}"])
        mse, sg, kn = orc.compress_ip(t(g[f"e{i}_K"]), Pi, kb, kc, S)
        vi, vn = orc.compress_mse(t(g[f"e{i}_V"]), Pi, vb)
        same(mse, g[f"e{i}_mse"]), same(sg, g[f"e{i}_qjl"]), same(vi, g[f"e{i}_val"])
        same(kn, g[f"e{i}_kn"]), same(vn, g[f"e{i}_vn"])
        out = orc.attention(t(g[f"e{i}_Q"]), mse, sg, kn, vi, vn, Pi, kc, vc, S, orc.QJL_COEFF / D,
                            causal=bool(causal), total_tokens=total)
        same(out, g[f"e{i}_out"])


def test_quantizers_and_edge_vectors(golden):
    g, c = golden("quantizers"), golden("constants")
    for d in (64, 128):
        x = t(g[f"x_d{d}"])
        Pi, S = t(c[f"Pi_d{d}_s42"]), t(c[f"S_d{d}_s42"])
        for bits in (1, 2, 3, 4):
            idx, nrm = orc.compress_mse(x, Pi, t(c[f"bnd_d{d}_b{bits}"]))
            same(idx, g[f"mse_idx_d{d}_b{bits}"]), same(nrm, g[f"mse_norm_d{d}_b{bits}"])
            same(orc.decompress_mse(idx, nrm, Pi, t(c[f"cent_d{d}_b{bits}"])), g[f"mse_rec_d{d}_b{bits}"])
        for bits in (2, 3, 4):
            cent, bnd = t(c[f"cent_d{d}_b{bits - 1}"]), t(c[f"bnd_d{d}_b{bits - 1}"])
            a, b, n = orc.compress_ip(x, Pi, bnd, cent, S)
            same(a, g[f"ip_mse_d{d}_b{bits}"]), same(b, g[f"ip_qjl_d{d}_b{bits}"]), same(n, g[f"ip_norm_d{d}_b{bits}"])
            same(orc.decompress_ip(a, b, n, Pi, cent, S, orc.QJL_COEFF / d), g[f"ip_rec_d{d}_b{bits}"])


def test_mixed_precision(golden):
    g, c = golden("mixed"), golden("constants")
    x, Pi = t(g["x"]), t(c["Pi_d128_s42"])
    ch = orc.outlier_channels(x[:1024], Pi, 32)
    same(ch, g["channels"])
    mask = torch.zeros(128, dtype=torch.bool)
    mask[ch] = True
    codes, norms = orc.compress_mixed(x[1024:], Pi, mask, t(c["bnd_d128_b3"]), t(c["bnd_d128_b2"]))
    same(codes, g["codes"]), same(norms, g["norms"])
    same(orc.decompress_mixed(codes, norms, Pi, mask, t(c["cent_d128_b3"]), t(c["cent_d128_b2"])), g["rec"])
    same(orc.compress_mixed(x[:64], Pi, None, t(c["bnd_d128_b3"]), t(c["bnd_d128_b2"]))[0], g["codes_uncal"])


def test_index_search_and_merge(golden):
    g, c = golden("index"), golden("constants")
    for tag in "abcd":
        d, n, m, k, bits = (int(v) for v in g[f"{tag}_meta"])
        Pi, S = t(c[f"Pi_d{d}_s42"]), t(c[f"S_d{d}_s42"])
        cent, bnd = t(c[f"cent_d{d}_b{bits - 1}"]), t(c[f"bnd_d{d}_b{bits - 1}"])
        mse, sg, nrm = orc.compress_ip(t(g[f"{tag}_db"]), Pi, bnd, cent, S)
        same(orc.pack_bits(mse, bits - 1), g[f"{tag}_mse_plane"])
        same(orc.pack_bits(sg, 1), g[f"{tag}_qjl_plane"])
        sc, ids = orc.index_search(t(g[f"{tag}_q"]), mse, sg, nrm, Pi, cent, S, orc.QJL_COEFF / d, k)
        same(orc.index_scores(t(g[f"{tag}_q"]), mse, sg, nrm, Pi, cent, S, orc.QJL_COEFF / d),
             g[f"{tag}_all_scores"])
        assert sc.shape == g[f"{tag}_scores"].shape
        # equal up to swaps between near-equal scores (BLAS rounding differs across hosts)
        for row, want in zip(ids.tolist(), g[f"{tag}_ids"].tolist()):
            assert len(set(row) ^ set(want)) <= 2
        # sharded search = per-shard top-k + merge
        kk = min(k, n // 2)
        if kk == min(k, n):
            half = n // 2
            parts = [orc.index_search(t(g[f"{tag}_q"]), mse[a:b], sg[a:b], nrm[a:b], Pi, cent, S,
                                      orc.QJL_COEFF / d, kk) for a, b in ((0, half), (half, n))]
            cs = torch.cat([p[0] for p in parts], 1)
            ci = torch.cat([parts[0][1], parts[1][1] + half], 1)
            ms, mi = orc.merge_topk(cs, ci, kk)
            assert (mi != ids).float().mean() < 1e-2


def test_hf_cache_keys_drop_sign_term(golden):
    g, c = golden("hf_cache"), golden("constants")
    seed = int(g["seed"])
    Pi, S = t(c[f"Pi_d64_s{seed}"]), orc.sign_vector(64, seed)
    K = torch.cat([t(g["k1"]), t(g["k2"])], 2)
    V = torch.cat([t(g["v1"]), t(g["v2"])], 2)
    mse, _, kn = orc.compress_ip(K, Pi, t(c["bnd_d64_b2"]), t(c["cent_d64_b2"]), S)
    vi, vn = orc.compress_mse(V, Pi, t(c["bnd_d64_b3"]))
    assert torch.allclose(orc.decompress_mse(mse, kn, Pi, t(c["cent_d64_b2"])), t(g["full_k"]), atol=1e-6)
    assert torch.allclose(orc.decompress_mse(vi, vn, Pi, t(c["cent_d64_b3"])), t(g["full_v"]), atol=1e-6)
