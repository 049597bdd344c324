"""Host-side checks that need no GPU: constants equal the reference's, the C-ABI library
loads and exports every declared symbol, argument errors carry the reference's texts, and
the hot methods refuse CPU tensors instead of falling back."""

import ctypes
import os
import re

import numpy as np
import pytest
import torch

import quashkv_b200 as qk
from quashkv_b200 import _lib, ops
from quashkv_b200.integrations.hf_cache import QuashKVCache
from quashkv_b200.packing import packed_size

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_codebook_matches_reference_values(golden):
    g = golden("constants")
    for d in (64, 96, 128):
        for bits in (1, 2, 3, 4):
            cb = qk.LloydMaxCodebook(d, bits)
            assert np.array_equal(cb.centroids.numpy(), g[f"cent_d{d}_b{bits}"])
            assert np.array_equal(cb.boundaries.numpy(), g[f"bnd_d{d}_b{bits}"])
    cb = qk.LloydMaxCodebook(64, 2, use_exact_pdf=True)
    assert np.array_equal(cb.centroids.numpy(), g["cent_exact_d64_b2"])
    with pytest.raises(ValueError, match="bits must be in"):
        qk.LloydMaxCodebook(64, 5)


def test_codebook_helpers_agree():
    cb = qk.LloydMaxCodebook(64, 3)
    x = torch.randn(1000) * 0.2
    assert torch.equal(cb.quantize(x), cb.quantize_boundary(x))
    assert torch.equal(cb.dequantize(cb.quantize(x)), cb.centroids[cb.quantize(x).long()])
    assert cb.n_levels == 8 and torch.all(cb.centroids[1:] > cb.centroids[:-1])


def test_sign_vector_and_rotation_match_reference(golden):
    g = golden("constants")
    for d, seed in ((128, 0), (128, 42), (64, 42), (96, 42), (64, 43)):
        q = qk.InnerProductQuantizer(d, 3, seed=seed)
        assert np.array_equal(q.S.numpy(), g[f"S_d{d}_s{seed}"])
        # QR goes through LAPACK: identical on the host that made the vectors, and orthogonal anywhere
        assert np.allclose(q.mse_quantizer.Pi.numpy(), g[f"Pi_d{d}_s{seed}"], atol=1e-5)
        eye = q.mse_quantizer.Pi @ q.mse_quantizer.Pi.T
        assert torch.allclose(eye, torch.eye(d), atol=1e-5)
        assert q.qjl_scale == pytest.approx((np.pi / 2) ** 0.5 / d)


def test_constructor_errors_have_reference_texts():
    with pytest.raises(ValueError, match="at least 2 total bits"):
        qk.InnerProductQuantizer(64, total_bits=1)
    with pytest.raises(ValueError, match="n_outliers must be in"):
        qk.MixedPrecisionMSEQuantizer(64, n_outliers=65)
    with pytest.raises(ValueError, match="outlier_bits should be >= regular_bits"):
        qk.MixedPrecisionMSEQuantizer(64, outlier_bits=2, regular_bits=3)
    with pytest.raises(ValueError, match="No compressed KV blocks in cache"):
        qk.QuashKVEngine(64).attention(torch.randn(1, 1, 1, 64))
    with pytest.raises(ValueError, match="Index is empty"):
        qk.QuashIndex(64).search(torch.randn(2, 64))
    with pytest.raises(ValueError, match=r"Expected \(N, 64\) tensor"):
        qk.QuashIndex(64).add(torch.randn(3, 32))
    with pytest.raises(ValueError, match="Unsupported bits"):
        qk.pack_bits(torch.zeros(2, 8, dtype=torch.uint8), 5)


def test_bookkeeping_without_gpu():
    e = qk.QuashKVEngine(128, 3, 3)
    assert e.total_tokens == 0 and e.num_blocks == 0 and e.compression_ratio() == 1.0
    assert e.actual_memory_bytes() == 0 and "cached_tokens=0" in repr(e)
    e._block_lens.append(1)   # ratio formula only needs a non-empty cache
    assert e.compression_ratio() == pytest.approx(2 * 128 * 16 / (3 * 128 + 32 + 3 * 128 + 32))
    idx = qk.QuashIndex(64, 3, pack_storage=True)
    assert len(idx) == 0 and idx.memory_bytes() == 0 and idx.compression_ratio() == 1.0
    cache = QuashKVCache(num_layers=4, head_dim=64)
    assert [e.seed for e in cache.engines] == [42, 43, 44, 45] and len(cache) == 4
    assert cache.get_seq_length() == 0 and cache.get_max_cache_length() is None
    k, v = cache[0]
    assert k.numel() == 0 and v.numel() == 0
    assert cache.compression_stats()["tokens_per_layer"] == [0, 0, 0, 0]
    m = qk.MixedPrecisionMSEQuantizer(128, 3, 2, 32)
    assert m.effective_bits == pytest.approx(2.25) and not m.calibrated
    m.set_outlier_channels(torch.tensor([5, 1, 9]))
    assert m.calibrated and m._outlier_indices.tolist() == [1, 5, 9]
    assert packed_size(128, 3) == 48 and packed_size(128, 1) == 16 and packed_size(64, 2) == 16
    assert ops.packed_row_bytes(65, 3) == 27 and ops.packed_row_bytes(100, 3) == 39
    assert ops.packed_row_bytes(63, 2) == 16 and ops.packed_row_bytes(129, 4) == 65


def test_hot_methods_refuse_cpu_tensors():
    q = qk.MSEQuantizer(64, 3)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        q.compress(torch.randn(4, 64))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        qk.pack_bits(torch.zeros(2, 8, dtype=torch.uint8), 3)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        qk.QuashKVEngine(64).append(torch.randn(1, 1, 2, 64), torch.randn(1, 1, 2, 64))
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        qk.QuashIndex(64).add(torch.randn(3, 64))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "quashkv_b200.h")).read()
    declared = set(re.findall(r"\b(qkv_[a-z_0-9]+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    L = _lib.lib()
    for name in declared:
        assert getattr(L, name) is not None
    assert L.qkv_abi_version() == 1
    assert L.qkv_strerror(0) == b"ok" and b"NULL" in L.qkv_strerror(-1)


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host before anything is launched."""
    L = _lib.lib()
    rows = _lib.Rows(1, 0, 0)
    one = ctypes.c_void_p(16)
    assert L.qkv_compress_mse(None, 0, 64, 1, 64, one, one, 3, one, 0, one, rows, None) == -1
    assert L.qkv_compress_mse(one, 0, 64, 1, 129, one, one, 3, one, 0, one, rows, None) == -2
    assert L.qkv_compress_mse(one, 0, 64, 1, 64, one, one, 5, one, 0, one, rows, None) == -3
    assert L.qkv_compress_mse(one, 7, 64, 1, 64, one, one, 3, one, 0, one, rows, None) == -4
    assert L.qkv_pack(one, one, 4, 64, 9, None) == -3
    assert L.qkv_topk_merge(one, one, 0, 4, 2, one, one, None) == -2
    assert L.qkv_attention_workspace_bytes(32, 32, 8, 1, 32768, 128) > 0
    assert L.qkv_index_workspace_bytes(1000, 4, 64, 10) > 0
    assert L.qkv_mixed_row_bytes(128, 32, 3, 2) == 36


def test_page_pool_bookkeeping_without_gpu():
    """Page allocation, block tables and the reference-shaped page manager need no GPU; the data path
    refuses CPU tensors."""
    from quashkv_b200.integrations.vllm_backend import (QuashKVModelManager, QuashKVPageConfig, QuashKVPagedCache,
                                                        QuashKVPageManager, register_quashkv_backend)
    cfg = QuashKVPageConfig()
    assert (cfg.key_bits, cfg.value_bits, cfg.block_size, cfg.seed) == (3, 3, 16, 42)   # reference defaults
    pool = QuashKVPagedCache(5, 2, 64, cfg, device="cpu")
    assert pool.planes["k_codes"].shape == (5, 2, 16, 16) and pool.planes["v_norms"].shape == (5, 2, 16)
    pool._grow("a", 17)
    pool._lens["a"] = 17
    pool._grow("b", 1)
    pool._lens["b"] = 1
    pool._grow("a", 15)                      # 32 tokens still fit two pages
    pool._lens["a"] = 32
    assert pool.blocks_of("a") == [0, 1] and pool.blocks_of("b") == [2] and pool.free_blocks == 2
    table, lens, longest = pool.block_table(["b", "a", "unknown"])
    assert table.dtype == torch.int32 and table.tolist() == [[2, 0], [0, 1], [0, 0]]
    assert lens.tolist() == [1, 32, 0] and longest == 32
    with pytest.raises(RuntimeError, match="pool exhausted"):
        pool._grow("b", 16 * 3)
    pool.free("a")
    assert pool.free_blocks == 4 and pool.seq_len("a") == 0
    pool._grow("c", 1)
    assert pool.blocks_of("c") == [0]        # freed pages are handed out again, lowest first
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        pool.append(["d"], torch.randn(1, 2, 3, 64), torch.randn(1, 2, 3, 64))

    mgr = QuashKVPageManager(2, 64, cfg, torch.device("cpu"), layer_idx=3)
    with pytest.raises(ValueError, match="No compressed KV blocks stored yet"):
        mgr.attention(torch.randn(1, 2, 1, 64))
    model = QuashKVModelManager(3, 2, 64, device="cpu")
    assert model.stats()["tokens_per_layer"] == [0, 0, 0] and model.stats()["config"]["block_size"] == 16
    with pytest.raises((ImportError, NotImplementedError)):
        register_quashkv_backend()


def test_index_file_checks_without_gpu(tmp_path):
    """An empty index round-trips on CPU; foreign or inconsistent files are refused."""
    qk.QuashIndex(64, 4, seed=7).save(tmp_path / "empty.pt")
    back = qk.QuashIndex.load(tmp_path / "empty.pt", device="cpu")
    assert (back.dim, back.bits, back.seed, len(back)) == (64, 4, 7, 0)
    torch.save({"something": 1}, tmp_path / "foreign.pt")
    with pytest.raises(ValueError, match="not a QuashIndex file"):
        qk.QuashIndex.load(tmp_path / "foreign.pt", device="cpu")
    torch.save({"format": 1, "dim": 64, "bits": 3, "seed": 1, "pack_storage": True, "n_vectors": 4,
                "codes": torch.zeros(4, 3, dtype=torch.uint8), "signs": torch.zeros(4, 8, dtype=torch.uint8),
                "norms": torch.zeros(4)}, tmp_path / "bad.pt")
    with pytest.raises(ValueError, match="plane shapes do not match"):
        qk.QuashIndex.load(tmp_path / "bad.pt", device="cpu")


def test_tile_record_format_decodes_to_the_expected_fragments(tmp_path):
    """The record layout, the tiling arithmetic and the register-level decode share one header; a small host
    program walks all 32 lanes of a random record and checks every fragment element (no GPU)."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host C++ compiler")
    here = os.path.dirname(os.path.abspath(__file__))
    exe = tmp_path / "tile_format_check"
    subprocess.run([gxx, "-O1", "-std=c++17", "-o", str(exe), os.path.join(here, "tile_format_check.cpp")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "tile emulation OK" in out.stdout, out.stdout + out.stderr


def test_tile_entry_points_refuse_bad_arguments_without_launching():
    L = _lib.lib()
    one, rec = ctypes.c_void_p(16), ctypes.c_void_p(256)
    rows = _lib.Rows(1, 0, 0)
    assert L.qkv_tile_rows(one, one, one, one, one, 0, rec, rows, None, None) == 0        # nothing to do
    assert L.qkv_tile_rows(None, one, one, one, one, 4, rec, rows, None, None) == -1
    assert L.qkv_tile_rows(one, one, one, one, one, 4, ctypes.c_void_p(24), rows, None, None) == -5   # records unaligned
    assert L.qkv_untile_rows(rec, _lib.Rows(0, 0, 0), None, 4, one, one, one, one, one, None) == -8
    cache = _lib.TiledCache(256, 64, None, None, 0, 0)
    args = (one, 0, cache, 1, 4, 1, 1, 64)
    tail = (one, one, one, one, 0.1, 0.1, 0, one, rec, 1 << 20, None)
    assert L.qkv_attention_tiled(*args, 64, 3, 3, *tail) == -3          # records exist for head_dim 128 at 3/3 bits only
    assert L.qkv_attention_tiled(*args, 128, 4, 3, *tail) == -3
    odd = _lib.TiledCache(256, 72, None, None, 0, 0)
    assert L.qkv_attention_tiled(one, 0, odd, 1, 4, 1, 1, 64, 128, 3, 3, *tail) == -8   # capacity not whole tiles
    assert L.qkv_attention_tiled(one, 0, _lib.TiledCache(None, 64, None, None, 0, 0), 1, 4, 1, 1, 64, 128, 3, 3, *tail) == -1


def test_engine_storage_choice_and_reset_shapes_without_gpu(monkeypatch):
    """Tile records are chosen for head_dim 128 at 3/3 bits, row-major planes otherwise or on request; clear()
    keeps nothing that pins the next sequence to the old (batch, heads)."""
    assert qk.QuashKVEngine(128, 3, 3)._tiled and not qk.QuashKVEngine(64, 3, 3)._tiled
    assert not qk.QuashKVEngine(128, 4, 3)._tiled and not qk.QuashKVEngine(128, 3, 2)._tiled
    monkeypatch.setenv("QUASHKV_B200_ROW_STORAGE", "1")
    assert not qk.QuashKVEngine(128, 3, 3)._tiled
    monkeypatch.delenv("QUASHKV_B200_ROW_STORAGE")
    # what the records presume of the tables: symmetric values, keys affine in the two bits of their code
    from quashkv_b200 import ops
    ref = qk.QuashKVEngine(128, 3, 3)
    kc, vc = ref.key_quantizer.mse_quantizer.codebook.centroids, ref.value_quantizer.codebook.centroids
    assert ops.tiled_tables_ok(kc, vc)
    bent = kc.clone(); bent[3] *= 1.01
    skew = vc.clone(); skew[0] *= 1.01
    assert not ops.tiled_tables_ok(bent, vc) and not ops.tiled_tables_ok(kc, skew)
    assert not ops.tiled_tables_ok(kc[:2], vc)
    eng = qk.QuashKVEngine(128, 3, 3)
    eng.reserve(2, 3, 100, "cpu")
    assert eng._planes["records"].shape == (6, 8, 1664) and eng._capacity == 128
    eng.reserve(2, 3, 300, "cpu")
    assert eng._planes["records"].shape == (6, 20, 1664)


def test_no_host_pointer_reaches_the_library():
    """The pointer helper refuses anything that is not device memory, and data tensors of one call have to share
    a device: a constant built on the CPU (a quantizer made with the default device) must never be handed to a
    kernel as if it were a device address."""
    from quashkv_b200 import ops
    with pytest.raises(ValueError, match="CUDA tensor"):
        ops._p(torch.zeros(4))
    assert ops._p(None) is None
    with pytest.raises(ValueError, match="different devices"):
        ops._same_device(torch.device("cpu"), torch.zeros(1), None, torch.zeros(1, device="meta"))
    ops._same_device(torch.device("cpu"), torch.zeros(1), None)
    keep = ops._Keep(torch.device("meta"))
    with pytest.raises(ValueError, match="CUDA tensor"):        # converted to the call's device first, then refused
        keep.f32(torch.zeros(3))
    assert keep.held[0].device.type == "meta"


def test_device_constants_follow_replaced_and_modified_tensors():
    """The per-device copies of a quantizer's constants are tied to the source tensor object and its version:
    a replaced or modified mask / rotation is copied again, never served stale."""
    from quashkv_b200.quantizer import _DeviceConstants
    c = _DeviceConstants()
    meta = torch.device("meta")
    a = torch.zeros(4)
    first = c.get("m", a, meta)
    assert c.get("m", a, meta) is first
    a.add_(1)                                   # modified in place: version changes
    second = c.get("m", a, meta)
    assert second is not first
    b = torch.zeros(4)                          # another tensor under the same name
    assert c.get("m", b, meta) is not second
    assert len(c._copies) == 1
    q = qk.MixedPrecisionMSEQuantizer(64, 3, 2, 8)
    q.set_outlier_channels(torch.tensor([1, 5, 9]))
    assert q._n_marked == 3 and q._mask_u8.tolist().count(1) == 3 and not q._consts._copies
    assert qk.MSEQuantizer(64, 3).Pi.is_contiguous()


def test_hf_cache_plumbing_with_a_stand_in_engine():
    """The transformers Cache over the engines and the attention function that reads them, on CPU with a stand-in
    engine that stores K / V and attends exactly: a tiny Llama must give the logits it gives with a DynamicCache,
    on the fused route (update appends only, attention reads the engine) and on the decompress-everything route."""
    transformers = pytest.importorskip("transformers")
    from quashkv_b200.integrations.hf_cache import QuashKVCache, make_hf_cache

    class StandIn:
        def __init__(self):
            self.K = self.V = None

        @property
        def total_tokens(self):
            return 0 if self.K is None else self.K.shape[2]

        def append(self, k, v):
            self.K = k.float() if self.K is None else torch.cat([self.K, k.float()], 2)
            self.V = v.float() if self.V is None else torch.cat([self.V, v.float()], 2)

        def clear(self):
            self.K = self.V = None

        def decompress_all(self, with_signs=False):
            return self.K, self.V

        def attention(self, q, scale=None, causal=False):
            G = q.shape[1] // self.K.shape[1]
            K, V = self.K.repeat_interleave(G, 1), self.V.repeat_interleave(G, 1)
            s = (q.float() @ K.transpose(-1, -2)) * scale
            if causal:
                n, Q = K.shape[2], q.shape[2]
                pos = torch.arange(Q) + n - Q
                s = s.masked_fill(torch.arange(n)[None, :] > pos[:, None], float("-inf"))
            return torch.softmax(s, -1) @ V

    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                                   head_dim=16, intermediate_size=128, vocab_size=100)
    model = transformers.LlamaForCausalLM(cfg).eval()
    ids = torch.randint(0, 100, (2, 7))
    with torch.no_grad():
        ref = model(input_ids=ids, use_cache=True)
        nxt = ref.logits[:, -1].argmax(-1, keepdim=True)
        ref2 = model(input_ids=nxt, past_key_values=ref.past_key_values, use_cache=True)
        for fused in (True, False):
            qc = QuashKVCache(2, 16)
            qc.engines = [StandIn(), StandIn()]
            cache = make_hf_cache(qc, fused=fused)
            previous = cache.attach(model)
            assert model.config._attn_implementation == ("quashkv_fused" if fused else previous)
            o1 = model(input_ids=ids, past_key_values=cache, use_cache=True)
            o2 = model(input_ids=nxt, past_key_values=cache, use_cache=True)
            cache.detach(model, previous)
            assert model.config._attn_implementation == previous
            assert torch.allclose(o1.logits, ref.logits, atol=1e-5) and torch.allclose(o2.logits, ref2.logits, atol=1e-5)
            assert cache.get_seq_length() == 8


def test_every_cuda_source_is_part_of_the_build():
    """A source file that is not in the build list would silently drop its kernels from the library."""
    import os
    from quashkv_b200 import _build
    on_disk = sorted(f for f in os.listdir(_build.CSRC) if f.endswith(".cu"))
    assert sorted(_build.SOURCES) == on_disk
