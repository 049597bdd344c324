"""The attention entry point that needs no workspace from the caller.

Some callers cannot allocate device memory at the moment they call into the library: a
serving loop whose memory plan already owns all of HBM, a plugin run by a framework that
forbids allocation on its streams, code between the begin and end of a stream capture.
``qkv_attention_static_scratch`` keeps its scratch in an array inside the library image; this
test calls it through the C ABI twice in a row (the second call reuses the array with the first
call's contents still in it) and holds both outputs to the ordinary entry point's results.
It also checks that a shape whose scratch need exceeds the array is refused, not launched.
The file name sorts last so that a run that stops at the first failure has run everything else.
"""

import ctypes

import pytest
import torch

import quashkv_b200 as qk
from quashkv_b200 import _lib, ops
from helpers import rel_l2

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _planes(eng):
    """The cache as the five row-major packed planes the entry point reads, over the whole capacity (exact
    copies when the engine stores tile records)."""
    return eng.row_planes(0, eng._capacity)


def _workspace_entry_point(eng, p, q, causal=False):
    """The ordinary entry point (qkv_attention, workspace from the caller) on the same planes."""
    kq, vq = eng.key_quantizer, eng.value_quantizer
    Pi, _, kc, S = kq._on(q.device)
    _, _, vc = vq._on(q.device)
    return ops.attention(q, p["k_codes"], p["k_signs"], p["k_norms"], p["v_codes"], p["v_norms"], eng.total_tokens,
                         eng._shape[1], eng.key_bits, eng.value_bits, Pi, kc, vc, S, kq.qjl_scale,
                         1.0 / q.shape[-1] ** 0.5, causal)


def _call(L, eng, p, q, causal=False):
    kq, vq = eng.key_quantizer, eng.value_quantizer
    dev = q.device
    Pi, _, kc, S = kq._on(dev)
    _, _, vc = vq._on(dev)
    B, Hq, Q, D = q.shape
    cache = _lib.Cache(p["k_codes"].data_ptr(), p["k_signs"].data_ptr(), p["k_norms"].data_ptr(),
                       p["v_codes"].data_ptr(), p["v_norms"].data_ptr(), eng._capacity)
    out = torch.full((B, Hq, Q, D), float("nan"), device=dev)
    qc = q.contiguous()
    rc = L.qkv_attention_static_scratch(
        ctypes.c_void_p(qc.data_ptr()), _lib.F32, cache, B, Hq, eng._shape[1], Q, eng.total_tokens, D,
        eng.key_bits, eng.value_bits, ctypes.c_void_p(Pi.data_ptr()), ctypes.c_void_p(kc.data_ptr()),
        ctypes.c_void_p(vc.data_ptr()), ctypes.c_void_p(S.data_ptr()), kq.qjl_scale, 1.0 / D ** 0.5,
        int(causal), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


@pytest.mark.parametrize("D,bits", [(128, 3), (64, 4)])   # tensor-core path and generic path
def test_static_scratch_attention_matches_workspace_entry_point(D, bits):
    L = _lib.lib()
    g = torch.Generator().manual_seed(21)
    eng = qk.QuashKVEngine(D, bits, bits, seed=42, pack_storage=True)
    eng.append(torch.randn(2, 2, 777, D, generator=g).to(DEV), torch.randn(2, 2, 777, D, generator=g).to(DEV))
    p = _planes(eng)
    for trial in range(2):      # two calls in a row share the scratch array
        q = torch.randn(2, 8, 1, D, generator=g).to(DEV)
        want = _workspace_entry_point(eng, p, q)
        assert rel_l2(want, eng.attention(q)) < 1e-3       # ... which agrees with the engine's own route
        rc, got = _call(L, eng, p, q)
        torch.cuda.synchronize()
        assert rc == 0, _lib.lib().qkv_strerror(rc)
        assert torch.isfinite(got).all()
        assert rel_l2(got, want) < 1e-6, (trial, rel_l2(got, want))
    # a longer cache between calls changes the split layout inside the same array
    eng.append(torch.randn(2, 2, 5000, D, generator=g).to(DEV), torch.randn(2, 2, 5000, D, generator=g).to(DEV))
    q = torch.randn(2, 8, 2, D, generator=g).to(DEV)
    p = _planes(eng)
    rc, got = _call(L, eng, p, q, causal=True)
    assert rc == 0 and rel_l2(got, _workspace_entry_point(eng, p, q, causal=True)) < 1e-6


def test_static_scratch_refuses_shapes_beyond_the_array():
    L = _lib.lib()
    limit = 8 << 20
    assert L.qkv_attention_workspace_bytes(32, 32, 8, 1, 32768, 128) <= limit      # the benchmark shape fits
    assert L.qkv_attention_workspace_bytes(64, 64, 8, 64, 4096, 128) > limit
    one = ctypes.c_void_p(256)
    cache = _lib.Cache(256, 256, 256, 256, 256, 4096)
    rc = L.qkv_attention_static_scratch(one, 0, cache, 64, 64, 8, 64, 4096, 128, 3, 3, one, one, one, one, 0.1, 0.1,
                                        0, one, None)
    assert rc == -6 and b"workspace" in L.qkv_strerror(rc)
