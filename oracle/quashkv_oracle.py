"""CPU oracle for the compressed-KV hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic of the reference project's
PyTorch path (QuashKV, TurboQuant-style quantisation).  It exists so the CUDA
kernels can be checked against it; it is never part of the product path and
only tests, the smoke check and the benchmark's CPU-baseline leg may import it.

Arithmetic library: the reference computes with ``torch`` on the CPU (matmul,
norm, compare, softmax, topk) and ``scipy.integrate.quad`` for the codebook.
The float parts of this restatement therefore use the same ``torch`` CPU
calls in the same order, so that results agree bit-for-bit with the reference
where both run on the same host; the byte/bit packing is plain numpy integer
arithmetic written from the layout rule (an LSB-first stream of w-bit fields).

Parity pin: every function here is checked against outputs of the reference
itself (imported read-only in the build container) by
``tests/golden/make_golden.py``; the resulting vectors are committed under
``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Each function cites the reference file:line (paths inside the reference
project) whose behaviour it follows.
"""

from __future__ import annotations

import math

import numpy as np
import torch

QJL_COEFF = math.sqrt(math.pi / 2.0)  # quashkv/constants.py:21


# ---------------------------------------------------------------------------
# constants generated on the host: rotation, sign vector, codebook
# ---------------------------------------------------------------------------

def rotation_matrix(d: int, seed: int) -> torch.Tensor:
    """Random orthogonal matrix: Q of QR(randn(d,d)), columns flipped by sign(diag R).

    Follows quashkv/quantizer.py:32-44.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    gauss = torch.randn(d, d, generator=g, dtype=torch.float32)
    q, r = torch.linalg.qr(gauss)
    return q * torch.sign(torch.diag(r)).unsqueeze(0)


def sign_vector(d: int, seed: int) -> torch.Tensor:
    """Length-d vector of +-1 drawn from seed + 1_000_000 (quashkv/quantizer.py:51-59)."""
    g = torch.Generator(device="cpu").manual_seed(seed + 1_000_000)
    bits = torch.randint(0, 2, (d,), generator=g, dtype=torch.float32, device="cpu")
    return bits * 2.0 - 1.0


def lloyd_max_tables(d: int, bits: int, *, exact_pdf: bool = False,
                     max_iter: int = 300, tol: float = 1e-12):
    """Lloyd-Max centroids and decision boundaries for one rotated coordinate.

    Follows quashkv/codebook.py:63-139 (solver) and :198-207 (fp32 tensors):
    density N(0, 1/d) (or the exact Beta-type density of a unit-vector
    coordinate), 2^bits centroids started uniformly in +-4 sigma, alternating
    midpoint boundaries and conditional means by ``scipy.integrate.quad``
    until the largest centroid shift is below ``tol``.
    """
    from scipy import integrate, special

    if bits not in (1, 2, 3, 4):
        raise ValueError(f"bits must be in {{1, 2, 3, 4}}, got {bits}")
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(d)
    if exact_pdf:
        log_c = (special.gammaln(d / 2.0) - 0.5 * math.log(math.pi)
                 - special.gammaln((d - 1) / 2.0))
        expo = (d - 3) / 2.0

        def pdf(t):
            if abs(t) >= 1.0:
                return 0.0
            if expo == 0:
                return math.exp(log_c)
            return math.exp(log_c + expo * math.log(1.0 - t * t))
        lo, hi = -1.0, 1.0
    else:
        def pdf(t):
            return (1.0 / (math.sqrt(2 * math.pi) * sigma)) * math.exp(-t * t / (2 * sigma * sigma))
        lo, hi = -4.0 * sigma, 4.0 * sigma

    cents = [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)]
    for _ in range(max_iter):
        mids = [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)]
        edges = [lo * 5] + mids + [hi * 5]
        nxt = []
        for i in range(levels):
            a, b = edges[i], edges[i + 1]
            num, _e = integrate.quad(lambda t: t * pdf(t), a, b, limit=100)
            den, _e = integrate.quad(pdf, a, b, limit=100)
            nxt.append(num / den if den > 1e-15 else cents[i])
        shift = max(abs(nxt[i] - cents[i]) for i in range(levels))
        cents = nxt
        if shift < tol:
            break
    mids = [(cents[i] + cents[i + 1]) / 2.0 for i in range(levels - 1)]
    return (torch.tensor(cents, dtype=torch.float32),
            torch.tensor(mids, dtype=torch.float32))


# ---------------------------------------------------------------------------
# scalar quantisation of rotated coordinates
# ---------------------------------------------------------------------------

def codes_from_boundaries(x_rot: torch.Tensor, boundaries: torch.Tensor) -> torch.Tensor:
    """code = number of boundaries strictly below the value (quashkv/codebook.py:239-259)."""
    count = torch.zeros_like(x_rot, dtype=torch.int32)
    for b in boundaries:
        count += (x_rot > b).to(torch.int32)
    return count.to(torch.uint8)


def _unit_rotated(x: torch.Tensor, Pi: torch.Tensor):
    norms = x.norm(dim=-1, keepdim=True).clamp(min=1e-8)
    return (x / norms) @ Pi.T, norms.squeeze(-1)


def compress_mse(x, Pi, boundaries):
    """normalise -> rotate -> bucketise (quashkv/quantizer.py:113-131,
    quashkv/triton_kernels/compress.py:34-58).  Returns (codes uint8, norms fp32)."""
    x_rot, norms = _unit_rotated(x.float(), Pi)
    return codes_from_boundaries(x_rot, boundaries), norms


def compress_ip(x, Pi, boundaries, centroids, S):
    """Two-stage key quantiser (quashkv/quantizer.py:211-242): codes at b-1 bits,
    then the sign bit of (x_rot - centroid) * S with ``>= 0`` mapping to 1."""
    x_rot, norms = _unit_rotated(x.float(), Pi)
    codes = codes_from_boundaries(x_rot, boundaries)
    resid = x_rot - centroids[codes.long()]
    signs = ((resid * S) >= 0).to(torch.uint8)
    return codes, signs, norms


def decompress_mse(codes, norms, Pi, centroids):
    """centroid gather -> un-rotate -> rescale (quashkv/quantizer.py:133-147)."""
    return (centroids[codes.long()] @ Pi) * norms.unsqueeze(-1)


def decompress_ip(codes, signs, norms, Pi, centroids, S, qjl_scale):
    """Key reconstruction including the sign term
    (quashkv/triton_kernels/decompress.py:58-96): two un-rotations, then the sum."""
    a = centroids[codes.long()] @ Pi
    b = (qjl_scale * (S * (signs.float() * 2.0 - 1.0))) @ Pi
    return (a + b) * norms.unsqueeze(-1)


# ---------------------------------------------------------------------------
# mixed precision (per-channel bit allocation)
# ---------------------------------------------------------------------------

def outlier_channels(sample: torch.Tensor, Pi: torch.Tensor, n_outliers: int) -> torch.Tensor:
    """Indices (sorted) of the n_outliers rotated channels of largest unbiased variance
    over the unit-normalised sample (quashkv/mixed_precision.py:92-115)."""
    x_rot, _ = _unit_rotated(sample.float(), Pi)
    _, top = x_rot.var(dim=0).topk(n_outliers)
    return top.sort().values


def compress_mixed(x, Pi, mask, bounds_outlier, bounds_regular):
    """Per-channel codebook choice (quashkv/mixed_precision.py:130-158).  ``mask`` is a
    bool (d,) tensor or None (regular codebook everywhere)."""
    x_rot, norms = _unit_rotated(x.float(), Pi)
    if mask is None:
        return codes_from_boundaries(x_rot, bounds_regular), norms
    codes = torch.empty_like(x_rot, dtype=torch.uint8)
    codes[..., mask] = codes_from_boundaries(x_rot[..., mask], bounds_outlier)
    codes[..., ~mask] = codes_from_boundaries(x_rot[..., ~mask], bounds_regular)
    return codes, norms


def compress_mixed_ip(x, Pi, mask, bounds_outlier, cents_outlier, bounds_regular, cents_regular, S):
    """Mixed-precision codes plus the sign bit of the rotated residual on every channel
    (quashkv/mixed_precision.py:270-322): codes as compress_mixed, residual against the centroid
    of the channel's own codebook, sign = (residual * S >= 0)."""
    x_rot, norms = _unit_rotated(x.float(), Pi)
    if mask is None:
        codes = codes_from_boundaries(x_rot, bounds_regular)
        hat = cents_regular[codes.long()]
    else:
        codes = torch.empty_like(x_rot, dtype=torch.uint8)
        codes[..., mask] = codes_from_boundaries(x_rot[..., mask], bounds_outlier)
        codes[..., ~mask] = codes_from_boundaries(x_rot[..., ~mask], bounds_regular)
        hat = torch.empty(*codes.shape, dtype=torch.float32)
        hat[..., mask] = cents_outlier[codes[..., mask].long()]
        hat[..., ~mask] = cents_regular[codes[..., ~mask].long()]
    signs = (((x_rot - hat) * S) >= 0).to(torch.uint8)
    return codes, signs, norms


def decompress_mixed(codes, norms, Pi, mask, cents_outlier, cents_regular):
    """quashkv/mixed_precision.py:160-187."""
    if mask is None:
        y = cents_regular[codes.long()]
    else:
        y = torch.empty(*codes.shape, dtype=torch.float32)
        y[..., mask] = cents_outlier[codes[..., mask].long()]
        y[..., ~mask] = cents_regular[codes[..., ~mask].long()]
    return (y @ Pi) * norms.unsqueeze(-1)


# ---------------------------------------------------------------------------
# bit packing: an LSB-first stream of w-bit fields over the last axis
# ---------------------------------------------------------------------------

def packed_size(d: int, bits: int) -> int:
    """ceil(d*bits/8) (quashkv/packing.py:162-165)."""
    return (d * bits + 7) // 8


def pack_bits(codes, bits: int):
    """Field i of a row occupies stream bits [i*w, (i+1)*w), byte k holds stream bits
    [8k, 8k+8), least significant first.  This reproduces every layout of
    quashkv/packing.py:22-94 (1-bit 8/byte, 2-bit 4/byte, 3-bit 8 values -> 24-bit
    word -> 3 bytes, 4-bit low nibble first); rows are zero-padded to a whole group
    (8 fields for 1- and 3-bit, 4 for 2-bit, 2 for 4-bit).  bits == 8 passes through."""
    was_tensor = isinstance(codes, torch.Tensor)
    a = codes.numpy() if was_tensor else np.asarray(codes)
    if bits == 8:
        return codes
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bits: {bits}")
    lead, d = a.shape[:-1], a.shape[-1]
    group = {1: 8, 2: 4, 3: 8, 4: 2}[bits]
    d_pad = -(-d // group) * group
    flat = np.zeros((int(np.prod(lead, dtype=np.int64)), d_pad), dtype=np.uint8)
    flat[:, :d] = a.reshape(-1, d)
    stream = ((flat[:, :, None] >> np.arange(bits, dtype=np.uint8)) & 1).reshape(flat.shape[0], -1)
    out = np.packbits(stream, axis=1, bitorder="little").reshape(*lead, -1)
    return torch.from_numpy(out) if was_tensor else out


def unpack_bits(packed, bits: int, d: int):
    """Inverse of :func:`pack_bits` (quashkv/packing.py:97-159)."""
    was_tensor = isinstance(packed, torch.Tensor)
    a = packed.numpy() if was_tensor else np.asarray(packed)
    if bits == 8:
        return packed
    if bits not in (1, 2, 3, 4):
        raise ValueError(f"Unsupported bits: {bits}")
    lead, nb = a.shape[:-1], a.shape[-1]
    stream = np.unpackbits(a.reshape(-1, nb), axis=1, bitorder="little")
    n_fields = stream.shape[1] // bits
    fields = stream[:, :n_fields * bits].reshape(-1, n_fields, bits)
    vals = (fields << np.arange(bits, dtype=np.uint8)).sum(axis=2).astype(np.uint8)
    out = np.ascontiguousarray(vals[:, :d]).reshape(*lead, d)
    return torch.from_numpy(out) if was_tensor else out


# ---------------------------------------------------------------------------
# attention over compressed keys and values
# ---------------------------------------------------------------------------

def attention(queries, key_codes, key_signs, key_norms, val_codes, val_norms,
              Pi, key_centroids, val_centroids, S, qjl_scale,
              scale=None, causal=False, total_tokens=None):
    """Full-softmax attention over unpacked codes (quashkv/engine.py:204-299).

    queries (B,H,Q,D); codes (B,H,KV,D) uint8; norms (B,H,KV).  Scores are
    ``k_norm * (q_rot.c[code] + qjl_scale * sum(|q_rot| * (2 sign - 1) * S)) * scale``;
    with ``causal`` the query at row i sits at position total_tokens - Q + i and
    sees keys at positions <= its own.  Values are reconstructed
    (c[code] @ Pi * v_norm) and combined with softmax weights.
    """
    B, H, Q, D = queries.shape
    KV = key_codes.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if total_tokens is None:
        total_tokens = KV
    q_rot = queries.float() @ Pi.T
    # The reference forms (B,H,Q,KV,D) products and sums the last axis
    # (quashkv/engine.py:252-267); the same is done here in KV slabs, which
    # leaves every per-(q,k) sum unchanged and bounds the temporary.
    slab = max(1, (1 << 26) // max(1, B * H * Q * D))
    pieces = []
    for k0 in range(0, KV, slab):
        k_hat = key_centroids[key_codes[:, :, k0:k0 + slab].long()]
        n = k_hat.shape[2]
        q_exp = q_rot.unsqueeze(3).expand(-1, -1, -1, n, -1)
        dots = (q_exp * k_hat.unsqueeze(2).expand(-1, -1, Q, -1, -1)).sum(dim=-1)
        sgn = key_signs[:, :, k0:k0 + slab].float() * 2.0 - 1.0
        corr = qjl_scale * (q_exp.abs() * sgn.unsqueeze(2).expand(-1, -1, Q, -1, -1) * S).sum(dim=-1)
        k_n = key_norms[:, :, k0:k0 + slab].unsqueeze(2).expand(-1, -1, Q, -1)
        pieces.append(k_n * (dots + corr) * scale)
    scores = torch.cat(pieces, dim=-1)
    if causal:
        q_pos = torch.arange(Q) + total_tokens - Q
        hidden = torch.arange(KV).unsqueeze(0) > q_pos.unsqueeze(1)
        scores = scores.masked_fill(hidden[None, None], float("-inf"))
    w = torch.softmax(scores, dim=-1)
    v = (val_centroids[val_codes.long()] @ Pi) * val_norms.unsqueeze(-1)
    return torch.einsum("bhqk,bhkd->bhqd", w, v)


def attention_gqa(queries, *planes, n_kv_heads, **kw):
    """Grouped-query form: query head h reads KV head h // G.  The reference has no
    GQA; this folds each group's G heads into the query-length axis of the
    per-KV-head call above (non-causal decode), which is the HuggingFace
    ``repeat_kv`` semantics."""
    B, Hq, Q, D = queries.shape
    G = Hq // n_kv_heads
    folded = queries.reshape(B, n_kv_heads, G * Q, D)
    out = attention(folded, *planes, **kw)
    return out.reshape(B, Hq, Q, D)


# ---------------------------------------------------------------------------
# maximum inner-product search over compressed vectors
# ---------------------------------------------------------------------------

def index_scores(queries, codes, signs, norms, Pi, centroids, S, qjl_scale):
    """(M,N) estimated inner products (quashkv/nn_search/index.py:145-161)."""
    q_rot = queries.float() @ Pi.T
    dots = q_rot @ centroids[codes.long()].T
    corr = qjl_scale * ((q_rot.abs() * S) @ (signs.float() * 2.0 - 1.0).T)
    return norms.unsqueeze(0) * (dots + corr)


def index_search(queries, codes, signs, norms, Pi, centroids, S, qjl_scale, k):
    """Top-k by estimated inner product, descending (quashkv/nn_search/index.py:121-163)."""
    k = min(k, codes.shape[0])
    return torch.topk(index_scores(queries, codes, signs, norms, Pi, centroids, S, qjl_scale), k, dim=1)


def merge_topk(scores, ids, k):
    """Merge per-shard candidate lists (M, g*k) into (M, k): higher score first, then
    lower id.  The reference has no sharded search; this is the rule the merge
    kernel is held to."""
    s = scores.double().numpy()
    i = ids.numpy()
    order = np.lexsort((i, -s), axis=1)[:, :k]
    return (torch.from_numpy(np.take_along_axis(s, order, 1)).float(),
            torch.from_numpy(np.take_along_axis(i, order, 1)))
