// Index scan on the fifth-generation tensor cores (tcgen05) for dim 128, 3 bits, k <= 12.
//
// Same contract as the mma.sync scan (index_scan_mma.cu): approximate fp16 scores only propose
// candidates under a proven error bound, the survivors are re-scored exactly afterwards.  What
// changes is who does the contraction.  One CTA per SM owns 64 queries (MMA N, the B operand: fp16 in
// shared memory) and a slice of the database; per tile of 128 rows (MMA M) the worker threads decode the
// packed rows ONCE into the A operand (K = 256: 128 centroid values, then the sign bits as the shift-free
// single-bit fp16 patterns), one thread issues 16 tcgen05.mma (128 x 64 x 16) into one of three
// tensor-memory accumulators, and two tiles later the workers read the accumulator back (thread = row, 32
// query columns per warp) and test every score against the query's threshold.  One decode serves 64 queries
// instead of 32 and needs no per-fragment shuffling, the MMAs leave the instruction stream, and the B
// operand is read by the tensor core instead of by LDS.
// Warp 0 only issues the MMAs (the issuing thread is held for about as long as they execute), warps 4-11 decode
// and test; the decoded rows go straight to tensor memory (tcgen05.st) and the MMA reads its A operand there;
// workers and issuer meet on mbarriers, there is no CTA barrier in the loop; three accumulators, so that the
// products a worker reads were issued two tiles earlier; a row's hits are filed by its own lane, one per round.
// 1M rows x 1024 queries: 1.67 ms for the whole search against 2.23 ms with the mma.sync scan; default for k <= 12
// (QUASHKV_B200_INDEX_TCGEN05=0 selects the mma.sync scan).
//
// Candidate bookkeeping is the mma.sync kernel's: per (row quarter, query) private buffers, a shared
// rising threshold, flagged queries redone by the CUDA-core scan.  A warp sees 32 rows per tile, so
// its first eight tiles are pushed in four lane groups with a prune in between.
#include "index_candidates.cuh"
#include "umma.cuh"

namespace qkv {

constexpr int kXQ = 64;                      // queries per CTA = MMA N
constexpr int kXRows = 128;                  // rows per tile = MMA M
constexpr int kXFirstWorker = 4;             // warp 0 issues the MMAs, warps 1-3 only help with the set-up and the lists
constexpr int kXWorkers = 256;               // worker warp w: row quarter w & 3 (its TMEM lanes), query block (w - 4) >> 2
constexpr int kXThreads = 32 * kXFirstWorker + kXWorkers;
constexpr int kXCap = 40;                    // candidate slots per (row quarter, query)
constexpr int kXSlack = 24;                  // a buffer is pruned when fewer slots than this are free: a tile can
                                             // add 32 rows at once, a handful in practice once the threshold is up
                                             // (64 slots, pruned at 40, measured slower: 1.76 against 1.67 ms at 1M x 1024)
constexpr uint32_t kXATile = kXRows * 256 * 2;   // 64 KB: four K blocks of 64 fp16
constexpr uint32_t kXBTile = kXQ * 256 * 2;      // 32 KB
constexpr uint32_t kXTmemCols = 512;         // three accumulators of 64 columns, two A operands of 128 (256 fp16 per row)
constexpr uint32_t kXTmemA = 256;            // first column of the A operands
constexpr int kXMaxK = kXCap - kXSlack - 4;  // k + a few extra rows must fit below the prune mark

constexpr size_t kXSmemBytes = 1024 + 2 * kXATile + kXBTile + static_cast<size_t>(kXQ) * 4 * kXCap * 6 + 5 * 8 + 16;

__device__ unsigned int g_index_umma_timeouts = 0;

// K position of the centroid part: k = 16 wd + 4 g + e  <->  coordinate 16 wd + g + 4 e (the order in which
// one PRMT per pair produces the values of a 32-bit code word).
__host__ __device__ constexpr int code_coord(int k) { return 16 * (k >> 4) + ((k & 15) >> 2) + 4 * (k & 3); }

__global__ void __launch_bounds__(kXThreads, 1) index_scan_umma_kernel(ScanMmaArgs a) {
  constexpr int D = 128;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float2 init_thr[kXQ];        // .x = kEps - sum of sign weights (unit query), .y = threshold
  __shared__ float inv_s[kXQ];
  __shared__ int cnt[4][kXQ];
  __shared__ float quart[4][kXQ];
  __shared__ float nmax_w[kXThreads / 32];
  unsigned char* base = smem_raw + ((1024u - (umma::smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* b_tile = base + 2 * kXATile;       // (the first 2 x 64 KB are not used: one CTA per SM, as its 512 tensor-memory columns require)
  float* buf_u = reinterpret_cast<float*>(b_tile + kXBTile);                      // [query][row quarter][kXCap]
  uint16_t* buf_r = reinterpret_cast<uint16_t*>(buf_u + kXQ * 4 * kXCap);
  uint64_t* mbar = reinterpret_cast<uint64_t*>(buf_r + kXQ * 4 * kXCap);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mbar + 5);   // mbar: accumulator 0 / 1 / 2 complete, A 0 / 1 written
  int* dead = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool worker = warp >= kXFirstWorker;
  const int rq = warp & 3, cb = worker ? (warp - kXFirstWorker) >> 2 : 0;
  const int row = 32 * rq + lane;           // row of the tile = tensor-memory lane
  const int slice = blockIdx.x, q0 = blockIdx.y * kXQ;
  const float inv_sk = __uint_as_float(a.tables[6]);
  const uint32_t kt_a = a.tables[0], kt_b = a.tables[1];
  constexpr int QS = 4 * kXCap;

  // ---- per query: unit scale, constant term, threshold ----------------------------------------------------
  if (tid < kXQ) {
    const int m = q0 + tid;
    const float* q = a.qk + static_cast<int64_t>(m < a.M ? m : 0) * 2 * D;
    float q2 = 0.f, ws = 0.f;
#pragma unroll 1
    for (int j0 = 0; j0 < D; j0 += 16) {             // sixteen loads of each half in flight, then the sums in order
      float4 x[4], w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        x[e] = __ldg(reinterpret_cast<const float4*>(q + j0) + e);
        w[e] = __ldg(reinterpret_cast<const float4*>(q + D + j0) + e);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        q2 = fmaf(x[e].x, x[e].x, q2); q2 = fmaf(x[e].y, x[e].y, q2); q2 = fmaf(x[e].z, x[e].z, q2); q2 = fmaf(x[e].w, x[e].w, q2);
        ws += w[e].x; ws += w[e].y; ws += w[e].z; ws += w[e].w;
      }
    }
    const float qn = sqrtf(q2);
    const bool usable = m < a.M && qn > 0.f && qn < INFINITY;
    const float inv = usable ? 1.f / qn : 0.f;
    inv_s[tid] = inv;
    init_thr[tid] = make_float2(kEps - ws * inv, usable ? -INFINITY : INFINITY);
    if (m < a.M && !usable) a.flags[m] = 1;
  }
  for (int i = tid; i < 4 * kXQ; i += kXThreads) { (&cnt[0][0])[i] = 0; (&quart[0][0])[i] = -INFINITY; }
  if (tid == 0) {
    umma::mbar_init(&mbar[0], 1);
    umma::mbar_init(&mbar[1], 1);
    umma::mbar_init(&mbar[2], 1);
    umma::mbar_init(&mbar[3], kXWorkers);
    umma::mbar_init(&mbar[4], kXWorkers);
    *dead = 0;
  }
  __syncthreads();
  // ---- B operand: 64 queries x 256 K, fp16, swizzled K-major (four blocks of 64 K = 8 KB each) ------------
#pragma unroll 8
  for (int idx = tid; idx < kXQ * 256; idx += kXThreads) {
    const int n = idx >> 8, k = idx & 255;
    const int m = q0 + n;
    const float* q = a.qk + static_cast<int64_t>(m < a.M ? m : 0) * 2 * D;
    float v;
    if (k < 128) {
      v = q[code_coord(k)] * inv_s[n] * inv_sk;
    } else {
      const int kk = k - 128, s = kk >> 5, t = (kk & 31) >> 1, hb = kk & 1;
      v = q[D + 32 * s + sign_coord(t) + 16 * hb] * inv_s[n] * (2.f / sign_v1(sign_pos(t)));
    }
    *reinterpret_cast<__half*>(b_tile + umma::sw128_offset(n, k, kXQ)) = __float2half_rn(v);
  }
  if (warp == 0) umma::tmem_alloc(tmem_slot, kXTmemCols);
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t n_begin = slice * a.slice_len;
  int64_t n_end = n_begin + a.slice_len;
  if (n_end > a.N) n_end = a.N;
  const int n_valid = static_cast<int>(n_end - n_begin);
  const int n_tiles = (n_valid + kXRows - 1) / kXRows;
  const uint4* codes = reinterpret_cast<const uint4*>(a.codes);
  const uint2* signs = reinterpret_cast<const uint2*>(a.signs);
  float my_nmax = 0.f;

  // raw packed words of this thread's half row: code words 4 cb .. 4 cb + 3, sign words 2 cb, 2 cb + 1
  auto fetch = [&](int tile, uint4& c, uint2& s, float& kn) {
    const int r = tile * kXRows + row;
    const bool ok = r < n_valid;
    const int64_t n = n_begin + (ok ? r : 0);
    c = ok ? __ldg(codes + n * 2 + cb) : make_uint4(0u, 0u, 0u, 0u);
    s = ok ? __ldg(signs + n * 2 + cb) : make_uint2(0u, 0u);
    kn = ok ? __ldg(a.norms + n) : 0.f;
  };

  // The decoded half row goes straight to tensor memory: 32-bit column c of the A operand holds K elements 2 c and
  // 2 c + 1, and a 16-byte chunk of the K-major row is four such columns.  Code part: columns 32 cb .. + 31, sign
  // part: 64 + 32 cb .. + 31 (lane = row).
  auto decode = [&](const uint4& c, const uint2& s, int buf) {
    const uint32_t ta = tmem_base + (static_cast<uint32_t>(32 * rq) << 16) + kXTmemA + buf * 128 + 32 * cb;
    const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int hw = 0; hw < 2; ++hw) {
      uint32_t o[16];
#pragma unroll
      for (int w2 = 0; w2 < 2; ++w2) {
        const int wd = 2 * hw + w2;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t y = (cw[wd] >> (2 * g)) & 0x03030303u;
          const uint32_t sl = y * 0x22u + 0x10101010u;
          o[8 * w2 + 2 * g] = prmt(kt_a, kt_b, sl);
          o[8 * w2 + 2 * g + 1] = prmt(kt_a, kt_b, sl >> 16);
        }
      }
      umma::tmem_st16(ta + 16 * hw, o);
    }
    const uint32_t sw[2] = {s.x, s.y};
#pragma unroll
    for (int w2 = 0; w2 < 2; ++w2) {
      const uint32_t cp[4] = {sw[w2], sw[w2] << 7, sw[w2] >> 1, sw[w2] << 13};
      uint32_t o[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const int cpy = t < 7 ? 0 : (t < 14 ? 1 : t - 12);
        o[t] = cp[cpy] & (0x00010001u << sign_pos(t));
      }
      umma::tmem_st16(ta + 64 + 16 * w2, o);
    }
  };

  auto issue_mmas = [&](int buf, int acc) {
    constexpr uint32_t idesc = umma::instr_desc(umma::kFmtF16, kXRows, kXQ);
    const uint32_t d = tmem_base + acc * kXQ;
    const uint32_t a_tmem = tmem_base + kXTmemA + buf * 128, b_addr = umma::smem_u32(b_tile);
#pragma unroll
    for (int ks = 0; ks < 16; ++ks) {
      const uint32_t b_off = (ks >> 2) * (kXQ * 128) + (ks & 3) * 32;
      umma::mma_f16_ts(d, a_tmem + 8 * ks, umma::smem_desc_sw128(b_addr + b_off), idesc, ks != 0);
    }
    umma::commit(&mbar[acc]);
  };

  // Shrink this warp's buffers that are close to full (same rule as the mma.sync kernel).
  auto prune = [&]() {
    unsigned need = __ballot_sync(QKV_FULL_MASK, cnt[rq][32 * cb + lane] > kXCap - kXSlack);
    if (!need) return;
    float nm = my_nmax;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(QKV_FULL_MASK, nm, o));
    const int k4 = (a.k + 3) / 4;
    while (need) {
      const int q = 32 * cb + __ffs(need) - 1;
      need &= need - 1;
      const int n = cnt[rq][q] < kXCap ? cnt[rq][q] : kXCap;
      float T, T4;
      const int kept = select_sorted<kXCap>(buf_u + q * QS + rq * kXCap, buf_r + q * QS + rq * kXCap, n, a.k,
                                            2.f * kEps * nm, kXCap - kXSlack, init_thr[q].y, k4, T, T4, lane);
      if (lane == 0) {
        if (kept > kXCap - kXSlack) {
          if (q0 + q < a.M) a.flags[q0 + q] = 1;
          init_thr[q].y = INFINITY;
          cnt[rq][q] = 0;
        } else {
          cnt[rq][q] = kept;
          quart[rq][q] = fmaxf(quart[rq][q], T4);
          const float all4 = fminf(fminf(*reinterpret_cast<volatile float*>(&quart[0][q]),
                                         *reinterpret_cast<volatile float*>(&quart[1][q])),
                                   fminf(*reinterpret_cast<volatile float*>(&quart[2][q]),
                                         *reinterpret_cast<volatile float*>(&quart[3][q])));
          const float bound = fmaxf(T, all4);
          raise_threshold(&init_thr[q].y, bound);
          if (q0 + q < a.M && bound > -INFINITY) publish_bound(a.gthr + q0 + q, bound);
        }
      }
    }
    __syncwarp();
  };

  // Scores of row `row` against this warp's 32 queries: optimistic score (c + kEps - sum w) * norm.
  auto epilogue = [&](int tile, int acc, float kn, float g, bool use_tmem) {   // g: the other slices' bound for query `lane`
    const int r = tile * kXRows + row;
    const bool valid = r < n_valid && use_tmem;
    uint32_t v[32];
    if (use_tmem) umma::tmem_ld32(tmem_base + (static_cast<uint32_t>(32 * rq) << 16) + acc * kXQ + 32 * cb, v);
    if (valid) my_nmax = fmaxf(my_nmax, kn);
    if (q0 + 32 * cb + lane < a.M) {                 // the other slices' progress: lane = query
      float* mine = &init_thr[32 * cb + lane].y;
      if (g > *mine && *mine != INFINITY) raise_threshold(mine, g);
    }
    __syncwarp();
    const int n_sub = tile < 8 ? 4 : 1;              // a warp's first rows arrive in four groups of eight lanes
    // Which of this row's 32 scores reach their query's threshold: one bit each, computed without a branch.  Then
    // every lane files its own hits, one per round: the rounds a warp needs are the LARGEST number of hits in one
    // row, not the number of (row, query) hits of the whole warp as with a branch per query (hits are spread over
    // rows and queries; the branch per query was 3000 of a tile's 5500 cycles).
    uint32_t hits = 0;
#pragma unroll
    for (int q = 0; q < 32; ++q) {
      const float2 it = init_thr[32 * cb + q];
      const float u = (__uint_as_float(v[q]) + it.x) * kn;
      hits |= (u >= it.y ? 1u : 0u) << q;
    }
    if (!valid) hits = 0;
#pragma unroll 1
    for (int sub = 0; sub < n_sub; ++sub) {
      uint32_t todo = (n_sub == 1 || (lane >> 3) == sub) ? hits : 0u;
      while (__any_sync(QKV_FULL_MASK, todo != 0u)) {
        if (todo) {
          const int q = __ffs(todo) - 1;
          todo &= todo - 1;
          uint32_t raw = v[0];                        // v[q] without a variable register index
#pragma unroll
          for (int j = 1; j < 32; ++j) raw = q == j ? v[j] : raw;
          const int qq = 32 * cb + q;
          const float2 it = init_thr[qq];
          const float u = (__uint_as_float(raw) + it.x) * kn;
          if (u >= it.y) {                            // the threshold may have risen since the first look
            const int pos = atomicAdd(&cnt[rq][qq], 1);
            if (pos < kXCap) {
              buf_u[qq * QS + rq * kXCap + pos] = u;
              buf_r[qq * QS + rq * kXCap + pos] = static_cast<uint16_t>(r);
            } else {                                  // buffer full before it could be pruned: redo this query
              if (q0 + qq < a.M) a.flags[q0 + qq] = 1;
              init_thr[qq].y = INFINITY;
            }
          }
        }
      }
      __syncwarp();
      prune();
    }
  };

  // ---- warp 0: per tile, wait until every worker has stored its part of A(i), then the 16 MMAs -----------------
  // (the thread that issues them is held for about as long as they execute; as a worker it would hold the
  // whole CTA back by that time)
  if (warp == 0) {
    if (lane == 0) {
      uint32_t full_phase[2] = {0u, 0u};
      for (int i = 0; i < n_tiles; ++i) {
        const int buf = i & 1;
        if (*reinterpret_cast<volatile int*>(dead)) break;
        if (!umma::mbar_wait(&mbar[3 + buf], full_phase[buf])) { *reinterpret_cast<volatile int*>(dead) = 1; break; }
        full_phase[buf] ^= 1u;
        if (*reinterpret_cast<volatile int*>(dead)) break;
        umma::fence_after_sync();
        issue_mmas(buf, i % 3);
      }
    }
    __syncwarp();
  }
  // ---- workers: wait(i-2); decode(i); arrive; epilogue(i-2).  No CTA barrier, and the products a worker waits
  // for were issued two tiles ago.  A(i) goes into the buffer of tile i-2, whose products this thread has waited
  // for; accumulator (i+1) % 3 = (i-2) % 3 is overwritten only after every worker has arrived for tile i+1, that
  // is after its epilogue of tile i-2.
  if (worker) {
    uint32_t phase[3] = {0u, 0u, 0u};
    auto wait_products = [&](int acc) -> bool {
      bool ok = *reinterpret_cast<volatile int*>(dead) == 0;
      if (ok) {
        const uint32_t ph = acc == 0 ? phase[0] : (acc == 1 ? phase[1] : phase[2]);
        ok = umma::mbar_wait(&mbar[acc], ph);
        if (acc == 0) phase[0] ^= 1u; else if (acc == 1) phase[1] ^= 1u; else phase[2] ^= 1u;
        if (!ok) *reinterpret_cast<volatile int*>(dead) = 1;
      }
      umma::fence_after_sync();
      return ok;
    };
    const bool have_q = q0 + 32 * cb + lane < a.M;
    uint4 rc; uint2 rs;
    float kn_next = 0.f, kn0 = 0.f, kn1 = 0.f, kn2 = 0.f;       // norms of tiles i, i-1, i-2
    if (n_tiles > 0) fetch(0, rc, rs, kn_next);
    for (int i = 0; i < n_tiles; ++i) {
      const int buf = i & 1;
      // the shared bound travels while the tile is decoded
      const float g = have_q ? *reinterpret_cast<const volatile float*>(a.gthr + q0 + 32 * cb + lane) : -INFINITY;
      bool ok = true;
      if (i >= 2) ok = wait_products((i - 2) % 3);
      decode(rc, rs, buf);
      kn2 = kn1; kn1 = kn0; kn0 = kn_next;
      if (i + 1 < n_tiles) fetch(i + 1, rc, rs, kn_next);
      umma::tmem_st_wait();
      umma::fence_before_sync();
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(umma::smem_u32(&mbar[3 + buf])) : "memory");
      if (i >= 2) epilogue(i - 2, (i - 2) % 3, kn2, g, ok);
    }
    for (int t = n_tiles >= 2 ? n_tiles - 2 : 0; t < n_tiles; ++t) {     // the last two tiles
      const bool ok = wait_products(t % 3);
      const float g = have_q ? *reinterpret_cast<const volatile float*>(a.gthr + q0 + 32 * cb + lane) : -INFINITY;
      epilogue(t, t % 3, t == n_tiles - 1 ? kn0 : kn1, g, ok);
    }
  }
  {
    float nm = my_nmax;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) nm = fmaxf(nm, __shfl_xor_sync(QKV_FULL_MASK, nm, o));
    if (lane == 0) nmax_w[warp] = nm;
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, kXTmemCols);
  const bool timed_out = *dead != 0;        // the tensor core never answered: every query of this CTA is redone
  if (timed_out && tid == 0) atomicAdd(&g_index_umma_timeouts, 1u);

  // ---- per (query, slice): union of the four row quarters, bounded once more, to the list -----------------
  constexpr int ENT = (kXCap + 31) / 32;
  const int out_k = a.k + kIExtra;
  float nm_cta = 0.f;
#pragma unroll
  for (int w = 0; w < kXThreads / 32; ++w) nm_cta = fmaxf(nm_cta, nmax_w[w]);
  for (int q = warp; q < kXQ; q += kXThreads / 32) {
    if (q0 + q >= a.M) continue;
    const int64_t o = (static_cast<int64_t>(q0 + q) * a.n_slices + slice) * out_k;
    const float T0 = init_thr[q].y;
    float u[4][ENT]; int r[4][ENT]; bool live[4][ENT];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int n_w = cnt[w][q] < kXCap ? cnt[w][q] : kXCap;
#pragma unroll
      for (int e = 0; e < ENT; ++e) {
        const int slot = lane + 32 * e;
        u[w][e] = slot < n_w ? buf_u[q * QS + w * kXCap + slot] : -INFINITY;
        r[w][e] = slot < n_w ? buf_r[q * QS + w * kXCap + slot] : 0;
        live[w][e] = slot < n_w && u[w][e] >= T0;
      }
    }
    __syncwarp();
    int total = 0;
    float* bu = buf_u + q * QS;
    uint16_t* br = buf_r + q * QS;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
#pragma unroll
      for (int e = 0; e < ENT; ++e) {
        const unsigned m = __ballot_sync(QKV_FULL_MASK, live[w][e]);
        const int dst = total + __popc(m & ((1u << lane) - 1u));
        if (live[w][e]) { bu[dst] = u[w][e]; br[dst] = static_cast<uint16_t>(r[w][e]); }
        total += __popc(m);
      }
    }
    __syncwarp();
    bool redo = T0 == INFINITY || timed_out;
    int kept = 0;
    if (!redo) {
      float T, T4;
      kept = select_sorted<QS>(bu, br, total, a.k, 2.f * kEps * nm_cta, out_k, T0, 1, T, T4, lane);
      redo = kept > out_k;
    }
    if (redo) { kept = 0; if (lane == 0) a.flags[q0 + q] = 1; }
    for (int s = lane; s < out_k; s += 32) {
      a.list_scores[o + s] = s < kept ? bu[s] : -INFINITY;
      a.list_ids[o + s] = s < kept ? n_begin + br[s] : -1;
    }
  }
}

unsigned int index_umma_timeouts() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_index_umma_timeouts, sizeof(v));
  return v;
}

bool index_umma_ok(int k) { return k <= kXMaxK; }

int index_umma_qtiles(int M) { return (M + kXQ - 1) / kXQ; }

int launch_index_scan_umma(const ScanMmaArgs& a, int n_qtiles, cudaStream_t st) {
  if (cudaFuncSetAttribute(index_scan_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(kXSmemBytes)) != cudaSuccess)
    return QKV_ELAUNCH;
  index_scan_umma_kernel<<<dim3(a.n_slices, n_qtiles), kXThreads, kXSmemBytes, st>>>(a);
  return QKV_OK;
}

}  // namespace qkv
