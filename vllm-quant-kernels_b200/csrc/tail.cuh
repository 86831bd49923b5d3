// Sampler tail of the streaming lm_head kernel at decode sizes: one CTA of the grid turns the
// records every CTA left in memory into the step's tokens, one warp per batch row, while those
// records are still in L2.
//
// Per batch row every CTA leaves one 64-byte record (CtaList, lm_head.cuh):
//   * the Gumbel (or greedy) winner of the CTA's vocab rows, for rows without top-k / top-p;
//   * the kCtaListM largest logits of the CTA's vocab rows with their token ids, and a WITNESS: every
//     logit of the CTA that is not listed is <= it, for rows with top-k.
// A top-k row is resolved from the records alone when they prove to hold every logit >= the k-th
// largest of the row: t_k = k-th largest of the listed values, and every witness of a CTA that
// could matter is < t_k.  Then top-k (ties kept), top-p and the Gumbel argmax run on those few
// values with the arithmetic of resolve_candidates in sampler.cu (same tokens, same scores).  A
// row the records cannot prove (more than kCtaListM of the top k in one CTA, or more than kListM in
// one warp group's slice; top-p without top-k; a threshold row with top-p; k > kTailMaxK) gets
// row_flag = 1 and is resolved from its fp16 logits row by the full-row kernel (k_select), which is
// launched behind every step and returns at once for rows whose flag is 0.
//
// WHO runs it: the LAST CTA of the grid to finish (an atomic ticket; nobody waits for anybody).
// HOW it is written: a single warp runs at the speed of its dependent latencies, not of its
// instruction count - an L2 round trip costs it more than a microsecond, a selection round some
// hundred cycles.  (Measured on B200 with %globaltimer stamps: a version that walked per-slice
// data in small loops took 16 us per row, one with two dependent trips - slice maxima, then the
// lists of the slices that can matter - 12 us.)  So a row costs ONE L2 trip: all the CTAs' records
// (9.5 KB for 148 CTAs) come into shared memory with asynchronous 16-byte copies that need no
// registers, and everything else runs on shared memory and registers: the k-th largest of the 148
// per-CTA maxima bounds the k-th largest logit from below, the few listed values above that bound are
// staged, and the k-th largest of those is t_k.
//
// All logits on this path are fp16 values, so their order is the order of 16-bit keys.
#pragma once

#include <type_traits>

#include "lm_head.cuh"
#include "peer_exchange.cuh"

namespace vqk {

constexpr int kTailMaxCtas = 160;     // CTAs (records per row) the tail can take; 5 per lane
constexpr int kTailCtaRegs = kTailMaxCtas / 32;
constexpr int kTailMaxK = 126;        // largest top-k resolved from the records (a shard record holds as many)
constexpr int kTailStageCap = 256;    // listed values >= the first bound a row may stage (k + ties + neighbours)
constexpr int kTailSurvCap = 192;     // survivors of top-k (k + ties) resolved per row
constexpr int kTailMaxWarps = 16;

// Per-warp scratch (bytes).  Region A holds the CTAs' records while a row is resolved, and afterwards
// the union of the shards' candidates (mv, mt); then the survivors and the top-p work arrays, which
// the staged entries borrow until the survivors are known.
constexpr int kTailOffRecs = 0;                                     // CtaList [kTailMaxCtas]
constexpr int kTailOffMv = 0;                                       // float  [kMergeCap]
constexpr int kTailOffMt = kTailOffMv + kMergeCap * 4;              // int    [kMergeCap]
constexpr int kTailRegionA = ((kTailOffMt + kMergeCap * 4 > kTailMaxCtas * 64 ? kTailOffMt + kMergeCap * 4 : kTailMaxCtas * 64) + 15) & ~15;
constexpr int kTailOffCv = kTailRegionA;                            // float  [kTailSurvCap]
constexpr int kTailOffCt = kTailOffCv + kTailSurvCap * 4;           // int    [kTailSurvCap]
constexpr int kTailOffY = kTailOffCt + kTailSurvCap * 4;            // float  [kTailSurvCap]
constexpr int kTailOffW = kTailOffY + kTailSurvCap * 4;             // uint64 [kTailSurvCap]
constexpr int kTailOffAlive = kTailOffW + kTailSurvCap * 8;         // uint8  [kTailSurvCap]
constexpr int kTailOffStage = kTailOffY;                            // uint2  [kTailStageCap]: key, local token
constexpr int kTailWarpBytes = (kTailOffAlive + kTailSurvCap + 15) & ~15;
static_assert(kTailStageCap * 8 <= kTailOffAlive - kTailOffY, "the staged entries fit the top-p work arrays");
static_assert(kTailOffW % 8 == 0, "mass array alignment");

// shared memory the tail wants from a CTA for `rows` batch rows (it makes do with less: fewer rows at a time)
__host__ __device__ inline size_t tail_smem_bytes(int rows) {
  return (size_t)(rows < kTailMaxWarps ? rows : kTailMaxWarps) * kTailWarpBytes;
}

// order-preserving 16-bit key of an fp16-representable float; -0 sorts with +0
__device__ __forceinline__ uint32_t h16_key(float v) {
  uint32_t b = __half_as_ushort(__float2half_rn(v));
  if ((b & 0x7fffu) == 0) b = 0;
  return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
}
__device__ __forceinline__ float h16_key_to_float(uint32_t k) {
  const uint32_t b = (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
  return __half2float(__ushort_as_half((unsigned short)b));
}
// the same key from the fp16 bits
__device__ __forceinline__ uint32_t h16_bits_key(uint32_t b) {
  b &= 0xffffu;
  if ((b & 0x7fffu) == 0) b = 0;
  return (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
}
constexpr uint32_t kKeyLowestFinite = 0x0400u;  // key(-65504); key(-inf) = 0x03ff sorts below

// k-th largest of the 16-bit keys a warp holds in registers (key[j] of lane l; unused slots hold 0,
// below every candidate >= kKeyLowestFinite that can win), three key bits per round: each round
// counts the keys >= seven thresholds at once (the counts packed ten bits apiece into three words,
// so a round costs three warp reductions instead of one per bit).  At least k keys must be
// >= kKeyLowestFinite.  The bits all those keys share (they usually agree in sign and exponent) are
// found with two reductions first and cost no round.  Result in every lane.
template <int R>
__device__ __forceinline__ uint32_t warp_kth_largest_reg(const uint32_t (&key)[R], int k) {
  static_assert(R * 32 < 1024, "a count must fit ten bits");
  uint32_t hi = 0, lo = 0xffffu;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    hi = max(hi, key[j]);
    if (key[j] >= kKeyLowestFinite) lo = min(lo, key[j]);
  }
  hi = __reduce_max_sync(0xffffffffu, hi);
  lo = __reduce_min_sync(0xffffffffu, lo);
  int nbits = 32 - __clz((hi ^ lo) | 0u);  // low bits in which the keys differ (0: all equal)
  if (hi == lo) return hi;
  uint32_t prefix = hi & ~((1u << nbits) - 1u);
#pragma unroll 1
  while (nbits > 0) {
    // thresholds prefix | t << sh, t = 1 .. nt
    const int w = nbits >= 3 ? 3 : nbits;
    const int sh = nbits - w;
    const int nt = (1 << w) - 1;
    uint32_t c0 = 0, c1 = 0, c2 = 0;  // counts of t = 1..3 | 4..6 | 7
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const uint32_t kj = key[j];
      c0 += (kj >= (prefix | (1u << sh))) + ((uint32_t)(nt > 1 && kj >= (prefix | (2u << sh))) << 10) +
            ((uint32_t)(nt > 2 && kj >= (prefix | (3u << sh))) << 20);
      c1 += (uint32_t)(nt > 3 && kj >= (prefix | (4u << sh))) + ((uint32_t)(nt > 3 && kj >= (prefix | (5u << sh))) << 10) +
            ((uint32_t)(nt > 3 && kj >= (prefix | (6u << sh))) << 20);
      c2 += (uint32_t)(nt > 3 && kj >= (prefix | (7u << sh)));
    }
    c0 = __reduce_add_sync(0xffffffffu, c0);
    c1 = __reduce_add_sync(0xffffffffu, c1);
    c2 = __reduce_add_sync(0xffffffffu, c2);
    // counts fall as t grows: take the largest t whose count still reaches k
    uint32_t t = 0;
    if ((int)(c0 & 1023u) >= k) t = 1;
    if ((int)((c0 >> 10) & 1023u) >= k) t = 2;
    if ((int)(c0 >> 20) >= k) t = 3;
    if ((int)(c1 & 1023u) >= k) t = 4;
    if ((int)((c1 >> 10) & 1023u) >= k) t = 5;
    if ((int)(c1 >> 20) >= k) t = 6;
    if ((int)c2 >= k) t = 7;
    prefix |= t << sh;
    nbits = sh;
  }
  return prefix;
}

// k-th largest of n keys in shared memory (n >= k >= 1) by bisection on the key bits `hi` down to
// `lo`: the largest x with count(key >= x) >= k.  Whole warp; result in every lane.
template <typename LoadKey>
__device__ __forceinline__ uint32_t warp_kth_largest_key(LoadKey key_at, int n, int k, int hi, int lo, int lane) {
  uint32_t prefix = 0;
#pragma unroll 1
  for (int bit = hi; bit >= lo; --bit) {
    const uint32_t cand = prefix | (1u << bit);
    int c = 0;
#pragma unroll 4
    for (int i = lane; i < n; i += 32) c += (key_at(i) >= cand);
    c = __reduce_add_sync(0xffffffffu, c);
    if (c >= k) prefix = cand;
  }
  return prefix;
}

__device__ __forceinline__ void warp_best_pair(float& s, int& t) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
    const int t2 = __shfl_xor_sync(0xffffffffu, t, o);
    if (better(s2, t2, s, t)) { s = s2; t = t2; }
  }
}

__device__ __forceinline__ void tail_write_header(uint8_t* records, int b, float score, int token, int n, int flags) {
  if (!records) return;
  RecordHeader* h = reinterpret_cast<RecordHeader*>(records + (size_t)b * VQK_RECORD_BYTES);
  h->score = score; h->token = token; h->n = n; h->flags = flags;
}

// Top-k over n <= kMergeCap candidates (raw logit, token) in shared memory, in place: those >= the
// K-th largest (ties kept; all of them when n <= K or K <= 0) move to the front.  Returns how many.
static __device__ __noinline__ int warp_topk_inplace(float* v, int* t, int n, int K, int lane) {
  if (K <= 0 || n <= K) return n;
  // fp16-representable values (every logit of the lm_head path) differ in the upper 19 key bits only
  int low = 1;
  for (int i = lane; i < n; i += 32) low &= ((__float_as_uint(v[i]) & 0x1fffu) == 0);
  low = __all_sync(0xffffffffu, low);
  float thr;  // the K-th largest value; entries >= it survive (float compare: -0 ties with +0)
  if (low && n <= 512) {  // the usual case: fp16 logits, a few per lane - select on registers, 16-bit keys
    // (as few registers as the count needs: a selection round costs in proportion to them)
    auto select = [&](auto rtag) {
      constexpr int R = decltype(rtag)::value;
      uint32_t key[R];
#pragma unroll
      for (int j = 0; j < R; ++j) key[j] = j * 32 + lane < n ? h16_key(v[j * 32 + lane]) : 0u;
      int fin = 0;
#pragma unroll
      for (int j = 0; j < R; ++j) fin += (key[j] >= kKeyLowestFinite);
      fin = __reduce_add_sync(0xffffffffu, fin);
      // (-inf entries can only come from an all -inf shard; with fewer than K finite values all of them survive)
      return fin >= K ? warp_kth_largest_reg(key, K) : kKeyLowestFinite;
    };
    uint32_t k16;
    if (n <= 128) k16 = select(std::integral_constant<int, 4>{});
    else if (n <= 256) k16 = select(std::integral_constant<int, 8>{});
    else k16 = select(std::integral_constant<int, 16>{});
    thr = h16_key_to_float(k16);
  } else {
    thr = key_f32(warp_kth_largest_key([&](int i) { return f32_key(v[i]); }, n, K, 31, low ? 13 : 0, lane));
  }
  const unsigned lt = (1u << lane) - 1u;
  int kept = 0;
#pragma unroll 1
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    float vi = 0.f;
    int ti = 0;
    bool keep = false;
    if (i < n) { vi = v[i]; ti = t[i]; keep = vi >= thr; }
    const unsigned mask = __ballot_sync(0xffffffffu, keep);  // every lane has read before anyone writes
    if (keep) { const int pos = kept + __popc(mask & lt); v[pos] = vi; t[pos] = ti; }
    kept += __popc(mask);
    __syncwarp();
  }
  return kept;
}

// Top-p over the n <= kTailSurvCap top-k survivors, then the Gumbel argmax: the arithmetic of
// resolve_candidates (sampler.cu), so both paths pick the same token with the same score.
struct TailWinner {
  float s;
  int t;
};
static __device__ __noinline__ TailWinner warp_topp_gumbel(const float* cv, const int* ct, int n, float T, float top_p, int seed,
                                                           float* y, unsigned long long* w, unsigned char* alive, int lane) {
#pragma unroll 1
  for (int i = lane; i < n; i += 32) { y[i] = cv[i] / T; alive[i] = 1; }
  __syncwarp();
  if (top_p < 1.f) {
    float mx = -INFINITY;
#pragma unroll 1
    for (int i = lane; i < n; i += 32) mx = fmaxf(mx, y[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    unsigned long long z = 0;
#pragma unroll 1
    for (int i = lane; i < n; i += 32) {
      const unsigned long long wi = __float2ull_rz(expf(y[i] - mx) * 1099511627776.0f);  // exact scaling: the value mass_of (sampler.cu) computes in double
      w[i] = wi;
      z += wi;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    __syncwarp();
    const double target = (double)top_p * (double)z;
#pragma unroll 1
    for (int i = lane; i < n; i += 32) {
      const float yi = y[i];
      unsigned long long above = 0;
#pragma unroll 4
      for (int j = 0; j < n; ++j)
        if (y[j] > yi) above += w[j];
      if (!((double)above < target)) alive[i] = 0;
    }
    __syncwarp();
  }
  float s = -INFINITY;
  int t = 0x7fffffff;
#pragma unroll 1
  for (int i = lane; i < n; i += 32) {
    if (!alive[i]) continue;
    const float sc = y[i] + gumbel_noise(seed, (uint32_t)ct[i]);
    if (better(sc, ct[i], s, t)) { s = sc; t = ct[i]; }
  }
  warp_best_pair(s, t);
  return TailWinner{s, t};
}

// The same for n <= 64 survivors (the usual case: k + ties), held two per lane in registers: the
// mass above each survivor is summed over shuffles, the two Gumbel draws of a lane run side by side.
static __device__ __noinline__ TailWinner warp_topp_gumbel64(const float* cv, const int* ct, int n, float T, float top_p,
                                                             int seed, int lane) {
  const bool h0 = lane < n, h1 = lane + 32 < n;
  const float y0 = h0 ? cv[lane] / T : -INFINITY, y1 = h1 ? cv[lane + 32] / T : -INFINITY;
  const int t0 = h0 ? ct[lane] : 0x7fffffff, t1 = h1 ? ct[lane + 32] : 0x7fffffff;
  bool a0 = h0, a1 = h1;
  if (top_p < 1.f) {
    float mx = fmaxf(y0, y1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const unsigned long long w0 = h0 ? __float2ull_rz(expf(y0 - mx) * 1099511627776.0f) : 0ull;  // = mass_of (sampler.cu): the scaling is exact
    const unsigned long long w1 = h1 ? __float2ull_rz(expf(y1 - mx) * 1099511627776.0f) : 0ull;
    unsigned long long z = w0 + w1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    const double target = (double)top_p * (double)z;
    unsigned long long ab0 = 0, ab1 = 0;
#pragma unroll 4
    for (int src = 0; src < 32; ++src) {
      const float ys0 = __shfl_sync(0xffffffffu, y0, src), ys1 = __shfl_sync(0xffffffffu, y1, src);
      const unsigned long long ws0 = __shfl_sync(0xffffffffu, w0, src), ws1 = __shfl_sync(0xffffffffu, w1, src);
      if (ys0 > y0) ab0 += ws0;
      if (ys1 > y0) ab0 += ws1;
      if (ys0 > y1) ab1 += ws0;
      if (ys1 > y1) ab1 += ws1;
    }
    a0 = a0 && ((double)ab0 < target);
    a1 = a1 && ((double)ab1 < target);
  }
  const float g0 = gumbel_noise(seed, (uint32_t)t0), g1 = gumbel_noise(seed, (uint32_t)t1);
  float s = a0 ? y0 + g0 : -INFINITY;
  int t = a0 ? t0 : 0x7fffffff;
  const float s1 = a1 ? y1 + g1 : -INFINITY;
  if (a1 && better(s1, t1, s, t)) { s = s1; t = t1; }
  warp_best_pair(s, t);
  return TailWinner{s, t};
}

// Sharded step: exchange this rank's record of row b and merge the shards.  Whole warp; writes the
// row's token / score.  `scratch` is the warp's scratch (region A is overwritten).
template <typename CandAt>
__device__ inline void tail_exchange_row(const PeerTable& pt, const RowMeta& m, int b, float score, int token, int n,
                                         int flags, CandAt cand, uint8_t* scratch, int lane, long long* tokens,
                                         float* scores, unsigned int step = 0) {
  float* mv = reinterpret_cast<float*>(scratch + kTailOffMv);
  int* mt = reinterpret_cast<int*>(scratch + kTailOffMt);
  const PeerRowResult r = peer_exchange_row(pt, b, score, token, n, flags, cand, mv, mt, lane, step);
  float s = -INFINITY;
  int t = -1;
  if (!r.late && !r.bad) {
    if (r.total == 0) {
      s = r.best_s;
      t = r.best_t;
    } else {
      __syncwarp();
      const int kept = warp_topk_inplace(mv, mt, r.total, m.top_k, lane);
      if (kept <= kTailSurvCap) {
        const TailWinner w = kept <= 64 ? warp_topp_gumbel64(mv, mt, kept, m.T, m.top_p, m.seed, lane)
                                        : warp_topp_gumbel(mv, mt, kept, m.T, m.top_p, m.seed,
                                                           reinterpret_cast<float*>(scratch + kTailOffY),
                                                           reinterpret_cast<unsigned long long*>(scratch + kTailOffW),
                                                           scratch + kTailOffAlive, lane);
        s = w.s;
        t = w.t;
      }
    }
  }
  if (lane == 0) {
    tokens[b] = t;
    if (scores) scores[b] = s;
  }
  __syncwarp();
}

// What the tail needs of the kernel's parameters (a small copy: the function below is not inlined)
struct TailArgs {
  SampleDev sp;
  const float* slice_max;
  const float* part_score;
  const int* part_token;
  const CtaList* lists;  // [rows][ncta]
  int nslices;
  int ncta;
  long long* tokens;
  float* scores;
  uint8_t* records;
  int single_shard;
  unsigned long long* dbg;  // null, or this CTA's 16 time stamps (measurement aid)
};

// One row, one warp.  Returns 1 when the row is done, 0 when it has to go to the full-row kernel,
// 2 when it is resolved as far as this shard goes and its record (survivors in cv / ct, count in
// *nsv_out, or the winner in *win_s / *win_t) still has to be exchanged.
struct TailRowResult {
  int status;  // 1 done, 0 to the full-row kernel, 2 record to be exchanged
  int nsv;     // survivors in cv / ct (status 2, top-k rows)
  float win_s; // the shard's winner (status 2, rows without top-k / top-p)
  int win_t;
};
// (`a` and `m` live in SHARED memory: in a kernel that takes nearly all of the SM's shared memory
// the L1 is too small to be relied on for stack traffic, and a single warp pays an L2 round trip
// for every miss)
static __device__ __noinline__ TailRowResult tail_resolve_row(const TailArgs& a, const RowMeta& m, int b, uint8_t* scratch,
                                                              int lane, bool exchange) {
  TailRowResult res{0, 0, -INFINITY, 0x7fffffff};
  const long long voff = a.sp.vocab_offset;
  const unsigned lt = (1u << lane) - 1u;
  const int ncta = a.ncta;
  if (!a.lists || ncta > kTailMaxCtas) {
    if (m.flags & ROW_CAND) return res;
    // no records (a kernel without them): per-slice winners -> row winner, as k_select merges them
    const int nsl = a.nslices;
    float s = -INFINITY;
    int t = 0x7fffffff;
#pragma unroll 4
    for (int i = lane; i < nsl; i += 32) {
      const float s2 = __ldcg(a.part_score + (long long)b * nsl + i);
      const int t2 = __ldcg(a.part_token + (long long)b * nsl + i);
      if (better(s2, t2, s, t)) { s = s2; t = t2; }
    }
    warp_best_pair(s, t);
    const long long tok = (long long)t + voff;
    res.win_s = s;
    res.win_t = (int)tok;
    res.status = exchange ? 2 : 1;
    if (!exchange && lane == 0) {
      tail_write_header(a.records, b, s, (int)tok, 0, 0);
      if (a.tokens) a.tokens[b] = tok;
      if (a.scores) a.scores[b] = s;
    }
    return res;
  }
  // 1. the one trip: every CTA's record of this row into shared memory (L2 -> shared, no registers held)
  CtaList* recs = reinterpret_cast<CtaList*>(scratch + kTailOffRecs);
  {
    const uint4* src = reinterpret_cast<const uint4*>(a.lists + (long long)b * ncta);
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(recs);
    for (int i = lane; i < ncta * 4; i += 32)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)i * 16u), "l"(src + i) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
  }
  if (a.dbg && b == 0 && lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory"); a.dbg[5] = t_; }
  if (!(m.flags & ROW_CAND)) {
    // the CTAs' winners -> row winner (the same merge k_select does for these rows)
    float s = -INFINITY;
    int t = 0x7fffffff;
    for (int c = lane; c < ncta; c += 32)
      if (better(recs[c].win_s, recs[c].win_t, s, t)) { s = recs[c].win_s; t = recs[c].win_t; }
    warp_best_pair(s, t);
    const long long tok = (long long)t + voff;
    res.win_s = s;
    res.win_t = (int)tok;
    res.status = exchange ? 2 : 1;
    if (!exchange && lane == 0) {
      tail_write_header(a.records, b, s, (int)tok, 0, 0);
      if (a.tokens) a.tokens[b] = tok;
      if (a.scores) a.scores[b] = s;
    }
    return res;
  }
  if (m.top_k <= 0 || m.top_k > kTailMaxK) return res;

  uint2* st = reinterpret_cast<uint2*>(scratch + kTailOffStage);
  float* cv = reinterpret_cast<float*>(scratch + kTailOffCv);
  int* ct = reinterpret_cast<int*>(scratch + kTailOffCt);
  const int K = m.top_k;
  // 2. key of a CTA = its largest logit; tau0 = K-th largest of those: K distinct logits are >= it,
  //    so the K-th largest logit of the row is too
  uint32_t qk[kTailCtaRegs];
  int nfin = 0;
#pragma unroll
  for (int j = 0; j < kTailCtaRegs; ++j) {
    const int c = j * 32 + lane;
    qk[j] = c < ncta ? h16_bits_key(__half_as_ushort(recs[c].v[0])) : 0u;
    nfin += (qk[j] >= kKeyLowestFinite);
  }
  nfin = __reduce_add_sync(0xffffffffu, nfin);
  uint32_t tau0 = kKeyLowestFinite;
  if (nfin >= K) tau0 = warp_kth_largest_reg(qk, K);
  if (tau0 < kKeyLowestFinite) tau0 = kKeyLowestFinite;
  if (a.dbg && b == 0 && lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory"); a.dbg[6] = t_; }
  // 3. every listed value >= tau0 is staged as (fp16 bits, token), in no particular order (a position
  //    counter in shared memory); the witnesses of the CTAs that reach tau0 are folded to a maximum (a
  //    CTA whose largest logit is below tau0 hides nothing that matters)
  int* stage_n = reinterpret_cast<int*>(scratch + kTailOffAlive);
  if (lane == 0) *stage_n = 0;
  __syncwarp();
  const float tau0f = h16_key_to_float(tau0);
  float wmax = -INFINITY;
  bool spill = false;
#pragma unroll 1
  for (int j = 0; j < kTailCtaRegs; ++j) {
    const int c = j * 32 + lane;
    if (c < ncta && __half2float(recs[c].v[0]) >= tau0f) {
      const uint4 hv = *reinterpret_cast<const uint4*>(recs[c].v);
      const __half2* h2 = reinterpret_cast<const __half2*>(&hv);
      int n = 0;  // descending values: those >= tau0 are a prefix
#pragma unroll
      for (int i = 0; i < kCtaListM / 2; ++i) {
        const float2 f = __half22float2(h2[i]);
        n += (f.x >= tau0f) + (f.y >= tau0f);
      }
      wmax = fmaxf(wmax, __half2float(recs[c].witness));
      const int pos = atomicAdd(stage_n, n);
      if (pos + n <= kTailStageCap) {
        const unsigned short* hb = reinterpret_cast<const unsigned short*>(recs[c].v);
        for (int i = 0; i < n; ++i) st[pos + i] = make_uint2((uint32_t)hb[i], (uint32_t)recs[c].t[i]);
      } else {
        spill = true;
      }
    }
  }
  __syncwarp();
  if (__any_sync(0xffffffffu, spill)) return res;
  const int ne = *stage_n;
  const uint32_t wkey = __reduce_max_sync(0xffffffffu, h16_key(wmax));
  __syncwarp();
  if (a.dbg && b == 0 && lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory"); a.dbg[7] = t_; }
  // 5. t_k: the K-th largest staged value (every staged value survives when fewer than K exist)
  uint32_t tk = kKeyLowestFinite;
  if (ne >= K) {
    if (ne <= 128) {  // the usual case: a handful of keys per lane, kept in registers
      uint32_t sk[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) sk[j] = j * 32 + lane < ne ? h16_bits_key(st[j * 32 + lane].x) : 0u;
      tk = warp_kth_largest_reg(sk, K);
    } else {
      uint32_t sk[kTailStageCap / 32];
#pragma unroll
      for (int j = 0; j < kTailStageCap / 32; ++j) sk[j] = j * 32 + lane < ne ? h16_bits_key(st[j * 32 + lane].x) : 0u;
      tk = warp_kth_largest_reg(sk, K);
    }
  }
  // 6. the proof: no CTA we looked at hides a value >= t_k (the others have maximum < tau0 <= t_k)
  if (wkey >= tk) return res;
  if (a.dbg && b == 0 && lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory"); a.dbg[10] = t_; }
  // 7. survivors (>= t_k, ties kept), with their GLOBAL token ids
  int nsv = 0;
#pragma unroll 1
  for (int i0 = 0; i0 < ne; i0 += 32) {
    const int i = i0 + lane;
    const uint2 e = i < ne ? st[i] : make_uint2(0u, 0u);
    const bool keep = i < ne && h16_bits_key(e.x) >= tk;
    const unsigned mask = __ballot_sync(0xffffffffu, keep);
    const int pos = nsv + __popc(mask & lt);
    if (keep && pos < kTailSurvCap) {
      cv[pos] = __half2float(__ushort_as_half((unsigned short)e.x));
      ct[pos] = (int)((long long)(int)e.y + voff);
    }
    nsv += __popc(mask);
  }
  if (nsv > kTailSurvCap) return res;
  __syncwarp();
  res.nsv = nsv;
  if (exchange) {
    res.status = nsv > VQK_RECORD_CAP ? 0 : 2;  // (the full-row kernel reports an overflowing record)
    return res;
  }
  if (a.records) {  // shard record: the local top-k survivors; top-p needs the union of the shards
    Cand* out = reinterpret_cast<Cand*>(a.records + (size_t)b * VQK_RECORD_BYTES + sizeof(RecordHeader));
    for (int i = lane; i < nsv && i < VQK_RECORD_CAP; i += 32) out[i] = Cand{cv[i], ct[i]};
    if (lane == 0)
      tail_write_header(a.records, b, -INFINITY, -1, min(nsv, VQK_RECORD_CAP), nsv > VQK_RECORD_CAP ? VQK_RECORD_FLAG_OVERFLOW : 0);
  }
  res.status = 1;
  if (!a.single_shard) return res;
  if (a.dbg && b == 0 && lane == 0) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_) :: "memory"); a.dbg[11] = t_; }
  // 8. top-p over the survivors, then the Gumbel argmax
  const TailWinner w = nsv <= 64 ? warp_topp_gumbel64(cv, ct, nsv, m.T, m.top_p, m.seed, lane)
                                 : warp_topp_gumbel(cv, ct, nsv, m.T, m.top_p, m.seed,
                                                    reinterpret_cast<float*>(scratch + kTailOffY),
                                                    reinterpret_cast<unsigned long long*>(scratch + kTailOffW),
                                                    scratch + kTailOffAlive, lane);
  if (lane == 0) {
    if (a.tokens) a.tokens[b] = w.t;
    if (a.scores) a.scores[b] = w.s;
  }
  return res;
}

// Everything the rows' resolution needs, in SHARED memory of the CTA that runs it (filled by one
// thread from the kernel's parameters), so that the code below can live in a function of its own:
// inlined into the lm_head kernels it cost them registers and instruction-cache room for nothing
// (147 of the 148 CTAs never run it).
struct TailShared {
  TailArgs a;
  PeerTable peer;
  RowMeta meta[kTailMaxBatch];      // a copy outside the scratch, which may overlay the kernel's own
  unsigned int step[kTailMaxBatch];  // sharded step: the rows' step numbers, fetched ahead of the exchange
  int* row_flag;
  int B, mode;
};

static __device__ __noinline__ void lm_head_tail_rows(const TailShared& sh, uint8_t* scratch, int nw) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp >= nw) return;
  uint8_t* mine = scratch + (size_t)warp * kTailWarpBytes;
  const bool exchange = sh.peer.G > 0;
  for (int b = warp; b < sh.B; b += nw) {
    TailRowResult rr{0, 0, 0.f, 0};
    if (sh.mode == 1) rr = tail_resolve_row(sh.a, sh.meta[b], b, mine, lane, exchange);  // 2: A/B runs, every row to the full-row kernel
    int r = rr.status;
    if (r == 2) {
      const float* cv = reinterpret_cast<const float*>(mine + kTailOffCv);
      const int* ct = reinterpret_cast<const int*>(mine + kTailOffCt);
      if (sh.meta[b].flags & ROW_CAND)
        tail_exchange_row(sh.peer, sh.meta[b], b, -INFINITY, -1, rr.nsv, 0, [&](int i) { return Cand{cv[i], ct[i]}; }, mine, lane,
                          sh.a.tokens, sh.a.scores, sh.step[b]);
      else
        tail_exchange_row(sh.peer, sh.meta[b], b, rr.win_s, rr.win_t, 0, 0, [](int) { return Cand{0.f, 0}; }, mine, lane,
                          sh.a.tokens, sh.a.scores, sh.step[b]);
      r = 1;
    }
    if (lane == 0) sh.row_flag[b] = r ? 0 : 1;
    __syncwarp();
  }
}

// Called by every thread of every CTA once its slice results are written.  `scratch` is shared
// memory of the CTA that is no longer in use, `scratch_bytes` of it (at least kTailWarpBytes).
// `meta`: the rows' sampling parameters as the kernel decoded them at its start (shared memory).
__device__ __forceinline__ void lm_head_tail(const LmHeadParams& p, const RowMeta* meta, uint8_t* scratch, size_t scratch_bytes) {
  __shared__ int s_last;
  __shared__ TailShared s_tail;
  __syncthreads();  // every thread's slice results are written ...
  if (threadIdx.x == 0) {
    __threadfence();  // ... and visible device-wide before the ticket is taken (the fence is cumulative over the barrier)
    s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    if (s_last) __threadfence();
  }
  __syncthreads();
  if (!s_last) return;
  dbg_stamp(p, 3);
  if (threadIdx.x < p.B && threadIdx.x < kTailMaxBatch) {
    s_tail.meta[threadIdx.x] = meta[threadIdx.x];
    s_tail.step[threadIdx.x] = p.peer.G > 0 ? p.peer.steps[threadIdx.x] + 1u : 0u;
  }
  if (threadIdx.x == 0) {
    TailArgs a;
    a.sp = p.sp; a.slice_max = p.slice_max; a.part_score = p.part_score; a.part_token = p.part_token;
    a.lists = p.lists; a.nslices = p.nslices; a.ncta = (int)gridDim.x; a.tokens = p.tokens; a.scores = p.scores;
    a.records = p.records; a.single_shard = p.single_shard;
    a.dbg = p.dbg ? p.dbg + (size_t)blockIdx.x * 16 : nullptr;
    s_tail.a = a;
    s_tail.peer = p.peer;
    s_tail.row_flag = p.row_flag;
    s_tail.B = p.B;
    s_tail.mode = p.fuse_tail;
  }
  __syncthreads();
  int nw = min((int)(blockDim.x >> 5), kTailMaxWarps);
  nw = min(nw, (int)(scratch_bytes / kTailWarpBytes));
  lm_head_tail_rows(s_tail, scratch, nw);
  __syncthreads();
  dbg_stamp(p, 4);
  if (threadIdx.x == 0) {  // ready for the next launch on this handle
    if (p.tile_counter) *p.tile_counter = 0u;
    __threadfence();
    *p.ticket = 0u;
  }
}

}  // namespace vqk
