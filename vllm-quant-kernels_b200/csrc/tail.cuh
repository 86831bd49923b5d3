// Sampler tail of the decode-sized lm_head kernels: the LAST CTA of the grid to finish (an atomic
// ticket; nobody waits for anybody) turns the per-slice results every CTA left in memory into
// the step's tokens, one warp per batch row, while those results are still in L2.
//
// Per (row, slice) the epilogues leave
//   * part_score / part_token   Gumbel (or greedy) winner of the slice, for rows without top-k / top-p;
//   * slice_max and a list of the kListLen largest logits of the slice (the first kListM with
//     their token ids), for rows with top-k.  The last list entry is the WITNESS: every logit of
//     the slice that is not in the list is <= it.  Layout: list_v [row][position][slice],
//     list_t [row][position][slice], so the tail reads runs of consecutive words.
// A top-k row is resolved from the lists alone when they prove to hold every logit >= the k-th
// largest of the row: t_k = k-th largest of the listed values, and every witness of a slice that
// could matter is < t_k.  Then top-k (ties kept), top-p and the Gumbel argmax run on those few
// values with the arithmetic of resolve_candidates in sampler.cu (same tokens, same scores).  A
// row the lists cannot prove (more than kListM of the top k in one slice, top-p without top-k, a
// threshold row with top-p, k > kTailMaxK) gets row_flag = 1 and is resolved from its fp16 logits
// row by the full-row kernel (k_select), which is launched behind every step and returns at once
// for rows whose flag is 0.
//
// The warp keeps its working sets in registers (a row's slice heads, the staged list entries, the
// union of the shards' candidates) and fetches them with unrolled batches of independent loads:
// the tail is a chain of L2 latencies, not of instructions.  All logits on this path are fp16
// values, so their order is the order of 16-bit keys.
#pragma once

#include "lm_head.cuh"
#include "peer_exchange.cuh"

namespace vqk {

constexpr int kTailMaxSlices = 1024;  // slices per row the tail can take (148 SMs x 4 = 592)
constexpr int kTailHeadRegs = kTailMaxSlices / 32;
constexpr int kTailMaxK = 126;        // largest top-k resolved from the lists (a shard record holds as many)
constexpr int kTailSliceCap = 160;    // slices whose head can reach the k-th largest (k + ties)
constexpr int kTailStageCap = kTailSliceCap * kListM;
constexpr int kTailStageRegs = kTailStageCap / 32;
constexpr int kTailSurvCap = 192;     // survivors of top-k (k + ties) resolved per row
constexpr int kTailSurvRegs = kTailSurvCap / 32;
constexpr int kTailMaxWarps = 16;
constexpr int kMergeRegs = (kMergeCap + 31) / 32;

// Per-warp scratch (bytes).  Region A holds the slice ids and staged list entries while a row is
// resolved from the lists, and afterwards the union of the shards' candidates (mv, mt); the
// survivors (cv, ct) follow it.
constexpr int kTailOffSlices = 0;                                   // uint16 [kTailSliceCap]
constexpr int kTailOffStage = kTailOffSlices + kTailSliceCap * 2;    // uint32 [kTailStageCap]: key << 16 | entry index
constexpr int kTailOffMv = 0;                                       // float  [kMergeCap]
constexpr int kTailOffMt = kTailOffMv + kMergeCap * 4;              // int    [kMergeCap]
constexpr int kTailRegionA = kTailOffMt + kMergeCap * 4;
static_assert(kTailOffStage + kTailStageCap * 4 <= kTailRegionA, "list staging fits region A");
constexpr int kTailOffCv = kTailRegionA;                            // float  [kTailSurvCap]
constexpr int kTailOffCt = kTailOffCv + kTailSurvCap * 4;           // int    [kTailSurvCap]
constexpr int kTailWarpBytes = (kTailOffCt + kTailSurvCap * 4 + 15) & ~15;

// shared memory the tail wants from a CTA of `warps` warps (it makes do with less: fewer rows at a time)
__host__ __device__ inline size_t tail_smem_bytes(int warps) {
  return (size_t)(warps < kTailMaxWarps ? warps : kTailMaxWarps) * kTailWarpBytes;
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
constexpr uint32_t kKeyLowestFinite = 0x0400u;  // key(-65504); key(-inf) = 0x03ff sorts below

// k-th largest of the keys a warp holds in registers, key[j] of lane l being element j * 32 + l
// (unused slots hold a key below every candidate), by bisection on the key bits `hi` down to
// `lo`: the largest x with count(key >= x) >= k.  Result in every lane.
template <int R>
__device__ __forceinline__ uint32_t warp_kth_largest_reg(const uint32_t (&key)[R], int used, int k, int hi, int lo) {
  uint32_t prefix = 0;
#pragma unroll 1
  for (int bit = hi; bit >= lo; --bit) {
    const uint32_t cand = prefix | (1u << bit);
    int c = 0;
#pragma unroll
    for (int j = 0; j < R; ++j)
      if (j < used) c += (key[j] >= cand);
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
__device__ inline int warp_topk_inplace(float* v, int* t, int n, int K, int lane) {
  if (K <= 0 || n <= K) return n;
  uint32_t key[kMergeRegs];
  const int used = (n + 31) >> 5;
  int low = 1;
#pragma unroll
  for (int j = 0; j < kMergeRegs; ++j) {
    key[j] = 0;
    if (j < used && j * 32 + lane < n) {
      const float x = v[j * 32 + lane];
      key[j] = f32_key(x);
      low &= ((__float_as_uint(x) & 0x1fffu) == 0);
    }
  }
  // fp16-representable values (every logit of the lm_head path) differ in the upper 19 key bits only
  low = __all_sync(0xffffffffu, low);
  const uint32_t tk = warp_kth_largest_reg(key, used, K, 31, low ? 13 : 0);
  const unsigned lt = (1u << lane) - 1u;
  int kept = 0;
#pragma unroll 1
  for (int j = 0; j < used; ++j) {
    const int i = j * 32 + lane;
    float vi = 0.f;
    int ti = 0;
    bool keep = false;
    if (i < n) { vi = v[i]; ti = t[i]; keep = f32_key(vi) >= tk; }
    const unsigned mask = __ballot_sync(0xffffffffu, keep);  // every lane has read before anyone writes
    if (keep) { const int pos = kept + __popc(mask & lt); v[pos] = vi; t[pos] = ti; }
    kept += __popc(mask);
    __syncwarp();
  }
  return kept;
}

// Top-p over the n <= kTailSurvCap top-k survivors (shared memory), then the Gumbel argmax: the
// arithmetic of resolve_candidates (sampler.cu), so both paths pick the same token with the same
// score.  The survivors sit in registers; the mass above each one is summed over shuffles.
__device__ inline void warp_topp_gumbel(const float* cv, const int* ct, int n, const RowMeta& m, int lane, float& s,
                                        int& t) {
  float y[kTailSurvRegs];
  int tok[kTailSurvRegs];
  bool alive[kTailSurvRegs];
  const int used = (n + 31) >> 5;
#pragma unroll
  for (int j = 0; j < kTailSurvRegs; ++j) {
    const int i = j * 32 + lane;
    alive[j] = j < used && i < n;
    y[j] = alive[j] ? cv[i] / m.T : -INFINITY;
    tok[j] = alive[j] ? ct[i] : 0x7fffffff;
  }
  if (m.top_p < 1.f) {
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kTailSurvRegs; ++j) mx = fmaxf(mx, y[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    unsigned long long w[kTailSurvRegs], above[kTailSurvRegs];
    unsigned long long z = 0;
#pragma unroll
    for (int j = 0; j < kTailSurvRegs; ++j) {
      w[j] = alive[j] ? (unsigned long long)((double)expf(y[j] - mx) * 1099511627776.0) : 0ull;
      above[j] = 0ull;
      z += w[j];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
    const double target = (double)m.top_p * (double)z;
#pragma unroll
    for (int jj = 0; jj < kTailSurvRegs; ++jj) {
      if (jj < used) {
#pragma unroll 4
        for (int src = 0; src < 32; ++src) {
          const float yj = __shfl_sync(0xffffffffu, y[jj], src);
          const unsigned long long wj = __shfl_sync(0xffffffffu, w[jj], src);
#pragma unroll
          for (int j = 0; j < kTailSurvRegs; ++j)
            if (yj > y[j]) above[j] += wj;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kTailSurvRegs; ++j)
      if (alive[j] && !((double)above[j] < target)) alive[j] = false;
  }
  s = -INFINITY;
  t = 0x7fffffff;
#pragma unroll
  for (int j = 0; j < kTailSurvRegs; ++j) {
    if (j < used && alive[j]) {
      const float sc = y[j] + gumbel_noise(m.seed, (uint32_t)tok[j]);
      if (better(sc, tok[j], s, t)) { s = sc; t = tok[j]; }
    }
  }
  warp_best_pair(s, t);
}

// Sharded step: exchange this rank's record of row b and merge the shards.  Whole warp; writes the
// row's token / score.  `scratch` is the warp's scratch (region A is overwritten).
template <typename CandAt>
__device__ inline void tail_exchange_row(const PeerTable& pt, const RowMeta& m, int b, float score, int token, int n,
                                         int flags, CandAt cand, uint8_t* scratch, int lane, long long* tokens,
                                         float* scores) {
  float* mv = reinterpret_cast<float*>(scratch + kTailOffMv);
  int* mt = reinterpret_cast<int*>(scratch + kTailOffMt);
  const PeerRowResult r = peer_exchange_row(pt, b, score, token, n, flags, cand, mv, mt, lane);
  float s = -INFINITY;
  int t = -1;
  if (!r.late && !r.bad) {
    if (r.total == 0) {
      s = r.best_s;
      t = r.best_t;
    } else {
      __syncwarp();
      const int kept = warp_topk_inplace(mv, mt, r.total, m.top_k, lane);
      if (kept <= kTailSurvCap) warp_topp_gumbel(mv, mt, kept, m, lane, s, t);
    }
  }
  if (lane == 0) {
    tokens[b] = t;
    if (scores) scores[b] = s;
  }
  __syncwarp();
}

// One row, one warp.  Returns false when the row has to go to the full-row kernel.
__device__ inline bool tail_resolve_row(const LmHeadParams& p, int b, uint8_t* scratch, int lane) {
  const RowMeta m = decode_row(p.sp, b);
  const int nsl = p.nslices;
  const long long voff = p.sp.vocab_offset;
  const bool exchange = p.peer.G > 0;
  const unsigned lt = (1u << lane) - 1u;
  if (!(m.flags & ROW_CAND)) {
    // per-slice winners -> row winner (the same merge k_select does for these rows)
    float s = -INFINITY;
    int t = 0x7fffffff;
    for (int i = lane; i < nsl; i += 32) {
      const float s2 = __ldcg(p.part_score + (long long)b * nsl + i);
      const int t2 = __ldcg(p.part_token + (long long)b * nsl + i);
      if (better(s2, t2, s, t)) { s = s2; t = t2; }
    }
    warp_best_pair(s, t);
    const long long tok = (long long)t + voff;
    if (exchange) {
      tail_exchange_row(p.peer, m, b, s, (int)tok, 0, 0, [](int) { return Cand{0.f, 0}; }, scratch, lane, p.tokens, p.scores);
    } else if (lane == 0) {
      tail_write_header(p.records, b, s, (int)tok, 0, 0);
      if (p.tokens) p.tokens[b] = tok;
      if (p.scores) p.scores[b] = s;
    }
    return true;
  }
  if (!p.list_v || m.top_k <= 0 || m.top_k > kTailMaxK || nsl > kTailMaxSlices) return false;

  uint16_t* sl = reinterpret_cast<uint16_t*>(scratch + kTailOffSlices);
  uint32_t* st = reinterpret_cast<uint32_t*>(scratch + kTailOffStage);
  float* cv = reinterpret_cast<float*>(scratch + kTailOffCv);
  int* ct = reinterpret_cast<int*>(scratch + kTailOffCt);
  const int K = m.top_k;
  const float* lv = p.list_v + (long long)b * kListLen * nsl;  // [position][slice]
  const int* ltok = p.list_t + (long long)b * kListM * nsl;

  // 1. slice heads (= list position 0) -> keys in registers, one batch of independent loads
  uint32_t hk[kTailHeadRegs];
  const int hused = (nsl + 31) >> 5;
  int nfin = 0;
#pragma unroll
  for (int j = 0; j < kTailHeadRegs; ++j) {
    float v = -INFINITY;
    if (j < hused && j * 32 + lane < nsl) v = __ldcg(lv + j * 32 + lane);
    hk[j] = h16_key(v);
    nfin += (hk[j] >= kKeyLowestFinite);
  }
  nfin = __reduce_add_sync(0xffffffffu, nfin);
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 5] = t_; }
  // 2. tau0 = K-th largest head: K slices hold a value >= it, so the K-th largest logit is >= it
  uint32_t tau0 = kKeyLowestFinite;
  if (nfin >= K) tau0 = warp_kth_largest_reg(hk, hused, K, 15, 0);
  if (tau0 < kKeyLowestFinite) tau0 = kKeyLowestFinite;
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 6] = t_; }
  // 3. the slices that can hold a logit >= tau0
  int ns = 0;
#pragma unroll
  for (int j = 0; j < kTailHeadRegs; ++j) {
    if (j < hused) {
      const bool hit = hk[j] >= tau0;  // unused slots hold key(-inf)
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      const int pos = ns + __popc(mask & lt);
      if (hit && pos < kTailSliceCap) sl[pos] = (uint16_t)(j * 32 + lane);
      ns += __popc(mask);
    }
  }
  if (ns > kTailSliceCap) return false;
  __syncwarp();
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 7] = t_; }
  // 4. their list entries, eight independent loads per lane at a time: values >= tau0 are staged as
  //    (key, entry index = slice slot * kListLen + position); witnesses are folded to a maximum
  const int nent = ns * kListLen;
  int ne = 0;
  uint32_t wkey = 0;
#pragma unroll 1
  for (int base = 0; base < nent; base += 256) {
    float v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = base + r * 32 + lane;
      v[r] = -INFINITY;
      if (i < nent) v[r] = __ldcg(lv + (i % kListLen) * nsl + (int)sl[i / kListLen]);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = base + r * 32 + lane;
      if (base + r * 32 < nent) {  // uniform
        const uint32_t k = h16_key(v[r]);
        const bool wit = i < nent && (i % kListLen) == kListM;
        if (wit) wkey = max(wkey, k);
        const bool take = i < nent && !wit && k >= tau0;
        const unsigned mask = __ballot_sync(0xffffffffu, take);
        if (take) st[ne + __popc(mask & lt)] = (k << 16) | (uint32_t)i;
        ne += __popc(mask);
      }
    }
  }
  wkey = __reduce_max_sync(0xffffffffu, wkey);
  __syncwarp();
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 8] = t_; }
  // 5. t_k: the K-th largest staged value (every staged value survives when fewer than K exist)
  uint32_t sk[kTailStageRegs];
  const int sused = (ne + 31) >> 5;
#pragma unroll
  for (int j = 0; j < kTailStageRegs; ++j) {
    sk[j] = 0;
    if (j < sused && j * 32 + lane < ne) sk[j] = st[j * 32 + lane];
  }
  uint32_t tk = kKeyLowestFinite;
  if (ne >= K) {
    uint32_t kk[kTailStageRegs];
#pragma unroll
    for (int j = 0; j < kTailStageRegs; ++j) kk[j] = sk[j] >> 16;
    tk = warp_kth_largest_reg(kk, sused, K, 15, 0);
  }
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 9] = t_; }
  // 6. the proof: no slice we looked at hides a value >= t_k (slices we skipped have head < tau0 <= t_k)
  if (wkey >= tk) return false;
  // 7. survivors (>= t_k, ties kept), with their GLOBAL token ids
  int nsv = 0;
#pragma unroll
  for (int j = 0; j < kTailStageRegs; ++j) {
    if (j < sused) {
      const bool keep = (sk[j] >> 16) >= tk && sk[j] != 0;
      const unsigned mask = __ballot_sync(0xffffffffu, keep);
      const int pos = nsv + __popc(mask & lt);
      if (keep && pos < kTailSurvCap) {
        const uint32_t e = sk[j] & 0xffffu;
        cv[pos] = h16_key_to_float(sk[j] >> 16);
        ct[pos] = (int)((long long)__ldcg(ltok + (e % kListLen) * nsl + (int)sl[e / kListLen]) + voff);
      }
      nsv += __popc(mask);
    }
  }
  if (nsv > kTailSurvCap) return false;
  __syncwarp();
  if (exchange) {
    if (nsv > VQK_RECORD_CAP) return false;  // the full-row kernel reports the overflow
    tail_exchange_row(p.peer, m, b, -INFINITY, -1, nsv, 0, [&](int i) { return Cand{cv[i], ct[i]}; }, scratch, lane,
                      p.tokens, p.scores);
    return true;
  }
  if (p.records) {  // shard record: the local top-k survivors; top-p needs the union of the shards
    Cand* out = reinterpret_cast<Cand*>(p.records + (size_t)b * VQK_RECORD_BYTES + sizeof(RecordHeader));
    for (int i = lane; i < nsv && i < VQK_RECORD_CAP; i += 32) out[i] = Cand{cv[i], ct[i]};
    if (lane == 0)
      tail_write_header(p.records, b, -INFINITY, -1, min(nsv, VQK_RECORD_CAP), nsv > VQK_RECORD_CAP ? VQK_RECORD_FLAG_OVERFLOW : 0);
  }
  if (!p.single_shard) return true;
  if (b == 0 && lane == 0 && p.dbg) { unsigned long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); p.dbg[(size_t)blockIdx.x * 16 + 10] = t_; }
  // 8. top-p over the survivors, then the Gumbel argmax
  float s;
  int t;
  warp_topp_gumbel(cv, ct, nsv, m, lane, s, t);
  if (lane == 0) {
    if (p.tokens) p.tokens[b] = t;
    if (p.scores) p.scores[b] = s;
  }
  return true;
}

// Called by every thread of every CTA once its slice results are written.  `scratch` is shared
// memory of the CTA that is no longer in use, `scratch_bytes` of it (at least kTailWarpBytes).
__device__ inline void lm_head_tail(const LmHeadParams& p, uint8_t* scratch, size_t scratch_bytes) {
  __shared__ int s_last;
  __threadfence();  // this thread's slice results are visible device-wide before the ticket is taken
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(p.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  dbg_stamp(p, 3);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int nw = min((int)(blockDim.x >> 5), kTailMaxWarps);
  nw = min(nw, (int)(scratch_bytes / kTailWarpBytes));
  if (warp < nw) {
    uint8_t* mine = scratch + (size_t)warp * kTailWarpBytes;
    for (int b = warp; b < p.B; b += nw) {
      const bool done = p.fuse_tail == 1 && tail_resolve_row(p, b, mine, lane);  // 2: every row to the full-row kernel (A/B runs)
      if (lane == 0) p.row_flag[b] = done ? 0 : 1;
      __syncwarp();
    }
  }
  __syncthreads();
  dbg_stamp(p, 4);
  if (threadIdx.x == 0) *p.ticket = 0u;  // ready for the next launch on this handle
}

// ---- sorted lists of the largest logits ------------------------------------------------------------
// `e` holds n entries in descending order of value; (v, t) goes in if v > e[n-1].v, the last falls out.
__device__ __forceinline__ void list_insert(Cand* e, int n, float v, int t) {
  if (!(v > e[n - 1].v)) return;
  int i = n - 1;
  while (i > 0 && v > e[i - 1].v) { e[i] = e[i - 1]; --i; }
  e[i] = Cand{v, t};
}

}  // namespace vqk
