// Record exchange between the vocab shards of one node over NVLink peer memory, one warp per
// batch row, callable from the tail of the lm_head kernels, from the full-row sampler kernel and
// from a kernel of its own.
//
// Every rank owns a landing buffer [2 parities][G source ranks][max_rows][kWireWords] of 64-bit
// words, zero when idle, mapped by its peers through CUDA IPC.  A row's record travels as
//   word 0      score bits | (0x80000000 | n << 8 | flags) << 32
//   word 1      token      | 1 << 63
//   word 2 + i  candidate i: raw-logit bits | (global token | 0x80000000) << 32
// Every word is non-zero and is written with ONE 8-byte store, so a word that reads non-zero is
// complete: there is no separate flag and no fence between payload and flag.  The warp of row b
// stores its rank's words into slot [parity][rank][b] of EVERY rank's buffer (plain peer stores,
// no multicast, no remote loads), then polls (bounded) the G slots of its own buffer, merges what
// it read, and zeroes the words it consumed.  The parity is the low bit of a per-row step counter
// in device memory, so a CUDA-graph replay advances it.  Two parities suffice: a rank writes a
// row's slot for step t + 2 only after it has read every peer's record of step t + 1, which a
// peer sends after it has consumed and cleared step t.
// All ranks must run the same sequence of steps with the same batch size.
#pragma once

#include "lm_head.cuh"

namespace vqk {

constexpr int kWireWords = 2 + VQK_RECORD_CAP;  // 1 KiB per (rank, row)
constexpr int kMergeCap = VQK_PEER_MAX_RANKS * VQK_RECORD_CAP;

__device__ __forceinline__ void st_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// bounded poll of one landing word; 0 = gave up
__device__ __forceinline__ unsigned long long peer_wait_word(const unsigned long long* p, unsigned int limit) {
  for (unsigned int it = 0; it < limit; ++it) {
    const unsigned long long v = ld_sys_u64(p);
    if (v) return v;
    if (it > 64) __nanosleep(it < 4096 ? 32 : 256);
  }
  return 0ull;
}

struct PeerRowResult {
  int total;     // candidates read into mv / mt (all ranks together)
  int bad;       // a record carried a flag, or the union does not fit: the row cannot be merged here
  int late;      // a peer's record never arrived
  float best_s;  // best (score, token) among the ranks' winners, for rows without candidates
  int best_t;
};

// One row, one warp.  This rank's record is (score, token, n, flags) with candidate i = cand(i)
// (raw logit, GLOBAL token).  The union of all ranks' candidates lands in mv / mt (kMergeCap each).
// `step`: this step's number for the row (the stored counter + 1) when the caller fetched the
// counter ahead of time, 0 to fetch it here.
template <typename CandAt>
__device__ inline PeerRowResult peer_exchange_row(const PeerTable& pt, int b, float score, int token, int n, int flags,
                                                  CandAt cand, float* mv, int* mt, int lane, unsigned int step = 0) {
  const int G = pt.G;
  if (lane == 0) {
    if (step == 0) step = pt.steps[b] + 1u;
    if (step == 0) step = 2u;  // the counter wrapped: keep the parity sequence, skip the reserved 0
    pt.steps[b] = step;
  }
  step = __shfl_sync(0xffffffffu, step, 0);
  const size_t parity_off = (size_t)(step & 1u) * G;
  // ---- push: this rank's words into every rank's buffer ------------------------------------------
  const size_t my_slot = ((parity_off + pt.rank) * pt.max_rows + b) * kWireWords;
  const int words = n + 2;
  for (int idx = lane; idx < G * words; idx += 32) {
    const int g = idx / words, i = idx % words;
    unsigned long long w;
    if (i == 0) w = (unsigned long long)__float_as_uint(score) | ((unsigned long long)(0x80000000u | ((unsigned)n << 8) | (unsigned)(flags & 0xff)) << 32);
    else if (i == 1) w = (unsigned long long)(unsigned int)token | (1ull << 63);
    else {
      const Cand c = cand(i - 2);
      w = (unsigned long long)__float_as_uint(c.v) | ((unsigned long long)((unsigned int)c.t | 0x80000000u) << 32);
    }
    st_sys_u64(pt.land[g] + my_slot + i, w);
  }
  // ---- wait for the G headers in the own buffer ----------------------------------------------------
  PeerRowResult r{};
  r.best_s = -INFINITY;
  r.best_t = 0x7fffffff;
  const unsigned long long* mine = pt.land[pt.rank];
  int ng = 0, fl = 0, late = 0;
  float sc = -INFINITY;
  int tk = 0x7fffffff;
  if (lane < G) {
    const unsigned long long* slot = mine + ((parity_off + lane) * pt.max_rows + b) * kWireWords;
    // both header words in flight at once; the bounded wait only for what has not landed yet
    unsigned long long w0 = ld_sys_u64(slot), w1 = ld_sys_u64(slot + 1);
    if (!w0) w0 = peer_wait_word(slot, pt.wait_polls);
    if (w0 && !w1) w1 = peer_wait_word(slot + 1, pt.wait_polls);
    if (!w0 || !w1) late = 1;
    else {
      const unsigned int hi = (unsigned int)(w0 >> 32);
      ng = (int)((hi >> 8) & 0xff);
      fl = (int)(hi & 0xff);
      sc = __uint_as_float((unsigned int)w0);
      tk = (int)(unsigned int)w1;
    }
  }
  r.late = __any_sync(0xffffffffu, late);
  if (r.late) {
    if (lane == 0) atomicExch(pt.error, 1);
    return r;
  }
  r.bad = __any_sync(0xffffffffu, fl != 0);
  // exclusive prefix of the candidate counts over the ranks
  int incl = ng;
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const int total = __shfl_sync(0xffffffffu, incl, G - 1);
  r.total = total;
  if (total > kMergeCap) r.bad = 1;
  {  // best winner over the ranks (rows without candidates)
    float s = (lane < G && ng == 0 && fl == 0) ? sc : -INFINITY;
    int t = (lane < G && ng == 0 && fl == 0) ? tk : 0x7fffffff;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
      const float s2 = __shfl_xor_sync(0xffffffffu, s, o);
      const int t2 = __shfl_xor_sync(0xffffffffu, t, o);
      if (better(s2, t2, s, t)) { s = s2; t = t2; }
    }
    r.best_s = __shfl_sync(0xffffffffu, s, 0);
    r.best_t = __shfl_sync(0xffffffffu, t, 0);
  }
  // ---- candidates of every rank ----------------------------------------------------------------------
  // A lane takes words lane, lane + 32, ... of every rank's list.  A rank's four loads are put in flight
  // together (each is an L2 round trip for this lone warp; one after the other they cost 0.7 us
  // apiece, 11 us at eight ranks); the bounded wait is only for words that have not landed yet.
  constexpr int kPer = (VQK_RECORD_CAP + 31) / 32;  // words per lane and rank at most
  constexpr int kFly = 4;                           // loads in flight together (a rank's worth)
  for (int t0 = 0; t0 < G * kPer; t0 += kFly) {
    unsigned long long w[kFly];
#pragma unroll
    for (int u = 0; u < kFly; ++u) {
      const int t = t0 + u, g = t / kPer, i = lane + 32 * (t % kPer);
      const int cnt = __shfl_sync(0xffffffffu, ng, g & 31);
      w[u] = 1ull;
      if (g < G && i < cnt) w[u] = ld_sys_u64(mine + ((parity_off + g) * pt.max_rows + b) * kWireWords + 2 + i);
    }
#pragma unroll
    for (int u = 0; u < kFly; ++u) {
      const int t = t0 + u, g = t / kPer, i = lane + 32 * (t % kPer);
      const int cnt = __shfl_sync(0xffffffffu, ng, g & 31);
      const int base = __shfl_sync(0xffffffffu, incl - ng, g & 31);
      if (g < G && i < cnt) {
        if (!w[u]) w[u] = peer_wait_word(mine + ((parity_off + g) * pt.max_rows + b) * kWireWords + 2 + i, pt.wait_polls);
        if (!w[u]) late = 1;
        else if (!r.bad) {
          mv[base + i] = __uint_as_float((unsigned int)w[u]);
          mt[base + i] = (int)((unsigned int)(w[u] >> 32) & 0x7fffffffu);
        }
      }
    }
  }
  r.late = __any_sync(0xffffffffu, late);
  if (r.late) {
    if (lane == 0) atomicExch(pt.error, 1);
    return r;
  }
  // ---- hand the slots back: zero what was read ---------------------------------------------------------
  for (int g = 0; g < G; ++g) {
    const int cnt = __shfl_sync(0xffffffffu, ng, g) + 2;
    unsigned long long* slot = const_cast<unsigned long long*>(mine) + ((parity_off + g) * pt.max_rows + b) * kWireWords;
    for (int i = lane; i < cnt; i += 32) slot[i] = 0ull;
  }
  // (no fence: a peer writes these words again only after it has read this rank's record of the NEXT
  // step, which a later launch sends; the end of this launch puts the zeroes in memory before that)
  __syncwarp();
  return r;
}

}  // namespace vqk
