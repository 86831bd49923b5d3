// Fused sampler: temperature, top-k, top-p and the Gumbel (exponential-race) argmax.
//
// Pass 1 (here k_slice_pass, or the lm_head epilogue) reduces every 256-column slice of a row
// to either a Gumbel winner (rows without top-k/top-p) or its maximum raw logit (rows with).
// Pass 2 (k_select, a cluster of 1 to 8 CTAs per row) turns the slice maxima into a lower bound tau
// on the k-th largest logit (the k-th largest slice maximum: k disjoint slices each hold a
// value >= it; the exact k-th largest logit when fewer than k slices hold data), re-reads the
// row, keeps the few columns >= tau, and resolves them exactly:
// top-k with ties kept (>=, as _sampler_kernels.py:88-90), vLLM's top-p, Philox noise only
// for the survivors.  Rows that do not fit (top-p without top-k, more ties than the candidate
// buffer) go through fullrow_resolve, an exact radix-select pass over the whole row.
#include <cooperative_groups.h>

#include <mutex>

#include "lm_head.cuh"
#include "tail.cuh"

namespace cg = cooperative_groups;

namespace vqk {

constexpr int kClusterSize = 8;
constexpr int kMaxSlices = 2048;
constexpr int kGlobalCap = 1024;  // candidates resolved per row
constexpr double kMassScale = 1099511627776.0;  // 2^40 fixed point for probability mass

// ---- small block-level helpers ------------------------------------------------------------
struct Best {
  float s;
  int t;
};

__device__ __forceinline__ Best warp_best(Best b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float s2 = __shfl_xor_sync(0xffffffffu, b.s, o);
    int t2 = __shfl_xor_sync(0xffffffffu, b.t, o);
    if (better(s2, t2, b.s, b.t)) { b.s = s2; b.t = t2; }
  }
  return b;
}

// all threads of the block must call; result valid in every thread
__device__ Best block_best(Best b, Best* red /* >= 32 */) {
  b = warp_best(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = b;
  __syncthreads();
  Best r = (l < nw) ? red[l] : Best{-INFINITY, 0x7fffffff};
  r = warp_best(r);
  return r;
}

__device__ float block_maxf(float v, float* red /* >= 32 */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  v = (l < nw) ? red[l] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T>
__device__ __forceinline__ float ldl(const T* row, int col) { return to_f32<T>(row[col]); }

__device__ __forceinline__ unsigned long long mass_of(float y, float m) {
  return (unsigned long long)((double)expf(y - m) * kMassScale);
}

// ---- pass 1 over materialised logits --------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) k_slice_pass(const T* __restrict__ logits, long long ld, int V, SampleDev sp,
                                                   float* __restrict__ slice_max, float* __restrict__ part_score,
                                                   int* __restrict__ part_token, int nslices, float* __restrict__ lp_max,
                                                   float* __restrict__ lp_sum) {
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const int slice = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (slice >= nslices) return;
  const RowMeta m = decode_row(sp, b);
  const T* row = logits + (long long)b * ld;
  const int c0 = slice * 256;
  float mx = -INFINITY;
  Best best{-INFINITY, 0x7fffffff};
  float lv[8];  // the lane's logits, kept for the sum of exponentials (log-probability requested)
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int col = c0 + j * 32 + lane;
    lv[j] = -INFINITY;
    if (col < V) {
      const float l = ldl(row, col);
      lv[j] = l;
      if (m.flags & ROW_CAND) {
        mx = fmaxf(mx, l);
      } else {
        float sc = l;
        if (!(m.flags & ROW_GREEDY)) {
          sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(col + sp.vocab_offset));
          if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
        }
        if (better(sc, col, best.s, best.t)) { best.s = sc; best.t = col; }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  best = warp_best(best);
  if (lane == 0) {
    slice_max[(long long)b * nslices + slice] = mx;
    part_score[(long long)b * nslices + slice] = best.s;
    part_token[(long long)b * nslices + slice] = best.t;
  }
  if (lp_max) {  // per-slice maximum and sum of exp(logit - maximum) of EVERY row kind, for the log-softmax
    float am = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, lv[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    float se = 0.f;
    if (am > -INFINITY) {
#pragma unroll
      for (int j = 0; j < 8; ++j) se += expf(lv[j] - am);  // exp(-inf) = 0 for the lanes beyond the row
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    if (lane == 0) {
      lp_max[(long long)b * nslices + slice] = am;
      lp_sum[(long long)b * nslices + slice] = se;
    }
  }
}

// log-softmax of the sampled token of every row: logit[token] - M - log(sum_s sum_s * exp(max_s - M)), one warp per row
template <typename T>
__global__ void __launch_bounds__(32) k_logprob(const T* __restrict__ logits, long long ld, int V, const float* __restrict__ lp_max,
                                                const float* __restrict__ lp_sum, int nslices,
                                                const long long* __restrict__ tokens, float* __restrict__ logprobs) {
  const int b = blockIdx.x, lane = threadIdx.x;
  float M = -INFINITY;
  for (int s = lane; s < nslices; s += 32) M = fmaxf(M, lp_max[(long long)b * nslices + s]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float z = 0.f;
  for (int s = lane; s < nslices; s += 32) {
    const float ms = lp_max[(long long)b * nslices + s];
    if (ms > -INFINITY) z += lp_sum[(long long)b * nslices + s] * expf(ms - M);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
  if (lane == 0) {
    const long long t = tokens[b];
    float lp = -INFINITY;
    if (t >= 0 && t < V && M > -INFINITY) lp = ldl(logits + (long long)b * ld, (int)t) - M - logf(z);
    logprobs[b] = lp;
  }
}

// ---- exact resolution of a small candidate set (one block) ------------------------------------
// cv/ct: candidate raw logits and GLOBAL token ids in shared memory; work arrays sized n.
// Returns the winner in every thread.  Must be called by all threads of the block.
__device__ Best resolve_candidates(const float* cv, const int* ct, int n, const RowMeta& m, float* y,
                                   unsigned long long* w, unsigned char* alive, Best* red_b, float* red_f,
                                   unsigned long long* zsum) {
  const int tid = threadIdx.x, nt = blockDim.x;
  // top-k with ties: alive iff fewer than k candidates are strictly larger
  for (int i = tid; i < n; i += nt) {
    bool a = true;
    if (m.top_k > 0) {
      const float vi = cv[i];
      int gcount = 0;
      for (int j = 0; j < n; ++j) gcount += (cv[j] > vi);
      a = gcount < m.top_k;
    } else if (m.flags & ROW_MASK_THR) {
      a = cv[i] >= m.thr;
    }
    alive[i] = a;
    y[i] = cv[i] / m.T;
  }
  __syncthreads();
  if (m.top_p < 1.f) {
    float mx = -INFINITY;
    for (int i = tid; i < n; i += nt)
      if (alive[i]) mx = fmaxf(mx, y[i]);
    mx = block_maxf(mx, red_f);
    if (tid == 0) *zsum = 0ull;
    __syncthreads();
    unsigned long long loc = 0;
    for (int i = tid; i < n; i += nt) {
      unsigned long long wi = alive[i] ? mass_of(y[i], mx) : 0ull;
      w[i] = wi;
      loc += wi;
    }
    atomicAdd(zsum, loc);
    __syncthreads();
    const double target = (double)m.top_p * (double)(*zsum);
    __syncthreads();
    // keep iff the mass strictly above is < p * Z (vLLM: drop while ascending cumsum <= 1 - p)
    for (int i = tid; i < n; i += nt) {
      if (!alive[i]) continue;
      const float yi = y[i];
      unsigned long long above = 0;
      for (int j = 0; j < n; ++j)
        if (alive[j] && y[j] > yi) above += w[j];
      if (!((double)above < target)) alive[i] = 2;  // dropped; stays non-zero while others still read it
    }
    __syncthreads();
    for (int i = tid; i < n; i += nt)
      if (alive[i] == 2) alive[i] = 0;
    __syncthreads();
  }
  Best best{-INFINITY, 0x7fffffff};
  for (int i = tid; i < n; i += nt) {
    if (!alive[i]) continue;
    const float sc = y[i] + gumbel_noise(m.seed, (uint32_t)ct[i]);
    if (better(sc, ct[i], best.s, best.t)) { best.s = sc; best.t = ct[i]; }
  }
  return block_best(best, red_b);
}

__device__ __forceinline__ void write_header(uint8_t* records, int b, float score, int token, int n, int flags) {
  if (!records) return;
  RecordHeader* h = reinterpret_cast<RecordHeader*>(records + (size_t)b * VQK_RECORD_BYTES);
  h->score = score; h->token = token; h->n = n; h->flags = flags;
}

// ---- exact full-row pass ---------------------------------------------------------------------------
// k-th largest raw logit of a row by 8-bit MSB radix select on order-preserving keys.
template <typename T>
__device__ float radix_kth_largest(const T* row, int V, int k, unsigned int* hist /* 256 */, unsigned int* bcast /* 2 */) {
  uint32_t prefix = 0, mask = 0;
  int kk = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int col = threadIdx.x; col < V; col += blockDim.x) {
      const uint32_t key = f32_key(ldl(row, col));
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned int cum = 0;
      int bin = 255;
      for (; bin > 0; --bin) {
        if (cum + hist[bin] >= (unsigned)kk) break;
        cum += hist[bin];
      }
      bcast[0] = (unsigned)bin;
      bcast[1] = cum;
    }
    __syncthreads();
    prefix |= bcast[0] << shift;
    mask |= 0xffu << shift;
    kk -= (int)bcast[1];
    __syncthreads();
  }
  return key_f32(prefix);
}

// Scratch of the full-row pass (shared memory of the calling block)
struct FullRowScratch {
  unsigned int hist[256];
  unsigned long long mass[256];
  unsigned int bc[2];
  unsigned long long z, above;
  Best redb[32];
  float redf[32];
};

// Exact sampler for one row by passes over the whole row: radix select of the k-th largest
// raw logit, probability-mass radix select of the nucleus cut, then the Gumbel argmax over
// the survivors.  Called by every thread of a block; the winner is returned in every thread.
template <typename T>
__device__ Best fullrow_resolve(const T* row, int V, const RowMeta& m, long long vocab_offset, FullRowScratch& S) {
  const int tid = threadIdx.x;
  unsigned int* s_hist = S.hist;
  unsigned long long* s_mass = S.mass;
  unsigned int* s_bc = S.bc;
  unsigned long long& s_z = S.z;
  unsigned long long& s_above = S.above;
  Best* s_redb = S.redb;
  float* s_redf = S.redf;

  float thr = -INFINITY;
  if (m.top_k > 0) thr = radix_kth_largest(row, V, m.top_k, s_hist, s_bc);
  else if (m.flags & ROW_MASK_THR) thr = m.thr;

  uint32_t cut = 0;  // smallest surviving key of y; 0 keeps everything
  if (m.top_p < 1.f) {
    float mx = -INFINITY;
    for (int col = tid; col < V; col += blockDim.x) {
      const float l = ldl(row, col);
      if (l >= thr) mx = fmaxf(mx, l / m.T);
    }
    mx = block_maxf(mx, s_redf);
    if (tid == 0) { s_z = 0ull; s_above = 0ull; }
    __syncthreads();
    unsigned long long loc = 0;
    for (int col = tid; col < V; col += blockDim.x) {
      const float l = ldl(row, col);
      if (l >= thr) loc += mass_of(l / m.T, mx);
    }
    atomicAdd(&s_z, loc);
    __syncthreads();
    const double target = (double)m.top_p * (double)s_z;
    uint32_t prefix = 0, mask = 0;
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int i = tid; i < 256; i += blockDim.x) s_mass[i] = 0ull;
      __syncthreads();
      for (int col = tid; col < V; col += blockDim.x) {
        const float l = ldl(row, col);
        if (l >= thr) {
          const float y = l / m.T;
          const uint32_t key = f32_key(y);
          if ((key & mask) == prefix) atomicAdd(&s_mass[(key >> shift) & 0xff], mass_of(y, mx));
        }
      }
      __syncthreads();
      if (tid == 0) {
        unsigned long long cum = s_above;
        int bin = 255;
        for (; bin > 0; --bin) {
          if ((double)(cum + s_mass[bin]) >= target) break;
          cum += s_mass[bin];
        }
        s_bc[0] = (unsigned)bin;
        s_above = cum;
      }
      __syncthreads();
      prefix |= s_bc[0] << shift;
      mask |= 0xffu << shift;
      __syncthreads();
    }
    cut = prefix;
  }

  Best best{-INFINITY, 0x7fffffff};
  for (int col = tid; col < V; col += blockDim.x) {
    const float l = ldl(row, col);
    if (!(l >= thr)) continue;
    const float y = l / m.T;
    if (f32_key(y) < cut) continue;
    const int tok = (int)(col + vocab_offset);
    const float sc = y + gumbel_noise(m.seed, (uint32_t)tok);
    if (better(sc, tok, best.s, best.t)) { best.s = sc; best.t = tok; }
  }
  return block_best(best, s_redb);
}

// k-th largest of n floats in shared memory (n >= k >= 1): 8-bit MSB radix select, one warp
// scans each 256-bin histogram.  Called by the whole block; result in every thread.
__device__ float smem_kth_largest(const float* v, int n, int k, unsigned int* hist /* 256 */, unsigned int* bc /* 2 */) {
  uint32_t prefix = 0, mask = 0;
  int kk = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = f32_key(v[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      unsigned int h[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = hist[lane * 8 + j]; tot += h[j]; }
      // suffix sum over lanes: above = number of keys in bins owned by higher lanes
      unsigned int incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned int t = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += t;
      }
      const unsigned int above = incl - tot;
      if (above < (unsigned)kk && incl >= (unsigned)kk) {  // exactly one lane
        unsigned int cum = above;
        int bin = 7;
        for (; bin > 0; --bin) {
          if (cum + h[bin] >= (unsigned)kk) break;
          cum += h[bin];
        }
        bc[0] = (unsigned)(lane * 8 + bin);
        bc[1] = cum;
      }
    }
    __syncthreads();
    prefix |= bc[0] << shift;
    mask |= 0xffu << shift;
    kk -= (int)bc[1];
    __syncthreads();
  }
  return key_f32(prefix);
}

// Sharded step: the record k_select just wrote for row b travels to every rank and the shards are
// merged, by the first warp of the row's CTA (peer_exchange.cuh).  `buf` is block shared memory of
// at least kTailWarpBytes.
struct SelectExchange {  // in shared memory: what the exchange needs of the kernel's parameters
  PeerTable peer;
  RowMeta m;
  const uint8_t* records;
  long long* tokens;
  float* scores;
};
static __device__ __noinline__ void select_exchange_row(const SelectExchange& x, int b, uint8_t* buf) {
  __syncthreads();  // the record of this row is complete (written by this block), and so is x
  if (threadIdx.x >= 32) return;
  const uint8_t* rec = x.records + (size_t)b * VQK_RECORD_BYTES;
  const RecordHeader h = *reinterpret_cast<const RecordHeader*>(rec);
  const Cand* cd = reinterpret_cast<const Cand*>(rec + sizeof(RecordHeader));
  tail_exchange_row(x.peer, x.m, b, h.score, h.token, h.n, h.flags, [&](int i) { return cd[i]; }, buf,
                    (int)threadIdx.x, x.tokens, x.scores);
}

// ---- pass 2: one cluster per row -----------------------------------------------------------------
// Two cluster barriers per row.  Every CTA first puts its share of the row in flight (16-byte
// loads into registers), then the cluster rank-counts the slice maxima for tau while those loads
// land; candidates >= tau go straight into rank 0's shared memory through DSMEM atomics, and
// rank 0 resolves them (or runs the exact full-row pass when the row does not fit).
// THREADS = 512 for a few rows (the kernel is a chain of block barriers there, which cost less with
// 16 warps), 1024 for many rows (each CTA then scans a long share of its row and wants the loads
// of 32 warps in flight).  Either way a CTA preloads 64 KB of its share before tau is known.
constexpr int kSelShare = 65536;

template <typename T, int kSelThreads>
__global__ void __launch_bounds__(kSelThreads) k_select(const SelectParams p) {
  constexpr int kSelPreload = kSelShare / 16 / kSelThreads;  // 16-byte vectors per thread fetched before tau is known
  cg::cluster_group cluster = cg::this_cluster();
  const int crank = (int)cluster.block_rank();
  const int csize = (int)cluster.num_blocks();  // 1, 2, 4 or 8: chosen by the launcher from the row length
  const int b = blockIdx.y, tid = threadIdx.x;
  pdl_wait();  // launched behind an lm_head kernel as its programmatic dependent: everything read below is that kernel's
  // rows the lm_head kernel's own tail already resolved (uniform over the cluster: no barrier is reached)
  if (p.row_flag && p.row_flag[b] == 0) return;
  const RowMeta m = decode_row(p.sp, b);
  const T* row = reinterpret_cast<const T*>(p.logits) + (long long)b * p.ld;

  __shared__ float s_sm[kMaxSlices];
  __shared__ float s_cv[kGlobalCap];
  __shared__ int s_ct[kGlobalCap];
  __shared__ float s_y[kGlobalCap];
  __shared__ unsigned long long s_w[kGlobalCap];
  __shared__ unsigned char s_alive[kGlobalCap];
  __shared__ Best s_redb[32];
  __shared__ float s_redf[32];
  __shared__ unsigned long long s_z;
  __shared__ int s_count;
  __shared__ int s_nrec;
  __shared__ FullRowScratch s_full;
  __shared__ __align__(16) uint8_t s_xbuf[kTailWarpBytes];  // sharded step: scratch of the record exchange
  __shared__ SelectExchange s_x;
  const bool exchange = p.peer.G > 0;
  if (exchange && tid == 0) {
    s_x.peer = p.peer;
    s_x.m = m;
    s_x.records = p.records;
    s_x.tokens = p.tokens;
    s_x.scores = p.scores;
  }

  if (!(m.flags & ROW_CAND)) {
    // row already reduced to per-slice winners: merge them (rank 0 only, no cluster traffic)
    if (crank != 0) return;
    Best best{-INFINITY, 0x7fffffff};
    for (int s = tid; s < p.nslices; s += blockDim.x) {
      const float sc = p.part_score[(long long)b * p.nslices + s];
      const int tk = p.part_token[(long long)b * p.nslices + s];
      if (better(sc, tk, best.s, best.t)) { best.s = sc; best.t = tk; }
    }
    best = block_best(best, s_redb);
    if (tid == 0) {
      const long long tok = (long long)best.t + p.sp.vocab_offset;
      write_header(p.records, b, best.s, (int)tok, 0, 0);
      if (p.tokens) p.tokens[b] = tok;
      if (p.scores) p.scores[b] = best.s;
    }
    if (exchange) select_exchange_row(s_x, b, s_xbuf);
    return;
  }

  // rows the candidate scheme cannot bound: top-p without top-k, or k beyond the slice count
  const bool needs_row = (m.flags & ROW_FULLROW) || (m.top_k > 0 && (m.top_k > p.nslices || p.nslices > kMaxSlices));
  if (needs_row) {  // uniform over the cluster: no barrier is ever reached
    if (crank != 0) return;
    if (p.single_shard) {
      Best w = fullrow_resolve(row, p.V, m, p.sp.vocab_offset, s_full);
      if (tid == 0) {
        write_header(p.records, b, -INFINITY, -1, 0, VQK_RECORD_FLAG_NEEDS_ROW);
        if (p.tokens) p.tokens[b] = w.t;
        if (p.scores) p.scores[b] = w.s;
      }
    } else if (tid == 0) {
      write_header(p.records, b, -INFINITY, -1, 0, VQK_RECORD_FLAG_NEEDS_ROW);
      if (p.tokens) p.tokens[b] = -1;
    }
    if (exchange) select_exchange_row(s_x, b, s_xbuf);
    return;
  }

  // ---- put this CTA's share of the row in flight -------------------------------------------
  constexpr int VEC = 16 / (int)sizeof(T);
  const int per = ((p.V + csize - 1) / csize + VEC - 1) / VEC * VEC;
  const int c0 = min(p.V, crank * per), c1 = min(p.V, c0 + per);
  const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  const int nvec = vec_ok ? (c1 - c0) / VEC : 0;
  uint4 pre[kSelPreload];
#pragma unroll
  for (int u = 0; u < kSelPreload; ++u) {
    const int v = tid + u * kSelThreads;
    pre[u] = v < nvec ? *reinterpret_cast<const uint4*>(row + c0 + v * VEC) : make_uint4(0, 0, 0, 0);
  }

  // ---- tau: k-th largest slice maximum, radix select in shared memory (every CTA for itself) ---
  if (tid == 0) s_count = 0;
  float tau = m.thr;
  if (m.top_k > 0) {
    const int ns = p.nslices;
    int nonempty = 0;  // slices that hold at least one finite logit
    for (int s0 = 0; s0 < ns; s0 += blockDim.x) {  // ns is uniform: every thread runs every round
      const int s = s0 + tid;
      bool finite = false;
      if (s < ns) {
        const float v = p.slice_max[(long long)b * ns + s];
        s_sm[s] = v;
        finite = v > -INFINITY;
      }
      nonempty += __syncthreads_count(finite);
    }
    if (nonempty >= m.top_k) {
      tau = smem_kth_largest(s_sm, ns, m.top_k, s_full.hist, s_full.bc);
    } else {
      // Fewer slices with data than k (a short vocab shard under a wide-tile kernel): the k-th
      // largest slice maximum is -inf and would admit the whole row.  Take the exact k-th
      // largest logit of the row instead (every CTA of the cluster computes the same value).
      tau = p.V >= m.top_k ? radix_kth_largest(row, p.V, m.top_k, s_full.hist, s_full.bc) : -INFINITY;
    }
  }
  cluster.sync();  // rank 0's candidate counter is zero before anybody pushes

  // ---- candidates >= tau go to rank 0 ---------------------------------------------------------
  int* r_count = cluster.map_shared_rank(&s_count, 0);
  float* r_cv = cluster.map_shared_rank(&s_cv[0], 0);
  int* r_ct = cluster.map_shared_rank(&s_ct[0], 0);
  auto push = [&](float l, int col) {
    if (l >= tau) {
      const int pos = atomicAdd(r_count, 1);
      if (pos < kGlobalCap) { r_cv[pos] = l; r_ct[pos] = (int)(col + p.sp.vocab_offset); }
    }
  };
#pragma unroll
  for (int u = 0; u < kSelPreload; ++u) {
    const int v = tid + u * kSelThreads;
    if (v < nvec) {
      const T* e = reinterpret_cast<const T*>(&pre[u]);
#pragma unroll
      for (int j = 0; j < VEC; ++j) push(to_f32<T>(e[j]), c0 + v * VEC + j);
    }
  }
  for (int v = tid + kSelPreload * kSelThreads; v < nvec; v += kSelThreads) {  // very long rows
    const uint4 raw = *reinterpret_cast<const uint4*>(row + c0 + v * VEC);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < VEC; ++j) push(to_f32<T>(e[j]), c0 + v * VEC + j);
  }
  for (int col = c0 + nvec * VEC + tid; col < c1; col += kSelThreads) push(ldl(row, col), col);  // tail / unaligned rows
  cluster.sync();  // all candidates are in rank 0's shared memory
  if (crank != 0) return;

  const int n = s_count;
  if (n > kGlobalCap) {  // more ties than the buffer holds: exact full-row pass instead
    if (p.single_shard) {
      Best w = fullrow_resolve(row, p.V, m, p.sp.vocab_offset, s_full);
      if (tid == 0) {
        write_header(p.records, b, -INFINITY, -1, 0, VQK_RECORD_FLAG_OVERFLOW);
        if (p.tokens) p.tokens[b] = w.t;
        if (p.scores) p.scores[b] = w.s;
      }
    } else if (tid == 0) {
      write_header(p.records, b, -INFINITY, -1, 0, VQK_RECORD_FLAG_OVERFLOW);
      if (p.tokens) p.tokens[b] = -1;
    }
    if (exchange) select_exchange_row(s_x, b, s_xbuf);
    return;
  }

  if (p.records) {
    // shard record: the local top-k survivors (ties kept); top-p needs the union, so it waits
    if (tid == 0) s_nrec = 0;
    __syncthreads();
    Cand* out = reinterpret_cast<Cand*>(p.records + (size_t)b * VQK_RECORD_BYTES + sizeof(RecordHeader));
    for (int i = tid; i < n; i += blockDim.x) {
      bool keep = true;
      if (m.top_k > 0) {
        int gc = 0;
        const float vi = s_cv[i];
        for (int j = 0; j < n; ++j) gc += (s_cv[j] > vi);
        keep = gc < m.top_k;
      }
      if (keep) {
        const int pos = atomicAdd(&s_nrec, 1);
        if (pos < VQK_RECORD_CAP) out[pos] = Cand{s_cv[i], s_ct[i]};
      }
    }
    __syncthreads();
    if (tid == 0) {
      const int nr = s_nrec;
      write_header(p.records, b, -INFINITY, -1, min(nr, VQK_RECORD_CAP), nr > VQK_RECORD_CAP ? VQK_RECORD_FLAG_OVERFLOW : 0);
    }
  }
  if (p.single_shard) {
    Best w = resolve_candidates(s_cv, s_ct, n, m, s_y, s_w, s_alive, s_redb, s_redf, &s_z);
    if (tid == 0) {
      if (p.tokens) p.tokens[b] = w.t;
      if (p.scores) p.scores[b] = w.s;
    }
  }
  if (exchange) select_exchange_row(s_x, b, s_xbuf);
}

// ---- merge of gathered shard records -----------------------------------------------------------
// record of rank g for row b: records + g * rank_stride + b * VQK_RECORD_BYTES
__device__ __forceinline__ void finalize_row(const uint8_t* records, size_t rank_stride, int G, int b,
                                             const SampleDev& sp, long long* tokens, float* scores) {
  const int tid = threadIdx.x;
  const RowMeta m = decode_row(sp, b);
  __shared__ float s_cv[kGlobalCap];
  __shared__ int s_ct[kGlobalCap];
  __shared__ float s_y[kGlobalCap];
  __shared__ unsigned long long s_w[kGlobalCap];
  __shared__ unsigned char s_alive[kGlobalCap];
  __shared__ Best s_redb[32];
  __shared__ float s_redf[32];
  __shared__ unsigned long long s_z;
  __shared__ int s_n, s_bad;
  if (tid == 0) {
    int n = 0, bad = 0;
    for (int g = 0; g < G; ++g) {
      const RecordHeader* h = reinterpret_cast<const RecordHeader*>(records + g * rank_stride + (size_t)b * VQK_RECORD_BYTES);
      if (h->flags) bad = 1;
      n += h->n;
    }
    if (n > kGlobalCap) bad = 1;
    s_n = n; s_bad = bad;
  }
  __syncthreads();
  if (s_bad) {
    if (tid == 0) { tokens[b] = -1; if (scores) scores[b] = -INFINITY; }
    return;
  }
  if (s_n == 0) {  // winners only
    if (tid == 0) {
      Best best{-INFINITY, 0x7fffffff};
      for (int g = 0; g < G; ++g) {
        const RecordHeader* h = reinterpret_cast<const RecordHeader*>(records + g * rank_stride + (size_t)b * VQK_RECORD_BYTES);
        if (better(h->score, h->token, best.s, best.t)) { best.s = h->score; best.t = h->token; }
      }
      tokens[b] = best.t;
      if (scores) scores[b] = best.s;
    }
    return;
  }
  int base = 0;
  for (int g = 0; g < G; ++g) {
    const uint8_t* rec = records + g * rank_stride + (size_t)b * VQK_RECORD_BYTES;
    const int c = reinterpret_cast<const RecordHeader*>(rec)->n;
    const Cand* cd = reinterpret_cast<const Cand*>(rec + sizeof(RecordHeader));
    for (int i = tid; i < c; i += blockDim.x) { s_cv[base + i] = cd[i].v; s_ct[base + i] = cd[i].t; }
    base += c;
  }
  __syncthreads();
  Best w = resolve_candidates(s_cv, s_ct, s_n, m, s_y, s_w, s_alive, s_redb, s_redf, &s_z);
  if (tid == 0) { tokens[b] = w.t; if (scores) scores[b] = w.s; }
}

__global__ void __launch_bounds__(256) k_finalize(const uint8_t* __restrict__ records, int G, int B, SampleDev sp,
                                                  long long* tokens, float* scores) {
  finalize_row(records, (size_t)B * VQK_RECORD_BYTES, G, blockIdx.x, sp, tokens, scores);
}

// ---- record exchange over peer memory + merge as a kernel of its own ---------------------------------
// One warp per row: the record the caller computed earlier (vqk_lm_head_forward / vqk_sample with
// `records`) is sent to every rank and the shards are merged (peer_exchange.cuh).
__global__ void __launch_bounds__(32) k_peer_exchange(const uint8_t* __restrict__ mine, PeerTable pt, SampleDev sp,
                                                      long long* tokens, float* scores) {
  __shared__ __align__(16) uint8_t s_xbuf[kTailWarpBytes];
  const int b = blockIdx.x;
  const RowMeta m = decode_row(sp, b);
  const uint8_t* rec = mine + (size_t)b * VQK_RECORD_BYTES;
  const RecordHeader h = *reinterpret_cast<const RecordHeader*>(rec);
  const Cand* cd = reinterpret_cast<const Cand*>(rec + sizeof(RecordHeader));
  tail_exchange_row(pt, m, b, h.score, h.token, h.n, h.flags, [&](int i) { return cd[i]; }, s_xbuf, (int)threadIdx.x,
                    tokens, scores);
}

template <typename T>
__global__ void __launch_bounds__(1024) k_topk_threshold(const T* __restrict__ logits, long long ld, int V,
                                                        const int32_t* __restrict__ top_k, float* __restrict__ thr) {
  const int b = blockIdx.x;
  __shared__ unsigned int s_hist[256];
  __shared__ unsigned int s_bc[2];
  const int k = top_k[b];
  if (k <= 0 || k >= V) {
    if (threadIdx.x == 0) thr[b] = -INFINITY;
    return;
  }
  float t = radix_kth_largest(logits + (long long)b * ld, V, k, s_hist, s_bc);
  if (threadIdx.x == 0) thr[b] = t;
}

// ---- host launchers ------------------------------------------------------------------------------------
#define VQK_DISPATCH_DTYPE(dt, CALL)                          \
  switch (dt) {                                               \
    case VQK_F16: { using T = __half; CALL; break; }          \
    case VQK_BF16: { using T = __nv_bfloat16; CALL; break; }  \
    case VQK_F32: { using T = float; CALL; break; }           \
    default: return VQK_ERR_INVALID;                          \
  }

int launch_slice_pass(const void* logits, int dtype, long long ld, int B, int V, const SampleDev& sp, float* slice_max,
                      float* part_score, int* part_token, int nslices, cudaStream_t st, float* lp_max, float* lp_sum) {
  if (B == 0 || V == 0) return VQK_OK;
  dim3 grid((unsigned)((nslices + 7) / 8), (unsigned)B);
  VQK_DISPATCH_DTYPE(dtype, (k_slice_pass<T><<<grid, 256, 0, st>>>((const T*)logits, ld, V, sp, slice_max, part_score,
                                                                   part_token, nslices, lp_max, lp_sum)));
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

int launch_logprob(const void* logits, int dtype, long long ld, int B, int V, const float* lp_max, const float* lp_sum,
                   int nslices, const long long* tokens, float* logprobs, cudaStream_t st) {
  if (B == 0 || V == 0) return VQK_OK;
  VQK_DISPATCH_DTYPE(dtype, (k_logprob<T><<<(unsigned)B, 32, 0, st>>>((const T*)logits, ld, V, lp_max, lp_sum, nslices, tokens,
                                                                      logprobs)));
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

int launch_select(const SelectParams& p, cudaStream_t st, bool after_lm_head) {
  if (p.B == 0) return VQK_OK;
  // CTAs per row: enough that a CTA's share fits the registers it preloads (kSelShare bytes),
  // at most kClusterSize; short rows (a vocab shard) take one CTA and
  // skip the cluster traffic altogether
  const size_t esz = p.dtype == VQK_F32 ? 4 : 2;
  const size_t share = kSelShare;
  int cs = 1;
  while (cs < kClusterSize && (size_t)p.V * esz > share * cs) cs <<= 1;
  // ... and no more CTAs in total than SMs (one 1024-thread CTA fits an SM): every CTA of a cluster repeats the
  // threshold search of its row, so with many rows narrow clusters (longer scans, fewer
  // repeats) finish sooner
  const int budget = device_sm_count();
  while (cs > 1 && (long long)cs * p.B > budget) cs >>= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cs, (unsigned)p.B);
  const bool narrow = (long long)cs * p.B <= 64;  // few CTAs in all: latency, not throughput, decides
  cfg.blockDim = dim3(narrow ? 512 : 1024);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cs;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = after_lm_head ? 2 : 1;
  cudaError_t le = cudaSuccess;
  if (narrow) {
    VQK_DISPATCH_DTYPE(p.dtype, (le = cudaLaunchKernelEx(&cfg, k_select<T, 512>, p)));
  } else {
    VQK_DISPATCH_DTYPE(p.dtype, (le = cudaLaunchKernelEx(&cfg, k_select<T, 1024>, p)));
  }
  VQK_CUDA(le);
  return VQK_OK;
}

int launch_finalize(const uint8_t* records, int G, int B, const SampleDev& sp, long long* tokens, float* scores,
                    cudaStream_t st) {
  if (B == 0) return VQK_OK;
  k_finalize<<<(unsigned)B, 256, 0, st>>>(records, G, B, sp, tokens, scores);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

int launch_peer_exchange(const uint8_t* mine, int B, const PeerTable& pt, const SampleDev& sp, long long* tokens,
                         float* scores, cudaStream_t st) {
  if (B == 0) return VQK_OK;
  k_peer_exchange<<<(unsigned)B, 32, 0, st>>>(mine, pt, sp, tokens, scores);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

int launch_topk_threshold(const void* logits, int dtype, long long ld, int B, int V, const int32_t* top_k, float* thr,
                          cudaStream_t st) {
  if (B == 0) return VQK_OK;
  VQK_DISPATCH_DTYPE(dtype, (k_topk_threshold<T><<<(unsigned)B, 1024, 0, st>>>((const T*)logits, ld, V, top_k, thr)));
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}


// ---- sampler entry that allocates nothing ---------------------------------------------------------
// Scratch for vqk_sample_static lives in this file-scope device array instead of a caller
// workspace.  Every GPU that loads the library keeps these bytes until the process exits.
// In host code the array's NAME is only a host-side stand-in: the device address is fetched
// once per device with cudaGetSymbolAddress (with that device current) and that pointer is
// what the kernels receive.
static __device__ __align__(256) unsigned char g_static_scratch[VQK_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_ptr[64];  // per device, filled on the first call there
static std::mutex g_static_scratch_mu;   // ... which may come from several host threads at once

int sample_static(const void* logits, int dtype, long long ld, int B, int V, const SampleDev& sp, long long* tokens,
                  float* scores, cudaStream_t st) {
  if (B > VQK_STATIC_MAX_ROWS || V > VQK_STATIC_MAX_VOCAB) return VQK_ERR_TOO_LARGE;
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (!g_static_scratch_ptr[dev]) {  // set-up: once per device, with that device current
      void* ptr = nullptr;
      VQK_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
      g_static_scratch_ptr[dev] = ptr;
    }
  }
  const int nslices = slice_pass_nslices(V);
  // three [B][nslices] arrays, each starting on a 256-byte boundary; all of them are fully
  // rewritten by the first pass before the second pass reads them, so nothing needs clearing
  const size_t each = (((size_t)B * nslices * sizeof(float)) + 255) & ~(size_t)255;
  if (3 * each > (size_t)VQK_STATIC_SCRATCH_BYTES) return VQK_ERR_TOO_LARGE;
  unsigned char* base = static_cast<unsigned char*>(g_static_scratch_ptr[dev]);
  float* slice_max = reinterpret_cast<float*>(base);
  float* part_score = reinterpret_cast<float*>(base + each);
  int* part_token = reinterpret_cast<int*>(base + 2 * each);
  int rc = launch_slice_pass(logits, dtype, ld, B, V, sp, slice_max, part_score, part_token, nslices, st);
  if (rc) return rc;
  SelectParams s{};
  s.logits = logits; s.dtype = dtype; s.ld = ld; s.V = V; s.B = B; s.sp = sp;
  s.slice_max = slice_max; s.part_score = part_score; s.part_token = part_token; s.nslices = nslices;
  s.records = nullptr; s.tokens = tokens; s.scores = scores;
  s.single_shard = 1;
  return launch_select(s, st);
}

}  // namespace vqk
