// Weight-streaming lm_head kernel for small batches (decode): one persistent CTA per SM,
// 16 warps = 4 groups x 4 warps.  A group owns one 16-row
// vocab tile at a time and its four warps split K; every lane streams 16 B (8 B / 4 B for the MX
// modes) of two weight rows straight from HBM into registers in the layout of a warp-level MMA A
// fragment, so the only per-byte ALU work is the int8 -> fp16 (or E2M1 -> e4m3) expansion.
// Activations sit in shared memory, pre-arranged as B fragments.
// The warps of a group do not run in lockstep: at the end of a tile each parks its split-K
// partial sums in shared memory (two buffers per group, handed over through mbarriers) and goes
// on with the next tile; the epilogue of a tile - add the partials, apply the mode's scale, round
// to fp16 exactly like the reference launchers, optionally store the logits, feed the sampler
// (per-slice lists of the largest logits, per-slice Gumbel winners) without a second pass - runs
// one tile later, when every warp's partials have long arrived, the batch columns dealt out to
// the four warps in rotation.  With the epilogue right behind its tile (two block barriers per
// tile) the W8A16 kernel ran 9 % slower; epilogue warps of their own (20 warps, 96 registers)
// could not keep up beyond four batch columns.  A warp keeps ONE set of weight registers and
// refills it unit by unit instead of double-buffering whole batches.
// Tiles: a group's first two are the static round-robin ones, the rest come from a per-launch
// counter (the CTAs stream at different rates); the leftover tiles, fewer than groups, are taken one
// per CTA with K split over all sixteen warps.  At its end every CTA merges its groups' sampler
// state into one record per batch row, and the last CTA to finish runs the sampler tail (tail.cuh).
//
// Replaces int8_gmv / int8_gemm / fp8_gemm / int8_w8a8_gemm / mxfp8_gemm / mxfp4_gemm of the
// reference (src/vllm_quant_kernels/_kernels.py) for batch <= 32.
#include <stdlib.h>

#include "async_helpers.cuh"
#include "lm_head.cuh"
#include "mma_helpers.cuh"
#include "tail.cuh"

namespace vqk {

// weight loads: evict-first (the read-only no-allocate form measured the same, and it too needs the L1:
// see stream_smem_total)
__device__ __forceinline__ uint4 ldg_stream16(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint2 ldg_stream8(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const uint2*>(p));
}
__device__ __forceinline__ uint32_t ldg_stream4(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const unsigned int*>(p));
}

template <int MODE>
struct AccT { using type = float; };
template <>
struct AccT<VQK_MODE_W8A8> { using type = int; };

// one batch of weight data in registers: U 64-byte k-steps of two rows (16 B per lane each), or
// U scale groups of two rows (8 B / 4 B per lane) plus their E8M0 bytes
template <int MODE, int U, bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4)>
struct StreamBuf {
  uint4 a[U], b[U];
};
template <int MODE, int U>
struct StreamBuf<MODE, U, true> {
  static constexpr int QW = (MODE == VQK_MODE_MXFP8) ? 2 : 1;
  uint32_t qa[U][QW], qb[U][QW];
  uint32_t scA[U / 4], scB[U / 4];
};

constexpr int kGroups = 4;
constexpr int kStreamWarps = 4 * kGroups;
constexpr int kThreads = kStreamWarps * 32;

// shared memory carve-up (bytes) -----------------------------------------------------------
__host__ __device__ inline size_t stream_xfrag_bytes(int mode, int K, int NT) {
  int k64 = (K + 63) / 64 * 64;
  return (size_t)k64 * NT * (mode == VQK_MODE_W8A16 ? 16 : 8);
}
__host__ __device__ inline size_t stream_sx_bytes(int mode, int K, int NT) {
  return (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4) ? (size_t)(K / GROUP) * NT * 8 * sizeof(float) : 0;
}
// split-K partial sums: [2 buffers][16 warps][NT][128] accumulators
__host__ __device__ inline size_t stream_red_bytes(int NT) { return (size_t)2 * kStreamWarps * NT * 128 * 4; }
// per warp group, batch column and tile row: running Gumbel (or greedy) winner of rows without top-k / top-p
__host__ __device__ inline size_t stream_win_bytes(int NT) { return (size_t)kGroups * NT * 8 * 16 * sizeof(Cand); }
constexpr size_t kStreamBarBytes = (size_t)(4 * kGroups + 1) * 8 + (size_t)kGroups * 8 * 4;  // full / free barriers of the partial-sum buffers, abort flag; per group four (tag, tile) slots of the tile hand-out
// Per warp group and batch column (sampler, top-k rows): the largest logits of the group's slice.
// A logit above the column's threshold is APPENDED to a small buffer (every passing lane at once, no
// order kept); when another pass might not fit, the buffer is cut back to its kListM largest and the
// threshold raised to the next one.  The threshold is the witness: every logit of the slice that is
// not in the buffer is <= it.  (A sorted list with one insertion per passing logit stalled its warp
// for some 300 cycles a time, 35 times per column.)
constexpr int kBufCap = 32;
struct ColCtl {
  int cnt;
  float thr;
};
__host__ __device__ inline size_t stream_tlist_bytes(int NT) {
  return (size_t)kGroups * NT * 8 * (kBufCap * sizeof(Cand) + sizeof(ColCtl));
}
__device__ __forceinline__ int stream_fkey(float f) {  // order-preserving float -> int (no NaN reaches it)
  const int i = __float_as_int(f);
  return i >= 0 ? i : (i ^ 0x7fffffff);
}
__device__ __forceinline__ float stream_fkey_inv(int k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }
// whole warp: keep the kListM largest entries (sorted, ties: lower token first) in buf[0 .. kListM), the
// rest of those slots at -inf; the threshold rises to the largest entry dropped
__device__ __forceinline__ void col_compact(Cand* buf, ColCtl* ctl, int lane) {
  const int n = ctl->cnt;  // warp-uniform, <= kBufCap
  Cand e{-INFINITY, 0x7fffffff};
  if (lane < n) e = buf[lane];
  const int key = stream_fkey(e.v);
  bool alive = lane < n;
  int myrank = -1;
  float dropped = -INFINITY;
#pragma unroll
  for (int r = 0; r <= kListM; ++r) {
    const int mk = __reduce_max_sync(0xffffffffu, alive ? key : (int)0x80000000);
    if (r < kListM) {
      const int mt = __reduce_min_sync(0xffffffffu, (alive && key == mk) ? e.t : 0x7fffffff);
      if (alive && key == mk && e.t == mt) { myrank = r; alive = false; }
    } else if (n > kListM) {
      dropped = stream_fkey_inv(mk);
    }
  }
  __syncwarp();
  if (myrank >= 0) buf[myrank] = e;
  if (lane >= n && lane < kListM) buf[lane] = Cand{-INFINITY, 0x7fffffff};
  if (lane == 0) {
    ctl->cnt = n < kListM ? n : kListM;
    if (n > kListM) ctl->thr = fmaxf(ctl->thr, dropped);
  }
  __syncwarp();
}
// (the sampler tail reuses the buffer once the main loop is over: one warp's scratch per batch row, as
// far as kStreamTailSmemCap allows - with fewer it takes the rows in rounds.  Shared memory is taken
// from the L1, and the weight stream needs the L1: its loads in flight occupy lines there.  Measured
// at batch 1: 119 us per launch with up to 180 KB of shared memory, 181 us with 200 KB or more; at batch
// 16 (two column tiles, 150 KB for the main loop) 135 us, but 172 us with 186 KB.)
constexpr size_t kStreamTailSmemCap = 128 * 1024;  // eight rows at a time
__host__ __device__ inline size_t stream_smem_total(int mode, int K, int NT, int B) {
  const size_t main_loop = stream_xfrag_bytes(mode, K, NT) + stream_sx_bytes(mode, K, NT) + stream_red_bytes(NT) +
                           (size_t)NT * 8 * sizeof(RowMeta) + stream_tlist_bytes(NT) + stream_win_bytes(NT) + kStreamBarBytes;
  size_t tail = tail_smem_bytes(B < NT * 8 ? B : NT * 8);
  if (tail > kStreamTailSmemCap) tail = kStreamTailSmemCap;
  return main_loop > tail ? main_loop : tail;
}
size_t stream_smem_bytes(int mode, int K, int NT) { return stream_smem_total(mode, K, NT, NT * 8); }

template <int MODE, int NT, int U, bool EVEN>
__global__ void __launch_bounds__(kThreads, 1) k_lm_head_stream(const LmHeadParams p) {
  using acc_t = typename AccT<MODE>::type;
  constexpr bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4);
  extern __shared__ __align__(16) uint8_t smem[];
  uint2* xfrag = reinterpret_cast<uint2*>(smem);
  float* sxf = reinterpret_cast<float*>(smem + stream_xfrag_bytes(MODE, p.K, NT));
  acc_t* red = reinterpret_cast<acc_t*>(smem + stream_xfrag_bytes(MODE, p.K, NT) + stream_sx_bytes(MODE, p.K, NT));
  RowMeta* meta = reinterpret_cast<RowMeta*>(reinterpret_cast<uint8_t*>(red) + stream_red_bytes(NT));
  Cand* sbuf_all = reinterpret_cast<Cand*>(meta + NT * 8);                        // [group][column][kBufCap]
  ColCtl* sctl_all = reinterpret_cast<ColCtl*>(sbuf_all + (size_t)kGroups * NT * 8 * kBufCap);  // [group][column]
  Cand* swin = reinterpret_cast<Cand*>(sctl_all + kGroups * NT * 8);               // [group][column][tile row]
  uint64_t* fullb = reinterpret_cast<uint64_t*>(swin + (size_t)kGroups * NT * 8 * 16);  // [group][buffer]: partial sums parked
  uint64_t* freeb = fullb + 2 * kGroups;                                           // [group][buffer]: partial sums read
  volatile int* abort_flag = reinterpret_cast<volatile int*>(freeb + 2 * kGroups);
  volatile int* seq_tag = reinterpret_cast<volatile int*>(freeb + 2 * kGroups + 1);  // [group][4]: 2 m = tile m is being fetched, 2 m + 1 = seq_val holds it
  volatile int* seq_val = seq_tag + kGroups * 4;                                       // [group][4]

  pdl_launch_dependents();  // the full-row sampler kernel behind this one may take its place as SMs come free
  dbg_stamp(p, 0);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp >> 2, wq = warp & 3;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K, V = p.V, B = p.B;
  const int ngroups = K / GROUP;
  const int nks = (K + 63) / 64;

  if (p.do_sample) {
    for (int i = tid; i < kGroups * NT * 8; i += kThreads) sctl_all[i] = ColCtl{0, -INFINITY};
    for (int i = tid; i < kGroups * NT * 8 * 16; i += kThreads) swin[i] = Cand{-INFINITY, 0x7fffffff};
  }
  if (tid == 0) {
    for (int i = 0; i < 2 * kGroups; ++i) {
      mbar_init(&fullb[i], 128);  // every thread of the group's four warps
      mbar_init(&freeb[i], 128);
    }
    *abort_flag = 0;
    // slot s is free for tile m (m & 3 == s) when it says "tile m - 4 was published"; tiles 0 and 1 are static
    for (int i = 0; i < kGroups * 4; ++i) seq_tag[i] = (i & 3) < 2 ? 2 * (i & 3) + 1 : 2 * ((i & 3) - 4) + 1;
  }

  const int ntiles = (V + 15) / 16;
  const size_t rowbytes = (MODE == VQK_MODE_MXFP4) ? (size_t)K / 2 : (size_t)K;
  constexpr int kRedBuf = kStreamWarps * NT * 128;  // accumulators per buffer
  acc_t* myred = red + (size_t)warp * NT * 128;

  // ---- main loop: a flat sequence of (tile, batch) steps per warp; a batch is U units.
  // EVEN (V % 16 == 0, every warp owns `per` whole units, per % U == 0) removes every bounds
  // test and zero fill from the inner loop; the instruction count per byte is what decides
  // whether this kernel reaches the HBM rate.
  constexpr int UB = MX ? (MODE == VQK_MODE_MXFP8 ? 32 : 16) : 64;   // weight bytes per row and unit
  constexpr int LB = MX ? (MODE == VQK_MODE_MXFP8 ? 8 : 4) : 16;     // bytes per lane, row and unit
  constexpr int MM = MX ? 1 : (MODE == VQK_MODE_W8A16 ? 4 : 2);      // MMAs (activation fragments) per unit
  const int units = MX ? ngroups : nks;
  const int per = (units + 3) / 4;         // units per warp, contiguous in K
  const int ubeg = wq * per, uend = EVEN ? ubeg + per : min(units, ubeg + per);
  const int nb = (per + U - 1) / U;        // batches per tile (same for the 4 warps of a group)
  const bool sc_aligned = MX && (EVEN || (((ngroups & 3) == 0) && ((per & 3) == 0)));
  StreamBuf<MODE, U> buf;

  // where batch `bi` of tile `tile` lies for this lane
  struct BatchAddr {
    const uint8_t *pA, *pB, *sA, *sB;
    int u0;
  };
  auto locate_at = [&](int tile, int u0) {
    const int row0 = tile * 16;
    const int rA = EVEN ? row0 + g : min(row0 + g, V - 1);
    const int rB = EVEN ? row0 + g + 8 : min(row0 + g + 8, V - 1);
    BatchAddr a;
    a.u0 = u0;
    a.pA = p.w + (size_t)rA * rowbytes + (size_t)a.u0 * UB + t * LB;
    a.pB = p.w + (size_t)rB * rowbytes + (size_t)a.u0 * UB + t * LB;
    a.sA = a.sB = nullptr;
    if constexpr (MX) {
      const uint8_t* ws = reinterpret_cast<const uint8_t*>(p.wscale);
      a.sA = ws + (size_t)rA * ngroups + a.u0;
      a.sB = ws + (size_t)rB * ngroups + a.u0;
    }
    return a;
  };
  auto locate = [&](int tile, int bi) { return locate_at(tile, ubeg + bi * U); };
  // unit u of a batch into its registers
  auto load_unit = [&](StreamBuf<MODE, U>& f, const BatchAddr& a, int u) {
    if constexpr (!MX) {
      if (EVEN || (a.u0 + u < uend && (a.u0 + u) * 64 + t * 16 + 16 <= K)) {
        f.a[u] = ldg_stream16(a.pA + u * UB);
        f.b[u] = ldg_stream16(a.pB + u * UB);
      } else {
        f.a[u] = make_uint4(0, 0, 0, 0);
        f.b[u] = make_uint4(0, 0, 0, 0);
      }
    } else {
      constexpr int QW = StreamBuf<MODE, U>::QW;
      if (EVEN || a.u0 + u < uend) {
        if constexpr (MODE == VQK_MODE_MXFP8) {
          uint2 va = ldg_stream8(a.pA + u * UB), vb = ldg_stream8(a.pB + u * UB);
          f.qa[u][0] = va.x; f.qa[u][QW - 1] = va.y; f.qb[u][0] = vb.x; f.qb[u][QW - 1] = vb.y;
        } else {
          f.qa[u][0] = ldg_stream4(a.pA + u * UB);
          f.qb[u][0] = ldg_stream4(a.pB + u * UB);
        }
      } else {
#pragma unroll
        for (int q = 0; q < QW; ++q) { f.qa[u][q] = 0; f.qb[u][q] = 0; }
      }
    }
  };
  // MX: the E8M0 bytes of units 4q .. 4q + 3
  auto load_scales = [&](StreamBuf<MODE, U>& f, const BatchAddr& a, int q) {
    if constexpr (MX) {
      if (EVEN || (sc_aligned && a.u0 + 4 * q + 4 <= uend)) {
        f.scA[q] = __ldg(reinterpret_cast<const unsigned int*>(a.sA + 4 * q));
        f.scB[q] = __ldg(reinterpret_cast<const unsigned int*>(a.sB + 4 * q));
      } else {
        f.scA[q] = 0; f.scB[q] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (a.u0 + 4 * q + j < uend) {
            f.scA[q] |= (uint32_t)__ldg(a.sA + 4 * q + j) << (8 * j);
            f.scB[q] |= (uint32_t)__ldg(a.sB + 4 * q + j) << (8 * j);
          }
      }
    }
  };

  acc_t acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0;

  // the MMAs of unit u of the batch that starts at unit u0
  auto consume_unit = [&](const StreamBuf<MODE, U>& f, int u0, int u) {
    if (!(EVEN || u0 + u < uend)) return;
    const uint2* xf = xfrag + (size_t)u0 * (MM * NT * 32) + lane;   // fragment (unit, i, nt) at ((u*MM+i)*NT+nt)*32
    if constexpr (!MX) {
      const uint32_t wa[4] = {f.a[u].x, f.a[u].y, f.a[u].z, f.a[u].w};
      const uint32_t wb[4] = {f.b[u].x, f.b[u].y, f.b[u].z, f.b[u].w};
      if constexpr (MODE == VQK_MODE_W8A16) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t a0, a1, a2, a3;
          int8x4_to_half2_even_odd(wa[i], a0, a2);
          int8x4_to_half2_even_odd(wb[i], a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint2 bf = xf[((u * MM + i) * NT + nt) * 32];
            mma_f16(acc[nt], a0, a1, a2, a3, bf.x, bf.y);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint2 bf = xf[((u * MM + i) * NT + nt) * 32];
            if constexpr (MODE == VQK_MODE_W8A8)
              mma_s8(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], bf.x, bf.y);
            else
              mma_e4m3(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], bf.x, bf.y);
          }
        }
      }
    } else {
      constexpr int QW = StreamBuf<MODE, U>::QW;
      const float* sxp = sxf + (size_t)u0 * (NT * 8) + 2 * t;
      uint32_t a0, a1, a2, a3;
      if constexpr (MODE == VQK_MODE_MXFP8) {
        a0 = f.qa[u][0]; a2 = f.qa[u][QW - 1]; a1 = f.qb[u][0]; a3 = f.qb[u][QW - 1];
      } else {
        e2m1x8_to_e4m3_even_odd(f.qa[u][0], a0, a2);
        e2m1x8_to_e4m3_even_odd(f.qb[u][0], a1, a3);
      }
      const float fa = e8m0_to_f32((f.scA[u >> 2] >> (8 * (u & 3))) & 0xff);
      const float fb = e8m0_to_f32((f.scB[u >> 2] >> (8 * (u & 3))) & 0xff);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        uint2 bf = xf[(u * NT + nt) * 32];
        float2 sx = *reinterpret_cast<const float2*>(sxp + (u * NT + nt) * 8);
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        mma_e4m3(d, a0, a1, a2, a3, bf.x, bf.y);
        acc[nt][0] = fmaf(d[0], fa * sx.x, acc[nt][0]);
        acc[nt][1] = fmaf(d[1], fa * sx.y, acc[nt][1]);
        acc[nt][2] = fmaf(d[2], fb * sx.x, acc[nt][2]);
        acc[nt][3] = fmaf(d[3], fb * sx.y, acc[nt][3]);
      }
    }
  };

  const int tstride = gridDim.x * kGroups;
  // Whole tiles go round-robin over the grid's warp groups as long as every group gets one; the
  // LEFTOVER tiles (fewer than groups) are taken one per CTA with K split over all sixteen warps, so the
  // last round costs a quarter of a tile's time instead of a whole one at a fraction of the HBM rate
  // (248320 rows on 148 CTAs: 26.2 rounds instead of 27; an eighth of those rows: 3.5 instead of 4).
  const int units16 = units / 16;
  const bool split_rest = !MX && EVEN && (units % 16) == 0 && units16 >= 1 && units16 <= U;
  const int main_end = split_rest ? (ntiles / tstride) * tstride : ntiles;
  const int rest_tile = main_end + (int)blockIdx.x;  // this CTA's first leftover tile
  const bool rest_have = split_rest && rest_tile < ntiles;
  bool rest_loaded = false;
  // Tile hand-out.  A group's first two tiles are the static round-robin ones; beyond them, when the launch
  // has a tile counter, groups take tiles as they get to them (the CTAs' streaming rates differ: their
  // finishing times spread over 9 us with static rounds).  The m-th tile of a group is fetched (one
  // atomicAdd) two tiles ahead by whichever of its warps gets there first, published through a shared
  // slot a batch later, and read by every warp at the end of tile m - 1.
  const bool dynamic = p.tile_counter != nullptr;
  volatile int* gtag = seq_tag + group * 4;
  volatile int* gval = seq_val + group * 4;
  bool fetching = false;      // lane 0: an atomicAdd of mine is in flight for tile `fetch_seq`
  int fetch_seq = 0, fetch_age = 0;
  unsigned int fetched = 0;
  auto publish_now = [&]() {
    gval[fetch_seq & 3] = 2 * tstride + (int)fetched;
    __threadfence_block();
    gtag[fetch_seq & 3] = 2 * fetch_seq + 1;
    fetching = false;
  };
  auto fetch_ahead = [&](int m) {  // at the start of tile m - 2
    if (!dynamic || m < 2 || lane != 0) return;
    if (fetching) publish_now();  // (one batch per tile: the earlier answer has not been passed on yet)
    if (atomicCAS(const_cast<int*>(&gtag[m & 3]), 2 * (m - 4) + 1, 2 * m) == 2 * (m - 4) + 1) {
      fetched = atomicAdd(p.tile_counter, 1u);
      fetching = true;
      fetch_seq = m;
      fetch_age = 0;
    }
  };
  auto publish = [&]() {  // at the top of every batch; acts one whole batch after fetch_ahead, when the counter's answer has arrived
    if (fetching && fetch_age++ >= 1) publish_now();
  };
  auto tile_of = [&](int m, int prev) -> int {  // the group's m-th tile (m >= 1), `prev` its (m - 1)-th
    if (!dynamic || m < 2) return prev + tstride;
    int v = -1;
    if (lane == 0) {
      for (uint32_t it = 0; it < kSpinLimit; ++it) {
        if (gtag[m & 3] == 2 * m + 1) { v = gval[m & 3]; break; }
        if ((it & 255u) == 255u && *abort_flag) break;
      }
      if (v < 0) {  // the wait ran out (it never should): flag the launch as failed and stop taking tiles
        *abort_flag = 1;
        atomicExch(&g_stream_error, 1);
        v = main_end;
      }
    }
    return __shfl_sync(0xffffffffu, v, 0);
  };
  int tile = blockIdx.x * kGroups + group, bi = 0;
  bool have = tile < main_end;
  if (have) {
    const BatchAddr a0 = locate(tile, 0);
#pragma unroll
    for (int u = 0; u < U; ++u) load_unit(buf, a0, u);
#pragma unroll
    for (int q = 0; q < U / 4; ++q) load_scales(buf, a0, q);
  }

  // ---- activations -> B fragments in shared memory, while the first weight loads are in flight ----
  if constexpr (MODE != VQK_MODE_W8A16) pdl_wait();  // the quantized activations come from the kernel before
  if constexpr (MODE == VQK_MODE_W8A16) {
    // one item = the four fragments (i = 0..3) a lane needs for a 64-wide k-step: the sixteen
    // consecutive activations k .. k + 15 of batch row b, fetched with two 16-byte loads when the
    // row allows it
    const int items = nks * NT * 32;
    const bool vec = p.x_dtype != VQK_BF16 && (K & 63) == 0 && ((p.ldx * 2) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;
    for (int s = tid; s < items; s += kThreads) {
      const int l = s & 31, nt = (s >> 5) % NT, ks = s / (32 * NT);
      const int b = nt * 8 + (l >> 2), k = ks * 64 + (l & 3) * 16;
      __align__(16) __half hv[16];
      if (b < B && vec) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.x) + (long long)b * p.ldx + k);
        *reinterpret_cast<uint4*>(hv) = src[0];
        *reinterpret_cast<uint4*>(hv + 8) = src[1];
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float v = 0.f;
          if (b < B && k + j < K) {
            v = p.x_dtype == VQK_BF16
                    ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.x)[(long long)b * p.ldx + k + j])
                    : __half2float(reinterpret_cast<const __half*>(p.x)[(long long)b * p.ldx + k + j]);
          }
          hv[j] = __float2half_rn(v);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // fragment order 0, 2, 1, 3: the weight expansion pairs bytes (0,2) and (1,3) of a word
        __align__(8) __half h[4] = {hv[4 * i], hv[4 * i + 2], hv[4 * i + 1], hv[4 * i + 3]};
        xfrag[((ks * 4 + i) * NT + nt) * 32 + l] = *reinterpret_cast<uint2*>(h);
      }
    }
  } else if constexpr (!MX) {
    const int total = nks * 2 * NT * 32;
    const uint8_t* xq = reinterpret_cast<const uint8_t*>(p.x);
    for (int s = tid; s < total; s += kThreads) {
      int l = s & 31, nt = (s >> 5) % NT, i = (s / (32 * NT)) & 1, ks = s / (64 * NT);
      int b = nt * 8 + (l >> 2), k = ks * 64 + (l & 3) * 16 + i * 8;
      uint2 v = make_uint2(0, 0);
      if (b < B && k < K) v = *reinterpret_cast<const uint2*>(xq + (long long)b * K + k);
      xfrag[s] = v;
    }
  } else {
    const int total = ngroups * NT * 32;
    const uint8_t* xq = reinterpret_cast<const uint8_t*>(p.x);
    const uint8_t* xs = reinterpret_cast<const uint8_t*>(p.xscale);
    for (int s = tid; s < total; s += kThreads) {
      int l = s & 31, nt = (s >> 5) % NT, G = s / (32 * NT);
      int b = nt * 8 + (l >> 2), k = G * 32 + (l & 3) * 8;
      uint2 v = make_uint2(0, 0);
      if (b < B) {
        v = *reinterpret_cast<const uint2*>(xq + (long long)b * K + k);
        if constexpr (MODE == VQK_MODE_MXFP4)  // bytes 0..7 -> (0,2,4,6), (1,3,5,7) like the E2M1 expansion
          v = make_uint2(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531));
      }
      xfrag[s] = v;
    }
    const float rescale = (MODE == VQK_MODE_MXFP4) ? kE2M1Rescale : 1.0f;
    for (int s = tid; s < ngroups * NT * 8; s += kThreads) {
      int c = s & 7, nt = (s >> 3) % NT, G = s / (8 * NT);
      int b = nt * 8 + c;
      sxf[s] = b < B ? e8m0_to_f32(xs[(long long)b * ngroups + G]) * rescale : 0.f;
    }
  }
  if (p.do_sample && tid < NT * 8) {
    RowMeta m;
    m.flags = 0; m.T = 1.f; m.thr = -INFINITY; m.top_p = 1.f; m.top_k = 0; m.seed = 0;
    if (tid < B) m = decode_row(p.sp, tid);
    meta[tid] = m;
  }
  float xs_w8a8 = 1.f;
  if constexpr (MODE == VQK_MODE_W8A8) xs_w8a8 = *reinterpret_cast<const float*>(p.xscale);
  __syncthreads();


  // ---- epilogue of the group's n-th tile (vocab rows etile * 16 ..), this warp's share of the columns:
  // lane -> row (lane & 15) of the tile; column b is taken by warp (b + n) & 3, two columns per pass
  // (one per half warp).  `rs`, `bias`: the row's scale and bias, fetched a tile ahead.
  const int er = lane & 15, eh = lane >> 4;
  auto duty = [&](int n) { return (wq - n) & 3; };  // first column of this warp in tile n
  auto fetch_row_scale = [&](int etile, float& rs, float& bias) {
    const int row = etile * 16 + er;
    rs = 1.f;
    bias = 0.f;
    if (row < V) {
      if constexpr (MODE == VQK_MODE_W8A16 || MODE == VQK_MODE_FP8)
        rs = __half2float(reinterpret_cast<const __half*>(p.wscale)[row]);
      if constexpr (MODE == VQK_MODE_W8A8) rs = reinterpret_cast<const float*>(p.wscale)[row];
      if (p.bias) bias = __half2float(p.bias[row]);
    }
  };
  // the columns bfirst, bfirst + bstep, ... of one tile: `nparts` partial sums per logit, NT * 128 apart
  // from gred; sampler state of warp group `sg`
  auto epilogue_cols = [&](int etile, float rs, float bias, const acc_t* gred, int nparts, int bfirst, int bstep, int sg) {
    Cand* sbuf = sbuf_all + (size_t)sg * NT * 8 * kBufCap;
    ColCtl* sctl = sctl_all + sg * NT * 8;
    Cand* win = swin + (size_t)sg * NT * 8 * 16;
    const int row = etile * 16 + er;
    const bool row_ok = row < V;
      for (int bb = bfirst; bb < B; bb += 2 * bstep) {
        const int b = bb + bstep * eh;
        bool pass = false;  // a top-k column's logit that beats the last entry of the slice's list
        float l = 0.f;
        if (row_ok && b < B) {
          const acc_t* q = gred + (b >> 3) * 128 + (b & 7) * 16 + er;
          acc_t sum = q[0];
          for (int k = 1; k < nparts; ++k) sum += q[k * NT * 128];
          float v;
          if constexpr (MODE == VQK_MODE_W8A8) v = ((float)sum * rs) * xs_w8a8;   // _kernels.py:471, left to right
          else if constexpr (MX) v = sum;
          else v = sum * rs;
          __half h = __float2half_rn(v);
          if (p.bias) h = __float2half_rn(__half2float(h) + bias);
          h = logit_post_ops(h, p.soft_cap, p.out_scale);
          if (p.logits) p.logits[(long long)b * p.ld_logits + row] = h;
          if (p.do_sample) {
            const RowMeta m = meta[b];
            l = __half2float(h);
            if (m.flags & ROW_CAND) {
              p.cand_logits[(long long)b * p.ld_cand + row] = h;
              pass = l > sctl[b].thr;
            } else {
              float sc = l;
              if (!(m.flags & ROW_GREEDY)) {
                sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(row + p.sp.vocab_offset));
                if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
              }
              const Cand w = win[b * 16 + er];  // (row, column)'s own entry: local token id, offset added by the consumer
              if (better(sc, row, w.v, w.t)) win[b * 16 + er] = Cand{sc, row};
            }
          }
        }
        if (p.do_sample) {
          // logits above their column's threshold go into the column's buffer, all at once
          const unsigned mask = __ballot_sync(0xffffffffu, pass);
          if (mask) {
            const unsigned hm = (mask >> (eh * 16)) & 0xffffu;  // this half warp's column
            const bool colok = b < B;
            int cnt = 0;
            if (colok) cnt = sctl[b].cnt;  // <= kBufCap - 16 between passes
            if (pass) sbuf[b * kBufCap + cnt + __popc(hm & ((1u << er) - 1u))] = Cand{l, row};
            const int ncnt = cnt + __popc(hm);
            __syncwarp();
            if (colok && er == 0 && hm) sctl[b].cnt = ncnt;
            __syncwarp();
            unsigned need = __ballot_sync(0xffffffffu, colok && er == 0 && ncnt > kBufCap - 16);
            while (need) {  // cut a buffer back before another pass might not fit
              const int src = __ffs(need) - 1;
              need &= need - 1;
              const int c = bb + bstep * (src >> 4);
              col_compact(sbuf + c * kBufCap, sctl + c, lane);
            }
          }
        }
    }
  };
  // epilogue of the group's n-th whole tile: column b is taken by warp (b + n) & 3
  auto epilogue = [&](int n, int etile, float rs, float bias) -> bool {
    const int bfirst = duty(n);
    const int par = n & 1;
    if (bfirst < B) {
      // every warp of the group has parked this tile's partial sums: a tile ago, as a rule
      if (!mbar_wait_warp(&fullb[group * 2 + par], ((uint32_t)n >> 1) & 1u, abort_flag)) return false;
      epilogue_cols(etile, rs, bias, red + par * kRedBuf + (size_t)(group * 4) * NT * 128, 4, bfirst, 4, group);
    }
    mbar_arrive(&freeb[group * 2 + par]);  // this thread is done with the buffer (also when it had no column)
    return true;
  };

  // ---- main loop ---------------------------------------------------------------------------------
  if (have) fetch_ahead(2);  // (behind the block barrier that follows the set-up of the hand-out slots)
  int tcount = 0;       // tiles this group has finished
  int ptile = 0;        // the previous one, whose epilogue is still due
  float prs = 1.f, pbias = 0.f;
  bool ok = true;
  while (have) {
    publish();
    int ntile = tile, nbi = bi + 1;
    if (nbi == nb) { nbi = 0; ntile = tile_of(tcount + 1, tile); }
    const bool nhave = ntile < main_end;
    // One set of registers, refilled unit by unit: as soon as a unit's MMAs have read it, the same
    // registers fetch that unit of the NEXT batch (also across tile boundaries), so U units per lane
    // are in flight all the time and the HBM stream of a warp never waits for its own arithmetic.
    const bool nrest = !nhave && rest_have;  // the last whole batch: its registers go on to the leftover tile
    const BatchAddr nxt = nrest ? locate_at(rest_tile, warp * units16) : locate(nhave ? ntile : tile, nhave ? nbi : bi);
    const int u0 = ubeg + bi * U;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      consume_unit(buf, u0, u);
      if (nhave || (nrest && u < units16)) load_unit(buf, nxt, u);
      if constexpr (MX)
        if ((u & 3) == 3 && nhave) load_scales(buf, nxt, u >> 2);
    }
    rest_loaded = rest_loaded || nrest;
    const bool tile_done = (bi == nb - 1);
    const int this_tile = tile;
    tile = ntile; bi = nbi; have = nhave;
    if (!tile_done) continue;

    // ---- the previous tile's epilogue, then park this tile's split-K partial sums and go on --------
    if (tcount > 0 && !epilogue(tcount - 1, ptile, prs, pbias)) { ok = false; break; }
    const int par = tcount & 1;
    // (the buffer's previous contents, two tiles back, have been read by every warp)
    if (!mbar_wait_warp(&freeb[group * 2 + par], (((uint32_t)tcount >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc_t* r = myred + par * kRedBuf + nt * 128;
      r[(2 * t) * 16 + g] = acc[nt][0];
      r[(2 * t + 1) * 16 + g] = acc[nt][1];
      r[(2 * t) * 16 + g + 8] = acc[nt][2];
      r[(2 * t + 1) * 16 + g + 8] = acc[nt][3];
      acc[nt][0] = 0; acc[nt][1] = 0; acc[nt][2] = 0; acc[nt][3] = 0;
    }
    mbar_arrive(&fullb[group * 2 + par]);
    ptile = this_tile;
    if (duty(tcount) < B) fetch_row_scale(this_tile, prs, pbias);  // in flight until the epilogue, a tile from now
    ++tcount;
    if (have) fetch_ahead(tcount + 2);
  }
  // ---- leftover tiles: one per CTA and sub-round, K split over the sixteen warps -------------------------
  if (split_rest) {
    for (int lt = rest_tile; lt < ntiles; lt += (int)gridDim.x) {  // CTA-uniform
      const BatchAddr la = locate_at(lt, warp * units16);
      if (!rest_loaded) {
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (u < units16) load_unit(buf, la, u);
      }
      rest_loaded = false;
      float lrs, lbias;
      fetch_row_scale(lt, lrs, lbias);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (u < units16) consume_unit(buf, la.u0, u);
      // the last whole tile's epilogue is still due (first sub-round); then both partial-sum buffers are free
      if (ok && tcount > 0) ok = epilogue(tcount - 1, ptile, prs, pbias);
      tcount = 0;
      __syncthreads();
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc_t* r = myred + nt * 128;
        r[(2 * t) * 16 + g] = acc[nt][0];
        r[(2 * t + 1) * 16 + g] = acc[nt][1];
        r[(2 * t) * 16 + g + 8] = acc[nt][2];
        r[(2 * t + 1) * 16 + g + 8] = acc[nt][3];
        acc[nt][0] = 0; acc[nt][1] = 0; acc[nt][2] = 0; acc[nt][3] = 0;
      }
      __syncthreads();
      // column b by warp b & 15; the tile counts as part of the CTA's first slice
      if (warp < B) epilogue_cols(lt, lrs, lbias, red, kStreamWarps, warp, kStreamWarps, 0);
    }
  }
  if (ok && tcount > 0) epilogue(tcount - 1, ptile, prs, pbias);
  __syncthreads();

  dbg_stamp(p, 1);
  if (p.do_sample) {
    // ---- every warp cuts its share of its group's column buffers back to the kListM largest (sorted);
    //      the threshold that remains is the group's witness
    for (int b = wq; b < B; b += 4)
      col_compact(sbuf_all + ((size_t)group * NT * 8 + b) * kBufCap, sctl_all + group * NT * 8 + b, lane);
    __syncthreads();
    // ---- per batch row (warp w takes rows w, w + 16): the per-slice results the full-row kernel reads,
    //      and the CTA's record for the tail
    for (int b = warp; b < B; b += kStreamWarps) {
      Cand gw[2];  // winners of groups eh and 2 + eh (rows without top-k / top-p), complete in lanes 0 and 16
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        Cand w = swin[((size_t)(2 * h + eh) * NT * 8 + b) * 16 + er];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
          const float s2 = __shfl_xor_sync(0xffffffffu, w.v, o);
          const int t2 = __shfl_xor_sync(0xffffffffu, w.t, o);
          if (better(s2, t2, w.v, w.t)) { w.v = s2; w.t = t2; }
        }
        gw[h] = w;
        if (er == 0) {
          const long long o = (long long)b * p.nslices + blockIdx.x * kGroups + 2 * h + eh;
          p.slice_max[o] = sbuf_all[((size_t)(2 * h + eh) * NT * 8 + b) * kBufCap].v;
          p.part_score[o] = w.v;
          p.part_token[o] = w.t;
        }
      }
      if (p.lists) {
        Cand cw = better(gw[1].v, gw[1].t, gw[0].v, gw[0].t) ? gw[1] : gw[0];
        {
          const float s2 = __shfl_xor_sync(0xffffffffu, cw.v, 16);
          const int t2 = __shfl_xor_sync(0xffffffffu, cw.t, 16);
          if (better(s2, t2, cw.v, cw.t)) { cw.v = s2; cw.t = t2; }
        }
        // the sixteen listed logits of the four groups (lane l < 16: group l / 4, entry l % 4), ranked
        Cand c{-INFINITY, 0x7fffffff};
        if (lane < 16) c = sbuf_all[((size_t)(lane >> 2) * NT * 8 + b) * kBufCap + (lane & 3)];
        int rank = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float vj = __shfl_sync(0xffffffffu, c.v, j);
          rank += (vj > c.v) || (vj == c.v && j < lane);
        }
        // witness: the groups' thresholds and the listed logits that do not fit the record
        float wv = (lane < 16 && rank >= kCtaListM) ? c.v : -INFINITY;
        if (lane >= 16 && lane < 16 + kGroups) wv = sctl_all[(lane - 16) * NT * 8 + b].thr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wv = fmaxf(wv, __shfl_xor_sync(0xffffffffu, wv, o));
        CtaList* rec = p.lists + (size_t)b * gridDim.x + blockIdx.x;
        if (lane < 16 && rank < kCtaListM) {
          rec->t[rank] = c.t;
          rec->v[rank] = __float2half_rn(c.v);
        }
        if (lane == 0) {
          rec->witness = __float2half_rn(wv);
          rec->pad = __float2half_rn(0.f);
          rec->win_s = cw.v;
          rec->win_t = cw.t;
          rec->pad2 = 0;
        }
      }
    }
    dbg_stamp(p, 2);
    if (p.fuse_tail) lm_head_tail(p, meta, smem, stream_smem_total(MODE, p.K, NT, B));
  }
  if (dynamic && !(p.do_sample && p.fuse_tail)) {
    // no tail, so nobody has taken the ticket: the last CTA to finish puts the tile counter back to zero
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(p.ticket, 1u) == gridDim.x - 1) {
        *p.tile_counter = 0u;
        __threadfence();
        *p.ticket = 0u;
      }
    }
  }
}

int stream_error_flag() { return read_stream_error(); }
int stream_error_clear() { return clear_stream_error(); }

// ---- host launch -------------------------------------------------------------------------
template <int MODE, int NT, int U, bool EVEN>
static int launch_stream(const LmHeadParams& p, int grid, cudaStream_t st) {
  size_t smem = stream_smem_total(MODE, p.K, NT, p.B);
  {  // measurement aid: VQK_STREAM_SMEM_KB asks for at least that much shared memory (the L1 shrinks accordingly)
    static const size_t want = [] { const char* e = getenv("VQK_STREAM_SMEM_KB"); return e ? (size_t)atoi(e) * 1024 : (size_t)0; }();
    if (want > smem && want <= 226 * 1024) smem = want;
  }
  static size_t configured[64] = {};  // per device: largest opt-in so far for this instantiation
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (smem > configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_stream<MODE, NT, U, EVEN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)smem));
    configured[dev] = smem;
  }
  VQK_CUDA(launch_kernel(k_lm_head_stream<MODE, NT, U, EVEN>, dim3(grid), dim3(kThreads), smem, st, p.pdl != 0, p));
  return VQK_OK;
}

// units per batch: the fast variant needs U to divide the units each warp owns
template <int MODE, int NT>
static int launch_stream_u(const LmHeadParams& p, int grid, cudaStream_t st) {
  constexpr bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4);
  const int units = MX ? p.K / GROUP : (p.K + 63) / 64;
  const int per = (units + 3) / 4;
  const bool whole = (p.V % 16 == 0) && (units % 4 == 0) && (MX || p.K % 64 == 0);
  if constexpr (MODE == VQK_MODE_MXFP4) {
    if (whole && per % 12 == 0 && per % 16 != 0) return launch_stream<MODE, NT, 12, true>(p, grid, st);
    if (whole && per % 16 == 0) return launch_stream<MODE, NT, 16, true>(p, grid, st);
    if (whole && per % 8 == 0) return launch_stream<MODE, NT, 8, true>(p, grid, st);
    return launch_stream<MODE, NT, 8, false>(p, grid, st);
  } else if constexpr (MODE == VQK_MODE_MXFP8) {
    if (whole && per % 8 == 0) return launch_stream<MODE, NT, 8, true>(p, grid, st);
    return launch_stream<MODE, NT, 8, false>(p, grid, st);
  } else {
    // six units (192 B per lane) in flight where the shape allows: 96 KB per SM (VQK_STREAM_U=4: A/B runs)
    static const bool u6 = [] { const char* e = getenv("VQK_STREAM_U"); return !(e && atoi(e) == 4); }();
    if (u6 && whole && per % 6 == 0) return launch_stream<MODE, NT, 6, true>(p, grid, st);
    if (whole && per % 4 == 0) return launch_stream<MODE, NT, 4, true>(p, grid, st);
    return launch_stream<MODE, NT, 4, false>(p, grid, st);
  }
}

template <int MODE>
static int launch_stream_nt(const LmHeadParams& p, int NT, int grid, cudaStream_t st) {
  switch (NT) {
    case 1: return launch_stream_u<MODE, 1>(p, grid, st);
    case 2: return launch_stream_u<MODE, 2>(p, grid, st);
    case 4:
      if constexpr (MODE != VQK_MODE_W8A16) return launch_stream_u<MODE, 4>(p, grid, st);
  }
  return VQK_ERR_INVALID;
}

int stream_max_cols(int mode, int K) {
  const size_t limit = 227 * 1024;
  int maxnt = (mode == VQK_MODE_W8A16) ? 2 : 4;
  for (int nt = maxnt; nt >= 1; nt >>= 1)
    if (stream_smem_bytes(mode, K, nt) <= limit) return nt * 8;
  return 0;
}

int launch_lm_head_stream(int mode, const LmHeadParams& p, int grid, cudaStream_t st) {
  int NT = p.B <= 8 ? 1 : (p.B <= 16 ? 2 : 4);
  if (NT * 8 > stream_max_cols(mode, p.K)) return VQK_ERR_UNSUPPORTED;
  switch (mode) {
    case VQK_MODE_W8A16: return launch_stream_nt<VQK_MODE_W8A16>(p, NT, grid, st);
    case VQK_MODE_W8A8: return launch_stream_nt<VQK_MODE_W8A8>(p, NT, grid, st);
    case VQK_MODE_FP8: return launch_stream_nt<VQK_MODE_FP8>(p, NT, grid, st);
    case VQK_MODE_MXFP8: return launch_stream_nt<VQK_MODE_MXFP8>(p, NT, grid, st);
    case VQK_MODE_MXFP4: return launch_stream_nt<VQK_MODE_MXFP4>(p, NT, grid, st);
  }
  return VQK_ERR_INVALID;
}

}  // namespace vqk
