// Pieces shared by the tcgen05 (UMMA) lm_head kernels: PTX wrappers, descriptors, epilogue.
#pragma once

#include <cuda.h>

#include "async_helpers.cuh"
#include "lm_head.cuh"

namespace vqk {
namespace umma {

constexpr int BM = 128;        // vocab rows per tile = TMEM lanes
constexpr int BK = 128;        // bytes of K per stage in shared memory: one 128-byte swizzle row
constexpr int kMaxStages = 8;
// sampler state of the four epilogue warps in shared memory: [4][3][BN] ints (slice maximum, best Gumbel
// score, its token)
__host__ __device__ inline size_t epi_state_bytes(int bn) { return (size_t)12 * bn * sizeof(int); }

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <bool INT8>
__device__ __forceinline__ void umma_8bit(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  if constexpr (INT8) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  }
}
// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread (lane = thread's TMEM lane)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with
// the 128-byte swizzle (what a TMA box {128 B, rows} with SWIZZLE_128B writes): 8-row groups
// are 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell), layout type 2.
// Stepping K by 32 bytes inside the swizzled row is a plain +32 on the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // descriptor version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// Instruction descriptor (dense, K-major A and B, M = 128): accumulator format at bit 4
// (1 = F32, 2 = S32), A / B formats at bits 7 / 10 (f8f6f4: 0 = E4M3; i8: 1 = signed), N >> 3 at
// bit 17, M >> 4 at bit 24.
__host__ __device__ inline uint32_t instr_desc(bool int8, int bn) {
  uint32_t d = 0;
  d |= (int8 ? 2u : 1u) << 4;
  d |= (int8 ? 1u : 0u) << 7;
  d |= (int8 ? 1u : 0u) << 10;
  d |= (uint32_t)(bn >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}

// Which vocab rows a CTA works on: its n-th tile is rows [(blockIdx.x + n * gridDim.x) * BM, + BM),
// whole 128-row tiles round-robin over the grid; the last tile of the matrix may be short.
struct TileSched {
  int row_begin, row_end, ntiles, stride_rows;
  __device__ __forceinline__ int count() const { return ntiles; }
  __device__ __forceinline__ int row0(int n) const { return row_begin + n * stride_rows; }
  __device__ __forceinline__ int limit(int n) const {  // one past the last row of tile n that exists
    const int r = row0(n) + BM;
    return r < row_end ? r : row_end;
  }
};
__device__ __forceinline__ TileSched sched_interleaved(int V) {
  TileSched t;
  const int ntiles = (V + BM - 1) / BM;
  t.row_begin = (int)blockIdx.x * BM;
  t.row_end = V;
  t.ntiles = (int)blockIdx.x < ntiles ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
  t.stride_rows = (int)gridDim.x * BM;
  return t;
}

__device__ __forceinline__ int ordered_key(float f) {  // order-preserving float -> signed int, NaN lowest
  if (f != f) return (int)0x80000000;
  int i = __float_as_int(f);
  return i >= 0 ? i : (i ^ 0x7fffffff);
}
__device__ __forceinline__ float key_to_float(int k) {
  return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff));
}

// Epilogue of the tensor-core lm_head kernels, run by the four epilogue warps (warp % 4 = TMEM
// lane quadrant).  EPI: 0 = fp32 accumulator x fp16/fp32 row scale, 1 = int32 accumulator x row
// scale x activation scale (W8A8), 2 = fp32 accumulator as is (MX modes).
// NI: independent MMA pipelines ("lanes") in the CTA.  The CTA's n-th tile is computed by lane
// n % NI into that lane's accumulator (n / NI) % 2, at TMEM columns ((n % NI) * 2 + buffer) * BN,
// and announced / released through tfull / tempty at the same index.
template <int EPI, int BN, int NI = 1>
__device__ __forceinline__ void umma_epilogue(const LmHeadParams& p, int warp, int lane, uint32_t tmem_base,
                                              uint64_t* tfull, uint64_t* tempty, volatile int* abort_flag,
                                              const RowMeta* meta, int* sstate, const TileSched& sched) {
  constexpr bool INT8 = (EPI == 1);
  const int V = p.V, B = p.B;
    // ================================ epilogue =========================================
    // Compact by design: a runtime loop over 16-column chunks (the fully unrolled form of a
    // 256-column epilogue does not fit the instruction cache and ran 10x slower than the MMAs).
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    int* st_max = sstate + (size_t)(q * 3 + 0) * BN;   // per warp, per batch column: slice maximum (ordered key)
    int* st_key = sstate + (size_t)(q * 3 + 1) * BN;   // best Gumbel score (ordered key)
    int* st_tok = sstate + (size_t)(q * 3 + 2) * BN;   // its local token id
    for (int b = lane; b < BN; b += 32) { st_max[b] = ordered_key(-INFINITY); st_key[b] = (int)0x80000000; st_tok[b] = 0x7fffffff; }
    __syncwarp();
    float xs_w8a8 = 1.f;
    if constexpr (INT8) xs_w8a8 = *reinterpret_cast<const float*>(p.xscale);
    const int nchunk = (B + 15) / 16;
    const bool post_ops = p.soft_cap > 0.f || p.out_scale != 1.f;

    const int mytiles = sched.count();
    for (int tcount = 0; tcount < mytiles; ++tcount) {
      const int buf = (tcount % NI) * 2 + ((tcount / NI) & 1);
      const uint32_t tph = (uint32_t)((tcount / NI) >> 1) & 1u;
      const int tile_row0 = sched.row0(tcount), tile_lim = sched.limit(tcount);
      const int row = tile_row0 + q * 32 + lane;
      const bool rok = row < tile_lim;
      const int rowc = rok ? row : tile_lim - 1;  // clamped: out-of-range lanes write nothing
      float rs = 1.f;
      if constexpr (EPI == 1) rs = reinterpret_cast<const float*>(p.wscale)[rowc];
      if constexpr (EPI == 0) rs = __half2float(reinterpret_cast<const __half*>(p.wscale)[rowc]);
      const float bias = p.bias ? __half2float(p.bias[rowc]) : 0.f;
      if (!mbar_wait_warp(&tfull[buf], tph, abort_flag)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      for (int ch = 0; ch < nchunk; ++ch) {
        const int c0 = ch * 16;
        uint32_t r[16];
        tmem_ld16(taddr + (uint32_t)c0, r);
        // which of the 16 columns take the candidate path / exist at all
        int myflags = 0;
        if (lane < 16 && c0 + lane < B && p.do_sample) myflags = meta[c0 + lane].flags | 0x100;
        const unsigned candmask = __ballot_sync(0xffffffffu, (myflags & ROW_CAND) != 0);
        const unsigned livemask = __ballot_sync(0xffffffffu, (myflags & 0x100) != 0);
        __half* lp = p.logits ? p.logits + (long long)c0 * p.ld_logits + rowc : nullptr;
        __half* cp = p.cand_logits + (long long)c0 * p.ld_cand + rowc;
        int mine_max = ordered_key(-INFINITY);
        tmem_ld_wait();
        if (!p.bias && !post_ops && c0 + 16 <= B && (!p.do_sample || (candmask & 0xffffu) == 0xffffu)) {
          // Fast path (all 16 columns exist and take the candidate path, or no sampling at all):
          // packed fp16 conversion, one store per column, and the 32-row maximum of every column
          // by a half2 butterfly over the warp instead of sixteen warp reductions.
          __half2 h2[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float v0, v1;
            if constexpr (INT8) {
              v0 = ((float)(int)r[2 * i] * rs) * xs_w8a8;
              v1 = ((float)(int)r[2 * i + 1] * rs) * xs_w8a8;
            } else {
              v0 = __uint_as_float(r[2 * i]) * rs;
              v1 = __uint_as_float(r[2 * i + 1]) * rs;
            }
            h2[i] = __floats2half2_rn(v0, v1);
          }
          if (rok) {
            __half* dst = cp;
            long long ldd = p.ld_cand;
            if (!p.do_sample) { dst = lp; ldd = p.ld_logits; }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              dst[(long long)(2 * i) * ldd] = __low2half(h2[i]);
              dst[(long long)(2 * i + 1) * ldd] = __high2half(h2[i]);
            }
            if (p.do_sample && lp && lp != cp) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                lp[(long long)(2 * i) * p.ld_logits] = __low2half(h2[i]);
                lp[(long long)(2 * i + 1) * p.ld_logits] = __high2half(h2[i]);
              }
            }
          }
          if (p.do_sample) {
            const __half2 ninf = __float2half2_rn(-INFINITY);
            __half2 a[4], bq[2], c;
#pragma unroll
            for (int i = 0; i < 8; ++i) h2[i] = rok ? h2[i] : ninf;
            const bool up16 = lane & 16, up8 = lane & 8, up4 = lane & 4;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __half2 send = up16 ? h2[i] : h2[i + 4], keep = up16 ? h2[i + 4] : h2[i];
              a[i] = __hmax2(keep, __shfl_xor_sync(0xffffffffu, send, 16));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const __half2 send = up8 ? a[i] : a[i + 2], keep = up8 ? a[i + 2] : a[i];
              bq[i] = __hmax2(keep, __shfl_xor_sync(0xffffffffu, send, 8));
            }
            {
              const __half2 send = up4 ? bq[0] : bq[1], keep = up4 ? bq[1] : bq[0];
              c = __hmax2(keep, __shfl_xor_sync(0xffffffffu, send, 4));
            }
            c = __hmax2(c, __shfl_xor_sync(0xffffffffu, c, 2));
            c = __hmax2(c, __shfl_xor_sync(0xffffffffu, c, 1));
            if ((lane & 3) == 0) {  // this lane group holds the column pair selected by lane bits 4, 3, 2
              const int pair = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
              const int k0 = ordered_key(__low2float(c)), k1 = ordered_key(__high2float(c));
              st_max[c0 + 2 * pair] = max(st_max[c0 + 2 * pair], k0);
              st_max[c0 + 2 * pair + 1] = max(st_max[c0 + 2 * pair + 1], k1);
            }
          }
          continue;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          float v;
          if constexpr (INT8) v = ((float)(int)r[j] * rs) * xs_w8a8;  // reference _kernels.py:471, left to right
          else v = __uint_as_float(r[j]) * rs;
          __half h = __float2half_rn(v);
          if (p.bias) h = __float2half_rn(__half2float(h) + bias);
          h = logit_post_ops(h, p.soft_cap, p.out_scale);
          if (c0 + j < B) {  // warp-uniform
            if (lp && rok) lp[(long long)j * p.ld_logits] = h;
            if (candmask & (1u << j)) {
              if (rok) cp[(long long)j * p.ld_cand] = h;
              const int mk = __reduce_max_sync(0xffffffffu, rok ? ordered_key(__half2float(h)) : ordered_key(-INFINITY));
              if (lane == j) mine_max = mk;
            } else if (livemask & (1u << j)) {
              const RowMeta m = meta[c0 + j];
              const float l = __half2float(h);
              float sc = l;
              if (!(m.flags & ROW_GREEDY)) {
                sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(row + p.sp.vocab_offset));
                if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
              }
              const int key = rok ? ordered_key(sc) : (int)0x80000000;
              const int mk = __reduce_max_sync(0xffffffffu, key);
              const unsigned eq = __ballot_sync(0xffffffffu, key == mk);
              const int tok = tile_row0 + q * 32 + (__ffs(eq) - 1);  // lowest row among equal scores
              if (lane == j && (mk > st_key[c0 + j] || (mk == st_key[c0 + j] && tok < st_tok[c0 + j]))) {
                st_key[c0 + j] = mk;
                st_tok[c0 + j] = tok;
              }
            }
          }
        }
        if (lane < 16 && (candmask & (1u << lane))) st_max[c0 + lane] = max(st_max[c0 + lane], mine_max);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    __syncwarp();
    if (p.do_sample) {
      const int slice = blockIdx.x * 4 + q;
      for (int b = lane; b < B; b += 32) {
        const long long o = (long long)b * p.nslices + slice;
        p.slice_max[o] = key_to_float(st_max[b]);
        p.part_score[o] = st_key[b] == (int)0x80000000 ? -INFINITY : key_to_float(st_key[b]);
        p.part_token[o] = st_tok[b];
      }
    }
}

}  // namespace umma
}  // namespace vqk
