// MXFP8 / MXFP4 lm_head for decode batches (up to 16 rows) on the block-scaled tensor-core path,
// with the WEIGHTS as the N-side operand: one tcgen05.mma covers 256 vocab rows.
//
// Why: a 128-row tcgen05.mma occupies the tensor pipe for about 128 cycles whatever its N (measured:
// 126 cycles for N = 16 ... 256, K = 32 bytes).  With the weights on the M side (lm_head_umma_mx.cu)
// the pipe therefore moves 128 rows x 32 container bytes per 126 cycles, which for MXFP4 (a byte
// of container per 4-bit code) is only ~0.7 of the HBM rate before any overhead.  On the N side the
// same instruction consumes 256 rows, and the pipe is no longer the limit.
//
// Layout of the product: D[batch row (TMEM lane), vocab row (TMEM column)], so the batch rows sit
// in lanes 0..15 of lane quadrant 0 and every epilogue warp must be one whose index is a multiple
// of four (the only warps that may read that quadrant).  The accumulator is single-buffered
// (2 x 256 columns plus the scale factors do not fit 512 TMEM columns); the epilogue warps copy
// it to shared memory at once and release it before they do their arithmetic.
//   * activations: [K/128][BPAD rows][128 B] resident in shared memory (TMA, 128-byte swizzle);
//     the M = 128 descriptor walks past the BPAD real rows into whatever follows, which only
//     produces accumulator lanes nobody reads;
//   * activation scales: arranged once and parked in TMEM for all K;
//   * weight scales: four warps arrange groups of four k-blocks (one 16-byte load per row) into a
//     three-slot ring, the MMA warp copies a group into one of two TMEM slots;
//   * MXFP4 weights stay packed in HBM, the 4-bit tensor-map type expands them into the padded
//     8-bit container layout.
// Replaces mxfp8_gemm / mxfp4_gemm of the reference (src/vllm_quant_kernels/_kernels.py:534-802)
// for decode-sized batches.
#include "umma_mx_common.cuh"

namespace vqk {
namespace umma {

constexpr int WN = 256;                 // vocab rows per tile
constexpr int kWideThreads = 13 * 32;   // warps 0,4,8,12: epilogue; 1: TMA; 2: MMA; 3,5,6,7: scales; 9-11 idle
constexpr int kWideStage = WN * BK;     // 32 KB of (expanded) weights per k-block
constexpr int kSfGroup = 4;             // k-blocks per weight-scale group
constexpr int kSfGroupBytes = kSfGroup * 2 * kSfBlock;
constexpr int kSfRing = 3;
constexpr int kStash = 65;              // words per (warp, lane) in the accumulator stash: 64 + 1 against bank conflicts

struct WideGeometry {
  int xa_bytes, stash_bytes, stages;
  size_t total;
};
__host__ __device__ inline WideGeometry wide_geometry(int bpad, int K, int cap = kMaxStages) {
  WideGeometry g;
  const int nkb = K / BK;
  g.xa_bytes = nkb * bpad * BK;
  const int sfx = nkb * kSfBlock, stash = 4 * bpad * kStash * 4;
  g.stash_bytes = ((sfx > stash ? sfx : stash) + 1023) & ~1023;  // the stash reuses the arranged activation scales
  const size_t fixed = 1024 + (size_t)g.xa_bytes + g.stash_bytes + kSfRing * kSfGroupBytes + 512 + (size_t)bpad * sizeof(RowMeta);
  const size_t limit = 227 * 1024;
  int s = fixed < limit ? (int)((limit - fixed) / kWideStage) : 0;
  g.stages = s > cap ? cap : s;
  g.total = fixed + (size_t)g.stages * kWideStage;
  return g;
}

// 32 lanes x 64 consecutive 32-bit columns
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
      "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,"
      "%62,%63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
        "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
        "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
        "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
        "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}

// A = activations (E4M3), B = weights (E2M1 or E4M3), N = 256
__host__ __device__ inline uint32_t instr_desc_wide(bool w_fp4) {
  uint32_t d = 0;
  d |= (w_fp4 ? 5u : 0u) << 10;
  d |= (uint32_t)(WN >> 3) << 17;
  d |= 1u << 23;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}

template <int MODE, int BPAD>
__global__ void __launch_bounds__(kWideThreads, 1)
k_lm_head_umma_wide(const LmHeadParams p, const __grid_constant__ CUtensorMap mapW, const __grid_constant__ CUtensorMap mapX,
                    const int stage_cap) {
  constexpr bool FP4 = (MODE == VQK_MODE_MXFP4);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const WideGeometry geo = wide_geometry(BPAD, p.K, stage_cap);
  const int S = geo.stages;
  uint8_t* xa = smem;                                         // [nkb][BPAD][128 B]
  uint8_t* stages = xa + geo.xa_bytes;                        // [S][256 rows][128 B]
  uint8_t* sfx = stages + (size_t)S * kWideStage;             // arranged activation scales, later the stash
  float* stash = reinterpret_cast<float*>(sfx);               // [4 warps][BPAD lanes][kStash]
  uint8_t* sfw = sfx + geo.stash_bytes;                       // [kSfRing][kSfGroupBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sfw + kSfRing * kSfGroupBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kMaxStages;
  uint64_t* sffull = bars + 2 * kMaxStages;                   // [kSfRing]
  uint64_t* sfempty = sffull + kSfRing;                       // [kSfRing]
  uint64_t* xfull = sfempty + kSfRing;
  uint64_t* tfull = xfull + 1;
  uint64_t* tempty = xfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xfull + 3);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  RowMeta* meta = reinterpret_cast<RowMeta*>(bars + 64);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = p.V, B = p.B;
  const int nkb = p.K / BK;
  const int ngroups = p.K / GROUP;
  const int ntiles = (V + WN - 1) / WN;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int r = 0; r < kSfRing; ++r) { mbar_init(&sffull[r], 4); mbar_init(&sfempty[r], 1); }
    mbar_init(xfull, 1); mbar_init(tfull, 1); mbar_init(tempty, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < BPAD) {
    RowMeta m;
    m.flags = 0; m.T = 1.f; m.thr = -INFINITY; m.top_p = 1.f; m.top_k = 0; m.seed = 0;
    if (p.do_sample && tid < B) m = decode_row(p.sp, tid);
    meta[tid] = m;
  }
  {  // activation scales: block kb holds groups 4kb..4kb+3 of the 128 accumulator rows
    const uint8_t* xs = reinterpret_cast<const uint8_t*>(p.xscale);
    for (int i = tid; i < nkb * 128; i += kWideThreads) {
      const int kb = i >> 7, n = i & 127;
      uint32_t w = 0x7f7f7f7fu;
      if (n < B) w = *reinterpret_cast<const uint32_t*>(xs + (size_t)n * ngroups + kb * 4);
      *reinterpret_cast<uint32_t*>(sfx + (size_t)kb * kSfBlock + (n & 31) * 16 + (n >> 5) * 4) = w;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tsfa_base = tmem_base + (uint32_t)WN;             // activation scales: 4 columns per k-block
  const uint32_t tsfb_base = tsfa_base + (uint32_t)(4 * nkb);      // weight scales: 2 slots x 4 k-blocks x 8 columns

  if (warp == 1) {
    // ================================ TMA producer =====================================
    if (lane == 0) {
      mbar_expect_tx(xfull, (uint32_t)geo.xa_bytes);  // rows past the batch are zero-filled and counted
      for (int kb = 0; kb < nkb; ++kb) tma_load_2d(xa + (size_t)kb * BPAD * BK, &mapX, kb * BK, 0, xfull);
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&empty[s], ((uint32_t)(it / S) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          // the 4-bit copy counts its packed size although it fills 128 bytes per row
          mbar_expect_tx(&full[s], (uint32_t)(FP4 ? kWideStage / 2 : kWideStage));
          tma_load_2d(stages + (size_t)s * kWideStage, &mapW, kb * BK, tile * WN, &full[s]);
        }
      }
    }
  } else if (warp == 2) {
    // ================================ MMA issuer =======================================
    if (lane == 0) {
      const uint32_t idesc = instr_desc_wide(FP4);
      for (int kb = 0; kb < nkb; ++kb) tmem_cp_sf(tsfa_base + (uint32_t)(4 * kb), sf_desc(smem_u32(sfx) + kb * kSfBlock));
      bool ok = mbar_wait(xfull, 0, abort_flag);
      int it = 0, gcount = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
        if (!mbar_wait(tempty, ((uint32_t)tcount & 1u) ^ 1u, abort_flag)) break;
        tc_fence_after();
        uint32_t tsfb = 0;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          if ((kb & (kSfGroup - 1)) == 0) {  // next group of weight scales into its TMEM slot
            const int slot = gcount % kSfRing;
            if (!mbar_wait(&sffull[slot], (uint32_t)(gcount / kSfRing) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            tsfb = tsfb_base + (uint32_t)((gcount & 1) * (kSfGroup * 8));
            const uint32_t src = smem_u32(sfw + (size_t)slot * kSfGroupBytes);
#pragma unroll
            for (int j = 0; j < kSfGroup * 2; ++j) tmem_cp_sf(tsfb + (uint32_t)(4 * j), sf_desc(src + j * kSfBlock));
            umma_commit(&sfempty[slot]);
            ++gcount;
          }
          const int s = it % S;
          if (!mbar_wait(&full[s], (uint32_t)(it / S) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t adesc = smem_desc_sw128(smem_u32(xa + (size_t)kb * BPAD * BK));
          const uint64_t bdesc = smem_desc_sw128(smem_u32(stages + (size_t)s * kWideStage));
          const uint32_t sfb = tsfb + (uint32_t)((kb & (kSfGroup - 1)) * 8);
          const uint32_t sfa = tsfa_base + (uint32_t)(4 * kb);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)  // scale byte k of the block for both operands
            umma_mx(tmem_base, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                    idesc | ((uint32_t)k << 29) | ((uint32_t)k << 4), sfa, sfb, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(tfull);
      }
    }
  } else if ((warp & 3) == 0) {
    // ================================ epilogue =========================================
    const int ew = warp >> 2;  // columns 64 ew .. 64 ew + 63 of the tile
    const bool live = lane < B;
    const RowMeta m = meta[lane < BPAD ? lane : 0];
    const bool cand = (m.flags & ROW_CAND) != 0;
    float* mine = stash + (size_t)(ew * BPAD + (lane < BPAD ? lane : 0)) * kStash;
    int smax = ordered_key(-INFINITY), bkey = (int)0x80000000, btok = 0x7fffffff;
    int tcount = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++tcount) {
      if (!mbar_wait_warp(tfull, (uint32_t)tcount & 1u, abort_flag)) break;
      tc_fence_after();
      {
        uint32_t r[64];
        tmem_ld64(tmem_base + (uint32_t)(ew * 64), r);
        tmem_ld_wait();
        if (lane < BPAD) {
#pragma unroll
          for (int j = 0; j < 64; ++j) mine[j] = __uint_as_float(r[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);  // the accumulator is free for the next tile
      if (!live) continue;
      const int row0 = tile * WN + ew * 64;
      __half* lp = p.logits ? p.logits + (long long)lane * p.ld_logits + row0 : nullptr;
      __half* cp = (p.do_sample && cand) ? p.cand_logits + (long long)lane * p.ld_cand + row0 : nullptr;
      if (cp == lp) cp = nullptr;  // the candidate logits alias the caller's buffer
      const bool full64 = row0 + 64 <= V;
      const bool lp16 = lp && full64 && ((reinterpret_cast<uintptr_t>(lp) & 15) == 0);
      const bool cp16 = cp && full64 && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0);
      for (int j0 = 0; j0 < 64; j0 += 8) {
        if (row0 + j0 >= V) break;
        __align__(16) __half h[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int row = row0 + j0 + j;
          const bool rok = row < V;
          __half hv = __float2half_rn(mine[j0 + j]);
          if (p.bias && rok) hv = __float2half_rn(__half2float(hv) + __half2float(p.bias[row]));
          h[j] = hv;
          if (p.do_sample && rok) {
            const float l = __half2float(hv);
            if (cand) {
              smax = max(smax, ordered_key(l));
            } else {
              float sc = l;
              if (!(m.flags & ROW_GREEDY)) {
                sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(row + p.sp.vocab_offset));
                if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
              }
              const int key = ordered_key(sc);
              if (key > bkey) { bkey = key; btok = row; }  // rows ascend: the lowest row wins ties
            }
          }
        }
        if (lp16) *reinterpret_cast<uint4*>(lp + j0) = *reinterpret_cast<const uint4*>(h);
        else if (lp) {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (row0 + j0 + j < V) lp[j0 + j] = h[j];
        }
        if (cp16) *reinterpret_cast<uint4*>(cp + j0) = *reinterpret_cast<const uint4*>(h);
        else if (cp) {
#pragma unroll
          for (int j = 0; j < 8; ++j) if (row0 + j0 + j < V) cp[j0 + j] = h[j];
        }
      }
    }
    if (p.do_sample && live) {
      const long long o = (long long)lane * p.nslices + (blockIdx.x * 4 + ew);
      p.slice_max[o] = key_to_float(smax);
      p.part_score[o] = bkey == (int)0x80000000 ? -INFINITY : key_to_float(bkey);
      p.part_token[o] = btok;
    }
  } else if (warp == 3 || (warp >= 5 && warp <= 7)) {
    // ================================ weight scales =====================================
    const int t = (warp == 3 ? 0 : warp - 4) * 32 + lane;  // 0..127
    const uint8_t* ws = reinterpret_cast<const uint8_t*>(p.wscale);
    int gcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
      for (int g4 = 0; g4 < nkb / kSfGroup; ++g4, ++gcount) {
        const int slot = gcount % kSfRing;
        if (!mbar_wait_warp(&sfempty[slot], ((uint32_t)(gcount / kSfRing) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        uint4 w[2];
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const int row = tile * WN + rr * 128 + t;
          w[rr] = make_uint4(0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu);
          if (row < V) w[rr] = __ldg(reinterpret_cast<const uint4*>(ws + (size_t)row * ngroups) + g4);
        }
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {  // row r = 128 rr + t of the tile -> block rr, lane t % 32, column t / 32
          uint8_t* dst = sfw + (size_t)slot * kSfGroupBytes + rr * kSfBlock + (t & 31) * 16 + (t >> 5) * 4;
          *reinterpret_cast<uint32_t*>(dst + 0 * 2 * kSfBlock) = w[rr].x;
          *reinterpret_cast<uint32_t*>(dst + 1 * 2 * kSfBlock) = w[rr].y;
          *reinterpret_cast<uint32_t*>(dst + 2 * 2 * kSfBlock) = w[rr].z;
          *reinterpret_cast<uint32_t*>(dst + 3 * 2 * kSfBlock) = w[rr].w;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&sffull[slot]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---- host side ------------------------------------------------------------------------------
static int wide_stage_cap() {
  static int cap = [] {
    const char* e = getenv("VQK_MX_STAGES");  // tuning knob: fewer pipeline stages
    const int v = e ? atoi(e) : 0;
    return v >= 2 && v <= kMaxStages ? v : kMaxStages;
  }();
  return cap;
}

template <int MODE, int BPAD>
static int wide_launch_one(const LmHeadParams& p, const CUtensorMap& w, const CUtensorMap& x, int grid, cudaStream_t st) {
  const WideGeometry geo = wide_geometry(BPAD, p.K, wide_stage_cap());
  static size_t configured[64] = {};
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (geo.total > configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_umma_wide<MODE, BPAD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)geo.total));
    configured[dev] = geo.total;
  }
  // every CTA of the grid runs (those without a tile still write their empty slice records)
  k_lm_head_umma_wide<MODE, BPAD><<<grid, kWideThreads, geo.total, st>>>(p, w, x, geo.stages);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

}  // namespace umma

// Batches and shapes the wide kernel takes: MX modes, up to 16 rows, K a multiple of 512 and at
// most 6144 (TMEM holds the activation scales of all K), at least three pipeline stages.
bool umma_wide_eligible(int mode, int K, int B) {
  if (mode != VQK_MODE_MXFP8 && mode != VQK_MODE_MXFP4) return false;
  if (B < 1 || B > 16 || K % (umma::BK * umma::kSfGroup) || K / umma::BK > 48) return false;
  return umma::wide_geometry(B <= 8 ? 8 : 16, K).stages >= 3;
}

int launch_lm_head_umma_wide(int mode, const LmHeadParams& p, int grid, cudaStream_t st) {
  using namespace umma;
  if (!umma_wide_eligible(mode, p.K, p.B)) return VQK_ERR_UNSUPPORTED;
  if (((uintptr_t)p.w & 31) || ((uintptr_t)p.x & 15) || ((uintptr_t)p.wscale & 15) || ((uintptr_t)p.xscale & 3))
    return VQK_ERR_UNSUPPORTED;
  const bool fp4 = mode == VQK_MODE_MXFP4;
  const int bpad = p.B <= 8 ? 8 : 16;
  CUtensorMap w, x;
  int rc = mx_make_map(&w, p.w, p.V, p.K, WN, fp4);
  if (rc) return rc;
  rc = mx_make_map(&x, p.x, p.B, p.K, bpad, false);
  if (rc) return rc;
  if (fp4) return bpad == 8 ? wide_launch_one<VQK_MODE_MXFP4, 8>(p, w, x, grid, st)
                            : wide_launch_one<VQK_MODE_MXFP4, 16>(p, w, x, grid, st);
  return bpad == 8 ? wide_launch_one<VQK_MODE_MXFP8, 8>(p, w, x, grid, st)
                   : wide_launch_one<VQK_MODE_MXFP8, 16>(p, w, x, grid, st);
}

int umma_wide_error_flag() { return read_stream_error(); }

}  // namespace vqk
