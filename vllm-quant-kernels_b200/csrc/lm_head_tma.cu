// Weight-streaming lm_head kernel, bulk-copy (TMA) pipeline: the decode path for H <= 4096.
//
// One persistent CTA per SM walks the 16-row vocab tiles (CTA c takes tiles c, c + grid, ...).
// A tile's rows are contiguous in HBM, so one producer thread fetches it with one
// cp.async.bulk per row into a ring of shared-memory stages (rows padded so that fragment
// reads are bank-conflict free); completion is signalled on an mbarrier.  Sixteen consumer
// warps split K sixteen ways: each reads its K slice of the tile from shared memory in the
// register layout of a warp-MMA A fragment, expands int8 -> fp16 (E2M1 -> e4m3) in
// registers, and multiplies with activation fragments that stay in registers for the whole
// kernel.  Four epilogue warps sum the sixteen partial tiles, apply the mode's scale, round
// to fp16 like the reference launchers, store logits if asked, and feed the sampler.
// No register staging of HBM loads, no L1 involvement: the bytes in flight are bounded by
// the ring (up to ~200 KB per SM), which is what a 7 TB/s stream needs.
//
// Every mbarrier wait is bounded; on expiry the kernel raises g_stream_error and drains.
#include <stdlib.h>

#include "lm_head.cuh"
#include "mma_helpers.cuh"
#include "async_helpers.cuh"

namespace vqk {


namespace tma {

constexpr int kConsumerWarps = 16;
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = (kConsumerWarps + kEpilogueWarps) * 32;  // 640: leaves 96 registers per thread
constexpr int kMaxStages = 8;

template <int MODE>
struct AccT { using type = float; };
template <>
struct AccT<VQK_MODE_W8A8> { using type = int; };

// ---- shared-memory geometry (host and device agree through these) ---------------------------
struct Geometry {
  int row_bytes;     // bytes of one quantized row
  int row_stride;    // padded stride of a row inside a stage
  int scale_bytes;   // MX: 16 rows of E8M0 scales, else 0
  int stage_bytes;   // 16 * row_stride + scale_bytes, rounded to 128
  int stages;
  size_t red_bytes;  // 2 buffers x 16 warps x NT x 128 x 4
  size_t sx_bytes;   // MX activation scales as floats
  size_t total;
};

__host__ __device__ inline Geometry geometry(int mode, int K, int NT) {
  Geometry g;
  const bool mx = (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4);
  g.row_bytes = (mode == VQK_MODE_MXFP4) ? K / 2 : K;
  // fragment reads are 16 B per lane (8 B MXFP8, 4 B MXFP4): consecutive rows must land
  // 64 / 32 / 16 bytes apart modulo the 128-byte bank window
  const int want = (mode == VQK_MODE_MXFP8) ? 32 : (mode == VQK_MODE_MXFP4 ? 16 : 64);
  int pad = (want - (g.row_bytes % 128) + 128) % 128;
  g.row_stride = g.row_bytes + pad;
  g.scale_bytes = mx ? 16 * (K / GROUP) : 0;
  g.stage_bytes = (16 * g.row_stride + g.scale_bytes + 127) & ~127;
  g.red_bytes = (size_t)2 * kConsumerWarps * NT * 128 * 4;
  g.sx_bytes = mx ? (size_t)(K / GROUP) * NT * 8 * sizeof(float) : 0;
  const size_t fixed = g.red_bytes + g.sx_bytes + (size_t)NT * 8 * sizeof(RowMeta) + 1024;
  const size_t limit = 227 * 1024;
  int s = fixed < limit ? (int)((limit - fixed) / g.stage_bytes) : 0;
  g.stages = s > kMaxStages ? kMaxStages : s;
  g.total = fixed + (size_t)g.stages * g.stage_bytes;
  return g;
}

// KPW: 64-byte k-steps per consumer warp (non-MX) or 32-element groups per warp (MX)
template <int MODE, int NT, int KPW>
__global__ void __launch_bounds__(kThreads, 1) k_lm_head_tma(const LmHeadParams p) {
  using acc_t = typename AccT<MODE>::type;
  constexpr bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4);
  extern __shared__ __align__(128) uint8_t smem[];
  const Geometry geo = geometry(MODE, p.K, NT);
  uint8_t* stage_base = smem;
  acc_t* red = reinterpret_cast<acc_t*>(smem + (size_t)geo.stages * geo.stage_bytes);
  float* sxf = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(red) + geo.red_bytes);
  RowMeta* meta = reinterpret_cast<RowMeta*>(reinterpret_cast<uint8_t*>(sxf) + geo.sx_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(meta) + (size_t)NT * 8 * sizeof(RowMeta));
  bars = reinterpret_cast<uint64_t*>(((uintptr_t)bars + 7) & ~(uintptr_t)7);
  uint64_t* full = bars;                   // [stages]
  uint64_t* empty = bars + kMaxStages;     // [stages]
  uint64_t* red_full = bars + 2 * kMaxStages;      // [2]
  uint64_t* red_empty = bars + 2 * kMaxStages + 2; // [2]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * kMaxStages + 4);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.K, V = p.V, B = p.B;
  const int ngroups = K / GROUP;
  const int S = geo.stages;
  const int ntiles = (V + 15) / 16;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kConsumerWarps); }
    for (int r = 0; r < 2; ++r) { mbar_init(&red_full[r], kConsumerWarps); mbar_init(&red_empty[r], kEpilogueWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (MX) {
    const uint8_t* xs = reinterpret_cast<const uint8_t*>(p.xscale);
    for (int s = tid; s < ngroups * NT * 8; s += kThreads) {
      int c = s & 7, nt = (s >> 3) % NT, G = s / (8 * NT);
      int b = nt * 8 + c;
      sxf[s] = b < B ? e8m0_to_f32(xs[(long long)b * ngroups + G]) * (MODE == VQK_MODE_MXFP4 ? kE2M1Rescale : 1.0f) : 0.f;
    }
  }
  if (p.do_sample && tid < NT * 8) {
    RowMeta m;
    m.flags = 0; m.T = 1.f; m.thr = -INFINITY; m.top_p = 1.f; m.top_k = 0; m.seed = 0;
    if (tid < B) m = decode_row(p.sp, tid);
    meta[tid] = m;
  }
  __syncthreads();

  if (warp < kConsumerWarps) {
    // ================================ consumers ========================================
    const int g = lane >> 2, t = lane & 3;
    // activation fragments for this warp's K slice, resident in registers for the whole kernel
    constexpr int MMAS = MX ? 1 : (MODE == VQK_MODE_W8A16 ? 4 : 2);
    uint2 xf[KPW][MMAS][NT];
#pragma unroll
    for (int j = 0; j < KPW; ++j)
#pragma unroll
      for (int i = 0; i < MMAS; ++i)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int b = nt * 8 + g;
          uint2 v = make_uint2(0, 0);
          if constexpr (MODE == VQK_MODE_W8A16) {
            const int k = (warp * KPW + j) * 64 + t * 16 + i * 4;
            if (b < B && k + 4 <= K) {
              __half h[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int kk = k + ((e & 1) * 2) + (e >> 1);  // order 0, 2, 1, 3 (see int8x4_to_half2_even_odd)
                float f = p.x_dtype == VQK_BF16
                              ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.x)[(long long)b * p.ldx + kk])
                              : __half2float(reinterpret_cast<const __half*>(p.x)[(long long)b * p.ldx + kk]);
                h[e] = __float2half_rn(f);
              }
              v = *reinterpret_cast<uint2*>(h);
            }
          } else if constexpr (!MX) {
            const int k = (warp * KPW + j) * 64 + t * 16 + i * 8;
            if (b < B && k + 8 <= K) v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.x) + (long long)b * K + k);
          } else {
            const int G = warp * KPW + j;
            if (b < B && G < ngroups) {
              v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.x) + (long long)b * K + G * 32 + t * 8);
              if constexpr (MODE == VQK_MODE_MXFP4)  // (0,2,4,6), (1,3,5,7) like the E2M1 expansion
                v = make_uint2(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531));
            }
          }
          xf[j][i][nt] = v;
        }

    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int s = it % S;
      const uint32_t ph = (uint32_t)(it / S) & 1u;
      const int rb = it & 1;
      const uint32_t rph = (uint32_t)(it >> 1) & 1u;
      acc_t acc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0;
      if (!mbar_wait_warp(&full[s], ph, abort_flag)) break;
      const uint8_t* st = stage_base + (size_t)s * geo.stage_bytes;
      const uint8_t* rowA = st + (size_t)g * geo.row_stride;
      const uint8_t* rowB = st + (size_t)(g + 8) * geo.row_stride;

      if constexpr (!MX) {
        uint4 a[KPW], b[KPW];
#pragma unroll
        for (int j = 0; j < KPW; ++j) {
          const int off = (warp * KPW + j) * 64 + t * 16;
          if (off + 16 <= K) {
            a[j] = *reinterpret_cast<const uint4*>(rowA + off);
            b[j] = *reinterpret_cast<const uint4*>(rowB + off);
          } else {
            a[j] = make_uint4(0, 0, 0, 0);
            b[j] = make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int j = 0; j < KPW; ++j) {
          const uint32_t wa[4] = {a[j].x, a[j].y, a[j].z, a[j].w};
          const uint32_t wb[4] = {b[j].x, b[j].y, b[j].z, b[j].w};
          if constexpr (MODE == VQK_MODE_W8A16) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint32_t a0, a1, a2, a3;
              int8x4_to_half2_even_odd(wa[i], a0, a2);
              int8x4_to_half2_even_odd(wb[i], a1, a3);
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) mma_f16(acc[nt], a0, a1, a2, a3, xf[j][i][nt].x, xf[j][i][nt].y);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                if constexpr (MODE == VQK_MODE_W8A8)
                  mma_s8(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], xf[j][i][nt].x, xf[j][i][nt].y);
                else
                  mma_e4m3(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], xf[j][i][nt].x, xf[j][i][nt].y);
              }
          }
        }
      } else {
        const uint8_t* sc = st + (size_t)16 * geo.row_stride;
#pragma unroll
        for (int j = 0; j < KPW; ++j) {
          const int G = warp * KPW + j;
          if (G < ngroups) {
            uint32_t a0, a1, a2, a3;
            if constexpr (MODE == VQK_MODE_MXFP8) {
              uint2 va = *reinterpret_cast<const uint2*>(rowA + G * 32 + t * 8);
              uint2 vb = *reinterpret_cast<const uint2*>(rowB + G * 32 + t * 8);
              a0 = va.x; a2 = va.y; a1 = vb.x; a3 = vb.y;
            } else {
              e2m1x8_to_e4m3_even_odd(*reinterpret_cast<const uint32_t*>(rowA + G * 16 + t * 4), a0, a2);
              e2m1x8_to_e4m3_even_odd(*reinterpret_cast<const uint32_t*>(rowB + G * 16 + t * 4), a1, a3);
            }
            const float fa = e8m0_to_f32(sc[g * ngroups + G]);
            const float fb = e8m0_to_f32(sc[(g + 8) * ngroups + G]);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              float2 sx = *reinterpret_cast<const float2*>(sxf + (size_t)(G * NT + nt) * 8 + 2 * t);
              float d[4] = {0.f, 0.f, 0.f, 0.f};
              mma_e4m3(d, a0, a1, a2, a3, xf[j][0][nt].x, xf[j][0][nt].y);
              acc[nt][0] = fmaf(d[0], fa * sx.x, acc[nt][0]);
              acc[nt][1] = fmaf(d[1], fa * sx.y, acc[nt][1]);
              acc[nt][2] = fmaf(d[2], fb * sx.x, acc[nt][2]);
              acc[nt][3] = fmaf(d[3], fb * sx.y, acc[nt][3]);
            }
          }
        }
      }
      // the stage has been read into registers: hand it back to the producer
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
      // partial tile -> reduction buffer rb (wait until the epilogue released it two tiles ago)
      if (!mbar_wait_warp(&red_empty[rb], rph ^ 1u, abort_flag)) break;
      acc_t* r = red + ((size_t)rb * kConsumerWarps + warp) * NT * 128;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        r[nt * 128 + (2 * t) * 16 + g] = acc[nt][0];
        r[nt * 128 + (2 * t + 1) * 16 + g] = acc[nt][1];
        r[nt * 128 + (2 * t) * 16 + g + 8] = acc[nt][2];
        r[nt * 128 + (2 * t + 1) * 16 + g + 8] = acc[nt][3];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[rb]);
    }
  } else {
    // ================================ epilogue =========================================
    const int e = tid - kConsumerWarps * 32;  // 0..127
    const int er = e & 15, ec = e >> 4;
    // four sampler slices per CTA (tile index modulo 4) keep the slice count at 4 x SMs
    float smax[NT][4], bs[NT][4];
    int bt[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int q = 0; q < 4; ++q) { smax[nt][q] = -INFINITY; bs[nt][q] = -INFINITY; bt[nt][q] = 0x7fffffff; }
    float xs_w8a8 = 1.f;
    if constexpr (MODE == VQK_MODE_W8A8) xs_w8a8 = *reinterpret_cast<const float*>(p.xscale);

    // Producer duty rides on one epilogue thread: it fills the ring up front, then refills a
    // stage right after the epilogue of the tile that used it (the consumers release a stage
    // before they publish that tile's partial sums, so the refill never waits).
    const bool producer = (e == 0);
    uint64_t policy = 0;
    auto issue = [&](int fill) {  // fill = index of this CTA's tile sequence
      const int tile = blockIdx.x + fill * gridDim.x;
      if (tile >= ntiles) return true;
      const int s = fill % S;
      const uint32_t ph = (uint32_t)(fill / S) & 1u;
      if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) return false;
      const int row0 = tile * 16;
      uint8_t* st = stage_base + (size_t)s * geo.stage_bytes;
      uint32_t bytes = 16u * (uint32_t)geo.row_bytes;
      if (MX) bytes += 16u * (uint32_t)ngroups;
      mbar_expect_tx(&full[s], bytes);
      const uint8_t* src = p.w + (size_t)row0 * geo.row_bytes;
#pragma unroll 4
      for (int r = 0; r < 16; ++r)
        bulk_g2s(st + (size_t)r * geo.row_stride, src + (size_t)r * geo.row_bytes, (uint32_t)geo.row_bytes, &full[s],
                 policy);
      if (MX)
        bulk_g2s(st + (size_t)16 * geo.row_stride, reinterpret_cast<const uint8_t*>(p.wscale) + (size_t)row0 * ngroups,
                 16u * (uint32_t)ngroups, &full[s], policy);
      return true;
    };
    if (producer) {
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
      for (int f = 0; f < S; ++f)
        if (!issue(f)) break;
    }
    __syncwarp();

    int it = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++it) {
      const int rb = it & 1;
      const uint32_t rph = (uint32_t)(it >> 1) & 1u;
      const int row = tile * 16 + er;
      // fetch the per-row constants while the consumers are still busy
      float rs = 1.f, bias = 0.f;
      if (row < V) {
        if constexpr (MODE == VQK_MODE_W8A16 || MODE == VQK_MODE_FP8)
          rs = __half2float(reinterpret_cast<const __half*>(p.wscale)[row]);
        if constexpr (MODE == VQK_MODE_W8A8) rs = reinterpret_cast<const float*>(p.wscale)[row];
        if (p.bias) bias = __half2float(p.bias[row]);
      }
      if (!mbar_wait_warp(&red_full[rb], rph, abort_flag)) break;
      const acc_t* r = red + (size_t)rb * kConsumerWarps * NT * 128;
      acc_t sum[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc_t s = 0;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += r[((size_t)w * NT + nt) * 128 + e];
        sum[nt] = s;
      }
      __syncwarp();
      if ((tid & 31) == 0) mbar_arrive(&red_empty[rb]);
      if (warp == kConsumerWarps) {  // warp-uniform exit if the refill gave up
        bool ok = true;
        if (producer) ok = issue(it + S);
        if (!__all_sync(0xffffffffu, ok)) break;
      }
      if (row < V) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int b = nt * 8 + ec;
          if (b < B) {
            float v;
            if constexpr (MODE == VQK_MODE_W8A8) v = ((float)sum[nt] * rs) * xs_w8a8;  // _kernels.py:471, left to right
            else if constexpr (MX) v = sum[nt];
            else v = sum[nt] * rs;
            __half h = __float2half_rn(v);
            if (p.bias) h = __float2half_rn(__half2float(h) + bias);
            if (p.logits) p.logits[(long long)b * p.ld_logits + row] = h;
            if (p.do_sample) {
              const RowMeta m = meta[b];
              const float l = __half2float(h);
              if (m.flags & ROW_CAND) {
                p.cand_logits[(long long)b * p.ld_cand + row] = h;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  if (q == (it & 3)) smax[nt][q] = fmaxf(smax[nt][q], l);
              } else {
                float sc = l;
                if (!(m.flags & ROW_GREEDY)) {
                  sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(row + p.sp.vocab_offset));
                  if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  if (q == (it & 3) && better(sc, row, bs[nt][q], bt[nt][q])) { bs[nt][q] = sc; bt[nt][q] = row; }
              }
            }
          }
        }
      }
    }
    // sampler slices: reduce the 16 row-threads of each column (a half warp), 4 slices per CTA
    if (p.do_sample) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float m = smax[nt][q], s = bs[nt][q];
          int tk = bt[nt][q];
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) {
            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            float s2 = __shfl_xor_sync(0xffffffffu, s, o);
            int t2 = __shfl_xor_sync(0xffffffffu, tk, o);
            if (better(s2, t2, s, tk)) { s = s2; tk = t2; }
          }
          const int b = nt * 8 + ec;
          if (er == 0 && b < B) {
            const long long o = (long long)b * p.nslices + blockIdx.x * 4 + q;
            p.slice_max[o] = m;
            p.part_score[o] = s;
            p.part_token[o] = tk;
          }
        }
    }
  }
}

template <int MODE, int NT, int KPW>
static int launch_one(const LmHeadParams& p, int grid, cudaStream_t st) {
  const Geometry geo = geometry(MODE, p.K, NT);
  static size_t configured[64] = {};
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (geo.total > configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_tma<MODE, NT, KPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)geo.total));
    configured[dev] = geo.total;
  }
  k_lm_head_tma<MODE, NT, KPW><<<grid, kThreads, geo.total, st>>>(p);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

template <int MODE, int NT>
static int launch_kpw(const LmHeadParams& p, int kpw, int grid, cudaStream_t st) {
  constexpr bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4);
  switch (kpw) {
    case 1: return launch_one<MODE, NT, 1>(p, grid, st);
    case 2: return launch_one<MODE, NT, 2>(p, grid, st);
    case 3: return launch_one<MODE, NT, 3>(p, grid, st);
    case 4: return launch_one<MODE, NT, 4>(p, grid, st);
    case 5: if constexpr (MX) return launch_one<MODE, NT, 6>(p, grid, st); break;
    case 6: if constexpr (MX) return launch_one<MODE, NT, 6>(p, grid, st); break;
    case 7: if constexpr (MX) return launch_one<MODE, NT, 8>(p, grid, st); break;
    case 8: if constexpr (MX) return launch_one<MODE, NT, 8>(p, grid, st); break;
  }
  return VQK_ERR_UNSUPPORTED;
}

}  // namespace tma

// units of K one consumer warp owns: 64-byte k-steps, or MX groups
static int tma_kpw(int mode, int K) {
  const bool mx = (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4);
  const int units = mx ? K / GROUP : (K + 63) / 64;
  return (units + tma::kConsumerWarps - 1) / tma::kConsumerWarps;
}

// batch columns one launch of the bulk-copy kernel can take for this shape (0: use the
// register-streaming kernel instead)
int tma_max_cols(int mode, int K) {
  const bool mx = (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4);
  const int kpw = tma_kpw(mode, K);
  if (kpw > (mx ? 8 : 4)) return 0;
  const int maxnt = 2;
  for (int nt = maxnt; nt >= 1; nt >>= 1)
    if (tma::geometry(mode, K, nt).stages >= 2) return nt * 8;
  return 0;
}

int launch_lm_head_tma(int mode, const LmHeadParams& p, int grid, cudaStream_t st) {
  using namespace tma;
  const int NT = p.B <= 8 ? 1 : 2;
  if (NT * 8 > tma_max_cols(mode, p.K)) return VQK_ERR_UNSUPPORTED;
  const int kpw = tma_kpw(mode, p.K);
  switch (mode) {
    case VQK_MODE_W8A16: return NT == 1 ? launch_kpw<VQK_MODE_W8A16, 1>(p, kpw, grid, st) : launch_kpw<VQK_MODE_W8A16, 2>(p, kpw, grid, st);
    case VQK_MODE_W8A8: return NT == 1 ? launch_kpw<VQK_MODE_W8A8, 1>(p, kpw, grid, st) : launch_kpw<VQK_MODE_W8A8, 2>(p, kpw, grid, st);
    case VQK_MODE_FP8: return NT == 1 ? launch_kpw<VQK_MODE_FP8, 1>(p, kpw, grid, st) : launch_kpw<VQK_MODE_FP8, 2>(p, kpw, grid, st);
    case VQK_MODE_MXFP8: return NT == 1 ? launch_kpw<VQK_MODE_MXFP8, 1>(p, kpw, grid, st) : launch_kpw<VQK_MODE_MXFP8, 2>(p, kpw, grid, st);
    case VQK_MODE_MXFP4: return NT == 1 ? launch_kpw<VQK_MODE_MXFP4, 1>(p, kpw, grid, st) : launch_kpw<VQK_MODE_MXFP4, 2>(p, kpw, grid, st);
  }
  return VQK_ERR_INVALID;
}

int stream_error_flag() { return read_stream_error(); }

}  // namespace vqk
