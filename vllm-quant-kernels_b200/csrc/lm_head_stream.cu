// Weight-streaming lm_head kernel for small batches (decode): one persistent CTA per SM,
// 16 warps = 4 groups x 4 warps.  A group owns one 16-row vocab tile at a time and its four
// warps split K; every lane streams 16 B (8 B / 4 B for the MX modes) of two weight rows
// straight from HBM into registers in the layout of a warp-level MMA A fragment, so the
// only per-byte ALU work is the int8 -> fp16 (or E2M1 -> e4m3) expansion.  Activations sit in
// shared memory, pre-arranged as B fragments.  The epilogue applies the mode's scale,
// rounds to fp16 exactly like the reference launchers, optionally stores the logits, and
// feeds the sampler (per-slice maxima, per-slice Gumbel winners) without a second pass.
//
// Replaces int8_gmv / int8_gemm / fp8_gemm / int8_w8a8_gemm / mxfp8_gemm / mxfp4_gemm of the
// reference (src/vllm_quant_kernels/_kernels.py) for batch <= 32.
#include <stdlib.h>

#include "lm_head.cuh"

namespace vqk {

__device__ __forceinline__ uint4 ldg_stream16(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ uint2 ldg_stream8(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const uint2*>(p));
}
__device__ __forceinline__ uint32_t ldg_stream4(const uint8_t* p) {
  return __ldcs(reinterpret_cast<const unsigned int*>(p));
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_e4m3(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// four int8 -> two half2 holding the exact integer values: (b ^ 0x80) | 0x6400 is 1024 + (b + 128)
__device__ __forceinline__ void int8x4_to_half2x2(uint32_t w, uint32_t& lo, uint32_t& hi) {
  uint32_t x = w ^ 0x80808080u;
  uint32_t l = __byte_perm(x, 0x64646464u, 0x4140);
  uint32_t h = __byte_perm(x, 0x64646464u, 0x4342);
  const uint32_t bias = 0x64806480u;  // half2(1152, 1152)
  __half2 lh = __hsub2(*reinterpret_cast<__half2*>(&l), *reinterpret_cast<const __half2*>(&bias));
  __half2 hh = __hsub2(*reinterpret_cast<__half2*>(&h), *reinterpret_cast<const __half2*>(&bias));
  lo = *reinterpret_cast<uint32_t*>(&lh);
  hi = *reinterpret_cast<uint32_t*>(&hh);
}

// eight packed E2M1 nibbles (element j in nibble j) -> two words of four e4m3 bytes
__device__ __forceinline__ void e2m1x8_to_e4m3x8(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t LUT_LO = 0x3C383000u;  // 0, 0.5, 1, 1.5
  const uint32_t LUT_HI = 0x4C484440u;  // 2, 3, 4, 6
  uint32_t m0 = __byte_perm(LUT_LO, LUT_HI, w & 0x7777u);
  uint32_t m1 = __byte_perm(LUT_LO, LUT_HI, (w >> 16) & 0x7777u);
  uint32_t w4 = w << 4;
  // msb-replicate mode: output byte j = 0xff if the sign bit of nibble j is set
  uint32_t s0 = __byte_perm(w4, w, 0xD9C8);
  uint32_t s1 = __byte_perm(w4, w, 0xFBEA);
  lo = m0 | (s0 & 0x80808080u);
  hi = m1 | (s1 & 0x80808080u);
}

template <int MODE>
struct AccT { using type = float; };
template <>
struct AccT<VQK_MODE_W8A8> { using type = int; };

constexpr int kThreads = 512;
constexpr int kGroups = 4;

// shared memory carve-up (bytes) -----------------------------------------------------------
__host__ __device__ inline size_t stream_xfrag_bytes(int mode, int K, int NT) {
  int k64 = (K + 63) / 64 * 64;
  return (size_t)k64 * NT * (mode == VQK_MODE_W8A16 ? 16 : 8);
}
__host__ __device__ inline size_t stream_sx_bytes(int mode, int K, int NT) {
  return (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4) ? (size_t)(K / GROUP) * NT * 8 * sizeof(float) : 0;
}
__host__ __device__ inline size_t stream_red_bytes(int NT) { return (size_t)16 * NT * 128 * 4; }
size_t stream_smem_bytes(int mode, int K, int NT) {
  return stream_xfrag_bytes(mode, K, NT) + stream_sx_bytes(mode, K, NT) + stream_red_bytes(NT) +
         (size_t)NT * 8 * sizeof(RowMeta);
}

template <int MODE, int NT>
__global__ void __launch_bounds__(kThreads, 1) k_lm_head_stream(const LmHeadParams p) {
  using acc_t = typename AccT<MODE>::type;
  constexpr bool MX = (MODE == VQK_MODE_MXFP8 || MODE == VQK_MODE_MXFP4);
  extern __shared__ __align__(16) uint8_t smem[];
  uint2* xfrag = reinterpret_cast<uint2*>(smem);
  float* sxf = reinterpret_cast<float*>(smem + stream_xfrag_bytes(MODE, p.K, NT));
  acc_t* red = reinterpret_cast<acc_t*>(smem + stream_xfrag_bytes(MODE, p.K, NT) + stream_sx_bytes(MODE, p.K, NT));
  RowMeta* meta = reinterpret_cast<RowMeta*>(reinterpret_cast<uint8_t*>(red) + stream_red_bytes(NT));

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = warp >> 2, wq = warp & 3;
  const int g = lane >> 2, t = lane & 3;
  const int K = p.K, V = p.V, B = p.B;
  const int ngroups = K / GROUP;
  const int nks = (K + 63) / 64;

  // ---- prologue: activations -> B fragments in shared memory -------------------------
  if constexpr (MODE == VQK_MODE_W8A16) {
    const int total = nks * 4 * NT * 32;
    for (int s = tid; s < total; s += kThreads) {
      int l = s & 31, nt = (s >> 5) % NT, i = (s / (32 * NT)) & 3, ks = s / (128 * NT);
      int b = nt * 8 + (l >> 2), k = ks * 64 + (l & 3) * 16 + i * 4;
      __half h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = 0.f;
        if (b < B && k + j < K) {
          v = p.x_dtype == VQK_BF16
                  ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.x)[(long long)b * p.ldx + k + j])
                  : __half2float(reinterpret_cast<const __half*>(p.x)[(long long)b * p.ldx + k + j]);
        }
        h[j] = __float2half_rn(v);
      }
      xfrag[s] = *reinterpret_cast<uint2*>(h);
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
      if (b < B) v = *reinterpret_cast<const uint2*>(xq + (long long)b * K + k);
      xfrag[s] = v;
    }
    for (int s = tid; s < ngroups * NT * 8; s += kThreads) {
      int c = s & 7, nt = (s >> 3) % NT, G = s / (8 * NT);
      int b = nt * 8 + c;
      sxf[s] = b < B ? e8m0_to_f32(xs[(long long)b * ngroups + G]) : 0.f;
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

  // ---- per-thread sampler state: epilogue thread e of a group owns (row e%16, col e/16) ----
  const int e = tid & 127;
  const int er = e & 15, ec = e >> 4;
  float smax[NT], bs[NT];
  int bt[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) { smax[nt] = -INFINITY; bs[nt] = -INFINITY; bt[nt] = 0x7fffffff; }

  const int ntiles = (V + 15) / 16;
  const size_t rowbytes = (MODE == VQK_MODE_MXFP4) ? (size_t)K / 2 : (size_t)K;
  acc_t* myred = red + (size_t)warp * NT * 128;
  const acc_t* gred = red + (size_t)(group * 4) * NT * 128;

  for (int tile = blockIdx.x * kGroups + group; tile < ntiles; tile += gridDim.x * kGroups) {
    const int row0 = tile * 16;
    const int rA = min(row0 + g, V - 1), rB = min(row0 + g + 8, V - 1);
    const uint8_t* pA = p.w + (size_t)rA * rowbytes;
    const uint8_t* pB = p.w + (size_t)rB * rowbytes;
    acc_t acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0;

    if constexpr (!MX) {
      constexpr int U = 6;
      const int per = (nks + 3) / 4;  // k-steps per warp
      for (int j0 = 0; j0 < per; j0 += U) {
        uint4 a[U], b[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = j0 + u;
          const int ks = p.contig ? wq * per + j : wq + 4 * j;
          const int off = ks * 64 + t * 16;
          if (j < per && off + 16 <= K) {
            a[u] = ldg_stream16(pA + off);
            b[u] = ldg_stream16(pB + off);
          } else {
            a[u] = make_uint4(0, 0, 0, 0);
            b[u] = make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = j0 + u;
          const int ks = p.contig ? wq * per + j : wq + 4 * j;
          if (j < per && ks < nks) {
            const uint32_t wa[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
            const uint32_t wb[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
            if constexpr (MODE == VQK_MODE_W8A16) {
              const uint2* xf = xfrag + (size_t)(ks * 4) * NT * 32 + lane;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint32_t a0, a1, a2, a3;
                int8x4_to_half2x2(wa[i], a0, a2);
                int8x4_to_half2x2(wb[i], a1, a3);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  uint2 bf = xf[(i * NT + nt) * 32];
                  mma_f16(acc[nt], a0, a1, a2, a3, bf.x, bf.y);
                }
              }
            } else {
              const uint2* xf = xfrag + (size_t)(ks * 2) * NT * 32 + lane;
#pragma unroll
              for (int i = 0; i < 2; ++i) {
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  uint2 bf = xf[(i * NT + nt) * 32];
                  if constexpr (MODE == VQK_MODE_W8A8)
                    mma_s8(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], bf.x, bf.y);
                  else
                    mma_e4m3(acc[nt], wa[2 * i], wb[2 * i], wa[2 * i + 1], wb[2 * i + 1], bf.x, bf.y);
                }
              }
            }
          }
        }
      }
    } else {
      // MX: one MMA per 32-element scale group; warps take chunks of 8 groups round-robin
      const uint8_t* ws = reinterpret_cast<const uint8_t*>(p.wscale);
      const uint8_t* sA = ws + (size_t)rA * ngroups;
      const uint8_t* sB = ws + (size_t)rB * ngroups;
      const bool sc_aligned = (ngroups & 7) == 0;
      const int nchunks = (ngroups + 7) / 8;
      for (int c = wq; c < nchunks; c += 4) {
        const int G0 = c * 8;
        uint32_t qa[8][2], qb[8][2];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int G = G0 + j;
          if (G < ngroups) {
            if constexpr (MODE == VQK_MODE_MXFP8) {
              uint2 va = ldg_stream8(pA + G * 32 + t * 8), vb = ldg_stream8(pB + G * 32 + t * 8);
              qa[j][0] = va.x; qa[j][1] = va.y; qb[j][0] = vb.x; qb[j][1] = vb.y;
            } else {
              qa[j][0] = ldg_stream4(pA + G * 16 + t * 4);
              qb[j][0] = ldg_stream4(pB + G * 16 + t * 4);
              qa[j][1] = 0; qb[j][1] = 0;
            }
          } else {
            qa[j][0] = qa[j][1] = qb[j][0] = qb[j][1] = 0;
          }
        }
        uint32_t scA[2], scB[2];
        if (sc_aligned) {
          uint2 va = __ldg(reinterpret_cast<const uint2*>(sA + G0));
          uint2 vb = __ldg(reinterpret_cast<const uint2*>(sB + G0));
          scA[0] = va.x; scA[1] = va.y; scB[0] = vb.x; scB[1] = vb.y;
        } else {
          scA[0] = scA[1] = scB[0] = scB[1] = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (G0 + j < ngroups) {
              scA[j >> 2] |= (uint32_t)__ldg(sA + G0 + j) << (8 * (j & 3));
              scB[j >> 2] |= (uint32_t)__ldg(sB + G0 + j) << (8 * (j & 3));
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int G = G0 + j;
          if (G < ngroups) {
            uint32_t a0, a1, a2, a3;
            if constexpr (MODE == VQK_MODE_MXFP8) {
              a0 = qa[j][0]; a2 = qa[j][1]; a1 = qb[j][0]; a3 = qb[j][1];
            } else {
              e2m1x8_to_e4m3x8(qa[j][0], a0, a2);
              e2m1x8_to_e4m3x8(qb[j][0], a1, a3);
            }
            const float fa = e8m0_to_f32((scA[j >> 2] >> (8 * (j & 3))) & 0xff);
            const float fb = e8m0_to_f32((scB[j >> 2] >> (8 * (j & 3))) & 0xff);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              uint2 bf = xfrag[(size_t)(G * NT + nt) * 32 + lane];
              float2 sx = *reinterpret_cast<const float2*>(sxf + (size_t)(G * NT + nt) * 8 + 2 * t);
              float d[4] = {0.f, 0.f, 0.f, 0.f};
              mma_e4m3(d, a0, a1, a2, a3, bf.x, bf.y);
              acc[nt][0] = fmaf(d[0], fa * sx.x, acc[nt][0]);
              acc[nt][1] = fmaf(d[1], fa * sx.y, acc[nt][1]);
              acc[nt][2] = fmaf(d[2], fb * sx.x, acc[nt][2]);
              acc[nt][3] = fmaf(d[3], fb * sx.y, acc[nt][3]);
            }
          }
        }
      }
    }

    // ---- cross-warp (split-K) reduction through shared memory --------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      acc_t* r = myred + nt * 128;
      r[(2 * t) * 16 + g] = acc[nt][0];
      r[(2 * t + 1) * 16 + g] = acc[nt][1];
      r[(2 * t) * 16 + g + 8] = acc[nt][2];
      r[(2 * t + 1) * 16 + g + 8] = acc[nt][3];
    }
    asm volatile("bar.sync %0, 128;" ::"r"(group + 1));

    // ---- epilogue: thread e -> (vocab row row0 + er, batch column nt*8 + ec) ------------
    const int row = row0 + er;
    if (row < V) {
      float rs = 1.f;
      if constexpr (MODE == VQK_MODE_W8A16 || MODE == VQK_MODE_FP8)
        rs = __half2float(reinterpret_cast<const __half*>(p.wscale)[row]);
      if constexpr (MODE == VQK_MODE_W8A8) rs = reinterpret_cast<const float*>(p.wscale)[row];
      float bias = p.bias ? __half2float(p.bias[row]) : 0.f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int b = nt * 8 + ec;
        if (b < B) {
          acc_t s = gred[0 * NT * 128 + nt * 128 + e] + gred[1 * NT * 128 + nt * 128 + e] +
                    gred[2 * NT * 128 + nt * 128 + e] + gred[3 * NT * 128 + nt * 128 + e];
          float v;
          if constexpr (MODE == VQK_MODE_W8A8) v = ((float)s * rs) * xs_w8a8;   // _kernels.py:471, left to right
          else if constexpr (MX) v = s;
          else v = s * rs;
          __half h = __float2half_rn(v);
          if (p.bias) h = __float2half_rn(__half2float(h) + bias);
          if (p.logits) p.logits[(long long)b * p.ld_logits + row] = h;
          if (p.do_sample) {
            const RowMeta m = meta[b];
            const float l = __half2float(h);
            if (m.flags & ROW_CAND) {
              p.cand_logits[(long long)b * p.ld_cand + row] = h;
              smax[nt] = fmaxf(smax[nt], l);
            } else {
              float sc = l;
              const int tok = row;  // local id; offset added by the consumer
              if (!(m.flags & ROW_GREEDY)) {
                sc = l / m.T + gumbel_noise(m.seed, (uint32_t)(row + p.sp.vocab_offset));
                if ((m.flags & ROW_MASK_THR) && !(l >= m.thr)) sc = -INFINITY;
              }
              if (better(sc, tok, bs[nt], bt[nt])) { bs[nt] = sc; bt[nt] = tok; }
            }
          }
        }
      }
    }
    asm volatile("bar.sync %0, 128;" ::"r"(group + 1));
  }

  // ---- per-slice sampler results: reduce over the 16 row-threads of each column ----------
  if (p.do_sample) {
    const int slice = blockIdx.x * kGroups + group;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float m = smax[nt], s = bs[nt];
      int tk = bt[nt];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        int t2 = __shfl_xor_sync(0xffffffffu, tk, o);
        if (better(s2, t2, s, tk)) { s = s2; tk = t2; }
      }
      const int b = nt * 8 + ec;
      if (er == 0 && b < B) {
        p.slice_max[(long long)b * p.nslices + slice] = m;
        p.part_score[(long long)b * p.nslices + slice] = s;
        p.part_token[(long long)b * p.nslices + slice] = tk;
      }
    }
  }
}

// ---- host launch -------------------------------------------------------------------------
template <int MODE, int NT>
static int launch_stream(const LmHeadParams& p, int grid, cudaStream_t st) {
  size_t smem = stream_smem_bytes(MODE, p.K, NT);
  static size_t configured[64] = {};  // per device: largest opt-in so far for this instantiation
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (smem > configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_stream<MODE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  k_lm_head_stream<MODE, NT><<<grid, kThreads, smem, st>>>(p);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

template <int MODE>
static int launch_stream_nt(const LmHeadParams& p, int NT, int grid, cudaStream_t st) {
  switch (NT) {
    case 1: return launch_stream<MODE, 1>(p, grid, st);
    case 2: return launch_stream<MODE, 2>(p, grid, st);
    case 4:
      if constexpr (MODE != VQK_MODE_W8A16) return launch_stream<MODE, 4>(p, grid, st);
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

int launch_lm_head_stream(int mode, const LmHeadParams& p_in, int grid, cudaStream_t st) {
  static const int contig = [] { const char* e = getenv("VQK_STREAM_CONTIG"); return e ? atoi(e) : 1; }();
  LmHeadParams p = p_in;
  p.contig = contig;
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
