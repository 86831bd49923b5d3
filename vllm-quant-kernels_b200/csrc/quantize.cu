// Offline weight quantizers and runtime activation quantizers (bit-exact with the
// reference's torch arithmetic: fp32 true division, round-half-even, non-saturating
// e4m3 cast, ceil(log2) MX scale, E2M1 midpoint ties toward the smaller magnitude).
#include "vqk_common.cuh"

namespace vqk {

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p, long long i) { return to_f32<T>(p[i]); }

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  int nw = (blockDim.x + 31) >> 5;
  v = (l < nw) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  return v;
}

// NaN-propagating |x| max is not needed: torch's amax propagates NaN, weights are finite.

// ---- per-row INT8 / FP8 (reference _quant.py:248-255, 285-292, 306-314) ---------------
// MODE 0: int8, fp16 scale; 1: int8, fp32 scale; 2: e4m3, fp16 scale
template <typename T, int MODE>
__global__ void __launch_bounds__(256) k_quant_rows(const T* __restrict__ w, long long ldw, int H,
                                                    uint8_t* __restrict__ q, void* __restrict__ scales) {
  __shared__ float red[32];
  long long row = blockIdx.x;
  const T* wr = w + row * ldw;
  float m = 0.f;
  for (int k = threadIdx.x; k < H; k += blockDim.x) m = fmaxf(m, fabsf(ld_f32(wr, k)));
  m = block_max(m, red);
  const float denom = (MODE == 2) ? 448.0f : 127.0f;
  float s = fmaxf(m / denom, 1e-12f);
  if (threadIdx.x == 0) {
    if (MODE == 1) reinterpret_cast<float*>(scales)[row] = s;
    else reinterpret_cast<__half*>(scales)[row] = __float2half_rn(s);
  }
  uint8_t* qr = q + row * (long long)H;
  for (int k = threadIdx.x; k < H; k += blockDim.x) {
    float v = ld_f32(wr, k) / s;
    if (MODE == 2) {
      v = fminf(fmaxf(v, -448.0f), 448.0f);
      qr[k] = f32_to_e4m3_nosat(v);
    } else {
      v = fminf(fmaxf(rintf(v), -127.0f), 127.0f);
      qr[k] = (uint8_t)(int8_t)(int)v;
    }
  }
}

// ---- MXFP8 / MXFP4: one warp per group of 32 (reference _quant.py:34-105) -------------
template <typename T, bool FP4>
__global__ void __launch_bounds__(256) k_quant_mx(const T* __restrict__ x, long long ldx, long long R, int H,
                                                  uint8_t* __restrict__ q, uint8_t* __restrict__ scales) {
  pdl_launch_dependents();  // an lm_head kernel behind this one may start its set-up now
  const int lane = threadIdx.x & 31;
  const int ngroups = H / GROUP;
  long long gid = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gid >= R * ngroups) return;
  long long row = gid / ngroups;
  int g = (int)(gid - row * ngroups);
  float v = ld_f32(x + row * ldx, (long long)g * GROUP + lane);
  float m = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  m = fmaxf(m, 1e-30f);
  int e = ceil_log2_clamped(m / (FP4 ? 6.0f : 448.0f));
  if (lane == 0) scales[row * ngroups + g] = (uint8_t)(e + 127);
  float sc = (e == -127) ? __uint_as_float(0x00400000u) : __uint_as_float((uint32_t)(e + 127) << 23);
  float sv = v / sc;
  if (!FP4) {
    sv = fminf(fmaxf(sv, -448.0f), 448.0f);
    q[row * (long long)H + (long long)g * GROUP + lane] = f32_to_e4m3_nosat(sv);
  } else {
    uint32_t sign = (sv < 0.f) ? 8u : 0u;
    float a = fminf(fabsf(sv), 6.0f);
    // number of midpoints strictly below |v| (torch.bucketize, right=False)
    uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
    uint32_t nib = sign | idx;
    uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
    if ((lane & 1) == 0)
      q[row * (long long)(H / 2) + (long long)g * (GROUP / 2) + (lane >> 1)] = (uint8_t)((other << 4) | nib);
  }
}

// ---- activations -----------------------------------------------------------------------
template <typename T>
__global__ void k_act_to_f16(const T* __restrict__ x, long long ldx, int H, __half* __restrict__ out) {
  long long row = blockIdx.y;
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < H; k += gridDim.x * blockDim.x)
    out[row * H + k] = __float2half_rn(ld_f32(x + row * ldx, k));
}

// `x.to(torch.float8_e4m3fn)`: for bf16 input torch converts bf16 -> e4m3 directly, for fp16
// likewise; both widen to fp32 exactly first, so one rounding either way.
template <typename T>
__global__ void k_act_fp8(const T* __restrict__ x, long long ldx, int H, uint8_t* __restrict__ out) {
  pdl_launch_dependents();
  long long row = blockIdx.y;
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < H; k += gridDim.x * blockDim.x)
    out[row * H + k] = f32_to_e4m3_nosat(ld_f32(x + row * ldx, k));
}

// per-tensor absmax: xs[1] holds the running max as uint bits (non-negative floats order
// like unsigned integers); zeroed by the host-side memset before this kernel.
template <typename T>
__global__ void __launch_bounds__(256) k_act_absmax(const T* __restrict__ x, long long ldx, int H, float* xs) {
  __shared__ float red[32];
  long long row = blockIdx.y;
  float m = 0.f;
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < H; k += gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(ld_f32(x + row * ldx, k)));
  m = block_max(m, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(xs + 1), __float_as_uint(m));
}

template <typename T>
__global__ void k_act_int8(const T* __restrict__ x, long long ldx, int H, int8_t* __restrict__ out, float* xs) {
  pdl_launch_dependents();
  long long row = blockIdx.y;
  float s = fmaxf(xs[1] / 127.0f, 1e-12f);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) xs[0] = s;
  for (int k = blockIdx.x * blockDim.x + threadIdx.x; k < H; k += gridDim.x * blockDim.x) {
    float v = rintf(ld_f32(x + row * ldx, k) / s);
    out[row * H + k] = (int8_t)(int)fminf(fmaxf(v, -127.0f), 127.0f);
  }
}

// Decode-sized batches: absmax and quantisation by ONE block (no memset, no second launch); the
// same arithmetic as the pair above.
constexpr long long kActInt8OneBlock = 32768;  // elements (B * H) the single block takes (beyond: one block per row is faster)
template <typename T>
__global__ void __launch_bounds__(1024) k_act_int8_one(const T* __restrict__ x, long long ldx, int B, int H,
                                                       int8_t* __restrict__ out, float* xs) {
  pdl_launch_dependents();
  __shared__ float red[32];
  __shared__ float s_scale;
  float m = 0.f;
  for (int r = 0; r < B; ++r)
    for (int c = threadIdx.x; c < H; c += blockDim.x) m = fmaxf(m, fabsf(ld_f32(x + (long long)r * ldx, c)));
  m = block_max(m, red);
  if (threadIdx.x == 0) {
    s_scale = fmaxf(m / 127.0f, 1e-12f);
    xs[0] = s_scale;
    xs[1] = m;
  }
  __syncthreads();
  const float s = s_scale;
  for (int r = 0; r < B; ++r)
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float v = rintf(ld_f32(x + (long long)r * ldx, c) / s);
      out[(long long)r * H + c] = (int8_t)(int)fminf(fmaxf(v, -127.0f), 127.0f);
    }
}

// ---- host dispatch ------------------------------------------------------------------------
template <typename T>
static int quantize_weight_t(int mode, const T* w, long long V, long long H, long long ldw, void* q, void* scales,
                             cudaStream_t st) {
  if (V == 0) return VQK_OK;
  switch (mode) {
    case VQK_MODE_W8A16: k_quant_rows<T, 0><<<(unsigned)V, 256, 0, st>>>(w, ldw, (int)H, (uint8_t*)q, scales); break;
    case VQK_MODE_W8A8: k_quant_rows<T, 1><<<(unsigned)V, 256, 0, st>>>(w, ldw, (int)H, (uint8_t*)q, scales); break;
    case VQK_MODE_FP8: k_quant_rows<T, 2><<<(unsigned)V, 256, 0, st>>>(w, ldw, (int)H, (uint8_t*)q, scales); break;
    case VQK_MODE_MXFP8:
    case VQK_MODE_MXFP4: {
      if (H % GROUP) return VQK_ERR_INVALID;
      long long groups = V * (H / GROUP);
      unsigned blocks = (unsigned)((groups + 7) / 8);
      if (mode == VQK_MODE_MXFP8)
        k_quant_mx<T, false><<<blocks, 256, 0, st>>>(w, ldw, V, (int)H, (uint8_t*)q, (uint8_t*)scales);
      else
        k_quant_mx<T, true><<<blocks, 256, 0, st>>>(w, ldw, V, (int)H, (uint8_t*)q, (uint8_t*)scales);
      break;
    }
    default: return VQK_ERR_INVALID;
  }
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

template <typename T>
static int quantize_act_t(int mode, const T* x, long long B, long long H, long long ldx, void* xq, void* xs,
                          cudaStream_t st) {
  if (B == 0) return VQK_OK;
  dim3 grid((unsigned)((H + 1023) / 1024), (unsigned)B);
  switch (mode) {
    case VQK_MODE_W8A16: k_act_to_f16<T><<<grid, 256, 0, st>>>(x, ldx, (int)H, (__half*)xq); break;
    case VQK_MODE_FP8: k_act_fp8<T><<<grid, 256, 0, st>>>(x, ldx, (int)H, (uint8_t*)xq); break;
    case VQK_MODE_W8A8:
      if (!xs) return VQK_ERR_INVALID;
      if (B * H <= kActInt8OneBlock) {
        k_act_int8_one<T><<<1, 1024, 0, st>>>(x, ldx, (int)B, (int)H, (int8_t*)xq, (float*)xs);
        break;
      }
      VQK_CUDA(cudaMemsetAsync(xs, 0, 2 * sizeof(float), st));
      k_act_absmax<T><<<grid, 256, 0, st>>>(x, ldx, (int)H, (float*)xs);
      k_act_int8<T><<<grid, 256, 0, st>>>(x, ldx, (int)H, (int8_t*)xq, (float*)xs);
      break;
    case VQK_MODE_MXFP8:
    case VQK_MODE_MXFP4: {
      if (H % GROUP || !xs) return VQK_ERR_INVALID;
      long long groups = B * (H / GROUP);
      k_quant_mx<T, false><<<(unsigned)((groups + 7) / 8), 256, 0, st>>>(x, ldx, B, (int)H, (uint8_t*)xq, (uint8_t*)xs);
      break;
    }
    default: return VQK_ERR_INVALID;
  }
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

int quantize_act_dispatch(int mode, const void* x, int dt, long long B, long long H, long long ldx, void* xq,
                          void* xs, cudaStream_t st) {
  switch (dt) {
    case VQK_F16: return quantize_act_t<__half>(mode, (const __half*)x, B, H, ldx, xq, xs, st);
    case VQK_BF16: return quantize_act_t<__nv_bfloat16>(mode, (const __nv_bfloat16*)x, B, H, ldx, xq, xs, st);
    case VQK_F32: return quantize_act_t<float>(mode, (const float*)x, B, H, ldx, xq, xs, st);
  }
  return VQK_ERR_INVALID;
}

}  // namespace vqk

using namespace vqk;

extern "C" int vqk_quantize_weight(int mode, const void* w, int w_dtype, int64_t V, int64_t H, int64_t ldw, void* q,
                                   void* scales, void* stream) {
  if (!w || !q || !scales || V < 0 || H <= 0 || ldw < H) return VQK_ERR_INVALID;
  if (V > 0x7fffffffLL || H > 0x7fffffffLL) return VQK_ERR_INVALID;
  if (mode == VQK_MODE_MXFP4 && (H & 1)) return VQK_ERR_INVALID;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  switch (w_dtype) {
    case VQK_F16: return quantize_weight_t<__half>(mode, (const __half*)w, V, H, ldw, q, scales, st);
    case VQK_BF16: return quantize_weight_t<__nv_bfloat16>(mode, (const __nv_bfloat16*)w, V, H, ldw, q, scales, st);
    case VQK_F32: return quantize_weight_t<float>(mode, (const float*)w, V, H, ldw, q, scales, st);
  }
  return VQK_ERR_INVALID;
}

extern "C" int vqk_quantize_act(int mode, const void* x, int x_dtype, int64_t B, int64_t H, int64_t ldx, void* xq,
                                void* xs, void* stream) {
  if (!x || !xq || B < 0 || H <= 0 || ldx < H) return VQK_ERR_INVALID;
  if (B > 65535) return VQK_ERR_TOO_LARGE;
  int rc = require_sm100();
  if (rc) return rc;
  return quantize_act_dispatch(mode, x, x_dtype, B, H, ldx, xq, xs, (cudaStream_t)stream);
}
