// Shared device/host helpers for libvqk (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/vqk.h"

namespace vqk {

// ---- host-side error plumbing ------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return VQK_ERR_CUDA;
}
#define VQK_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e__ = (call);                            \
    if (e__ != cudaSuccess) return ::vqk::cuda_fail(e__); \
  } while (0)
#define VQK_LAUNCH_CHECK() VQK_CUDA(cudaPeekAtLastError())

int device_sm_count();  // SMs of the current device (cached per device)
int require_sm100();    // VQK_OK or VQK_ERR_ARCH

constexpr int GROUP = 32;  // MX block size (reference: _kernels.py:488,646)

// ---- programmatic dependent launch ------------------------------------------------------
// The lm_head kernels follow the activation quantizer on the stream.  Launched as its
// programmatic dependents they start while it still runs (barrier set-up, TMEM allocation, the
// first weight loads need nothing from it) and wait right before they first touch its output;
// the quantizer lets them go at its own start.  Both instructions are no-ops in a kernel that was
// launched the plain way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool pdl_enabled();  // VQK_PDL=0 switches it off (A/B runs)

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- numeric helpers ------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }

// e4m3fn byte -> fp32, exact (0x7f/0xff -> NaN)
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

// fp32 -> e4m3fn byte, RNE, NON-saturating like torch's cast: |x| <= 464 -> finite,
// larger / inf / NaN -> 0x7f | sign.
__device__ __forceinline__ uint8_t f32_to_e4m3_nosat(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_NOSAT, __NV_E4M3);
}

// E8M0 byte -> 2^(b-127) as fp32 (b = 0 is the subnormal 2^-127; b = 255 never produced)
__device__ __forceinline__ float e8m0_to_f32(uint32_t b) {
  return __uint_as_float(b == 0 ? 0x00400000u : (b << 23));
}

// ceil(log2(r)) for positive normal fp32 r by the integer rule (exponent, +1 unless the
// mantissa is zero); clamps to [-127, 127] as the reference does (_quant.py:54-55).
__device__ __forceinline__ int ceil_log2_clamped(float r) {
  uint32_t u = __float_as_uint(r);
  int e = (int)((u >> 23) & 0xFF) - 127;
  if (u & 0x7FFFFF) e += 1;
  return max(-127, min(127, e));
}

// order-preserving map fp32 -> uint32 (larger float <-> larger key); NaN sorts above +inf
__device__ __forceinline__ uint32_t f32_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_f32(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k;
  return __uint_as_float(u);
}

// ---- Philox-4x32-10 as Triton's tl.rand uses it -----------------------------------
// counter (offset, 0, 0, 0), key (seed_lo, seed_hi); returns word 0.
__device__ __forceinline__ uint32_t philox_word0(uint32_t seed_lo, uint32_t seed_hi, uint32_t offset) {
  uint32_t c0 = offset, c1 = 0, c2 = 0, c3 = 0, k0 = seed_lo, k1 = seed_hi;
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    uint32_t hiB = __umulhi(0xCD9E8D57u, c2), loB = 0xCD9E8D57u * c2;
    uint32_t hiA = __umulhi(0xD2511F53u, c0), loA = 0xD2511F53u * c0;
    c0 = hiB ^ c1 ^ k0;
    c2 = hiA ^ c3 ^ k1;
    c1 = loB;
    c3 = loA;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}

// Gumbel noise of the reference sampler: u = tl.rand(seed, idx) clamped to 2^-126,
// g = -log(-log(u)) in fp32 (_sampler_kernels.py:104-106).  int32 seeds sign-extend to
// 64 bits, so a negative seed has seed_hi = 0xffffffff.
__device__ __forceinline__ float gumbel_noise(int32_t seed, uint32_t global_idx) {
  uint32_t w = philox_word0((uint32_t)seed, seed < 0 ? 0xFFFFFFFFu : 0u, global_idx);
  int32_t x = (int32_t)w;
  x = x < 0 ? -x - 1 : x;
  float u = (float)x * 4.6566127342e-10f;
  u = fmaxf(u, 1.17549435e-38f);
  return -logf(-logf(u));
}

// (score, token) comparator: higher score wins, equal scores -> lower token
__device__ __forceinline__ bool better(float s, int t, float bs, int bt) {
  return s > bs || (s == bs && t < bt);
}

// ---- per-row sampling description, decoded once per kernel --------------------------
enum : int {
  ROW_GREEDY = 1,    // score = raw logit
  ROW_MASK_THR = 2,  // keep only logit >= thr (reference-style threshold given by caller)
  ROW_CAND = 4,      // needs the candidate path (device top-k and/or top-p)
  ROW_FULLROW = 8    // top-p without top-k: needs a pass over the whole row
};

struct RowMeta {
  float T;
  float thr;
  float top_p;   // >= 1 disabled
  int32_t top_k; // 0 disabled
  int32_t seed;
  int flags;
};

struct SampleDev {  // vqk_sample_params with device pointers, passed by value
  const float* temperature;
  const int32_t* seeds;
  const int32_t* top_k;
  const float* top_p;
  const float* thr;
  long long vocab_offset;
  long long vocab_total;
  float* logprobs;  // optional out [B]: raw log-softmax of the sampled token (stand-alone sampler)
};

__device__ __forceinline__ RowMeta decode_row(const SampleDev& sp, int b) {
  RowMeta m;
  m.T = sp.temperature ? sp.temperature[b] : 0.f;
  m.seed = sp.seeds ? sp.seeds[b] : 0;
  m.thr = -INFINITY;
  m.top_k = 0;
  m.top_p = 1.f;
  m.flags = 0;
  bool greedy = (sp.temperature == nullptr) || (m.T < 1e-5f);
  if (greedy) {
    m.flags = ROW_GREEDY;
    return m;
  }
  if (sp.thr) {
    m.thr = sp.thr[b];
    m.flags |= ROW_MASK_THR;
  } else if (sp.top_k) {
    int k = sp.top_k[b];
    if (k > 0 && (long long)k < sp.vocab_total) m.top_k = k;
  }
  if (sp.top_p) {
    float p = sp.top_p[b];
    if (p < 1.f) m.top_p = p;
  }
  if (m.top_k > 0 || m.top_p < 1.f) {
    m.flags |= ROW_CAND;
    if (m.top_k == 0 && !(m.flags & ROW_MASK_THR)) m.flags |= ROW_FULLROW;
  }
  return m;
}

// exchange record (see vqk.h)
struct RecordHeader {
  float score;
  int32_t token;
  int32_t n;
  int32_t flags;
};
struct Cand {
  float v;
  int32_t t;
};
static_assert(sizeof(RecordHeader) + VQK_RECORD_CAP * sizeof(Cand) == VQK_RECORD_BYTES, "record layout");

}  // namespace vqk
