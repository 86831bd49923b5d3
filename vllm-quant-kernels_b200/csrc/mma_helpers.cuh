// Warp-level MMA wrappers and the in-register weight expansions shared by the lm_head kernels.
#pragma once

#include "vqk_common.cuh"

namespace vqk {

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
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four int8 (bytes 0..3 of w) -> two half2 holding the exact integers:
//   even = (b0, b2), odd = (b1, b3).
// (byte ^ 0x80) | 0x6400 is the fp16 number 1024 + (b + 128); one LOP3 does mask and both
// constants at once, then 1152 is subtracted.  Shift and logic ops only: on B200 the byte
// permute instruction runs on the quarter-rate XU pipe and capped this path at half the
// HBM rate.  The even/odd split is free: the activation fragments are built in the same order.
__device__ __forceinline__ void int8x4_to_half2_even_odd(uint32_t w, uint32_t& even, uint32_t& odd) {
  uint32_t e = (w & 0x00ff00ffu) ^ 0x64806480u;
  uint32_t o = ((w >> 8) & 0x00ff00ffu) ^ 0x64806480u;
  const uint32_t bias = 0x64806480u;  // half2(1152, 1152)
  __half2 eh = __hsub2(*reinterpret_cast<__half2*>(&e), *reinterpret_cast<const __half2*>(&bias));
  __half2 oh = __hsub2(*reinterpret_cast<__half2*>(&o), *reinterpret_cast<const __half2*>(&bias));
  even = *reinterpret_cast<uint32_t*>(&eh);
  odd = *reinterpret_cast<uint32_t*>(&oh);
}

// Eight packed E2M1 nibbles (element j in nibble j of w) -> two words of four e4m3 bytes:
//   even = elements (0, 2, 4, 6), odd = elements (1, 3, 5, 7), each SCALED BY 2^-6.
// An E2M1 code s.e1e0.m placed as the e4m3 byte s00e1e0m00 is the same number times 2^-6,
// subnormals included (0.5 = code 001 becomes the e4m3 subnormal 4/8 * 2^-6), so the
// expansion is two shifts and three logic ops per word; the constant 2^6 is folded into the
// activation-side scale.  No byte-permute (XU pipe) instructions.
constexpr float kE2M1Rescale = 64.0f;
__device__ __forceinline__ void e2m1x8_to_e4m3_even_odd(uint32_t w, uint32_t& even, uint32_t& odd) {
  even = ((w << 4) & 0x80808080u) | ((w << 2) & 0x1c1c1c1cu);
  odd = (w & 0x80808080u) | ((w >> 2) & 0x1c1c1c1cu);
}

}  // namespace vqk
