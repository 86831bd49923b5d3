// Pieces shared by the block-scaled (MXFP8 / MXFP4) tcgen05 kernels: the block-scaled MMA and
// scale-copy wrappers, their descriptors, and the tensor-map encoder.
#pragma once

#include "umma_common.cuh"

namespace vqk {
namespace umma {

constexpr int kSfBlock = 512;    // bytes of one 128-row x 4-group scale block

__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                        uint32_t sfb, uint32_t acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %6, 0;\n"
      " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(acc)
      : "memory");
}
// 32 rows x 128 bits from shared memory into 32 TMEM lanes x 4 columns, replicated to all four
// lane quadrants
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// descriptor of a 512-byte scale block: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)(128 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;           // descriptor version
  return d;
}
// block-scaled instruction descriptor: B scale id at bit 4, A / B formats at bits 7 / 10 (0 = E4M3,
// 5 = E2M1), N >> 3 at bit 17, scale format E8M0 at bit 23, M >> 4 at bit 24, A scale id at bit 29
__host__ __device__ inline uint32_t instr_desc_mx(bool a_fp4, int bn) {
  uint32_t d = 0;
  d |= (a_fp4 ? 5u : 0u) << 7;
  d |= (uint32_t)(bn >> 3) << 17;
  d |= 1u << 23;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}

// ---- host side: tensor maps ----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn mx_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return (EncodeTiledFn)f;
  }();
  return fn;
}

// [rows, K elements] row-major, 8-bit or packed 4-bit elements; box {128 elements, box_rows}; the
// 4-bit type lands in shared memory as sixteen codes per 16-byte chunk, i.e. 128 bytes per box row
static int mx_make_map(CUtensorMap* m, const void* base, long long rows, long long K, int box_rows, bool fp4) {
  EncodeTiledFn fn = mx_encode_fn();
  if (!fn) return VQK_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(fp4 ? K / 2 : K)};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = (int)r;
    return VQK_ERR_CUDA;
  }
  return VQK_OK;
}

}  // namespace umma
}  // namespace vqk
