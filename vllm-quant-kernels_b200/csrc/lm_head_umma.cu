// Large-batch lm_head on the 5th-generation tensor cores (tcgen05), "swap-AB" form:
// the 128 vocab rows of a tile are the M side of the MMA, the (padded) batch is the N side,
// so the weight matrix is streamed exactly once whatever the batch.
//
//   warp 0      TMA producer: per 128-byte K block one 2-D tensor copy of the weight tile
//               (128 rows x 128 B, 128-byte swizzle) and one of the activations (BN rows x 128 B)
//               into a ring of shared-memory stages, completion on an mbarrier.
//   warp 1      MMA issuer: one thread issues tcgen05.mma (kind::i8 for W8A8, kind::f8f6f4 for
//               FP8) from shared-memory descriptors into a TMEM accumulator (128 lanes x BN
//               fp32/int32 columns, two buffers), tcgen05.commit hands stages back / signals
//               the epilogue.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (a warp owns the 32 TMEM lanes = 32 vocab
//               rows of its quadrant), apply the mode's scale, round to fp16 like the reference
//               launchers, store logits if asked, feed the sampler (per-slice maxima / Gumbel
//               winners), overlapped with the next tile's MMAs through the second TMEM buffer.
//
// Replaces fp8_gemm / int8_w8a8_gemm of the reference (src/vllm_quant_kernels/_kernels.py:299-477)
// for batches above 16.  Every mbarrier wait is bounded (async_helpers.cuh).
#include "umma_common.cuh"

namespace vqk {
namespace umma {

constexpr int kThreads = 192;  // producer warp, MMA warp, four epilogue warps

struct Geometry {
  int stage_bytes;  // A tile + B tile
  int stages;
  size_t total;
};
__host__ __device__ inline Geometry geometry(int bn) {
  Geometry g;
  g.stage_bytes = BM * BK + bn * BK;
  const size_t fixed = 1024 /* alignment slack */ + 256 /* barriers */ + (size_t)bn * sizeof(RowMeta) +
                       (size_t)12 * bn * sizeof(int) /* sampler state */;
  const size_t limit = 227 * 1024;
  int s = (int)((limit - fixed) / g.stage_bytes);
  g.stages = s > kMaxStages ? kMaxStages : s;
  g.total = fixed + (size_t)g.stages * g.stage_bytes;
  return g;
}


template <int MODE, int BN>
__global__ void __launch_bounds__(kThreads, 1)
k_lm_head_umma(const LmHeadParams p, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB) {
  constexpr bool INT8 = (MODE == VQK_MODE_W8A8);
  constexpr uint32_t TCOLS = (2 * BN <= 32) ? 32u : (uint32_t)(2 * BN);  // power of two for BN in {16..256}
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const Geometry geo = geometry(BN);
  const int S = geo.stages;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)S * geo.stage_bytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kMaxStages;
  uint64_t* tfull = bars + 2 * kMaxStages;
  uint64_t* tempty = bars + 2 * kMaxStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  RowMeta* meta = reinterpret_cast<RowMeta*>(bars + 32);
  int* sstate = reinterpret_cast<int*>(meta + BN);  // [4 warps][3][BN] sampler state of the epilogue warps

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = p.V, B = p.B;
  const int nkb = p.K / BK;
  const int ntiles = (V + BM - 1) / BM;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int r = 0; r < 2; ++r) { mbar_init(&tfull[r], 1); mbar_init(&tempty[r], 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (p.do_sample)
    for (int b = tid; b < BN; b += kThreads) {
      RowMeta m;
      m.flags = 0; m.T = 1.f; m.thr = -INFINITY; m.top_p = 1.f; m.top_k = 0; m.seed = 0;
      if (b < B) m = decode_row(p.sp, b);
      meta[b] = m;
    }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================================ TMA producer =====================================
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (uint32_t)(it / S) & 1u;
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + (size_t)s * geo.stage_bytes;
          uint8_t* sb = sa + BM * BK;
          mbar_expect_tx(&full[s], (uint32_t)geo.stage_bytes);
          tma_load_2d(sa, &mapA, kb * BK, tile * BM, &full[s]);
          tma_load_2d(sb, &mapB, kb * BK, 0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer =======================================
    if (lane == 0) {
      const uint32_t idesc = instr_desc(INT8, BN);
      int it = 0, tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++tcount) {
        const int buf = tcount & 1;
        const uint32_t tph = (uint32_t)(tcount >> 1) & 1u;
        if (!mbar_wait(&tempty[buf], tph ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (uint32_t)(it / S) & 1u;
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)s * geo.stage_bytes);
          const uint64_t adesc = smem_desc_sw128(sa);
          const uint64_t bdesc = smem_desc_sw128(sa + BM * BK);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)  // +32 bytes of K = +2 in the 16-byte address field
            umma_8bit<INT8>(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[buf]);  // accumulator complete
      }
    }
  } else {
    umma_epilogue<INT8 ? 1 : 0, BN>(p, warp, lane, tmem_base, tfull, tempty, abort_flag, meta, sstate, ntiles);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TCOLS);
  }
}


// ---- host side ------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
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

// bytes [rows, K] row-major -> tensor map with a {128 B, box_rows} box and the 128-byte swizzle;
// rows past `rows` read as zeros
static int make_map(CUtensorMap* m, const void* base, long long rows, long long K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return VQK_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VQK_OK : VQK_ERR_CUDA;
}

template <int MODE, int BN>
static int launch_one(const LmHeadParams& p, const CUtensorMap& a, const CUtensorMap& b, int grid, cudaStream_t st) {
  const Geometry geo = geometry(BN);
  static bool configured[64] = {};
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (!configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_umma<MODE, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)geo.total));
    configured[dev] = true;
  }
  k_lm_head_umma<MODE, BN><<<grid, kThreads, geo.total, st>>>(p, a, b);
  VQK_LAUNCH_CHECK();
  return VQK_OK;
}

template <int MODE>
static int launch_bn(const LmHeadParams& p, const CUtensorMap& a, const CUtensorMap& b, int bn, int grid, cudaStream_t st) {
  switch (bn) {
    case 16: return launch_one<MODE, 16>(p, a, b, grid, st);
    case 32: return launch_one<MODE, 32>(p, a, b, grid, st);
    case 64: return launch_one<MODE, 64>(p, a, b, grid, st);
    case 128: return launch_one<MODE, 128>(p, a, b, grid, st);
    case 256: return launch_one<MODE, 256>(p, a, b, grid, st);
  }
  return VQK_ERR_INVALID;
}

}  // namespace umma

// Shapes the tensor-core kernel takes: FP8 / W8A8, K a multiple of 128 bytes, 16-byte aligned bases.
int umma_max_cols(int mode, int K) {
  if (mode != VQK_MODE_FP8 && mode != VQK_MODE_W8A8) return 0;
  if (K % umma::BK) return 0;
  return 256;
}

int launch_lm_head_umma(int mode, const LmHeadParams& p, int grid, cudaStream_t st) {
  using namespace umma;
  if (p.B < 1 || p.B > 256 || umma_max_cols(mode, p.K) == 0) return VQK_ERR_UNSUPPORTED;
  if (((uintptr_t)p.w & 15) || ((uintptr_t)p.x & 15)) return VQK_ERR_UNSUPPORTED;
  int bn = 16;
  while (bn < p.B) bn <<= 1;
  CUtensorMap a, b;
  int rc = make_map(&a, p.w, p.V, p.K, BM);
  if (rc) return rc;
  rc = make_map(&b, p.x, p.B, p.K, bn);
  if (rc) return rc;
  if (mode == VQK_MODE_W8A8) return launch_bn<VQK_MODE_W8A8>(p, a, b, bn, grid, st);
  return launch_bn<VQK_MODE_FP8>(p, a, b, bn, grid, st);
}

int umma_error_flag() { return read_stream_error(); }

}  // namespace vqk
