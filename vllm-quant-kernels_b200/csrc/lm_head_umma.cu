// Large-batch lm_head on the 5th-generation tensor cores (tcgen05), "swap-AB" form:
// the 128 vocab rows of a tile are the M side of the MMA, the (padded) batch is the N side,
// so the weight matrix is streamed exactly once whatever the batch.
//
//   producers   one thread per pipeline: per 128-byte K block one 2-D tensor copy of the weight
//               tile (128 rows x 128 B, 128-byte swizzle) and one of the activations (BN rows x
//               128 B) into the pipeline's ring of shared-memory stages, completion on an mbarrier.
//   issuers     one thread per pipeline issues tcgen05.mma (kind::i8 for W8A8, kind::f8f6f4 for
//               FP8) from shared-memory descriptors into a TMEM accumulator (128 lanes x BN
//               fp32/int32 columns, two buffers per pipeline), tcgen05.commit hands stages back /
//               signals the epilogue.
//   4 warps     epilogue: tcgen05.ld the accumulator (a warp owns the 32 TMEM lanes = 32 vocab
//               rows of its quadrant), apply the mode's scale, round to fp16 like the reference
//               launchers, store logits if asked, feed the sampler (per-slice maxima / Gumbel
//               winners), overlapped with the next tiles' MMAs through the second TMEM buffers.
//
// Replaces fp8_gemm / int8_w8a8_gemm of the reference (src/vllm_quant_kernels/_kernels.py:299-477)
// for batches above 8.  Every mbarrier wait is bounded (async_helpers.cuh).
#include "umma_common.cuh"

namespace vqk {
namespace umma {

// NI independent MMA pipelines ("lanes") per CTA, each with its own TMA producer thread, issuing
// thread, stage ring and pair of accumulators, each on its own tile (the CTA's n-th tile belongs
// to lane n % NI).  One thread issues a tcgen05 instruction about every 54 cycles and also has a
// barrier wait and a commit per k-block, while the tensor pipe needs only 39 cycles for a
// 128 x N x 32-byte MMA with N <= 32 (64 for N = 128): narrow batches are issue-bound with one
// issuer, and extra lanes hide each other's bookkeeping.
__host__ __device__ inline int umma_threads(int ni) { return (2 * ni + 4) * 32; }
constexpr int kPerLane = 2 * kMaxStages;  // barriers per lane: full, empty

struct Geometry {
  int stage_bytes;  // A tile + B tile
  int stages_per_lane;
  size_t total;
};
__host__ __device__ inline Geometry geometry(int bn, int ni) {
  Geometry g;
  g.stage_bytes = BM * BK + bn * BK;
  const size_t fixed = 1024 /* alignment slack */ + 1024 /* barriers */ + (size_t)bn * sizeof(RowMeta) +
                       epi_state_bytes(bn) /* sampler state */;
  const size_t limit = 227 * 1024;
  int s = (int)((limit - fixed) / g.stage_bytes) / ni;
  g.stages_per_lane = s > kMaxStages ? kMaxStages : s;
  g.total = fixed + (size_t)ni * g.stages_per_lane * g.stage_bytes;
  return g;
}

template <int MODE, int BN, int NI>
__global__ void __launch_bounds__((2 * NI + 4) * 32, 1)
k_lm_head_umma(const LmHeadParams p, const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB) {
  constexpr bool INT8 = (MODE == VQK_MODE_W8A8);
  constexpr int kThreadsHere = (2 * NI + 4) * 32;
  constexpr uint32_t kNeed = (uint32_t)(NI * 2 * BN);
  constexpr uint32_t TCOLS = kNeed <= 32 ? 32u : kNeed <= 64 ? 64u : kNeed <= 128 ? 128u : kNeed <= 256 ? 256u : 512u;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const Geometry geo = geometry(BN, NI);
  const int S = geo.stages_per_lane;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NI * S * geo.stage_bytes);
  uint64_t* tfull = bars;            // [NI * 2]
  uint64_t* tempty = bars + 2 * NI;  // [NI * 2]
  uint64_t* drained = bars + 4 * NI;   // [NI]: an issuer's last commit, waited for before the CTA exits
  uint64_t* lane_bars = bars + 5 * NI;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(lane_bars + NI * kPerLane);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  RowMeta* meta = reinterpret_cast<RowMeta*>(bars + 128);
  int* sstate = reinterpret_cast<int*>(meta + BN);  // [4 warps][3][BN] sampler state of the epilogue warps

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int V = p.V, B = p.B;
  const int nkb = p.K / BK;
  const int ntiles = (V + BM - 1) / BM;

  if (tid == 0) {
    for (int i = 0; i < 2 * NI; ++i) { mbar_init(&tfull[i], 1); mbar_init(&tempty[i], 4); }
    for (int l = 0; l < NI; ++l) mbar_init(&drained[l], 1);
    for (int l = 0; l < NI; ++l)
      for (int s = 0; s < S; ++s) { mbar_init(&lane_bars[l * kPerLane + s], 1); mbar_init(&lane_bars[l * kPerLane + kMaxStages + s], 1); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (p.do_sample)
    for (int b = tid; b < BN; b += kThreadsHere) {
      RowMeta m;
      m.flags = 0; m.T = 1.f; m.thr = -INFINITY; m.top_p = 1.f; m.top_k = 0; m.seed = 0;
      if (b < B) m = decode_row(p.sp, b);
      meta[b] = m;
    }
  if (warp == NI) {  // the first issuing warp owns the TMEM allocation
    tmem_alloc(tmem_slot, TCOLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // this CTA's n-th tile is blockIdx.x + n * gridDim.x; lane l takes n = l, l + NI, ...
  const int mytiles = (int)blockIdx.x < ntiles ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (warp < NI) {
    // ================================ TMA producers =====================================
    if (lane == 0) {
      pdl_wait();  // the quantized activations come from the kernel before
      const int l = warp;
      uint64_t* full = lane_bars + l * kPerLane;
      uint64_t* empty = full + kMaxStages;
      uint8_t* my = smem + (size_t)l * S * geo.stage_bytes;
      int s = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int n = l; n < mytiles && ok; n += NI) {
        const int row0 = (blockIdx.x + n * gridDim.x) * BM;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty[s], ph ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = my + (size_t)s * geo.stage_bytes;
          mbar_expect_tx(&full[s], (uint32_t)geo.stage_bytes);
          tma_load_2d(sa, &mapA, kb * BK, row0, &full[s]);
          tma_load_2d(sa + BM * BK, &mapB, kb * BK, 0, &full[s]);
          ++issued;
          if (++s == S) { s = 0; ph ^= 1u; }
        }
      }
      // no copy of this thread may still be in flight when the CTA exits: the last min(issued, S)
      // stages are the only ones that can be (on the normal path they have all been consumed)
      for (int i = issued > S ? issued - S : 0; i < issued; ++i) mbar_drain(&full[i % S], (uint32_t)(i / S) & 1u);
    }
  } else if (warp < 2 * NI) {
    // ================================ MMA issuers =======================================
    // Counters and constant increments only: everything in this loop delays the next MMA.
    if (lane == 0) {
      const int l = warp - NI;
      uint64_t* full = lane_bars + l * kPerLane;
      uint64_t* empty = full + kMaxStages;
      const uint32_t idesc = instr_desc(INT8, BN);
      const uint64_t adesc0 = smem_desc_sw128(smem_u32(smem + (size_t)l * S * geo.stage_bytes));
      const uint64_t kStageStep = (uint64_t)geo.stage_bytes >> 4;
      int s = 0, u = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int n = l; n < mytiles && ok; n += NI, ++u) {
        const int acc = l * 2 + (u & 1);
        if (!mbar_wait(&tempty[acc], ((uint32_t)(u >> 1) & 1u) ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          const uint64_t adesc = adesc0 + (uint64_t)s * kStageStep;
          const uint64_t bdesc = adesc + ((uint64_t)(BM * BK) >> 4);
          // +32 bytes of K = +2 in the 16-byte address field
          umma_8bit<INT8>(d_tmem, adesc, bdesc, idesc, kb != 0 ? 1u : 0u);
          umma_8bit<INT8>(d_tmem, adesc + 2, bdesc + 2, idesc, 1u);
          umma_8bit<INT8>(d_tmem, adesc + 4, bdesc + 4, idesc, 1u);
          umma_8bit<INT8>(d_tmem, adesc + 6, bdesc + 6, idesc, 1u);
          umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
          if (++s == S) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(&tfull[acc]);  // accumulator complete
      }
      // nothing this thread issued may still be running when the CTA frees its TMEM and exits
      umma_commit(&drained[l]);
      mbar_drain(&drained[l], 0);
    }
  } else {
    pdl_wait();  // W8A8: the activation scale comes from the kernel before
    umma_epilogue<INT8 ? 1 : 0, BN, NI>(p, warp, lane, tmem_base, tfull, tempty, abort_flag, meta, sstate, sched_interleaved(V));
  }

  tc_fence_before();
  __syncthreads();
  if (warp == NI) {
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

template <int MODE, int BN, int NI>
static int launch_lanes(const LmHeadParams& p, const CUtensorMap& a, const CUtensorMap& b, int grid, cudaStream_t st) {
  const Geometry geo = geometry(BN, NI);
  if (geo.stages_per_lane < 2) return VQK_ERR_UNSUPPORTED;
  static bool configured[64] = {};
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (!configured[dev]) {
    VQK_CUDA(cudaFuncSetAttribute(k_lm_head_umma<MODE, BN, NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)geo.total));
    configured[dev] = true;
  }
  // every CTA of the grid runs (those without a tile still write their empty slice records)
  VQK_CUDA(launch_kernel(k_lm_head_umma<MODE, BN, NI>, dim3(grid), dim3(umma_threads(NI)), geo.total, st, p.pdl != 0, p, a, b));
  return VQK_OK;
}
// three pipelines for narrow batch tiles (issue-bound), two at 64, one from 128 columns on (the
// MMAs are long enough, and the accumulators fill TMEM)
template <int MODE, int BN>
static int launch_one(const LmHeadParams& p, const CUtensorMap& a, const CUtensorMap& b, int grid, cudaStream_t st) {
  static const int cap = [] {
    const char* e = getenv("VQK_UMMA_LANES");  // tuning knob: fewer MMA pipelines per CTA
    const int v = e ? atoi(e) : 0;
    return v >= 1 && v <= 3 ? v : 3;
  }();
  constexpr int kWant = BN <= 32 ? 3 : BN <= 64 ? 2 : 1;
  if (kWant >= 3 && cap >= 3) return launch_lanes<MODE, BN, 3>(p, a, b, grid, st);
  if (kWant >= 2 && cap >= 2) return launch_lanes<MODE, BN, (BN <= 128 ? 2 : 1)>(p, a, b, grid, st);
  return launch_lanes<MODE, BN, 1>(p, a, b, grid, st);
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
int umma_error_clear() { return clear_stream_error(); }

}  // namespace vqk
