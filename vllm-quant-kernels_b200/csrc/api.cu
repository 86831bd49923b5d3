// C ABI of libvqk.so: argument checks, workspace carving, kernel dispatch.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "lm_head.cuh"

namespace vqk {

thread_local int g_last_cuda_error = 0;

static int g_sm_count[64];
static int g_cc_major[64];

static int query_device(int* dev_out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e);
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  if (g_cc_major[dev] == 0) {
    int major = 0, sms = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e);
    g_sm_count[dev] = sms;
    g_cc_major[dev] = major;
  }
  *dev_out = dev;
  return VQK_OK;
}

int require_sm100() {
  int dev;
  int rc = query_device(&dev);
  if (rc) return rc;
  return g_cc_major[dev] == 10 ? VQK_OK : VQK_ERR_ARCH;
}

int device_sm_count() {
  int dev;
  if (query_device(&dev)) return 0;
  return g_sm_count[dev];
}

// ---- workspace bump allocator -----------------------------------------------------------
struct Carver {
  uint8_t* base;
  size_t off = 0;
  explicit Carver(void* b) : base((uint8_t*)b) {}
  template <typename T>
  T* take(size_t count) {
    off = (off + 255) & ~(size_t)255;
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += count * sizeof(T);
    return p;
  }
};

struct LmHeadWs {
  uint8_t* xq;
  uint8_t* xs;
  float* slice_max;
  float* part_score;
  int* part_token;
  __half* cand;
  long long ld_cand;
  size_t total;
};

static LmHeadWs carve_lm_head(void* base, int mode, long long V, long long K, long long B, int sample, int nslices) {
  Carver c(base);
  LmHeadWs w{};
  if (mode != VQK_MODE_W8A16) w.xq = c.take<uint8_t>((size_t)B * K);
  if (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4) w.xs = c.take<uint8_t>((size_t)B * (K / GROUP));
  if (mode == VQK_MODE_W8A8) w.xs = (uint8_t*)c.take<float>(2);
  if (sample) {
    w.slice_max = c.take<float>((size_t)B * nslices);
    w.part_score = c.take<float>((size_t)B * nslices);
    w.part_token = c.take<int>((size_t)B * nslices);
    w.ld_cand = (V + 7) & ~7LL;
    w.cand = c.take<__half>((size_t)B * w.ld_cand);
  }
  w.total = (c.off + 255) & ~(size_t)255;
  return w;
}

}  // namespace vqk

using namespace vqk;

// batches above this go to the tensor-core kernel (FP8 / W8A8)
static const int kUmmaMinBatch = 8;

struct vqk_lm_head {
  int mode;
  const uint8_t* q;
  const void* scales;
  long long V, H;
  cudaEvent_t ev_start, ev_stop;
};

extern "C" int vqk_version(void) { return VQK_VERSION; }

extern "C" const char* vqk_strerror(int s) {
  switch (s) {
    case VQK_OK: return "ok";
    case VQK_ERR_INVALID: return "invalid argument";
    case VQK_ERR_UNSUPPORTED: return "unsupported shape or mode";
    case VQK_ERR_CUDA: return "CUDA runtime error";
    case VQK_ERR_WORKSPACE: return "workspace missing or too small";
    case VQK_ERR_ARCH: return "device is not sm_100 (B200); there is no fallback path";
    case VQK_ERR_COMM: return "NCCL unavailable or collective failed";
    case VQK_ERR_TOO_LARGE:
      return "size exceeds a fixed maximum (vqk_sample_static: at most 64 rows of at most 262144 columns)";
  }
  return "unknown status";
}

extern "C" int vqk_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int vqk_device_error(void) {
  const int b = umma_error_flag(), c = umma_mx_error_flag(), d = peer_error_flag();
  return (b < 0 || c < 0 || d < 0) ? -1 : (b | c | d);
}

extern "C" int vqk_lm_head_create(int mode, const void* q, const void* scales, int64_t V, int64_t H,
                                  vqk_lm_head** out) {
  if (!out) return VQK_ERR_INVALID;
  *out = nullptr;
  if (mode < VQK_MODE_W8A16 || mode > VQK_MODE_MXFP4 || !q || !scales || V <= 0 || H <= 0) return VQK_ERR_INVALID;
  if (V > 0x7ffffff0LL || H > (1 << 20)) return VQK_ERR_TOO_LARGE;
  // rows are streamed with 16-byte loads (8 / 4 bytes for the MX modes)
  if (H % 16) return VQK_ERR_UNSUPPORTED;
  if ((mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4) && (H % GROUP)) return VQK_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)scales & 7)) return VQK_ERR_INVALID;
  vqk_lm_head* h = new (std::nothrow) vqk_lm_head;
  if (!h) return VQK_ERR_INVALID;
  h->mode = mode; h->q = (const uint8_t*)q; h->scales = scales; h->V = V; h->H = H;
  h->ev_start = nullptr; h->ev_stop = nullptr;
  *out = h;
  return VQK_OK;
}

extern "C" int vqk_lm_head_destroy(vqk_lm_head* h) {
  delete h;
  return VQK_OK;
}

extern "C" int vqk_lm_head_set_kernel_events(vqk_lm_head* h, void* start_event, void* stop_event) {
  if (!h || (!start_event != !stop_event)) return VQK_ERR_INVALID;
  h->ev_start = (cudaEvent_t)start_event;
  h->ev_stop = (cudaEvent_t)stop_event;
  return VQK_OK;
}

extern "C" int64_t vqk_lm_head_workspace_bytes(const vqk_lm_head* h, int64_t B, int sample) {
  if (!h || B < 0) return VQK_ERR_INVALID;
  int sms = device_sm_count();
  if (sms <= 0) return VQK_ERR_CUDA;
  return (int64_t)carve_lm_head(nullptr, h->mode, h->V, h->H, B, sample, sms * 4).total;
}

extern "C" int vqk_lm_head_forward(vqk_lm_head* h, const void* x, int x_dtype, int64_t B, int64_t ldx,
                                   const void* bias, void* logits, int64_t ld_logits, const vqk_sample_params* sp,
                                   int64_t* tokens, float* scores, void* records, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  if (!h || !x || B < 0 || ldx < h->H) return VQK_ERR_INVALID;
  if (x_dtype != VQK_F16 && x_dtype != VQK_BF16) return VQK_ERR_INVALID;
  if (logits && ld_logits < h->V) return VQK_ERR_INVALID;
  if (!logits && !sp) return VQK_ERR_INVALID;
  if (sp && !tokens && !records) return VQK_ERR_INVALID;
  if (sp && sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (sp && tokens && (sp->vocab_total != h->V || sp->vocab_offset != 0)) return VQK_ERR_INVALID;
  if (sp && (sp->vocab_offset < 0 || sp->vocab_offset + h->V > sp->vocab_total || sp->vocab_total > 0x7fffffffLL))
    return VQK_ERR_INVALID;
  if (B > 65535) return VQK_ERR_TOO_LARGE;
  if (B == 0) return VQK_OK;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
  const int nslices = sms * 4;
  const int mode = h->mode;
  // Kernel choice: the register-streaming kernel for decode batches, the tcgen05 tensor-core
  // kernel once the batch is large enough that re-streaming the weights per 32 columns (or the
  // warp-MMA rate) would cost more.  VQK_LM_HEAD_KERNEL = stream | umma pins one (A/B runs).
  const char* kenv = getenv("VQK_LM_HEAD_KERNEL");
  const bool want_umma = kenv && !strcmp(kenv, "umma");
  const bool want_stream = kenv && !strcmp(kenv, "stream");
  int maxcols = 0;
  const bool mx_mode = (mode == VQK_MODE_MXFP8 || mode == VQK_MODE_MXFP4);
  const int umma_cols = mx_mode ? umma_mx_max_cols(mode, (int)h->H) : umma_max_cols(mode, (int)h->H);
  // the block-scaled modes take the tensor-core path at every batch size: the hardware applies
  // the E8M0 scales, which the register kernel has to do with ALU work per element
  // the tensor maps want aligned operands (32 bytes for the packed 4-bit rows); anything else
  // stays on the streaming kernel, which only needs 16-byte aligned rows
  const bool umma_aligned = (((uintptr_t)h->q & (mx_mode ? 31 : 15)) == 0) && (!mx_mode || ((uintptr_t)h->scales & 3) == 0);
  const bool use_umma = !want_stream && umma_cols > 0 && umma_aligned && (want_umma || mx_mode || B > kUmmaMinBatch);
  if (use_umma) maxcols = umma_cols;
  else maxcols = stream_max_cols(mode, (int)h->H);
  if (maxcols <= 0) return VQK_ERR_UNSUPPORTED;

  LmHeadWs ws = carve_lm_head(workspace, mode, h->V, h->H, B, sp != nullptr, nslices);
  const bool needs_ws = ws.total > 0 && (mode != VQK_MODE_W8A16 || sp);
  if (needs_ws && (!workspace || (size_t)workspace_bytes < ws.total)) return VQK_ERR_WORKSPACE;
  if (needs_ws && ((uintptr_t)workspace & 255)) return VQK_ERR_INVALID;

  if (mode != VQK_MODE_W8A16) {
    rc = quantize_act_dispatch(mode, x, x_dtype, B, h->H, ldx, ws.xq, ws.xs, st);
    if (rc) return rc;
  }
  SampleDev sd{};
  if (sp) sd = to_dev(sp);

  if (h->ev_start) VQK_CUDA(cudaEventRecord(h->ev_start, st));
  for (long long b0 = 0; b0 < B; b0 += maxcols) {
    const int Bc = (int)((B - b0 < maxcols) ? (B - b0) : maxcols);
    LmHeadParams p{};
    p.w = h->q;
    p.wscale = h->scales;
    p.V = (int)h->V; p.K = (int)h->H; p.B = Bc;
    p.x_dtype = x_dtype;
    if (mode == VQK_MODE_W8A16) {
      p.x = (const uint8_t*)x + (size_t)b0 * ldx * 2;
      p.ldx = ldx;
    } else {
      p.x = ws.xq + (size_t)b0 * h->H;
      p.ldx = h->H;
      if (mode == VQK_MODE_W8A8) p.xscale = ws.xs;
      else if (mode != VQK_MODE_FP8) p.xscale = ws.xs + (size_t)b0 * (h->H / GROUP);
    }
    p.bias = (const __half*)bias;
    p.logits = logits ? (__half*)logits + (size_t)b0 * ld_logits : nullptr;
    p.ld_logits = ld_logits;
    p.do_sample = sp ? 1 : 0;
    if (sp) {
      p.sp = offset_rows(sd, b0);
      p.slice_max = ws.slice_max + (size_t)b0 * nslices;
      p.part_score = ws.part_score + (size_t)b0 * nslices;
      p.part_token = ws.part_token + (size_t)b0 * nslices;
      p.nslices = nslices;
      // rows that take the candidate path need their fp16 logits in memory: the caller's logits
      // buffer when there is one, scratch otherwise
      if (logits) {
        p.cand_logits = p.logits;
        p.ld_cand = ld_logits;
      } else {
        p.cand_logits = ws.cand + (size_t)b0 * ws.ld_cand;
        p.ld_cand = ws.ld_cand;
      }
    }
    rc = use_umma ? (mx_mode ? launch_lm_head_umma_mx(mode, p, sms, st) : launch_lm_head_umma(mode, p, sms, st))
                   : launch_lm_head_stream(mode, p, sms, st);
    if (rc) return rc;
  }
  if (h->ev_stop) VQK_CUDA(cudaEventRecord(h->ev_stop, st));
  if (!sp) return VQK_OK;

  SelectParams s{};
  s.logits = logits ? logits : (void*)ws.cand; s.dtype = VQK_F16; s.ld = logits ? ld_logits : ws.ld_cand;
  s.V = (int)h->V; s.B = (int)B; s.sp = sd;
  s.slice_max = ws.slice_max; s.part_score = ws.part_score; s.part_token = ws.part_token; s.nslices = nslices;
  s.records = (uint8_t*)records; s.tokens = (long long*)tokens; s.scores = scores;
  s.single_shard = tokens ? 1 : 0;
  return launch_select(s, st);
}

// ---- stand-alone sampler ----------------------------------------------------------------------
namespace {
struct SampleWs {
  float* slice_max;
  float* part_score;
  int* part_token;
  size_t total;
};
SampleWs carve_sample(void* base, long long B, int nslices) {
  Carver c(base);
  SampleWs w{};
  w.slice_max = c.take<float>((size_t)B * nslices);
  w.part_score = c.take<float>((size_t)B * nslices);
  w.part_token = c.take<int>((size_t)B * nslices);
  w.total = (c.off + 255) & ~(size_t)255;
  return w;
}
}  // namespace

extern "C" int64_t vqk_sample_workspace_bytes(int64_t B, int64_t V) {
  if (B < 0 || V <= 0) return VQK_ERR_INVALID;
  return (int64_t)carve_sample(nullptr, B, slice_pass_nslices(V)).total;
}

extern "C" int vqk_sample(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld, const vqk_sample_params* sp,
                          int64_t* tokens, float* scores, void* records, void* workspace, int64_t workspace_bytes,
                          void* stream) {
  if (!logits || !sp || B < 0 || V <= 0 || ld < V || (!tokens && !records)) return VQK_ERR_INVALID;
  if (dtype < VQK_F16 || dtype > VQK_F32) return VQK_ERR_INVALID;
  if (sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (V > 0x7ffffff0LL || sp->vocab_total > 0x7fffffffLL) return VQK_ERR_TOO_LARGE;
  if (sp->vocab_offset < 0 || sp->vocab_offset + V > sp->vocab_total) return VQK_ERR_INVALID;
  if (tokens && (sp->vocab_total != V || sp->vocab_offset != 0)) return VQK_ERR_INVALID;
  if (B > 65535) return VQK_ERR_TOO_LARGE;
  if (B == 0) return VQK_OK;
  int rc = require_sm100();
  if (rc) return rc;
  const int nslices = slice_pass_nslices(V);
  SampleWs ws = carve_sample(workspace, B, nslices);
  if (!workspace || (size_t)workspace_bytes < ws.total) return VQK_ERR_WORKSPACE;
  if ((uintptr_t)workspace & 255) return VQK_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  SampleDev sd = to_dev(sp);
  rc = launch_slice_pass(logits, dtype, ld, (int)B, (int)V, sd, ws.slice_max, ws.part_score, ws.part_token, nslices, st);
  if (rc) return rc;
  SelectParams s{};
  s.logits = logits; s.dtype = dtype; s.ld = ld; s.V = (int)V; s.B = (int)B; s.sp = sd;
  s.slice_max = ws.slice_max; s.part_score = ws.part_score; s.part_token = ws.part_token; s.nslices = nslices;
  s.records = (uint8_t*)records; s.tokens = (long long*)tokens; s.scores = scores;
  s.single_shard = tokens ? 1 : 0;
  return launch_select(s, st);
}

extern "C" int vqk_sample_static(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
                                 const vqk_sample_params* sp, int64_t* tokens, float* scores, void* stream) {
  if (!logits || !sp || !tokens || B < 0 || V <= 0 || ld < V) return VQK_ERR_INVALID;
  if (dtype < VQK_F16 || dtype > VQK_F32) return VQK_ERR_INVALID;
  if (sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (B > VQK_STATIC_MAX_ROWS || V > VQK_STATIC_MAX_VOCAB) return VQK_ERR_TOO_LARGE;
  if (sp->vocab_total != V || sp->vocab_offset != 0) return VQK_ERR_INVALID;
  if (B == 0) return VQK_OK;
  int rc = require_sm100();
  if (rc) return rc;
  return sample_static(logits, dtype, ld, (int)B, (int)V, to_dev(sp), (long long*)tokens, scores, (cudaStream_t)stream);
}

extern "C" int vqk_sample_finalize(const void* records, int G, int64_t B, const vqk_sample_params* sp, int64_t* tokens,
                                   float* scores, void* stream) {
  if (!records || !sp || !tokens || G <= 0 || G > 8 || B < 0) return VQK_ERR_INVALID;
  if (B > 65535) return VQK_ERR_TOO_LARGE;
  int rc = require_sm100();
  if (rc) return rc;
  return launch_finalize((const uint8_t*)records, G, (int)B, to_dev(sp), (long long*)tokens, scores,
                         (cudaStream_t)stream);
}

extern "C" int vqk_topk_threshold(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
                                  const int32_t* top_k, float* threshold, void* stream) {
  if (!logits || !top_k || !threshold || B < 0 || V <= 0 || ld < V) return VQK_ERR_INVALID;
  if (V > 0x7ffffff0LL || B > 0x7fffffffLL) return VQK_ERR_TOO_LARGE;
  int rc = require_sm100();
  if (rc) return rc;
  return launch_topk_threshold(logits, dtype, ld, (int)B, (int)V, top_k, threshold, (cudaStream_t)stream);
}

// ---- NCCL, bound at run time ---------------------------------------------------------------------
namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm_t;
struct NcclApi {
  int (*GetUniqueId)(nccl_uid*);
  int (*CommInitRank)(nccl_comm_t*, int, nccl_uid, int);
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
  int (*CommDestroy)(nccl_comm_t);
  bool ok = false;
};
NcclApi* nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api.ok ? &api : nullptr;
  tried = true;
  void* hnd = nullptr;
  const char* env = getenv("VQK_NCCL_LIB");
  if (env && *env) hnd = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
  if (!hnd) hnd = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy PyTorch already mapped
  if (!hnd) hnd = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!hnd) return nullptr;
  api.GetUniqueId = (int (*)(nccl_uid*))dlsym(hnd, "ncclGetUniqueId");
  api.CommInitRank = (int (*)(nccl_comm_t*, int, nccl_uid, int))dlsym(hnd, "ncclCommInitRank");
  api.AllGather = (int (*)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t))dlsym(hnd, "ncclAllGather");
  api.CommDestroy = (int (*)(nccl_comm_t))dlsym(hnd, "ncclCommDestroy");
  api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy;
  return api.ok ? &api : nullptr;
}
}  // namespace

struct vqk_comm {
  nccl_comm_t comm;
  int rank, nranks;
};

extern "C" int vqk_comm_unique_id(void* id_out) {
  if (!id_out) return VQK_ERR_INVALID;
  NcclApi* a = nccl();
  if (!a) return VQK_ERR_COMM;
  nccl_uid id;
  if (a->GetUniqueId(&id) != 0) return VQK_ERR_COMM;
  memcpy(id_out, &id, sizeof(id));
  return VQK_OK;
}

extern "C" int vqk_comm_create(const void* id_host, int rank, int nranks, vqk_comm** out) {
  if (!id_host || !out || nranks <= 0 || rank < 0 || rank >= nranks) return VQK_ERR_INVALID;
  *out = nullptr;
  NcclApi* a = nccl();
  if (!a) return VQK_ERR_COMM;
  nccl_uid id;
  memcpy(&id, id_host, sizeof(id));
  nccl_comm_t c = nullptr;
  if (a->CommInitRank(&c, nranks, id, rank) != 0) return VQK_ERR_COMM;
  vqk_comm* vc = new (std::nothrow) vqk_comm;
  if (!vc) return VQK_ERR_INVALID;
  vc->comm = c; vc->rank = rank; vc->nranks = nranks;
  *out = vc;
  return VQK_OK;
}

extern "C" int vqk_comm_allgather(vqk_comm* c, const void* send, void* recv, int64_t bytes_per_rank, void* stream) {
  if (!c || !send || !recv || bytes_per_rank < 0) return VQK_ERR_INVALID;
  NcclApi* a = nccl();
  if (!a) return VQK_ERR_COMM;
  if (a->AllGather(send, recv, (size_t)bytes_per_rank, /*ncclInt8*/ 0, c->comm, (cudaStream_t)stream) != 0)
    return VQK_ERR_COMM;
  return VQK_OK;
}

extern "C" int vqk_comm_destroy(vqk_comm* c) {
  if (!c) return VQK_OK;
  NcclApi* a = nccl();
  if (a) a->CommDestroy(c->comm);
  delete c;
  return VQK_OK;
}

// ---- record exchange over peer memory ---------------------------------------------------------------
struct vqk_peer {
  int rank, nranks;
  long long max_rows;
  void* local;       // own landing buffer | flag words | step counters
  void* mapped[8];   // peers' buffers opened through CUDA IPC (null for the own rank)
  PeerTable pt;
  bool connected;
};
namespace {
size_t peer_data_bytes(int G, long long rows) { return (size_t)2 * G * rows * VQK_RECORD_BYTES; }
size_t peer_flag_bytes(int G, long long rows) { return (((size_t)G * rows * sizeof(unsigned int)) + 255) & ~(size_t)255; }
}  // namespace

extern "C" int vqk_peer_create(int rank, int nranks, int64_t max_rows, vqk_peer** out, void* handle_out_host) {
  if (!out || !handle_out_host || nranks <= 0 || nranks > VQK_PEER_MAX_RANKS || rank < 0 || rank >= nranks ||
      max_rows <= 0 || max_rows > 65535)
    return VQK_ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == VQK_PEER_HANDLE_BYTES, "IPC handle size");
  *out = nullptr;
  int rc = require_sm100();
  if (rc) return rc;
  const size_t bytes = peer_data_bytes(nranks, max_rows) + peer_flag_bytes(nranks, max_rows) + (size_t)max_rows * sizeof(unsigned int);
  void* base = nullptr;
  VQK_CUDA(cudaMalloc(&base, bytes));
  cudaError_t e = cudaMemset(base, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    cudaFree(base);
    return VQK_ERR_CUDA;
  }
  vqk_peer* p = new (std::nothrow) vqk_peer();
  if (!p) { cudaFree(base); return VQK_ERR_INVALID; }
  p->rank = rank; p->nranks = nranks; p->max_rows = max_rows; p->local = base; p->connected = false;
  memcpy(handle_out_host, &h, sizeof(h));
  *out = p;
  return VQK_OK;
}

extern "C" int vqk_peer_connect(vqk_peer* p, const void* all_handles_host) {
  if (!p || !all_handles_host || p->connected) return VQK_ERR_INVALID;
  const size_t data = peer_data_bytes(p->nranks, p->max_rows), flags = peer_flag_bytes(p->nranks, p->max_rows);
  for (int g = 0; g < p->nranks; ++g) {
    void* base = p->local;
    if (g != p->rank) {
      cudaIpcMemHandle_t h;
      memcpy(&h, (const uint8_t*)all_handles_host + (size_t)g * VQK_PEER_HANDLE_BYTES, sizeof(h));
      cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        for (int q = 0; q < g; ++q)
          if (p->mapped[q]) { cudaIpcCloseMemHandle(p->mapped[q]); p->mapped[q] = nullptr; }
        return VQK_ERR_COMM;
      }
      p->mapped[g] = base;
    }
    p->pt.land[g] = (uint8_t*)base;
    p->pt.flags[g] = (unsigned int*)((uint8_t*)base + data);
  }
  p->pt.steps = (unsigned int*)((uint8_t*)p->local + data + flags);
  p->connected = true;
  return VQK_OK;
}

extern "C" int vqk_peer_exchange_finalize(vqk_peer* p, const void* records, int64_t B, const vqk_sample_params* sp,
                                          int64_t* tokens, float* scores, void* stream) {
  if (!p || !p->connected || !records || !sp || !tokens || B < 0) return VQK_ERR_INVALID;
  if (B > p->max_rows) return VQK_ERR_TOO_LARGE;
  return launch_peer_exchange((const uint8_t*)records, (int)B, p->rank, p->nranks, (int)p->max_rows, p->pt, to_dev(sp),
                              (long long*)tokens, scores, (cudaStream_t)stream);
}

extern "C" int vqk_peer_destroy(vqk_peer* p) {
  if (!p) return VQK_OK;
  for (int g = 0; g < p->nranks; ++g)
    if (p->mapped[g]) cudaIpcCloseMemHandle(p->mapped[g]);
  if (p->local) cudaFree(p->local);
  delete p;
  return VQK_OK;
}
