// C ABI of libvqk.so: argument checks, workspace carving, kernel dispatch.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <new>

#include "lm_head.cuh"
#include "peer_exchange.cuh"

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

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("VQK_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
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
  CtaList* lists;  // decode-sized batches only: [B][CTAs]
  int* row_flag;
  __half* cand;
  long long ld_cand;
  size_t total;
};

// Ticket counters of the fused sampler tail: one slot per vqk_lm_head, handed out round-robin.
// Zero at load; the last CTA of every launch puts its slot back to zero.  In host code the array's
// name is only a stand-in: the device address is looked up once per device.
constexpr int kTicketSlots = 256;
static __device__ unsigned int g_tickets[kTicketSlots * 2];  // per slot: the end-of-kernel ticket, the streaming kernel's tile counter
static unsigned int* g_tickets_ptr[64];
static std::mutex g_symbol_mu;  // the once-per-device address look-ups may come from several host threads
static int ticket_base(unsigned int** out) {
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  std::lock_guard<std::mutex> lock(g_symbol_mu);
  if (!g_tickets_ptr[dev]) {
    void* ptr = nullptr;
    VQK_CUDA(cudaGetSymbolAddress(&ptr, g_tickets));
    g_tickets_ptr[dev] = (unsigned int*)ptr;
  }
  *out = g_tickets_ptr[dev];
  return VQK_OK;
}

// Error word of the peer exchange (a wait that ran out), one per device, same address rule.
static __device__ int g_peer_error;
static int* g_peer_error_ptr[64];
static int peer_error_word(int** out) {
  int dev = 0;
  VQK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return VQK_ERR_INVALID;
  std::lock_guard<std::mutex> lock(g_symbol_mu);
  if (!g_peer_error_ptr[dev]) {
    void* ptr = nullptr;
    VQK_CUDA(cudaGetSymbolAddress(&ptr, g_peer_error));
    g_peer_error_ptr[dev] = (int*)ptr;
  }
  *out = g_peer_error_ptr[dev];
  return VQK_OK;
}
static int peer_error_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_peer_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

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
    if (B <= kTailMaxBatch) w.lists = c.take<CtaList>((size_t)B * (nslices / 4));
    w.row_flag = c.take<int>((size_t)B);
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
  int ticket_slot;
  unsigned long long* dbg;
  float soft_cap, out_scale;
  // vqk_lm_head_step_host: pinned (mapped) host staging [inputs | tokens | scores] and its device mirror
  uint8_t* host_stage;
  uint8_t* dev_stage;
  long long* host_tokens_dev;  // device address of the mapped token words
  size_t stage_in_cap;  // bytes of the input part
  long long stage_rows; // rows the output part holds
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
      return "size exceeds a fixed maximum (vqk_sample_static: at most 64 rows of at most 262144 columns; "
             "vqk_peer: the max_rows it was created with)";
  }
  return "unknown status";
}

extern "C" int vqk_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int vqk_device_error(void) {
  const int a = stream_error_flag(), b = umma_error_flag(), c = umma_mx_error_flag(), d = peer_error_flag();
  return (a < 0 || b < 0 || c < 0 || d < 0) ? -1 : (a | b | c | d);
}

extern "C" int vqk_device_error_clear(void) {
  const int zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return VQK_ERR_CUDA;
  if (stream_error_clear() || umma_error_clear() || umma_mx_error_clear()) return VQK_ERR_CUDA;
  VQK_CUDA(cudaMemcpyToSymbol(g_peer_error, &zero, sizeof(int)));
  {  // a launch that gave up may have left its ticket or tile counter behind
    void* tp = nullptr;
    VQK_CUDA(cudaGetSymbolAddress(&tp, g_tickets));
    VQK_CUDA(cudaMemset(tp, 0, sizeof(unsigned int) * kTicketSlots * 2));
  }
  return VQK_OK;
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
  h->ev_start = nullptr; h->ev_stop = nullptr; h->dbg = nullptr;
  h->soft_cap = 0.f; h->out_scale = 1.f;
  h->host_stage = nullptr; h->dev_stage = nullptr; h->stage_in_cap = 0; h->stage_rows = 0;
  static unsigned int next_slot = 0;
  h->ticket_slot = (int)(__atomic_fetch_add(&next_slot, 1u, __ATOMIC_RELAXED) % kTicketSlots);
  *out = h;
  return VQK_OK;
}

extern "C" int vqk_lm_head_destroy(vqk_lm_head* h) {
  if (h) {
    if (h->host_stage) cudaFreeHost(h->host_stage);
    if (h->dev_stage) cudaFree(h->dev_stage);
  }
  delete h;
  return VQK_OK;
}

extern "C" int vqk_lm_head_set_kernel_events(vqk_lm_head* h, void* start_event, void* stop_event) {
  if (!h || (!start_event != !stop_event)) return VQK_ERR_INVALID;
  h->ev_start = (cudaEvent_t)start_event;
  h->ev_stop = (cudaEvent_t)stop_event;
  return VQK_OK;
}

extern "C" int vqk_lm_head_set_post_ops(vqk_lm_head* h, float soft_cap, float scale) {
  if (!h || soft_cap != soft_cap || scale != scale) return VQK_ERR_INVALID;
  h->soft_cap = soft_cap > 0.f ? soft_cap : 0.f;
  h->out_scale = scale;
  return VQK_OK;
}

extern "C" int vqk_lm_head_set_debug_times(vqk_lm_head* h, void* device_buffer) {
  if (!h) return VQK_ERR_INVALID;
  h->dbg = (unsigned long long*)device_buffer;
  return VQK_OK;
}

extern "C" int64_t vqk_lm_head_workspace_bytes(const vqk_lm_head* h, int64_t B, int sample) {
  if (!h || B < 0) return VQK_ERR_INVALID;
  int sms = device_sm_count();
  if (sms <= 0) return VQK_ERR_CUDA;
  return (int64_t)carve_lm_head(nullptr, h->mode, h->V, h->H, B, sample, sms * 4).total;
}

struct vqk_peer;
static int peer_table_of(const vqk_peer* p, int64_t B, PeerTable* out);

// lm_head (+ sampler) of one shard; with `peer` the step is sharded: records travel over peer memory
// and `tokens` receives the merged result.
static int lm_head_forward_impl(vqk_lm_head* h, const void* x, int x_dtype, int64_t B, int64_t ldx, const void* bias,
                                void* logits, int64_t ld_logits, const vqk_sample_params* sp, int64_t* tokens,
                                float* scores, void* records, const vqk_peer* peer, void* workspace,
                                int64_t workspace_bytes, void* stream) {
  if (!h || !x || B < 0 || ldx < h->H) return VQK_ERR_INVALID;
  if (x_dtype != VQK_F16 && x_dtype != VQK_BF16) return VQK_ERR_INVALID;
  if (logits && ld_logits < h->V) return VQK_ERR_INVALID;
  if (!logits && !sp) return VQK_ERR_INVALID;
  if (sp && !tokens && !records) return VQK_ERR_INVALID;
  if (sp && sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (sp && sp->logprobs) return VQK_ERR_UNSUPPORTED;  // stand-alone sampler only (vqk_sample)
  if (sp && tokens && !peer && (sp->vocab_total != h->V || sp->vocab_offset != 0)) return VQK_ERR_INVALID;
  if (sp && (sp->vocab_offset < 0 || sp->vocab_offset + h->V > sp->vocab_total || sp->vocab_total > 0x7fffffffLL))
    return VQK_ERR_INVALID;
  if (B > 65535) return VQK_ERR_TOO_LARGE;
  if (B == 0) return VQK_OK;
  int rc = require_sm100();
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int sms = device_sm_count();
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
  const int grid = sms;  // persistent kernels: one CTA per SM (144 CTAs, which fill the last round of 248320 rows, were no faster)
  const int nslices = grid * 4;  // one slice per warp group (streaming kernel) or epilogue warp (tensor-core kernels)

  PeerTable pt{};
  if (peer) {
    rc = peer_table_of(peer, B, &pt);
    if (rc) return rc;
  }
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
  // Decode-sized batches: the lm_head kernel's last CTA resolves the rows itself (tail.cuh); the
  // full-row kernel behind it only picks up rows the tail flagged.
  // The streaming kernel only: inside the tensor-core kernels the same tail ran slower than the
  // full-row kernel it replaces, and the per-column lists cost their epilogues registers.
  // VQK_TAIL_MODE (A/B runs): 0 = never, 2 = the tail hands every row to the full-row kernel.
  static const int tail_mode = [] {
    const char* e = getenv("VQK_TAIL_MODE");
    const int v = e ? atoi(e) : 1;
    return v >= 0 && v <= 2 ? v : 1;
  }();
  const bool tail_here = !use_umma;
  const bool fuse_tail = tail_mode && tail_here && sp && B <= kTailMaxBatch && B <= maxcols && nslices <= 1024;
  unsigned int* tickets = nullptr;
  int* error_word = nullptr;
  // the streaming kernel hands its tiles out dynamically beyond the first two rounds (VQK_STREAM_DYNAMIC=0:
  // static rounds, for A/B runs); the counter sits next to the handle's ticket and is reset by the last CTA
  static const bool dynamic_tiles = [] { const char* e = getenv("VQK_STREAM_DYNAMIC"); return !(e && atoi(e) == 0); }();
  const bool want_counter = !use_umma && dynamic_tiles;
  if (fuse_tail || want_counter) {
    rc = ticket_base(&tickets);
    if (rc) return rc;
  }
  if (fuse_tail) {
    rc = peer_error_word(&error_word);
    if (rc) return rc;
  }

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
    p.dbg = h->dbg;
    p.pdl = (mode != VQK_MODE_W8A16 && b0 == 0 && pdl_enabled()) ? 1 : 0;
    p.bias = (const __half*)bias;
    p.soft_cap = h->soft_cap;
    p.out_scale = h->out_scale;
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
      if (fuse_tail) {
        p.fuse_tail = tail_mode == 2 ? 2 : 1;
        p.lists = ws.lists;
        p.ticket = tickets + 2 * h->ticket_slot;
        p.error = error_word;
        p.row_flag = ws.row_flag;
        p.tokens = (long long*)tokens; p.scores = scores; p.records = (uint8_t*)records;
        p.single_shard = (tokens && !peer) ? 1 : 0;
        p.peer = pt;
      }
    }
    if (want_counter) {
      p.ticket = tickets + 2 * h->ticket_slot;
      p.tile_counter = tickets + 2 * h->ticket_slot + 1;
    }
    rc = use_umma ? (mx_mode ? launch_lm_head_umma_mx(mode, p, grid, st) : launch_lm_head_umma(mode, p, grid, st))
                   : launch_lm_head_stream(mode, p, grid, st);
    if (rc) return rc;
  }
  if (h->ev_stop) VQK_CUDA(cudaEventRecord(h->ev_stop, st));
  if (!sp) return VQK_OK;

  SelectParams s{};
  s.logits = logits ? logits : (void*)ws.cand; s.dtype = VQK_F16; s.ld = logits ? ld_logits : ws.ld_cand;
  s.V = (int)h->V; s.B = (int)B; s.sp = sd;
  s.slice_max = ws.slice_max; s.part_score = ws.part_score; s.part_token = ws.part_token; s.nslices = nslices;
  s.records = (uint8_t*)records; s.tokens = (long long*)tokens; s.scores = scores;
  s.single_shard = (tokens && !peer) ? 1 : 0;
  s.row_flag = fuse_tail ? ws.row_flag : nullptr;
  s.peer = pt;
  // behind the streaming kernel as its programmatic dependent: its CTAs are in place when that kernel ends (1.8 us
  // per step; behind the tensor-core kernels the same cost the MXFP4 step 4 - 7 us, so there it is launched
  // the plain way).  An event record in between would separate the two.
  return launch_select(s, st, !use_umma && pdl_enabled() && !h->ev_stop);
}

extern "C" int vqk_lm_head_forward(vqk_lm_head* h, const void* x, int x_dtype, int64_t B, int64_t ldx,
                                   const void* bias, void* logits, int64_t ld_logits, const vqk_sample_params* sp,
                                   int64_t* tokens, float* scores, void* records, void* workspace,
                                   int64_t workspace_bytes, void* stream) {
  return lm_head_forward_impl(h, x, x_dtype, B, ldx, bias, logits, ld_logits, sp, tokens, scores, records, nullptr,
                              workspace, workspace_bytes, stream);
}

// ---- stand-alone sampler ----------------------------------------------------------------------
namespace {
struct SampleWs {
  float* slice_max;
  float* part_score;
  int* part_token;
  float* lp_max;  // per-slice maximum and sum of exponentials (log-probability of the sampled token)
  float* lp_sum;
  size_t total;
};
SampleWs carve_sample(void* base, long long B, int nslices) {
  Carver c(base);
  SampleWs w{};
  w.slice_max = c.take<float>((size_t)B * nslices);
  w.part_score = c.take<float>((size_t)B * nslices);
  w.part_token = c.take<int>((size_t)B * nslices);
  w.lp_max = c.take<float>((size_t)B * nslices);
  w.lp_sum = c.take<float>((size_t)B * nslices);
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
  if (sd.logprobs && !tokens) return VQK_ERR_UNSUPPORTED;  // the log-probability is of the merged token: single shard only
  rc = launch_slice_pass(logits, dtype, ld, (int)B, (int)V, sd, ws.slice_max, ws.part_score, ws.part_token, nslices, st,
                         sd.logprobs ? ws.lp_max : nullptr, sd.logprobs ? ws.lp_sum : nullptr);
  if (rc) return rc;
  SelectParams s{};
  s.logits = logits; s.dtype = dtype; s.ld = ld; s.V = (int)V; s.B = (int)B; s.sp = sd;
  s.slice_max = ws.slice_max; s.part_score = ws.part_score; s.part_token = ws.part_token; s.nslices = nslices;
  s.records = (uint8_t*)records; s.tokens = (long long*)tokens; s.scores = scores;
  s.single_shard = tokens ? 1 : 0;
  rc = launch_select(s, st);
  if (rc || !sd.logprobs) return rc;
  return launch_logprob(logits, dtype, ld, (int)B, (int)V, ws.lp_max, ws.lp_sum, nslices, (const long long*)tokens, sd.logprobs, st);
}

extern "C" int vqk_sample_static(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
                                 const vqk_sample_params* sp, int64_t* tokens, float* scores, void* stream) {
  if (!logits || !sp || !tokens || B < 0 || V <= 0 || ld < V) return VQK_ERR_INVALID;
  if (dtype < VQK_F16 || dtype > VQK_F32) return VQK_ERR_INVALID;
  if (sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (sp->logprobs) return VQK_ERR_UNSUPPORTED;  // the fixed scratch has no room for the per-slice sums
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
  if (sp->logprobs) return VQK_ERR_UNSUPPORTED;
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
  void* local;       // own landing buffer | step counters
  void* mapped[8];   // peers' buffers opened through CUDA IPC (null for the own rank and for caller-owned pointers)
  unsigned long long* land[8];
  unsigned int wait_polls;
  bool connected;
};
namespace {
size_t peer_data_bytes(int G, long long rows) { return (size_t)2 * G * rows * kWireWords * sizeof(unsigned long long); }
constexpr unsigned int kPeerDefaultPolls = 1u << 22;  // about a second of polling, then the row reports -1
}  // namespace

static int peer_table_of(const vqk_peer* p, int64_t B, PeerTable* out) {
  if (!p->connected) return VQK_ERR_INVALID;
  if (B > p->max_rows) return VQK_ERR_TOO_LARGE;
  PeerTable pt{};
  for (int g = 0; g < p->nranks; ++g) pt.land[g] = p->land[g];
  pt.steps = (unsigned int*)((uint8_t*)p->local + peer_data_bytes(p->nranks, p->max_rows));
  int rc = peer_error_word(&pt.error);
  if (rc) return rc;
  pt.wait_polls = p->wait_polls;
  pt.rank = p->rank; pt.G = p->nranks; pt.max_rows = (int)p->max_rows;
  *out = pt;
  return VQK_OK;
}

extern "C" int vqk_peer_create(int rank, int nranks, int64_t max_rows, vqk_peer** out, void* handle_out_host) {
  if (!out || !handle_out_host || nranks <= 0 || nranks > VQK_PEER_MAX_RANKS || rank < 0 || rank >= nranks ||
      max_rows <= 0 || max_rows > 65535)
    return VQK_ERR_INVALID;
  static_assert(sizeof(cudaIpcMemHandle_t) == VQK_PEER_HANDLE_BYTES, "IPC handle size");
  static_assert(kWireWords * sizeof(unsigned long long) == VQK_RECORD_BYTES, "a record's wire form fills a record slot");
  *out = nullptr;
  int rc = require_sm100();
  if (rc) return rc;
  const size_t bytes = peer_data_bytes(nranks, max_rows) + (size_t)max_rows * sizeof(unsigned int);
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
  p->wait_polls = kPeerDefaultPolls;
  memcpy(handle_out_host, &h, sizeof(h));
  *out = p;
  return VQK_OK;
}

extern "C" int vqk_peer_connect(vqk_peer* p, const void* all_handles_host) {
  if (!p || !all_handles_host || p->connected) return VQK_ERR_INVALID;
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
    p->land[g] = (unsigned long long*)base;
  }
  p->connected = true;
  return VQK_OK;
}

extern "C" void* vqk_peer_local_buffer(vqk_peer* p) { return p ? p->local : nullptr; }

extern "C" int vqk_peer_connect_pointers(vqk_peer* p, void* const* buffers_host) {
  if (!p || !buffers_host || p->connected) return VQK_ERR_INVALID;
  for (int g = 0; g < p->nranks; ++g) {
    void* base = g == p->rank ? p->local : buffers_host[g];
    if (!base || ((uintptr_t)base & 7)) return VQK_ERR_INVALID;
    p->land[g] = (unsigned long long*)base;
  }
  p->connected = true;
  return VQK_OK;
}

extern "C" int vqk_peer_set_wait_limit(vqk_peer* p, int64_t polls) {
  if (!p || polls < 1 || polls > 0x7fffffffLL) return VQK_ERR_INVALID;
  p->wait_polls = (unsigned int)polls;
  return VQK_OK;
}

extern "C" int vqk_peer_exchange_finalize(vqk_peer* p, const void* records, int64_t B, const vqk_sample_params* sp,
                                          int64_t* tokens, float* scores, void* stream) {
  if (!p || !p->connected || !records || !sp || !tokens || B < 0) return VQK_ERR_INVALID;
  if (sp->temperature && !sp->seeds) return VQK_ERR_INVALID;
  if (sp->logprobs) return VQK_ERR_UNSUPPORTED;
  if (B > p->max_rows) return VQK_ERR_TOO_LARGE;
  int rc = require_sm100();
  if (rc) return rc;
  PeerTable pt{};
  rc = peer_table_of(p, B, &pt);
  if (rc) return rc;
  return launch_peer_exchange((const uint8_t*)records, (int)B, pt, to_dev(sp), (long long*)tokens, scores,
                              (cudaStream_t)stream);
}

extern "C" int vqk_lm_head_step_sharded(vqk_lm_head* h, vqk_peer* peer, const void* x, int x_dtype, int64_t B,
                                        int64_t ldx, const void* bias, const vqk_sample_params* sp, int64_t* tokens,
                                        float* scores, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!peer || !sp || !tokens) return VQK_ERR_INVALID;
  // the workspace holds the records of the rows the full-row kernel resolves, after the rest
  const int64_t base = vqk_lm_head_workspace_bytes(h, B, 1);
  if (base < 0) return (int)base;
  const int64_t need = base + B * VQK_RECORD_BYTES;
  if (!workspace || workspace_bytes < need) return VQK_ERR_WORKSPACE;
  void* records = (uint8_t*)workspace + base;
  return lm_head_forward_impl(h, x, x_dtype, B, ldx, bias, nullptr, 0, sp, tokens, scores, records, peer, workspace,
                              base, stream);
}

// ---- host-buffer step -----------------------------------------------------------------------------
extern "C" int64_t vqk_lm_head_step_host_workspace_bytes(const vqk_lm_head* h, int64_t B) {
  return vqk_lm_head_step_sharded_workspace_bytes(h, B);
}

static inline size_t pad16(size_t n) { return (n + 15) & ~(size_t)15; }
constexpr long long kHostTokenPending = (long long)0x8000000000000000ull;  // no token has this value

extern "C" int vqk_lm_head_step_host(vqk_lm_head* h, vqk_peer* peer, const void* x_host, int x_dtype, int64_t B,
                                     const void* bias, const vqk_sample_params* sp_host, int64_t* tokens_host,
                                     float* scores_host, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!h || !x_host || !sp_host || !tokens_host || B <= 0) return VQK_ERR_INVALID;
  if (x_dtype != VQK_F16 && x_dtype != VQK_BF16) return VQK_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  // staging layout: x | temperature | seeds | top_k | top_p | topk_threshold (absent arrays take no room)
  const size_t xb = pad16((size_t)B * h->H * 2), ab = pad16((size_t)B * 4);
  const void* arr[5] = {sp_host->temperature, sp_host->seeds, sp_host->top_k, sp_host->top_p, sp_host->topk_threshold};
  size_t off[5], in_bytes = xb;
  for (int i = 0; i < 5; ++i) {
    off[i] = in_bytes;
    if (arr[i]) in_bytes += ab;
  }
  if (in_bytes > h->stage_in_cap || B > h->stage_rows) {  // (re)allocate: first call, or a larger batch
    VQK_CUDA(cudaStreamSynchronize(st));
    if (h->host_stage) cudaFreeHost(h->host_stage);
    if (h->dev_stage) cudaFree(h->dev_stage);
    h->host_stage = nullptr; h->dev_stage = nullptr; h->stage_in_cap = 0; h->stage_rows = 0;
    const size_t cap = pad16(xb + 5 * ab);
    VQK_CUDA(cudaHostAlloc((void**)&h->host_stage, cap + pad16((size_t)B * 8) + pad16((size_t)B * 4), cudaHostAllocMapped));
    VQK_CUDA(cudaMalloc((void**)&h->dev_stage, cap + pad16((size_t)B * 8) + pad16((size_t)B * 4)));
    h->stage_in_cap = cap;
    h->stage_rows = B;
    void* dp = nullptr;
    VQK_CUDA(cudaHostGetDevicePointer(&dp, h->host_stage + cap, 0));
    h->host_tokens_dev = reinterpret_cast<long long*>(dp);
  }
  uint8_t* hs = h->host_stage;
  memcpy(hs, x_host, (size_t)B * h->H * 2);
  for (int i = 0; i < 5; ++i)
    if (arr[i]) memcpy(hs + off[i], arr[i], (size_t)B * 4);
  volatile long long* tok_pinned = reinterpret_cast<volatile long long*>(hs + h->stage_in_cap);
  float* sc_pinned = reinterpret_cast<float*>(hs + h->stage_in_cap + pad16((size_t)h->stage_rows * 8));
  VQK_CUDA(cudaMemcpyAsync(h->dev_stage, hs, in_bytes, cudaMemcpyHostToDevice, st));
  vqk_sample_params sp = *sp_host;
  const uint8_t* ds = h->dev_stage;
  sp.temperature = arr[0] ? reinterpret_cast<const float*>(ds + off[0]) : nullptr;
  sp.seeds = arr[1] ? reinterpret_cast<const int32_t*>(ds + off[1]) : nullptr;
  sp.top_k = arr[2] ? reinterpret_cast<const int32_t*>(ds + off[2]) : nullptr;
  sp.top_p = arr[3] ? reinterpret_cast<const float*>(ds + off[3]) : nullptr;
  sp.topk_threshold = arr[4] ? reinterpret_cast<const float*>(ds + off[4]) : nullptr;
  const bool watch = scores_host == nullptr;
  int64_t* tok_out;
  float* sc_out = nullptr;
  if (watch) {
    // the kernels store every token straight into the mapped pinned words the host watches
    for (int64_t b = 0; b < B; ++b) tok_pinned[b] = kHostTokenPending;
    tok_out = reinterpret_cast<int64_t*>(h->host_tokens_dev);
  } else {
    tok_out = reinterpret_cast<int64_t*>(h->dev_stage + h->stage_in_cap);
    sc_out = reinterpret_cast<float*>(h->dev_stage + h->stage_in_cap + pad16((size_t)h->stage_rows * 8));
  }
  int rc;
  if (peer) rc = vqk_lm_head_step_sharded(h, peer, ds, x_dtype, B, h->H, bias, &sp, tok_out, sc_out, workspace, workspace_bytes, stream);
  else rc = vqk_lm_head_forward(h, ds, x_dtype, B, h->H, bias, nullptr, 0, &sp, tok_out, sc_out, nullptr, workspace, workspace_bytes, stream);
  if (rc) return rc;
  if (watch) {
    // bounded watch (about two seconds of polls), then the ordinary blocking wait
    bool all = false;
    for (long long it = 0; it < (1LL << 28) && !all; ++it) {
      all = true;
      for (int64_t b = 0; b < B; ++b)
        if (tok_pinned[b] == kHostTokenPending) { all = false; break; }
    }
    if (!all) VQK_CUDA(cudaStreamSynchronize(st));
    for (int64_t b = 0; b < B; ++b) tokens_host[b] = tok_pinned[b];
  } else {
    const size_t out_bytes = pad16((size_t)h->stage_rows * 8) + (size_t)B * 4;
    VQK_CUDA(cudaMemcpyAsync(hs + h->stage_in_cap, h->dev_stage + h->stage_in_cap, out_bytes, cudaMemcpyDeviceToHost, st));
    VQK_CUDA(cudaStreamSynchronize(st));
    for (int64_t b = 0; b < B; ++b) { tokens_host[b] = tok_pinned[b]; scores_host[b] = sc_pinned[b]; }
  }
  return VQK_OK;
}

extern "C" int64_t vqk_lm_head_step_sharded_workspace_bytes(const vqk_lm_head* h, int64_t B) {
  const int64_t base = vqk_lm_head_workspace_bytes(h, B, 1);
  return base < 0 ? base : base + B * VQK_RECORD_BYTES;
}

extern "C" int vqk_peer_destroy(vqk_peer* p) {
  if (!p) return VQK_OK;
  for (int g = 0; g < p->nranks; ++g)
    if (p->mapped[g]) cudaIpcCloseMemHandle(p->mapped[g]);
  if (p->local) cudaFree(p->local);
  delete p;
  return VQK_OK;
}
