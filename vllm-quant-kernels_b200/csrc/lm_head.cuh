// Internal interface between the lm_head kernels, the sampler kernels and the C ABI.
#pragma once

#include "vqk_common.cuh"

namespace vqk {

constexpr int kListM = 4;     // logits a warp group keeps per top-k column (its slice's largest), besides the witness
constexpr int kCtaListM = 8;  // logits a CTA hands to the tail per top-k row: the largest of its groups' lists
// What a CTA of the streaming kernel leaves per batch row for the sampler tail: four 16-byte words.
// Every logit of the CTA's rows that is not among the kCtaListM listed ones is <= the witness.
struct __align__(16) CtaList {
  int t[kCtaListM];      // local token ids of the CTA's largest logits
  __half v[kCtaListM];   // their values, descending (-inf: no entry)
  __half witness;
  __half pad;
  float win_s;           // rows without top-k / top-p: the CTA's Gumbel (or greedy) winner
  int win_t;             // its local token id
  int pad2;
};
static_assert(sizeof(CtaList) == 64, "four 16-byte words per CTA and row");

// Record exchange over peer memory (peer_exchange.cuh).  G == 0: no exchange.
struct PeerTable {
  unsigned long long* land[8];  // every rank's landing buffer [2][G][max_rows][kWireWords] words (own one included)
  unsigned int* steps;          // this rank's per-row step counters [max_rows]
  int* error;                   // device error word, set when a wait runs out
  unsigned int wait_polls;      // bound of every wait, in polls
  int rank, G, max_rows;
};

struct LmHeadParams {
  const uint8_t* w;    // quantized rows [V, K] bytes (MXFP4: [V, K/2])
  const void* wscale;  // fp16 [V] / fp32 [V] / E8M0 [V, K/32]
  const void* x;       // W8A16: caller's activations [B, ldx] (x_dtype); else quantized bytes [B, K]
  const void* xscale;  // W8A8: const float* (xs[0]); MX: E8M0 [B, K/32]
  int x_dtype;
  int V, K, B;
  long long ldx;
  const __half* bias;  // [V] or null
  float soft_cap;      // > 0: logits = tanh(logits / soft_cap) * soft_cap after the bias (0: off)
  float out_scale;     // logits *= out_scale after that (1: off)
  __half* logits;      // [B, ld_logits] or null
  long long ld_logits;
  int do_sample;
  SampleDev sp;        // per-row arrays already offset to this launch's first batch row
  float* slice_max;    // [B][nslices] max raw logit of candidate-path rows
  float* part_score;   // [B][nslices] per-slice winner of the other rows
  int* part_token;     // [B][nslices] local token id of that winner
  int nslices;
  __half* cand_logits; // [B, ld_cand] fp16 logits of candidate-path rows (scratch or == logits)
  long long ld_cand;
  int pdl;             // launched as a programmatic dependent of the activation quantizer
  unsigned long long* dbg;  // null, or [gridDim.x][16] time stamps (vqk_lm_head_set_debug_times)
  // decode-sized batches: the last CTA to finish resolves the rows (tail.cuh)
  int fuse_tail;
  CtaList* lists;        // [B][gridDim.x] what every CTA hands to the tail (decode-sized batches); null: no tail
  unsigned int* ticket;  // device counter, zero between launches
  unsigned int* tile_counter;  // streaming kernel: tiles handed out beyond the first two rounds (zero between launches); null: static rounds
  int* error;            // device error word, set when the tail's bounded wait for the grid runs out
  int* row_flag;         // [B] written by the tail: 1 = the row still needs the full-row kernel
  long long* tokens;     // outputs of the tail (as SelectParams)
  float* scores;
  uint8_t* records;
  int single_shard;
  PeerTable peer;        // sharded step: the tail also exchanges the row's record and merges (G > 0)
};

// vLLM's LogitsProcessor.forward post-ops (vllm/model_executor/layers/logits_processor.py:66-72) on an
// fp16 logit, with upstream's roundings: it runs them as separate fp16 tensor ops (divide, tanh,
// multiply, multiply), each computed in fp32 and rounded to fp16; torch turns the division of a
// tensor by a host scalar into a multiplication by the scalar's fp32 reciprocal.
__device__ __forceinline__ __half logit_post_ops(__half h, float soft_cap, float out_scale) {
  if (soft_cap > 0.f) {
    h = __float2half_rn(__half2float(h) * __fdiv_rn(1.0f, soft_cap));
    h = __float2half_rn(tanhf(__half2float(h)));
    h = __float2half_rn(__half2float(h) * soft_cap);
  }
  if (out_scale != 1.f) h = __float2half_rn(__half2float(h) * out_scale);
  return h;
}

// time stamp i of this CTA (measurement aid; %globaltimer, nanoseconds)
__device__ __forceinline__ void dbg_stamp(const LmHeadParams& p, int i) {
  if (p.dbg && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) :: "memory");
    p.dbg[(size_t)blockIdx.x * 16 + i] = t;
  }
}


constexpr int kTailMaxBatch = 16;    // largest batch whose rows the lm_head kernel resolves itself

// lm_head_stream.cu
size_t stream_smem_bytes(int mode, int K, int NT);
int stream_max_cols(int mode, int K);  // batch columns one launch can take (0: K too large)
int launch_lm_head_stream(int mode, const LmHeadParams& p, int grid, cudaStream_t st);
int stream_error_flag();
int stream_error_clear();


// lm_head_umma.cu: tcgen05 tensor-core kernel for larger batches (FP8, W8A8; K % 128 == 0)
int umma_max_cols(int mode, int K);    // 256, or 0 when the mode / shape is not covered
int launch_lm_head_umma(int mode, const LmHeadParams& p, int grid, cudaStream_t st);
int umma_error_flag();
int umma_error_clear();
// lm_head_umma_mx.cu: block-scaled tcgen05 kernel (MXFP8, MXFP4; K % 128 == 0; up to 128 columns)
int umma_mx_max_cols(int mode, int K);
int launch_lm_head_umma_mx(int mode, const LmHeadParams& p, int grid, cudaStream_t st);
int umma_mx_error_flag();
int umma_mx_error_clear();

// quantize.cu
int quantize_act_dispatch(int mode, const void* x, int dt, long long B, long long H, long long ldx, void* xq,
                          void* xs, cudaStream_t st);

// sampler.cu -------------------------------------------------------------------------------
struct SelectParams {
  const void* logits;   // [B, ld] rows in `dtype` (local shard)
  int dtype;
  long long ld;
  int V;                // local columns
  int B;
  SampleDev sp;
  const float* slice_max;   // [B][nslices]
  const float* part_score;  // [B][nslices]
  const int* part_token;    // [B][nslices]
  int nslices;
  uint8_t* records;     // [B] exchange records (always written)
  long long* tokens;    // final answers when single shard (may be null)
  float* scores;
  int single_shard;     // 1: also resolve candidate rows to a final token here
  const int* row_flag;  // null, or [B]: rows whose flag is 0 were resolved by the lm_head kernel's tail
  PeerTable peer;       // G > 0: rank 0 of the row's cluster also exchanges the record and merges (sharded step)
};

// first pass over materialised logits: per-slice maxima / Gumbel winners (slices of 256 columns)
int launch_slice_pass(const void* logits, int dtype, long long ld, int B, int V, const SampleDev& sp, float* slice_max,
                      float* part_score, int* part_token, int nslices, cudaStream_t st, float* lp_max = nullptr,
                      float* lp_sum = nullptr);
// log-softmax of the sampled tokens from the first pass's per-slice (max, sum of exponentials): lp_* [B][nslices]
int launch_logprob(const void* logits, int dtype, long long ld, int B, int V, const float* lp_max, const float* lp_sum,
                   int nslices, const long long* tokens, float* logprobs, cudaStream_t st);
inline int slice_pass_nslices(long long V) { return (int)((V + 255) / 256); }
// cluster-per-row selection: tau from slice maxima, candidate collection, final choice / record;
// rows that do not fit the candidate scheme are resolved by an exact full-row pass inside
// `after_lm_head`: launched as a programmatic dependent of the lm_head kernel before it on the stream (its CTAs are
// in place, waiting, when that kernel ends)
int launch_select(const SelectParams& p, cudaStream_t st, bool after_lm_head = false);
// merge gathered records
int launch_finalize(const uint8_t* records, int G, int B, const SampleDev& sp, long long* tokens, float* scores,
                    cudaStream_t st);
int launch_peer_exchange(const uint8_t* mine, int B, const PeerTable& pt, const SampleDev& sp, long long* tokens,
                         float* scores, cudaStream_t st);
// sampler on materialised logits with its scratch in a static device array (no allocation)
int sample_static(const void* logits, int dtype, long long ld, int B, int V, const SampleDev& sp, long long* tokens,
                  float* scores, cudaStream_t st);
int launch_topk_threshold(const void* logits, int dtype, long long ld, int B, int V, const int32_t* top_k, float* thr,
                          cudaStream_t st);

inline SampleDev to_dev(const vqk_sample_params* sp) {
  SampleDev d;
  d.temperature = sp->temperature;
  d.seeds = sp->seeds;
  d.top_k = sp->top_k;
  d.top_p = sp->top_p;
  d.thr = sp->topk_threshold;
  d.vocab_offset = sp->vocab_offset;
  d.vocab_total = sp->vocab_total;
  d.logprobs = sp->logprobs;
  return d;
}
inline SampleDev offset_rows(SampleDev d, long long b0) {
  if (d.temperature) d.temperature += b0;
  if (d.seeds) d.seeds += b0;
  if (d.top_k) d.top_k += b0;
  if (d.top_p) d.top_p += b0;
  if (d.thr) d.thr += b0;
  return d;
}

}  // namespace vqk
