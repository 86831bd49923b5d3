/*
 * vqk.h - C ABI of libvqk.so: quantized lm_head + fused sampler for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host binds instead of the reference plugin's Triton
 * kernels (project himikk/vllm-quant-kernels).  Every entry point cites the
 * reference interface it replaces as `path:line` inside that project.
 *
 * Conventions
 *   - plain pointers and sizes only; `stream` is a cudaStream_t passed as void*
 *     (NULL = the legacy default stream);
 *   - all data pointers are DEVICE pointers unless a comment says host;
 *   - every function returns VQK_OK (0) or a negative vqk_status; nothing throws,
 *     nothing calls exit();
 *   - work is enqueued on `stream` and the call returns without synchronising;
 *   - the caller owns every buffer, including the workspace whose size the
 *     *_workspace_bytes functions report; a vqk_lm_head owns no device memory;
 *   - there is no CPU fallback: on a device that is not compute capability 10.x
 *     the compute entry points return VQK_ERR_ARCH.
 */
#ifndef VQK_H_
#define VQK_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VQK_VERSION 100

typedef enum {
  VQK_OK = 0,
  VQK_ERR_INVALID = -1,      /* bad argument (null pointer, size, alignment, enum) */
  VQK_ERR_UNSUPPORTED = -2,  /* valid request this build does not implement (e.g. H % 16 != 0) */
  VQK_ERR_CUDA = -3,         /* a CUDA runtime call failed; see vqk_last_cuda_error */
  VQK_ERR_WORKSPACE = -4,    /* workspace missing or too small */
  VQK_ERR_ARCH = -5,         /* current device is not sm_100 */
  VQK_ERR_COMM = -6,         /* NCCL not loadable or a collective failed */
  VQK_ERR_TOO_LARGE = -7     /* size beyond a stated fixed maximum */
} vqk_status;

/* lm_head modes, in the reference's priority order from lowest to highest
 * (src/vllm_quant_kernels/_registration.py:57-68). */
typedef enum {
  VQK_MODE_W8A16 = 0,  /* int8 rows + fp16 scale   (_quant.py:245-255)  kernels int8_gmv / int8_gemm */
  VQK_MODE_W8A8 = 1,   /* int8 rows + fp32 scale   (_quant.py:285-292)  kernel  int8_w8a8_gemm */
  VQK_MODE_FP8 = 2,    /* e4m3 rows + fp16 scale   (_quant.py:306-314)  kernel  fp8_gemm */
  VQK_MODE_MXFP8 = 3,  /* e4m3 + E8M0 per 32       (_quant.py:34-61)    kernel  mxfp8_gemm */
  VQK_MODE_MXFP4 = 4   /* E2M1 x2/byte + E8M0/32   (_quant.py:64-105)   kernel  mxfp4_gemm (W4A8) */
} vqk_mode;

typedef enum { VQK_F16 = 0, VQK_BF16 = 1, VQK_F32 = 2 } vqk_dtype;

int vqk_version(void);
const char* vqk_strerror(int status);
/* cudaError_t of the most recent failing CUDA call on this host thread (0 if none). */
int vqk_last_cuda_error(void);
/* Synchronises the device and returns 1 if a bounded wait inside a kernel ever ran out
 * (the kernel then drained and left its outputs undefined), 0 if not, -1 on a CUDA error.
 * For tests and post-mortems; not for the hot path. */
int vqk_device_error(void);
/* Synchronises the device and puts the flag vqk_device_error reports back to 0 (after a wait ran
 * out the flag would otherwise stay set for the life of the process). */
int vqk_device_error_clear(void);

/* ---------------------------------------------------------------------------
 * Offline weight quantisation.  Replaces the torch code in
 * QuantizedLogitsProcessor._init_int8_weights / _init_w8a8 / _init_fp8 /
 * _init_mxfp8 / _init_mxfp4 (src/vllm_quant_kernels/_quant.py:245-380) and
 * _quantize_to_mxfp8 / _quantize_to_mxfp4 (_quant.py:34-105).  Bit-exact.
 *   w      [V, H] fp16 or bf16 (or fp32), row stride ldw elements
 *   q      W8A16/W8A8: int8 [V,H]; FP8/MXFP8: e4m3 bytes [V,H]; MXFP4: uint8 [V,H/2],
 *          even element in the low nibble
 *   scales W8A16/FP8: fp16 [V]; W8A8: fp32 [V]; MX: uint8 E8M0 [V, H/32]
 * ------------------------------------------------------------------------- */
int vqk_quantize_weight(int mode, const void* w, int w_dtype, int64_t V, int64_t H, int64_t ldw,
                        void* q, void* scales, void* stream);

/* ---------------------------------------------------------------------------
 * Runtime activation quantisation.  Replaces the torch code inside the
 * launchers: `x.to(float8_e4m3fn)` (_quant.py:413), `_quantize_to_mxfp8(x)`
 * (_quant.py:448,495), per-tensor int8 (_quant.py:536-540, without the
 * `.item()` host sync of :548 - the scale stays on the device).
 *   xq  W8A16: fp16 [B,H] (dtype conversion only); FP8/MX: e4m3 bytes [B,H]; W8A8: int8 [B,H]
 *   xs  W8A8: float[2] ([0] = scale, [1] = scratch); MX: uint8 [B, H/32]; else ignored
 * ------------------------------------------------------------------------- */
int vqk_quantize_act(int mode, const void* x, int x_dtype, int64_t B, int64_t H, int64_t ldx,
                     void* xq, void* xs, void* stream);

/* ---------------------------------------------------------------------------
 * Sampling parameters (all arrays on the device, length B).  Semantics follow
 * _gumbel_block_argmax_kernel (src/vllm_quant_kernels/_sampler_kernels.py:38-120)
 * with Triton's Philox (`tl.rand(seed, global_vocab_index)`):
 *   temperature NULL        -> every row is plain argmax (HAS_TEMPERATURE=False)
 *   temperature[i] < 1e-5   -> row i is greedy
 *   topk_threshold          -> reference style raw-logit threshold, keep l >= thr[i]
 *                              (_sampler.py:62-93); overrides top_k
 *   top_k[i]                -> computed on the device; <= 0 or >= vocab_total disables
 *   top_p[i]                -> nucleus AFTER temperature and top-k, vLLM semantics
 *                              (vllm/v1/sample/ops/topk_topp_sampler.py:349-369);
 *                              >= 1 disables.  Not on the reference's fast path.
 * Token ids are global: local column + vocab_offset; noise uses the global id, so
 * the result does not depend on how the vocabulary is sharded.
 * ------------------------------------------------------------------------- */
typedef struct {
  const float* temperature;
  const int32_t* seeds;
  const int32_t* top_k;
  const float* top_p;
  const float* topk_threshold;
  int64_t vocab_offset; /* global id of local column 0 */
  int64_t vocab_total;  /* global vocabulary size (== V when not sharded) */
  float* logprobs;      /* optional OUT [B] (device): raw log-softmax of the sampled token, i.e. of the
                         * logits as given, before temperature / top-k / top-p (what vLLM reports by default;
                         * the reference sends such batches back to vLLM, _sampler.py:158-169).  From the first
                         * pass's per-slice maxima and sums of exponentials, no second pass over the row.
                         * vqk_sample on a single shard only; every other entry point returns
                         * VQK_ERR_UNSUPPORTED when it is set. */
} vqk_sample_params;

/* Per (rank, row) exchange record of a vocab-sharded step: 16-byte header
 * {float score; int32 token; int32 n; int32 flags} followed by VQK_RECORD_CAP
 * candidates {float raw_logit; int32 token}.  n == 0: the header holds the
 * shard's winner; n > 0: the shard's top-k candidate set. */
#define VQK_RECORD_CAP 126
#define VQK_RECORD_BYTES 1024
#define VQK_RECORD_FLAG_OVERFLOW 1  /* more candidates than VQK_RECORD_CAP */
#define VQK_RECORD_FLAG_NEEDS_ROW 2 /* row needs a full-row pass (top-p without top-k) */

/* ---------------------------------------------------------------------------
 * lm_head operator.  Replaces QuantizedLogitsProcessor._quantized_forward and the
 * five launchers _int8/_w8a8/_fp8/_mxfp8/_mxfp4_forward
 * (src/vllm_quant_kernels/_quant.py:382-643) plus their Triton kernels
 * (src/vllm_quant_kernels/_kernels.py:21-84,189-248,299-358,412-477,534-632,701-802).
 * ------------------------------------------------------------------------- */
typedef struct vqk_lm_head vqk_lm_head;

/* Describe one vocab shard: quantized rows [V, H] and their scales in the layouts
 * of vqk_quantize_weight.  Host-side object; allocates no device memory (it is given one of a
 * few counters that live inside the library).  One call at a time per handle: calls on the same
 * handle must be ordered on one stream. */
int vqk_lm_head_create(int mode, const void* q, const void* scales, int64_t V, int64_t H,
                       vqk_lm_head** out);
int vqk_lm_head_destroy(vqk_lm_head* h);

/* Workspace for vqk_lm_head_forward at batch B (sample != 0 if sampling is requested). */
int64_t vqk_lm_head_workspace_bytes(const vqk_lm_head* h, int64_t B, int sample);

/* logits[b, v] = x[b, :] . dequant(W[v, :]) with the mode's epilogue, rounded to fp16
 * (_quant.py:409,445,492,533,570), plus bias in fp16 (_quant.py:428-429).
 *   x        [B, H] fp16 or bf16, row stride ldx
 *   bias     fp16 [V] or NULL
 *   logits   fp16 [B, ld_logits] or NULL (not written when NULL)
 *   sp       NULL -> logits only.  Otherwise the sampler runs on the fp16-rounded
 *            logits inside the same pass (up to 16 rows: inside the same KERNEL, whose last
 *            CTA resolves the rows from per-slice lists of the largest logits; a row those
 *            lists cannot decide, and every top-k / top-p row of a larger batch, is resolved
 *            by a second kernel from its fp16 logits row, kept in the workspace):
 *              tokens/scores non-NULL -> final int64 token ids / fp32 winning scores
 *                                        (single shard: vocab_total == V);
 *              records non-NULL       -> [B] exchange records for a sharded step, to
 *                                        be all-gathered and given to vqk_sample_finalize.
 */
int vqk_lm_head_forward(vqk_lm_head* h, const void* x, int x_dtype, int64_t B, int64_t ldx,
                        const void* bias, void* logits, int64_t ld_logits,
                        const vqk_sample_params* sp, int64_t* tokens, float* scores, void* records,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* The post-ops vLLM's LogitsProcessor.forward applies to the logits after the matmul and the bias
 * (vllm/model_executor/layers/logits_processor.py:66-72; the reference left them to upstream, i.e.
 * to extra passes over [B, V]): soft_cap > 0 -> tanh(logits / soft_cap) * soft_cap, then
 * logits *= scale.  Set on the handle, applied in the epilogue of every following
 * vqk_lm_head_forward with upstream's fp16 roundings (each of its tensor ops rounds to fp16), so
 * both the logits written and the tokens sampled see them.  (0, 1) switches them off. */
int vqk_lm_head_set_post_ops(vqk_lm_head* h, float soft_cap, float scale);

/* Measurement aid (no counterpart in the reference): when both are non-NULL cudaEvent_t
 * handles, every following vqk_lm_head_forward on `h` records `start` right before and
 * `stop` right after its weight-streaming kernel launch(es) on the call's stream, so a
 * benchmark can time that kernel in place.  Pass NULLs to switch it off. */
int vqk_lm_head_set_kernel_events(vqk_lm_head* h, void* start_event, void* stop_event);
/* Measurement aid (no counterpart in the reference): a device buffer of gridDim x 16 uint64
 * (148 x 16 on B200) in which CTA c of the streaming and block-scaled lm_head kernels leaves
 * %globaltimer stamps at [c][0] entry, [c][1] weight stream done, [c][2] slice results written,
 * and the CTA that ran the sampler tail [c][3] tail start, [c][4] tail end, [c][5..] phases of row 0.  NULL switches it off. */
int vqk_lm_head_set_debug_times(vqk_lm_head* h, void* device_buffer);

/* ---------------------------------------------------------------------------
 * Stand-alone sampler on materialised logits.  Replaces fused_gumbel_sample
 * (src/vllm_quant_kernels/_sampler_kernels.py:123-182) and, with top_k / top_p,
 * the vLLM chain behind FusedSampler.sample (_sampler.py:144-206).
 *   logits [B, V] fp32 / bf16 / fp16, row stride ld
 * ------------------------------------------------------------------------- */
int64_t vqk_sample_workspace_bytes(int64_t B, int64_t V);
int vqk_sample(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
               const vqk_sample_params* sp, int64_t* tokens, float* scores, void* records,
               void* workspace, int64_t workspace_bytes, void* stream);

/* The same sampler for callers that must not allocate (no counterpart in the reference).
 * Some hosts cannot call cudaMalloc where they sample: an engine that measured its memory
 * once and handed every remaining byte to its KV cache has nothing left to ask for, and a
 * call made between the begin and end of a stream capture may not allocate at all.  This
 * entry point takes no workspace and makes no allocation of any kind: its scratch (the
 * per-slice arrays vqk_sample keeps in the caller's workspace) is a fixed array inside the
 * library, VQK_STATIC_SCRATCH_BYTES per GPU, held from library load until process exit.
 * Limits: B <= VQK_STATIC_MAX_ROWS and V <= VQK_STATIC_MAX_VOCAB, else VQK_ERR_TOO_LARGE;
 * single shard only (vocab_offset 0, vocab_total == V); tokens are required.
 * The first call on each device looks up the array's device address; make that first
 * call before any stream capture begins on that device.
 * All calls share the one array: the library rewrites every element it later reads, so
 * nothing carries over between calls, but two calls whose kernels overlap on the GPU
 * (different streams) race on it - serialise them. */
#define VQK_STATIC_MAX_ROWS 64
#define VQK_STATIC_MAX_VOCAB 262144
#define VQK_STATIC_SCRATCH_BYTES (3 * VQK_STATIC_MAX_ROWS * (VQK_STATIC_MAX_VOCAB / 256) * 4)
int vqk_sample_static(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
                      const vqk_sample_params* sp, int64_t* tokens, float* scores, void* stream);

/* Merge all-gathered records [G][B] into final tokens; every rank computes the same
 * answer.  Higher score wins, equal scores go to the lower token id (the first-index
 * rule of _sampler_kernels.py:116-120,180-181).  Rows whose records carry an overflow
 * flag get token -1. */
int vqk_sample_finalize(const void* records, int G, int64_t B, const vqk_sample_params* sp,
                        int64_t* tokens, float* scores, void* stream);

/* k-th largest raw logit per row; replaces _compute_topk_threshold (_sampler.py:62-93)
 * without its host sync.  top_k[i] <= 0 or >= V gives -inf for that row. */
int vqk_topk_threshold(const void* logits, int dtype, int64_t B, int64_t V, int64_t ld,
                       const int32_t* top_k, float* threshold, void* stream);

/* ---------------------------------------------------------------------------
 * Winner exchange between vocab shards (no counterpart in the reference, which is
 * single-GPU; the shape follows vLLM's LogitsProcessor.get_top_tokens,
 * vllm/model_executor/layers/logits_processor.py:106-156).  NCCL is loaded at run
 * time from the process (the copy PyTorch already loaded) or from libnccl.so.2.
 * ------------------------------------------------------------------------- */
typedef struct vqk_comm vqk_comm;
#define VQK_COMM_ID_BYTES 128
int vqk_comm_unique_id(void* id_out_host /* VQK_COMM_ID_BYTES */);
int vqk_comm_create(const void* id_host, int rank, int nranks, vqk_comm** out);
int vqk_comm_allgather(vqk_comm* c, const void* send, void* recv, int64_t bytes_per_rank, void* stream);
int vqk_comm_destroy(vqk_comm* c);

/* ---------------------------------------------------------------------------
 * The same exchange without NCCL, fused with the merge (no counterpart in the
 * reference): every rank (one process per GPU, all on one node) owns a landing
 * buffer that its peers map through CUDA IPC.  The warp that holds a row's record
 * stores it into every rank's buffer with plain 8-byte peer stores over NVLink (every
 * word is self-validating, so there is no flag and no fence), waits (bounded: a peer
 * that never arrives gives token -1 and sets vqk_device_error) for the other ranks'
 * records of the same step, merges them and hands the slots back.  No multicast, no
 * remote loads.  All ranks must make the same sequence of calls with the same B.  Safe
 * to capture in a CUDA graph (the step number lives in device memory).
 *   vqk_peer_create            allocates the landing buffer (not on the hot path) and returns
 *                              the handle to hand to every other rank (any transport).
 *   vqk_peer_connect           takes all ranks' handles, rank-major, own one included.
 *   vqk_peer_connect_pointers  the same for landing buffers the caller can already address
 *                              (several vqk_peer in one process: vqk_peer_local_buffer of each).
 *   vqk_peer_set_wait_limit    bound of every wait in polls (default about a second).
 *   vqk_lm_head_step_sharded   the whole sharded step in one call: this rank's lm_head shard,
 *                              its sampling stage, the exchange and the merge.  Up to 16 rows
 *                              ALL of it runs inside the lm_head kernel (its last CTA: one warp
 *                              per row); beyond, and for rows the lists cannot decide, the
 *                              full-row sampler kernel behind it does the exchange.  sp carries
 *                              this rank's vocab_offset and the global vocab_total; tokens and
 *                              scores are the merged result, identical on every rank.
 *   vqk_peer_exchange_finalize exchange + merge of records computed earlier (vqk_lm_head_forward
 *                              or vqk_sample with `records`), as a kernel of its own.
 * ------------------------------------------------------------------------- */
typedef struct vqk_peer vqk_peer;
#define VQK_PEER_HANDLE_BYTES 64
#define VQK_PEER_MAX_RANKS 8
int vqk_peer_create(int rank, int nranks, int64_t max_rows, vqk_peer** out,
                    void* handle_out_host /* VQK_PEER_HANDLE_BYTES */);
int vqk_peer_connect(vqk_peer* p, const void* all_handles_host /* nranks * VQK_PEER_HANDLE_BYTES */);
int vqk_peer_connect_pointers(vqk_peer* p, void* const* buffers_host /* nranks device pointers; own entry ignored */);
void* vqk_peer_local_buffer(vqk_peer* p);
int vqk_peer_set_wait_limit(vqk_peer* p, int64_t polls);
int64_t vqk_lm_head_step_sharded_workspace_bytes(const vqk_lm_head* h, int64_t B);
int vqk_lm_head_step_sharded(vqk_lm_head* h, vqk_peer* peer, const void* x, int x_dtype, int64_t B, int64_t ldx,
                             const void* bias, const vqk_sample_params* sp, int64_t* tokens, float* scores,
                             void* workspace, int64_t workspace_bytes, void* stream);
/* One decode step from HOST memory (no counterpart in the reference, whose hooks get device
 * tensors from vLLM): `x_host` [B, H] (x_dtype, rows contiguous) and the per-row arrays of
 * `sp_host` (HOST pointers; null where vqk_sample_params allows it) are staged through a pinned
 * buffer the handle owns and travel in ONE host-to-device copy; the step runs as
 * vqk_lm_head_forward would (vqk_lm_head_step_sharded when `peer` is given: sp_host then carries
 * this rank's vocab_offset and the global vocab_total); the tokens land in `tokens_host` [B], and the
 * call returns when they are there.  Without `scores_host` the kernels write the tokens straight
 * into mapped pinned memory and the host watches them arrive (bounded: then it falls back to a
 * stream synchronise), which saves the device-to-host copy and the wake-up of a blocking wait;
 * with `scores_host` [B] tokens and scores come back by one copy and a stream synchronise.
 * `workspace`: device memory of vqk_lm_head_step_host_workspace_bytes(h, B) (or more).  The
 * first call, and a call with a larger B than any before, allocate the staging buffers: not
 * inside a stream capture.  `bias` is a device pointer, as in vqk_lm_head_forward. */
int64_t vqk_lm_head_step_host_workspace_bytes(const vqk_lm_head* h, int64_t B);
int vqk_lm_head_step_host(vqk_lm_head* h, vqk_peer* peer /* or NULL */, const void* x_host, int x_dtype, int64_t B,
                          const void* bias, const vqk_sample_params* sp_host, int64_t* tokens_host,
                          float* scores_host /* or NULL */, void* workspace, int64_t workspace_bytes, void* stream);
int vqk_peer_exchange_finalize(vqk_peer* p, const void* records /* [B, VQK_RECORD_BYTES] device */, int64_t B,
                               const vqk_sample_params* sp, int64_t* tokens, float* scores, void* stream);
int vqk_peer_destroy(vqk_peer* p);

#ifdef __cplusplus
}
#endif
#endif /* VQK_H_ */
