/*
 * blockrank_b200 -- C ABI of the B200 (sm_100a) BlockRank prefill kernels.
 *
 * Every entry point is `extern "C"`, takes plain pointers, sizes and strides,
 * never allocates or frees device memory, and is asynchronous on the CUDA
 * stream it is given (a `cudaStream_t` passed as `void*`).  Functions return
 * 0 on success and a negative BRK_E_* code on failure; brk_last_error() gives
 * the message of the calling thread's last failure.
 *
 * Vocabulary.  A prompt is a sequence of S token slots split into M blocks:
 * block 0 is the instruction prefix, blocks 1..M-2 are documents, block M-1 is
 * the query block (M == 1: a single causal block; M == 2: prefix + query).
 * Block m of prompt b occupies slots [blk_start[b*M+m], +blk_len[b*M+m]);
 * blocks are ordered and do not overlap; slots outside every block are
 * padding.  This covers both the reference's left-padded (B, M, H) grid and a
 * padding-free packed layout.  Allowed (query, key) pairs -- the pattern of
 * src/blockrank/blockrank_std_attention.py:158-237 in the reference:
 *   same block and key slot <= query slot;
 *   query in a document block and key in block 0;
 *   query in the last block and key in any earlier block.
 *
 * Tensors are addressed as ptr[b*stride_b + s*stride_s + h*stride_h + d] in
 * elements (innermost stride 1), so the HF layout [B, S, heads, D] viewed as
 * (B, heads, S, D) is passed without a copy, and grouped-query K/V heads are
 * shared inside the kernels (no repeat_kv copy).
 */
#ifndef BLOCKRANK_B200_H_
#define BLOCKRANK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BRK_VERSION 102

#if defined(__GNUC__)
#define BRK_API __attribute__((visibility("default")))
#else
#define BRK_API
#endif

enum {
  BRK_OK = 0,
  BRK_E_ARG = -1,        /* bad shape / stride / alignment / null pointer */
  BRK_E_UNSUPPORTED = -2,/* head_dim, dtype or algorithm not available */
  BRK_E_WORKSPACE = -3,  /* workspace too small */
  BRK_E_CUDA = -4,       /* a CUDA call failed (launch, attribute, tensor map) */
  BRK_E_DEVICE = -5,     /* device is not sm_100 */
  BRK_E_TIMEOUT = -6     /* a bounded device-side wait gave up (reported by brk_status_poll) */
};

enum { BRK_BF16 = 0, BRK_F32 = 1 };

/* attention algorithm selector */
enum {
  BRK_ALGO_AUTO = 0,  /* tcgen05 kernel for bf16 / head_dim 128, otherwise SIMT */
  BRK_ALGO_SIMT = 1,  /* CUDA-core fp32-accumulate kernel: bf16 and fp32, head_dim 64 or 128 */
  BRK_ALGO_TC = 2     /* tcgen05 + TMEM + TMA kernel: bf16, head_dim 128 */
};

/* A (B, heads, S, D) tensor view; strides in elements, innermost stride 1. */
typedef struct brk_view {
  void* ptr;
  int64_t stride_b;
  int64_t stride_h;
  int64_t stride_s;
} brk_view;

/* Replaces the attention call made by the registered attention functions
 * (reference: eager_blockrank_attention_forward,
 * src/blockrank/blockrank_std_attention.py:96-262, and
 * kernelized_blockrank_attention_forward_with_full_mask,
 * src/blockrank/blockrank_triton_kernel_attention.py:609-746). */
typedef struct brk_attn_params {
  int32_t dtype;          /* BRK_BF16 or BRK_F32 (q, k, v, o share it) */
  int32_t algo;           /* BRK_ALGO_* */
  int32_t B, N, Nk, D;    /* prompts, query heads, KV heads, head dim */
  int32_t S;              /* token slots per prompt */
  int32_t M;              /* blocks per prompt */
  int32_t max_block_len;  /* upper bound on blk_len (sizes the grid) */
  float scale;            /* softmax scale (the model's `scaling`) */
  brk_view q, k, v, o;    /* o is written as [B, S, N, D] through its strides */
  float* lse;             /* optional [B, N, S] natural-log sum-exp of scaled logits; NULL to skip */
  const int32_t* blk_start; /* device, [B*M] */
  const int32_t* blk_len;   /* device, [B*M] */
  int32_t* status;        /* optional device word, zeroed by the caller once; see brk_status_poll */
  int32_t max_query_len;  /* upper bound on blk_len of the LAST block, or 0 if unknown (then max_block_len
                             is used); a tight bound shrinks the tensor-core path's workspace */
} brk_attn_params;

/* Requirements on the data that no call can check cheaply:
 *  - K and V must hold FINITE values in every slot the kernels may load: the slots of all blocks and up to 63
 *    slots behind the end of any block (tiles are loaded 64 keys at a time; slots past S are never read).  Keys
 *    outside a row's visible set get a probability of exactly zero, but 0 x Inf or 0 x NaN in V would still
 *    poison the row.  Zero-filled or token-filled padding (what a model produces) is fine.
 * What IS checked, on the device, by a small kernel in front of every attention call: every block lies inside
 * [0, S), is no longer than max_block_len (the last one: max_query_len, if given), and starts at or after the end
 * of its predecessor.  If not, the call writes nothing and the status word (if given) is set. */

BRK_API int brk_version(void);
BRK_API const char* brk_last_error(void);
/* 0 if the current device is sm_100, BRK_E_DEVICE otherwise. */
BRK_API int brk_device_check(void);

/* Block spans from the collator's left-padded (B, M, H) boolean mask (one byte
 * per slot).  Replaces the (B,1,M,H,H) additive mask built by
 * eager_blockrank_attention_mask (src/blockrank/blockrank_std_attention.py:264-309):
 * the kernels need only start/length per block. */
BRK_API int brk_spans_from_mask(const uint8_t* mask, int32_t B, int32_t M, int32_t H,
                        int32_t* blk_start, int32_t* blk_len, void* stream);

/* Device scratch the call needs (16-byte aligned; contents need not be initialised or
 * preserved between calls, but two calls in flight must not share it).  Every path needs at
 * least a 256-byte header (work counter, verdict of the span check); the tensor-core path adds
 * the partial results of the query block's key chunks for long prompts. */
BRK_API size_t brk_attn_fwd_workspace_bytes(const brk_attn_params* p);
BRK_API int brk_attn_fwd(const brk_attn_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Backward of the attention call, for training through the registered attention function.  Replaces what
 * autograd derives from the reference's differentiable paths (eager_blockrank_attention_forward and
 * sdpa_blockrank_attention_forward, src/blockrank/blockrank_std_attention.py:96-262, 472-650; the reference's
 * Triton path has no backward, src/blockrank/blockrank_triton_kernel_attention.py:759-761), as used by the
 * auxiliary-loss trainer (src/blockrank/trainer.py:51-107).
 * Inputs are the forward's q, k, v, its output o and its lse ([B, N, S], natural log) and the gradient d_o of o
 * (same layout as o).  Outputs dq (like q), dk and dv (like k, v; summed over the query heads of each KV group);
 * slots outside every block get zero gradients.  bf16: warp-level tensor-core MMA (fp32 accumulation);
 * fp32: CUDA cores (there N / Nk must divide 64). */
typedef struct brk_attn_bwd_params {
  int32_t dtype;          /* BRK_BF16 or BRK_F32 (q, k, v, o, d_o, dq, dk, dv share it) */
  int32_t B, N, Nk, D;    /* D = 64 or 128 */
  int32_t S, M, max_block_len;
  float scale;
  brk_view q, k, v, o, d_o;
  const float* lse;       /* [B, N, S] from the forward call */
  const int32_t* blk_start;
  const int32_t* blk_len;
  brk_view dq, dk, dv;    /* written through their strides; dk, dv: (B, Nk, S, D) views */
} brk_attn_bwd_params;

/* fp32 scratch: the rows' dot(d_o, o), the dk / dv accumulators and (bf16) the last block's dq; cleared by the call */
BRK_API size_t brk_attn_bwd_workspace_bytes(const brk_attn_bwd_params* p);
BRK_API int brk_attn_bwd(const brk_attn_bwd_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Device-side status.  The kernels never trap: a bounded wait that gives up, or malformed block spans, set
 * the caller's status word (brk_attn_params.status; first event wins) and the kernel returns normally.
 * brk_status_poll synchronises `stream`, reads the word and clears it: BRK_OK if it was zero,
 * BRK_E_TIMEOUT after a wait gave up (the outputs of that call are incomplete), BRK_E_ARG after malformed
 * spans (nothing was written); brk_last_error() names the event.  Call it where the host synchronises
 * anyway (e.g. when the scores are copied back).  No counterpart in the reference, which has no device-side
 * error reporting. */
BRK_API int brk_status_poll(int32_t* status, void* stream);
/* Self-test of that give-up path: one thread waits `budget` (1..65536) polls on a barrier nothing arrives
 * at, then records its code in *status and returns; a following brk_status_poll returns BRK_E_TIMEOUT.
 * Nothing faults or hangs. */
BRK_API int brk_selftest_bounded_wait(int32_t* status, uint32_t budget, void* stream);

/* Fused score epilogue.  Replaces _compute_last_block_scores_kernel +
 * compute_last_block_attention_scores
 * (src/blockrank/blockrank_triton_kernel_attention.py:432-606) followed by
 * compute_auxiliary_attention_loss(..., return_logits=True)
 * (src/blockrank/losses.py:37-78): for each signal row the softmax over all
 * valid document tokens is summed per document, without materialising the
 * (B, N, R, S) logit slab.
 *   rows      device [B*R] slot indices of the signal rows (inside the query block)
 *   doc_mass  device [B, N, R, M-2] fp32 out: per head / row normalised mass per document
 *   logits    device [B, M-2] fp32 out, optional: mean over heads and rows / temperature
 * workspace: brk_doc_scores_workspace_bytes() bytes of device scratch, 8-byte aligned, contents
 * need not be initialised.  One kernel launch (plus a memset of B counters): the CTA that finishes
 * a prompt last merges its per-document partials and writes doc_mass and logits. */
typedef struct brk_score_params {
  int32_t dtype;
  int32_t B, N, Nk, D, S, M, R;
  float scale;
  float temperature;
  brk_view q, k;
  const int32_t* rows;
  const int32_t* blk_start;
  const int32_t* blk_len;
  float* doc_mass;
  float* logits;
} brk_score_params;

BRK_API size_t brk_doc_scores_workspace_bytes(const brk_score_params* p);
BRK_API int brk_doc_scores(const brk_score_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* Allocation-free variant of brk_doc_scores.  It has no counterpart in the reference.
 *
 * Same inputs, outputs and results as brk_doc_scores, but the scratch between its two kernels
 * is a fixed BRK_STATIC_SCRATCH_BYTES array inside the library, so neither the library nor the
 * caller has to obtain device memory for it.  It is meant for callers that must not allocate
 * at the point of the call: a serving loop that reserved all of its device memory at start-up
 * and treats any later cudaMalloc as a bug (it synchronises the device and can fail under
 * memory pressure), or an embedding of the library into a host (another language runtime, a
 * plugin sandbox) that owns no device allocator at all and can only pass through the input and
 * output buffers it was given.
 *
 * Limits and rules:
 *  - 16384 + B*N*R*(M-2)*8 bytes must fit in BRK_STATIC_SCRATCH_BYTES (4 MiB; e.g. 8 prompts x 32
 *    heads x 2 rows x 1000 documents) and B*(Nk+1) <= 4096; larger problems are refused with
 *    BRK_E_WORKSPACE and a message that names both sizes.  Each GPU that loads the library holds
 *    the array until exit.
 *  - The first call on a device looks up the array's device address; make that first call
 *    outside any stream capture.
 *  - All calls on a device share the one array.  Nothing needs clearing between calls (every
 *    (max, sum) pair is rewritten before it is read, and the per-prompt completion counters count
 *    back to zero by the end of a call), but two calls that can run at the same time on the
 *    GPU -- different streams, or different host threads -- race on it: serialise them.  A call
 *    that was aborted half-way (device reset, a fault elsewhere) leaves the counters undefined.
 *  - `stream` must belong to the device that is current when the call is made.
 *  - No cudaMalloc / cudaFree / allocating library routine is called. */
#define BRK_STATIC_SCRATCH_BYTES (4u << 20)
BRK_API int brk_doc_scores_static(const brk_score_params* p, void* stream);

/* Compatibility output of the reference's second return value: raw scaled,
 * masked logits of the last R slots of the prompt against every slot,
 * out[B, N, R, S] in `dtype`, masked entries = 0.7 * lowest finite value of the
 * dtype (src/blockrank/blockrank_std_attention.py:233, :256-262, :306).
 * Uses q, k, scale, blk_* of brk_score_params; rows/doc_mass/logits ignored. */
BRK_API int brk_raw_scores(const brk_score_params* p, void* out, void* stream);

/* Runner helpers (the model code around the attention call; the reference
 * relies on transformers' modeling_mistral.py for these). All row-major. */
/* out = weight * (x * rsqrt(mean(x^2) + eps)); if residual != NULL first
 * residual += x (stored) and the norm is taken of the sum. */
BRK_API int brk_rmsnorm(int32_t dtype, const void* x, void* residual, const void* weight, void* out,
                int64_t rows, int32_t hidden, float eps, void* stream);
/* In-place rotate-half RoPE on q [T, N, D] and k [T, Nk, D] (row stride given
 * in elements), angle = pos[t] * inv_freq[i].  q may be NULL when N == 0, k when Nk == 0. */
BRK_API int brk_rope(int32_t dtype, void* q, int64_t q_row_stride, int32_t N, void* k, int64_t k_row_stride,
             int32_t Nk, int32_t D, const int32_t* pos, const float* inv_freq, int64_t T, void* stream);
/* out[r, c] = silu(gate_up[r, c]) * gate_up[r, inter + c]. */
BRK_API int brk_silu_mul(int32_t dtype, const void* gate_up, void* out, int64_t rows, int32_t inter, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BLOCKRANK_B200_H_ */
