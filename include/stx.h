/*
 * stx.h — C ABI of the B200 (sm_100a) contextual-sparsity MLP library (libstx.so).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes (no torch types),
 * returns an `int` status (STX_OK == 0) and never throws.  Unless stated otherwise all
 * data pointers are DEVICE pointers, every call is asynchronous on the `stream` it is
 * given (a `cudaStream_t` passed as `void*`), performs no allocation and no host
 * synchronisation, and may therefore be captured in a CUDA graph.  Entry points that
 * allocate, synchronise or touch host memory say so.
 *
 * The comment on each declaration names the interface of the reference project
 * (NimbleEdge/sparse_transformers, paths relative to that project) which it replaces.
 *
 * Conventions
 *   H  hidden size, I intermediate size, r predictor rank, B flattened batch rows,
 *   K  number of active neurons (lives on the device; read back only on request).
 *   dtype: element type of weights and activations (stx_dtype); accumulation is fp32.
 *   mask bits: uint32 words, neuron n is bit (n & 31) of word (n >> 5); unused high
 *   bits of the last word are zero.
 */
#ifndef STX_H_
#define STX_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define STX_VERSION 100

typedef enum {
  STX_OK = 0,
  STX_ERR_INVALID_ARG = 1,   /* null pointer, bad size, bad enum                         */
  STX_ERR_UNSUPPORTED = 2,   /* shape/dtype combination this build has no kernel for     */
  STX_ERR_CUDA = 3,          /* a CUDA runtime call failed; see stx_last_error()         */
  STX_ERR_NO_ACTIVE = 4,     /* mask left zero active neurons ("No active weights")      */
  STX_ERR_CACHE_INVALID = 5, /* getters used before any successful update                */
  STX_ERR_ALLOC = 6,         /* device allocation failed                                 */
  STX_ERR_TIMEOUT = 7,       /* a bounded device-side wait expired                       */
  STX_ERR_TOO_LARGE = 8      /* size exceeds a documented fixed limit                    */
} stx_status;

typedef enum { STX_F32 = 0, STX_F16 = 1, STX_BF16 = 2 } stx_dtype;

/* Activation applied to the gate (or, without a gate, to the up) projection.
 * Names follow transformers.activations.ACT2FN as used by src/modeling_skip.py:64-65. */
typedef enum {
  STX_ACT_RELU = 0,      /* "relu"  — also what the reference CPU op always applies (sparse_mlp_op.cpp:157,183) */
  STX_ACT_SILU = 1,      /* "silu"                                                   */
  STX_ACT_GELU_TANH = 2, /* "gelu_pytorch_tanh" (src/models/gemma3n/modelling_gemma_skip.py:61) */
  STX_ACT_SIGMOID = 3,   /* what the reference's unfinished CUDA kernels apply (sparse_mlp_cuda.cu:82-86) */
  STX_ACT_GELU = 4       /* "gelu" (erf form)                                        */
} stx_act;

/* Rule that turns predictor scores into a per-row boolean mask
 * (src/modeling_skip.py:204-213).                                                  */
typedef enum {
  STX_MASK_THRESHOLD = 0,  /* scores >= param  (param = 0 is the reference's "naive")           */
  STX_MASK_TOPK = 1,       /* exact top-k per row, k = (int)param                               */
  STX_MASK_STATISTICAL = 2 /* scores > mean + std_pop * param per row ("statistical_topk")      */
} stx_mask_method;

typedef struct stx_cache stx_cache_t;   /* differential weight cache (one per MLP layer) */
typedef struct stx_layer stx_layer_t;   /* predictor + cache + scratch of one sparse layer */
typedef struct stx_stack stx_stack_t;   /* a sequence of layers replayed as one CUDA graph */
typedef struct stx_peer stx_peer_t;     /* peer-memory exchange of the GPUs that share a layer */

/* ------------------------------------------------------------------ misc */

/* Thread-local description of the last non-OK status returned on this thread. */
const char* stx_last_error(void);
int stx_version(void);
const char* stx_status_string(int status);
/* Parse an activation name ("relu", "silu", "gelu_pytorch_tanh", "sigmoid", "gelu").
 * Returns the stx_act value or -1.                                                     */
int stx_act_from_name(const char* name);

/* ------------------------------------------------------------------ weight cache
 * Replaces class WeightCache (sparse_transformers/csrc/weight_cache.h:13-381).        */

/* Flags for stx_cache_create. */
#define STX_CACHE_ALIAS_GATE_UP 1u /* use the caller's gate/up [I,H] buffers as the pool instead of
                                      copying them; the caller must keep them alive and unchanged  */

/* Bytes of device memory stx_cache_create will allocate for these sizes (host function). */
int stx_cache_bytes(int64_t I, int64_t H, int dtype, int has_gate, unsigned flags, size_t* bytes_out);

/* WeightCache::WeightCache / init (weight_cache.h:148-227).  Allocates device memory
 * (cudaMalloc) for: the full pools gate/up [I,H] (unless aliased) and down transposed to
 * [I,H]; the packed pools gate/up/down [I,H]; index arrays.  gate_w/up_w are row-major
 * [I,H]; down_w is row-major [H,I] (nn.Linear layout) and is transposed on the device.
 * gate_w may be NULL when has_gate == 0.  The cache starts with an all-zero current mask;
 * if init_mask_bytes != NULL (device, I bytes, 0/1) it is applied exactly like
 * update_active_weights(init_mask) (weight_cache.h:223-226), else the cache is left
 * empty and invalid.  Work is enqueued on `stream`; the function does not synchronise. */
int stx_cache_create(stx_cache_t** out, int64_t I, int64_t H, int dtype, int has_gate,
                     const void* gate_w, const void* up_w, const void* down_w,
                     const uint8_t* init_mask_bytes, unsigned flags, void* stream);
int stx_cache_destroy(stx_cache_t* c);

/* WeightCache::update_active_weights (weight_cache.h:229-359) with a torch-style bool
 * mask: `mask_bytes` is I bytes on the device, non-zero = active.                      */
int stx_cache_update(stx_cache_t* c, const uint8_t* mask_bytes, void* stream);
/* Same with an already bit-packed mask (ceil(I/32) words on the device).               */
int stx_cache_update_bits(stx_cache_t* c, const uint32_t* mask_bits, void* stream);

/* WeightCache::get_num_active (weight_cache.h:374-377).  SYNCHRONISES `stream`, reads
 * K and the device status word.  Returns STX_ERR_NO_ACTIVE if an update left K == 0
 * (the reference throws "No active weights", weight_cache.h:117-118) and
 * STX_ERR_CACHE_INVALID before the first effective update (weight_cache.h:364).        */
int stx_cache_num_active(stx_cache_t* c, int64_t* k_out, void* stream);

/* WeightCache::get_concat_weight (weight_cache.h:362-366): rows 0..K-1 are the gate rows
 * of the active neurons in cache order, rows K..2K-1 their up rows ([2K,H] contiguous;
 * [K,H] without a gate).  The packed pools are kept per matrix, so this entry point
 * gathers them into the cache's concat buffer when that buffer is stale (one device copy
 * of 2*K*H elements) and returns its address.  SYNCHRONISES `stream` to learn K.       */
int stx_cache_concat_weight(stx_cache_t* c, void** ptr_out, int64_t* rows_out, void* stream);

/* WeightCache::get_active_down_weight (weight_cache.h:368-372): returns the packed down
 * pool; row j (H contiguous elements) is column active[j] of the [H,I] down matrix, i.e.
 * the reference tensor [H,K] with strides (1,H).  Zero-copy.  SYNCHRONISES `stream`.   */
int stx_cache_active_down(stx_cache_t* c, void** ptr_out, int64_t* k_out, void* stream);

/* Brings the packed rows up to date when layer steps ran with lazy row copies (see
 * stx_layer_set_lazy_cache); the getters above do this themselves.  Asynchronous.       */
int stx_cache_flush(stx_cache_t* c, void* stream);

/* Device addresses of the packed per-matrix pools ([I,H] capacity, first K rows valid)
 * and of the cache's device-resident K.  No synchronisation (and no flush).             */
int stx_cache_packed_ptrs(stx_cache_t* c, void** gate_out, void** up_out, void** down_out,
                          const int32_t** k_dev_out);

/* Copies the ordered list of active neuron ids (the reference's private `active_indices`,
 * weight_cache.h:44) to HOST memory `host_out` (capacity `cap` entries).  SYNCHRONISES. */
int stx_cache_active_indices(stx_cache_t* c, int32_t* host_out, int64_t cap, int64_t* k_out, void* stream);

/* Counters of the most recent update (HOST out-params; SYNCHRONISES): rows added,
 * rows removed, packed rows rewritten.                                                   */
int stx_cache_last_update_stats(stx_cache_t* c, int64_t* added, int64_t* removed, int64_t* rows_copied, void* stream);

/* ------------------------------------------------------------------ predictor + mask
 * Replaces FastLoRAProjection.forward (src/modeling_skip.py:52-53) and
 * SkipDecoderLayer._compute_binary_mask / _gaussian_topk (src/modeling_skip.py:197-214). */

/* Bytes of scratch stx_predict_mask needs (host function). */
int stx_predict_scratch_bytes(int64_t B, int64_t I, int64_t r, size_t* bytes_out);

/* scores = (x A^T) Bm^T with x [B,H], A [r,H] (predictor "down.weight"), Bm [I,r]
 * (predictor "up.weight"), all row-major in `dtype`; t = x A^T and the scores are rounded
 * to `dtype` like the reference's two nn.Linear calls; then the per-row rule `method`
 * with `param`, then OR over the B rows (mask.any(dim=0), modeling_skip.py:214).
 * mask_bits_out: ceil(I/32) words.  scores_out: optional [B,I] in `dtype` (may be NULL
 * for STX_MASK_THRESHOLD).  scratch: stx_predict_scratch_bytes() bytes, 16-byte aligned. */
int stx_predict_mask(const void* x, int64_t B, int64_t H, const void* A, int64_t r,
                     const void* Bm, int64_t I, int dtype, int method, float param,
                     uint32_t* mask_bits_out, void* scores_out, void* scratch, void* stream);

/* Expand a bit mask to I bytes (0/1), e.g. to hand it to torch as a bool tensor.        */
int stx_mask_bits_to_bytes(const uint32_t* bits, int64_t I, uint8_t* bytes_out, void* stream);
int stx_mask_bytes_to_bits(const uint8_t* bytes, int64_t I, uint32_t* bits_out, void* stream);

/* Replaces approx_topk_threshold (sparse_transformers/csrc/approx_topk.h:10-87):
 * scores [B,I] in `dtype` -> threshold [B] in `dtype` (the reference returns [B,1]).
 * scratch: stx_approx_topk_scratch_bytes() bytes.                                       */
int stx_approx_topk_scratch_bytes(int64_t B, int64_t I, size_t* bytes_out);
int stx_approx_topk_threshold(const void* scores, int64_t B, int64_t I, int64_t k, int dtype,
                              void* threshold_out, void* scratch, void* stream);

/* ------------------------------------------------------------------ sparse MLP forward
 * Replaces sparse_mlp_forward / sparse_mlp_forward_cpu / sparse_mlp_forward_cuda
 * (sparse_mlp_op.cpp:53-192, sparse_mlp_cuda.cu:284-361) and the expression the models
 * run, SkipMLP._forward_sparse_weight_cache (src/modeling_skip.py:114-117).             */

/* Bytes of scratch stx_sparse_mlp_forward needs for up to K active neurons (host function). */
int stx_mlp_scratch_bytes(int64_t B, int64_t H, int64_t K, size_t* bytes_out);

/* x [B,H]; concat_w [2K,H] (gate rows then up rows; [K,H] when has_gate == 0) with row
 * stride H; down_packed [K,H]: row j = column j of the [H,K] active down weight (pass
 * the storage of a [H,K] tensor whose strides are (1,H)).
 * combined_buf [B,2K] (or [B,K]): on return columns 0..K-1 hold act(gate)*up and columns
 * K..2K-1 hold up, as the reference leaves them (sparse_mlp_op.cpp:151-158).
 * down_buf [B,H]: the result.  scratch: stx_mlp_scratch_bytes() bytes, 16-byte aligned,
 * ZERO on the first call; its leading (256 + 4*B*H rounded up to 256) bytes are an fp32
 * accumulator and a counter that every call leaves zeroed again, the rest holds the
 * fp32 activations a[K][B] between the two kernels.  The extent of that leading region
 * depends on B and H: a buffer that is reused for a call with a different B or H must have
 * the new call's leading region zeroed again first (cudaMemsetAsync on the same stream).  Row blocks of 9 and more in
 * fp16/bf16 (prefill) run as two tcgen05 tensor-core GEMMs instead and keep their
 * activation matrix and a transposed copy of the down rows behind those regions.         */
int stx_sparse_mlp_forward(const void* x, int64_t B, int64_t H, const void* concat_w,
                           const void* down_packed, int64_t K, void* down_buf,
                           void* combined_buf, int act, int has_gate, int dtype,
                           void* scratch, void* stream);

/* No counterpart in the reference.  The same computation as stx_sparse_mlp_forward for
 * callers that may not allocate device memory (a server that fixes its HBM budget at
 * start-up, a plugin whose host owns the allocator): the scratch lives in a fixed
 * ~256 KiB device array inside the library image, held by every GPU that loads it.
 * Limit: B*(H+K) <= 65536 elements, else STX_ERR_TOO_LARGE.  The first call on a device
 * resolves the array's address; make it outside stream capture.  All calls on a device
 * share the array (it is cleared at the start of each call), so calls whose GPU work
 * overlaps race: keep them ordered on one stream.  Allocates nothing.                   */
int stx_sparse_mlp_forward_noalloc(const void* x, int64_t B, int64_t H, const void* concat_w,
                                   const void* down_packed, int64_t K, void* down_buf,
                                   void* combined_buf, int act, int has_gate, int dtype,
                                   void* stream);

/* SkipMLP._forward_sparse_weight_cache (src/modeling_skip.py:114-117) WITHOUT the two getters:
 * the sparse MLP of x [B,H] over the cache's packed rows, the number of active neurons read
 * on the device.  What get_concat_weight + get_active_down_weight + sparse_mlp_forward compute,
 * but asynchronous: no host read-back of K, no allocation, graph-capturable.  out [B,H].
 * scratch: stx_mlp_scratch_bytes(B, H, I) bytes, zeroed once (see stx_sparse_mlp_forward for the
 * reuse rule).  Row blocks of 9 and more (16-bit, gated) take the tensor-core path.  Rows that
 * lazy layer steps left stale are brought up to date first.                                  */
int stx_cache_mlp_forward(stx_cache_t* c, const void* x, int64_t B, void* out, int act, void* scratch, void* stream);

/* ------------------------------------------------------------------ fused layer step
 * One decode step of one sparse layer: predictor -> mask -> cache update -> sparse MLP
 * (SkipDecoderLayer.forward's sparse branch, src/modeling_skip.py:236-238,258, with K
 * never leaving the device).                                                            */

/* Creates the per-layer object (ALLOCATES scratch with cudaMalloc).  The layer keeps
 * pointers to A [r,H] and Bm [I,r]; the caller keeps them alive.  `cache` stays owned
 * by the caller.                                                                        */
int stx_layer_create(stx_layer_t** out, stx_cache_t* cache, const void* A, int64_t r,
                     const void* Bm, int method, float param, int act, int64_t max_batch);
int stx_layer_destroy(stx_layer_t* l);

/* x_pred [B,H]: input of the predictor (the layer's normed input, modeling_skip.py:235-238);
 * x_mlp [B,H]: input of the MLP (modeling_skip.py:257-258); they may be the same buffer.
 * out [B,H].  Asynchronous, no allocation, graph-capturable.                            */
int stx_layer_step(stx_layer_t* l, const void* x_pred, const void* x_mlp, int64_t B,
                   void* out, void* stream);
/* The same step restricted to some of its stages (bit mask); used to time stages apart.
 * Stages that are skipped leave their outputs as the previous call left them.  Up to 8
 * rows under the threshold rule (2..8 rows: 16-bit gated weights) run PREDICT_MASK and
 * MLP_GATEUP as ONE kernel when both bits are set (the mask never leaves the chip before
 * the rows are fetched); MLP_DOWN is then the deterministic sum of that kernel's per-CTA
 * partial outputs.  9 rows and more (16-bit, gated) run the MLP stage as tensor-core
 * GEMMs over the packed cache; for such a row block the MLP stage owns the cache upkeep:
 * it runs the index plan and the row copies itself, on its own stream, and a call that
 * names PLAN and/or COPY without MLP does nothing (so upkeep issued on a side stream can
 * never run concurrently with the upkeep of the MLP stage).                             */
#define STX_STAGE_PREDICT_T 1u     /* predictor, first half: t = A x            */
#define STX_STAGE_PREDICT_MASK 32u /* predictor, second half: scores -> mask bits */
#define STX_STAGE_PREDICT 33u      /* both                                      */
#define STX_STAGE_PLAN 2u    /* mask diff -> cache index plan             */
#define STX_STAGE_COPY 4u    /* rewrite the changed packed rows           */
#define STX_STAGE_MLP_GATEUP 8u  /* sparse gate/up projection + activation  */
#define STX_STAGE_MLP_DOWN 16u   /* sparse down projection                   */
#define STX_STAGE_MLP 24u        /* both                                     */
#define STX_STAGE_ALL 63u
int stx_layer_step_stages(stx_layer_t* l, const void* x_pred, const void* x_mlp, int64_t B,
                          void* out, void* stream, unsigned stages);
/* lazy != 0: a layer step advances the cache's index plan but defers the packed-row
 * copies until a cache getter (or stx_cache_flush) asks for the rows; the step's own MLP
 * gathers its rows from the full pools and never needs them.  Default: 0 (rows are copied
 * every step, as WeightCache::update_active_weights does).  Set before capturing a stack. */
int stx_layer_set_lazy_cache(stx_layer_t* l, int lazy);
/* Device pointer to the layer's current mask bits (ceil(I/32) words), valid after a step. */
int stx_layer_mask_bits(stx_layer_t* l, const uint32_t** bits_out);
/* *fused_out = 1 when a step of B rows runs PREDICT_MASK and the MLP as the one-kernel
 * pair described above (B <= 8, threshold rule, shape fits), else 0.  No reference
 * counterpart; bench and tests use it to name the kernels they time.                    */
int stx_layer_single_row_fused(stx_layer_t* l, int64_t B, int* fused_out);

/* Same step with HOST buffers: copies x (B*H elements, used for both inputs) to the
 * device, runs the step, copies the result back and SYNCHRONISES the stream.           */
int stx_layer_step_host(stx_layer_t* l, const void* x_host, int64_t B, void* out_host, void* stream);

/* A stack of L layers, every layer fed the same x [B,H]; out [L,B,H].  The L steps are
 * captured once into a CUDA graph and replayed.  stx_stack_create ALLOCATES and runs one
 * capture; the layers stay owned by the caller.
 *
 * One row (B == 1) under the threshold rule, all layers of one shape: the whole stack runs
 * as ONE persistent, cooperatively launched kernel; each cache then gets a second copy of
 * its pools with one contiguous record per neuron (ALLOCATED at create time).
 * Because every layer reads the same x, no layer waits for another one: the kernel
 * (k_stack_flow) forms the masks of all layers first and then streams the active rows of
 * layer after layer without a grid barrier in between; the output sums come last, and then
 * the caches' index plans and row copies, inside the same launch.  Sharded
 * (stx_layer_set_peer), the layers' sums are exchanged side by side in one go, which needs
 * L*H elements in the peer object (max_elems of stx_peer_create); with less room the layers
 * run one after the other (k_stack_b1: two grid barriers and one exchange per layer).
 * Environment, read when a stack is created:
 *   STX_STACK_STRICT=1        nothing of layer l+1 starts before out[l] is complete: the order
 *                             a model needs that feeds a layer's output forward (k_stack_b1,
 *                             four grid barriers per layer)
 *   STX_STACK_ORDER=layerwise k_stack_b1 in its overlapped order: layer after layer, t of
 *                             layer l+1 and the sum of layer l formed while rows stream
 *   STX_STACK_UPKEEP=kernels  index plans and row copies of the layers' caches in kernels of their
 *                             own behind k_stack_flow (default: inside its launch, where a CTA
 *                             has the shared memory for the plan's work space)
 *   STX_STACK_KERNEL=layers   keep the per-layer kernels (k_pred_t, k_mlp_b1, k_partial_reduce)
 *   STX_STACK_GROUP=n         at most n layers per launch of the persistent kernel (1..36)
 * Other shapes and batch sizes: the per-layer kernels, serialised on one stream, each layer's
 * cache upkeep on side branches.                                                         */
int stx_stack_create(stx_stack_t** out, stx_layer_t* const* layers, int64_t L, int64_t B);
/* Same, capturing only the given STX_STAGE_* bits of every layer step.                  */
int stx_stack_create_stages(stx_stack_t** out, stx_layer_t* const* layers, int64_t L, int64_t B,
                            unsigned stages);
int stx_stack_destroy(stx_stack_t* s);
/* Device addresses of the stack's own input [B,H] and output [L,B,H] buffers, which the
 * captured graph reads and writes.                                                     */
int stx_stack_buffers(stx_stack_t* s, void** x_in_out, void** out_out);
/* x: device [B,H], copied into the stack's input buffer first (NULL or the buffer itself:
 * use what is already there).  out: device [L,B,H] to copy the result to (NULL or the
 * stack's own buffer: leave it in place).                                              */
/* Every step ends by collecting the layers' device error bits (a bounded wait that expired,
 * a bounds check that skipped an access) into pinned host memory; a later call of
 * stx_stack_step / stx_stack_step_host that finds them set returns STX_ERR_TIMEOUT /
 * STX_ERR_INVALID_ARG instead of stepping (no synchronisation: the error surfaces one or
 * two calls late).  The bits are sticky in the caches' status words.                     */
int stx_stack_step(stx_stack_t* s, const void* x, void* out, void* stream);
int stx_stack_step_host(stx_stack_t* s, const void* x_host, void* out_host, void* stream);
/* Number of kernel launches one stack step replays (for launch accounting).            */
int stx_stack_launches_per_step(stx_stack_t* s, int64_t* n_out);

/* ------------------------------------------------------------------------------------------
 * Intermediate-dimension sharding over the GPUs of one node: the sum of the shards' partial
 * down projections.  The reference has no multi-GPU path; these entries implement the
 * all-reduce that sharding its MLP (sparse_mlp_op.cpp:66-94, the down projection sums over
 * neurons) needs.  One process per GPU.  Every rank creates a peer object (it ALLOCATES a
 * buffer of 16 * world * max_elems bytes on the current device), the host side exchanges the
 * 64-byte handles by any means (torch.distributed in this package) and connects.  A call of
 * stx_peer_allreduce - or a layer step after stx_layer_set_peer - is collective: every rank
 * must make the same calls in the same order.  The sum runs in fp32 in ascending rank order
 * (bit-identical on all ranks) inside ONE kernel that stores to the peers' memory over
 * NVLink and polls its own; there is no library collective underneath.  Waits are bounded
 * (environment STX_PEER_WAIT_ITERS at create time, default 2^22 polls, a few seconds): a
 * rank that never arrives makes the others finish with a wrong sum and STX_ERR_TIMEOUT in
 * stx_peer_status, it does not hang them.                                                */
#define STX_PEER_HANDLE_BYTES 64
int stx_peer_create(stx_peer_t** out, int rank, int world, int64_t max_elems);
int stx_peer_destroy(stx_peer_t* p);
/* Writes the STX_PEER_HANDLE_BYTES-byte interprocess handle of this rank's buffer.       */
int stx_peer_ipc_handle(stx_peer_t* p, void* handle_out);
/* handles: world * STX_PEER_HANDLE_BYTES bytes, rank-major (the own entry is ignored).
 * Every rank must have created its object before any rank connects.                     */
int stx_peer_connect_ipc(stx_peer_t* p, const void* handles);
/* Same-process alternative (one process driving several GPUs with peer access enabled):
 * buffers[q] = stx_peer_local_buffer of rank q's object.                                */
int stx_peer_connect_ptrs(stx_peer_t* p, void* const* buffers);
int stx_peer_local_buffer(stx_peer_t* p, void** buffer_out);
/* data[0..n) <- element-wise sum over ranks, in place; n <= max_elems.  Asynchronous,
 * allocation-free, graph-capturable.                                                    */
int stx_peer_allreduce(stx_peer_t* p, void* data, int64_t n, int dtype, void* stream);
/* SYNCHRONISES the stream; *status_out = STX_OK or STX_ERR_TIMEOUT (sticky).             */
int stx_peer_status(stx_peer_t* p, int* status_out, void* stream);
/* After this call a step of the layer ends with the all-reduce of its output over the
 * peer object's ranks: inside the step's last kernel for the single-row path, as one more
 * kernel otherwise.  peer == NULL detaches.  Set before capturing a stack.               */
int stx_layer_set_peer(stx_layer_t* l, stx_peer_t* peer);

/* ---- decode-time glue of the decoder layer around the MLP (one token, graph-capturable)
 * What SkipDecoderLayer.forward does between the predictor's input and the MLP
 * (src/modeling_skip.py:235-256): input RMSNorm -> self-attention with a KV cache ->
 * residual -> post-attention RMSNorm.  The projections stay GEMV calls of the caller.
 *
 * stx_attn_decode: qkv [ (n_heads + 2 n_kv_heads) * head_dim ] = the token's q, k, v
 * projections.  Rotates q and k by row *pos_dev of cos/sin [max_len, head_dim] (fp32,
 * rotate-half layout), stores k and v at position *pos_dev of k_cache / v_cache
 * [n_kv_heads, max_len, head_dim], attends over the positions 0..*pos_dev with scale
 * head_dim^-1/2 (grouped-query: n_heads / n_kv_heads query heads per cache head) and writes
 * out [n_heads * head_dim].  head_dim 64, 128 or 256; max_len <= 8192.  A position outside
 * 0..max_len-1 leaves everything untouched.  workspace: device memory of
 * stx_attn_decode_workspace_bytes bytes, zeroed once by the caller and then owned by the calls
 * (the keys of a head are split over several CTAs; their partial results meet in shared
 * memory of the CTAs' cluster, or in the workspace with STX_ATTN_MERGE=workspace in the
 * environment); calls that share a workspace must be ordered on one stream.
 * stx_add_rmsnorm: h_out = h + a (rounded to dtype; a == NULL: no add, h_out unused),
 * x_out = round(h_out * rsqrt(mean(h_out^2) + eps)) * w, the operation order of
 * LlamaSkipRMSNorm (src/models/llama/modelling_llama_skip.py:39-44).  h_out may alias h;
 * H <= 8192.                                                                               */
int stx_attn_decode(const void* qkv, const float* cos_table, const float* sin_table, const int64_t* pos_dev, void* k_cache,
                    void* v_cache, void* out, int n_heads, int n_kv_heads, int head_dim, int64_t max_len, int dtype,
                    void* workspace, void* stream);
int stx_attn_decode_workspace_bytes(int n_heads, int head_dim, int64_t* bytes_out);
int stx_add_rmsnorm(const void* h, const void* a, const void* w, float eps, void* h_out, void* x_out, int64_t H, int dtype,
                    void* stream);
/* y [N] = W [N,H] (row-major) times x, where x = h when w_norm == NULL, else
 * x = RMSNorm(h + a) * w_norm as in stx_add_rmsnorm, computed inside the same kernel (a may be
 * NULL).  With w_norm, h + a is also written to h_out and x to x_out when those are given;
 * h_out must not alias h.  H <= 8192, a multiple of the 16-byte vector; fp32 accumulation,
 * one rounding of y (NaN if a row's bulk copy did not arrive within the bounded wait).  The
 * projection in front of which SkipDecoderLayer.forward applies its
 * input RMSNorm (src/modeling_skip.py:235-241).                                            */
int stx_norm_gemv(const void* h, const void* a, const void* w_norm, float eps, const void* W, void* y, void* h_out,
                  void* x_out, int64_t H, int64_t N, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* STX_H_ */
