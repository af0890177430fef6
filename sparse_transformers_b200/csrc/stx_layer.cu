// Fused decode step of one sparse layer, and a stack of layers replayed as one CUDA graph.
//
// A layer step is: predictor -> mask bits -> cache plan -> row copies -> sparse MLP, all on
// one stream with K resident on the device (no host read-back, no allocation), i.e. the
// sparse branch of SkipDecoderLayer.forward (src/modeling_skip.py:236-238 and :258).
#include "stx_cache.cuh"
#include "stx_peer.cuh"
#include "stx_stack_b1.cuh"
#include "stx_cache_plan.cuh"

#include <cstdlib>

#include <algorithm>
#include <new>
#include <vector>

namespace stx {
int predict_mask(const void* x, int64_t B, int64_t H, const void* A, int64_t r, const void* Bm, int64_t I,
                 int dtype, int method, float param, uint32_t* bits, void* scores_out, void* scratch, unsigned parts,
                 cudaStream_t s);
float* b1_partial_region(void* scratch, int64_t H, int64_t K_cap);
void* mlp_prefill_region(void* scratch, int64_t B, int64_t H, int64_t K);
bool prefill_wanted(int64_t B, int64_t H, int64_t K, int dtype, int has_gate);
int prefill_forward(const void* x, int64_t B, int64_t H, const void* concat, const void* down_packed, int64_t K,
                    void* out, void* combined, int act, int dtype, void* scratch, int* status, const int* k_dev,
                    cudaStream_t s);
bool layer_b1_supported(int64_t B, int64_t H, int64_t I, int64_t r, int has_gate, int dtype, const void* gate,
                        const void* up, const void* down, const void* Bm);
int layer_b1_forward(const void* x, int64_t B, int64_t H, int64_t I, const void* gate, const void* up, const void* down,
                     const float* t, const void* Bm, int64_t r, float tau, uint32_t* bits, void* out, int act,
                     int has_gate, int dtype, float* partial, int* xchg, int* status, unsigned parts, const stx_peer* peer,
                     cudaStream_t s);
size_t layer_bn_xchg_bytes();
int peer_allreduce(const stx_peer* p, void* data, int64_t n, int dtype, cudaStream_t s);
int mlp_forward(const void* x, int64_t B, int64_t H, const void* gate, const void* up, const void* down,
                const int32_t* K_dev, int64_t K_host, int64_t K_cap, int up_after_gate, void* out, void* combined,
                int act, int has_gate, int dtype, void* scratch, int* status, unsigned parts,
                const uint32_t* mask_bits, int32_t* idx_out, int32_t* count_out, bool scratch_has_partial,
                cudaStream_t s);
}  // namespace stx

struct stx_layer {
  stx_cache* cache = nullptr;
  const void* A = nullptr;
  const void* Bm = nullptr;
  int64_t r = 0;
  int method = 0;
  float param = 0.f;
  int act = 0;
  int64_t max_batch = 0;
  uint32_t* bits = nullptr;
  int32_t* idx = nullptr;        // [I] active neuron ids in ascending order (set bits of `bits`)
  int32_t* count = nullptr;      // [0] number of active neurons, [1] last-block ticket of the predictor
  bool gather = true;            // MLP gathers rows from the full pools (needs H*elem >= 512 bytes)
  bool lazy = false;             // gather mode only: defer the packed-row copies until somebody reads them
  void* scores = nullptr;        // [max_batch, I], only for rules that need whole rows
  void* pred_scratch = nullptr;
  void* mlp_scratch = nullptr;
  float* partial = nullptr;  // per-CTA partial outputs of the fused kernels: [SMs][partial_rows][H] fp32
  int64_t partial_rows = 0;
  int* xchg = nullptr;  // count/id exchange between the CTAs of the 2..8-row kernel
  stx_peer* peer = nullptr;  // not owned: the shards' exchange; a step then ends with the all-reduce
  void* x_stage = nullptr;       // [max_batch, H] for the host-buffer entry point
  void* out_stage = nullptr;
};

struct stx_stack {
  std::vector<stx_layer*> layers;
  int64_t B = 0, H = 0;
  size_t es = 2;
  void* x_in = nullptr;   // [B,H]
  void* out = nullptr;    // [L,B,H]
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int64_t kernel_nodes = 0;
  std::vector<cudaEvent_t> events;  // [0,L) fork points, [L] join, [L+1, 2L+1) plan-done points, [2L+1] second join
  std::vector<void*> b1_scratch;    // persistent single-row kernel: counters, t and partial vectors per group of layers
  bool persistent = false;
  // Device status of the step (bounded waits that expired, bounds checks that skipped an access): the last
  // node of the graph ORs the layers' status words into status_dev and copies it to the pinned status_host,
  // which the NEXT stx_stack_step call reads without synchronising.
  stx::UpkeepArgs* upkeep_args = nullptr;  // device [L]: the layers' caches for upkeep that runs inside the flow kernel
  int** status_ptrs = nullptr;  // device [L]
  int* status_dev = nullptr;
  int* status_host = nullptr;
};

using namespace stx;

// ORs the layers' device status words into one (error bits only).
__global__ void k_stack_status(int* const* __restrict__ ptrs, int n, int* __restrict__ out) {
  int v = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) v |= *ptrs[i] & (DEV_TIMEOUT | DEV_BAD_INDEX);
  v = __reduce_or_sync(0xffffffffu, v);
  if (threadIdx.x == 0) *out = v;
}

extern "C" {

int stx_cache_mlp_forward(stx_cache_t* c, const void* x, int64_t B, void* out, int act, void* scratch, void* stream) {
  STX_CHECK_ARG(c && x && out && scratch, "stx_cache_mlp_forward: null pointer");
  STX_CHECK_ARG(B > 0, "stx_cache_mlp_forward: B must be positive");
  STX_CHECK_ARG(act >= STX_ACT_RELU && act <= STX_ACT_GELU, "stx_cache_mlp_forward: bad activation %d", act);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = cache_flush(c, s);
  if (rc != STX_OK) return rc;
  if (c->pk_gate && prefill_wanted(B, c->H, c->I, c->dtype, c->has_gate))
    return prefill_forward(x, B, c->H, c->pk_gate, c->pk_down, c->I, out, nullptr, act, c->dtype,
                           mlp_prefill_region(scratch, B, c->H, c->I), c->state + ST_STATUS, c->state + ST_K, s);
  return mlp_forward(x, B, c->H, c->pk_gate, c->pk_up, c->pk_down, c->state + ST_K, 0, c->I, 0, out, nullptr, act, c->has_gate,
                     c->dtype, scratch, c->state + ST_STATUS, 3u, nullptr, nullptr, nullptr, true, s);
}

int stx_layer_destroy(stx_layer_t* l) {
  if (!l) return STX_OK;
  cudaFree(l->bits);
  cudaFree(l->idx);
  cudaFree(l->count);
  cudaFree(l->scores);
  cudaFree(l->pred_scratch);
  cudaFree(l->mlp_scratch);
  cudaFree(l->partial);
  cudaFree(l->xchg);
  cudaFree(l->x_stage);
  cudaFree(l->out_stage);
  delete l;
  return STX_OK;
}

int stx_layer_create(stx_layer_t** out, stx_cache_t* cache, const void* A, int64_t r, const void* Bm, int method,
                     float param, int act, int64_t max_batch) {
  STX_CHECK_ARG(out, "stx_layer_create: out is null");
  *out = nullptr;
  STX_CHECK_ARG(cache && A && Bm, "stx_layer_create: null pointer");
  STX_CHECK_ARG(r > 0 && max_batch > 0, "stx_layer_create: r and max_batch must be positive");
  STX_CHECK_ARG(method >= STX_MASK_THRESHOLD && method <= STX_MASK_STATISTICAL, "stx_layer_create: bad method %d", method);
  STX_CHECK_ARG(act >= STX_ACT_RELU && act <= STX_ACT_GELU, "stx_layer_create: bad activation %d", act);
  stx_layer* l = new (std::nothrow) stx_layer();
  if (!l) {
    set_error("stx_layer_create: out of host memory");
    return STX_ERR_ALLOC;
  }
  l->cache = cache;
  l->A = A;
  l->Bm = Bm;
  l->r = r;
  l->method = method;
  l->param = param;
  l->act = act;
  l->max_batch = max_batch;
  const int64_t I = cache->I, H = cache->H;
  size_t pred_bytes = 0, mlp_bytes = 0;
  stx_predict_scratch_bytes(max_batch, I, r, &pred_bytes);
  // The scratch layout depends on the row count of a call (a single row keeps per-CTA partial
  // vectors, few rows on the tensor-core path keep split-contraction partials whose size is not
  // monotonic in B): size the buffer for the worst case over 1..max_batch.  Within a bucket of
  // equal output-tile count the need grows with B, so the bucket tops are enough.
  stx_mlp_scratch_bytes(max_batch, H, I, &mlp_bytes);
  for (int64_t b = 1; b < max_batch; b = (b < 128 ? 128 : b + 256 - b % 256)) {
    size_t need = 0;
    stx_mlp_scratch_bytes(b, H, I, &need);
    mlp_bytes = std::max(mlp_bytes, need);
  }
  const size_t es = dtype_size(cache->dtype);
  // 16-bit rows narrower than 32 chunks fall back to the packed cache inside the MLP
  cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&l->bits), ((I + 31) / 32) * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&l->idx), I * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&l->count), 64);
  if (e == cudaSuccess) e = cudaMemset(l->count, 0, 64);
  if (e == cudaSuccess) e = cudaMemset(l->idx, 0, I * sizeof(int32_t));
  if (e == cudaSuccess) e = cudaMemset(l->bits, 0, ((I + 31) / 32) * sizeof(uint32_t));
  l->gather = (H * es) >= 512 && (H * es) % 16 == 0 && I <= 65536 && (I + 131) / 132 + 4 <= 512;
  if (e == cudaSuccess) e = cudaMalloc(&l->pred_scratch, pred_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&l->mlp_scratch, mlp_bytes);
  if (e == cudaSuccess) e = cudaMemset(l->mlp_scratch, 0, mlp_bytes);
  if (e == cudaSuccess) {
    l->partial_rows = std::min<int64_t>(max_batch, 8);
    e = cudaMalloc(reinterpret_cast<void**>(&l->partial), sizeof(float) * num_sms() * l->partial_rows * H);
  }
  if (e == cudaSuccess && max_batch > 1) {
    e = cudaMalloc(reinterpret_cast<void**>(&l->xchg), layer_bn_xchg_bytes());
    if (e == cudaSuccess) e = cudaMemset(l->xchg, 0, layer_bn_xchg_bytes());
  }
  if (e == cudaSuccess && method != STX_MASK_THRESHOLD) e = cudaMalloc(&l->scores, static_cast<size_t>(max_batch) * I * es);
  if (e != cudaSuccess) {
    set_error("stx_layer_create: device allocation failed: %s", cudaGetErrorString(e));
    stx_layer_destroy(l);
    return STX_ERR_ALLOC;
  }
  *out = l;
  return STX_OK;
}

// Up to 8 rows under the threshold rule: scores, mask, gather and MLP of a neuron stay in one CTA
// (k_mlp_b1 for one row, k_mlp_bn for 2..8), followed by the sum of the per-CTA partials.
static bool single_row_fusable(const stx_layer* l, int64_t B) {
  const stx_cache* c = l->cache;
  return l->partial && B <= l->partial_rows && l->gather && l->method == STX_MASK_THRESHOLD &&
         layer_b1_supported(B, c->H, c->I, l->r, c->has_gate, c->dtype, c->pool_gate, c->pool_up, c->pool_down, l->Bm);
}

// One step with the cache maintenance (plan + row copies) optionally on a second stream.
// With `gather` the MLP reads the active rows straight from the full pools through the list
// of set mask bits, so it needs neither the index plan nor the copied rows: the differential
// cache is then kept current off the critical path (side stream), which is where a GPU wants
// it — contiguity of the active rows buys nothing when every row is a multi-KB burst.
static int layer_step_streams(stx_layer* l, const void* x_pred, const void* x_mlp, int64_t B, void* out, cudaStream_t s,
                              cudaStream_t side, cudaEvent_t fork_ev, unsigned stages, cudaStream_t side2 = nullptr,
                              cudaEvent_t plan_ev = nullptr, bool* used_side2 = nullptr) {
  stx_cache* c = l->cache;
  int rc = STX_OK;
  // One row under the threshold rule: scores, mask, gather and MLP of a neuron stay in one CTA.
  float* partial = single_row_fusable(l, B) ? l->partial : nullptr;
  const bool fuse = partial && (stages & STX_STAGE_PREDICT_MASK) && (stages & STX_STAGE_MLP) && x_mlp && out;
  if (stages & STX_STAGE_PREDICT) {
    STX_CHECK_ARG(x_pred, "stx_layer_step: x_pred is null");
    const unsigned pparts = ((stages & STX_STAGE_PREDICT_T) ? 1u : 0u) | (((stages & STX_STAGE_PREDICT_MASK) && !fuse) ? 2u : 0u);
    if (pparts) {
      rc = predict_mask(x_pred, B, c->H, l->A, l->r, l->Bm, c->I, c->dtype, l->method, l->param, l->bits, l->scores,
                        l->pred_scratch, pparts, s);
      if (rc != STX_OK) return rc;
    }
  }
  // Row blocks of 9 and more (16-bit, gated): the packed cache IS the operand of two tensor-core
  // GEMMs, so its maintenance comes first, on the same stream; the GEMMs are shaped for all I
  // slots and follow the device-side K (no host read-back, graph-capturable).
  const bool big = !fuse && c->pk_gate && prefill_wanted(B, c->H, c->I, c->dtype, c->has_gate);
  const bool gather = l->gather && !big;
  const bool forked = side != s && gather;
  cudaStream_t cs = forked ? side : s;  // stream of the cache maintenance
  const bool fork_needed = forked && (stages & (STX_STAGE_PLAN | STX_STAGE_COPY));
  if (fork_needed && !fuse) {
    STX_CUDA(cudaEventRecord(fork_ev, s));
    STX_CUDA(cudaStreamWaitEvent(side, fork_ev, 0));
  }
  if (fuse) {
    const float* t = static_cast<const float*>(l->pred_scratch);
    if (stages & STX_STAGE_MLP_GATEUP) {
      rc = layer_b1_forward(x_mlp, B, c->H, c->I, c->pool_gate, c->pool_up, c->pool_down, t, l->Bm, l->r, l->param, l->bits,
                            out, l->act, c->has_gate, c->dtype, partial, l->xchg, c->state + ST_STATUS, 1u, l->peer, s);
      if (rc != STX_OK) return rc;
    }
    if (fork_needed) {  // the mask exists once that kernel is done
      STX_CUDA(cudaEventRecord(fork_ev, s));
      STX_CUDA(cudaStreamWaitEvent(side, fork_ev, 0));
    }
    if (stages & STX_STAGE_MLP_DOWN) {
      rc = layer_b1_forward(x_mlp, B, c->H, c->I, c->pool_gate, c->pool_up, c->pool_down, t, l->Bm, l->r, l->param, l->bits,
                            out, l->act, c->has_gate, c->dtype, partial, l->xchg, c->state + ST_STATUS, 2u, l->peer, s);
      if (rc != STX_OK) return rc;
    }
  }
  if (!gather) {
    // The MLP reads the packed cache: plan and copies come first, on the same stream.  For a big row
    // block the MLP stage OWNS the maintenance: a call that asks for PLAN and/or COPY without the MLP
    // stage does nothing, so a caller that issues those stages on side streams (as it must for the
    // gathering kernels) can never run a second plan concurrently with the one of the MLP stage.
    const bool plan_here = big ? (stages & STX_STAGE_MLP) != 0 : (stages & STX_STAGE_PLAN) != 0;
    const bool copy_here = big ? (stages & STX_STAGE_MLP) != 0 : (stages & STX_STAGE_COPY) != 0;
    if (plan_here) {
      rc = cache_plan(c, l->bits, s);
      if (rc != STX_OK) return rc;
    }
    if (copy_here) {
      rc = cache_copy_rows(c, s);
      if (rc != STX_OK) return rc;
    }
  }
  if ((stages & STX_STAGE_MLP) && big) {
    STX_CHECK_ARG(x_mlp && out, "stx_layer_step: x_mlp/out is null");
    rc = prefill_forward(x_mlp, B, c->H, c->pk_gate, c->pk_down, c->I, out, nullptr, l->act, c->dtype,
                         mlp_prefill_region(l->mlp_scratch, B, c->H, c->I), c->state + ST_STATUS, c->state + ST_K, s);
    if (rc != STX_OK) return rc;
    if (l->peer && l->peer->world > 1) {
      rc = peer_allreduce(l->peer, out, B * c->H, c->dtype, s);
      if (rc != STX_OK) return rc;
    }
  }
  if ((stages & STX_STAGE_MLP) && !fuse && !big) {
    STX_CHECK_ARG(x_mlp && out, "stx_layer_step: x_mlp/out is null");
    const unsigned parts = ((stages & STX_STAGE_MLP_GATEUP) ? 1u : 0u) | ((stages & STX_STAGE_MLP_DOWN) ? 2u : 0u);
    if (gather)
      rc = mlp_forward(x_mlp, B, c->H, c->pool_gate, c->pool_up, c->pool_down, l->count, 0, c->I, 0, out, nullptr, l->act,
                       c->has_gate, c->dtype, l->mlp_scratch, c->state + ST_STATUS, parts, l->bits, l->idx, l->count, true, s);
    else
      rc = mlp_forward(x_mlp, B, c->H, c->pk_gate, c->pk_up, c->pk_down, c->state + ST_K, 0, c->I, 0, out, nullptr, l->act,
                       c->has_gate, c->dtype, l->mlp_scratch, c->state + ST_STATUS, parts, nullptr, nullptr, nullptr, true, s);
    if (rc != STX_OK) return rc;
    if ((stages & STX_STAGE_MLP_DOWN) && l->peer && l->peer->world > 1) {
      rc = peer_allreduce(l->peer, out, B * c->H, c->dtype, s);
      if (rc != STX_OK) return rc;
    }
  }
  if (gather) {
    if (stages & STX_STAGE_PLAN) {
      rc = cache_plan(c, l->bits, cs, l->lazy);
      if (rc != STX_OK) return rc;
    }
    if ((stages & STX_STAGE_COPY) && !l->lazy) {
      // With a second side stream the row copies of this layer leave the plan's stream, so the next
      // layer's index plan (a single block, latency-bound) does not queue behind them.
      cudaStream_t ccs = cs;
      if (forked && side2 && plan_ev) {
        STX_CUDA(cudaEventRecord(plan_ev, cs));
        STX_CUDA(cudaStreamWaitEvent(side2, plan_ev, 0));
        ccs = side2;
        if (used_side2) *used_side2 = true;
      }
      rc = cache_copy_rows(c, ccs);
      if (rc != STX_OK) return rc;
    }
  }
  return rc;
}

int stx_layer_step_stages(stx_layer_t* l, const void* x_pred, const void* x_mlp, int64_t B, void* out, void* stream,
                          unsigned stages) {
  STX_CHECK_ARG(l, "stx_layer_step: null layer");
  STX_CHECK_ARG(B > 0 && B <= l->max_batch, "stx_layer_step: B=%lld outside 1..max_batch=%lld", static_cast<long long>(B),
                static_cast<long long>(l->max_batch));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return layer_step_streams(l, x_pred, x_mlp, B, out, s, s, nullptr, stages);
}

int stx_layer_step(stx_layer_t* l, const void* x_pred, const void* x_mlp, int64_t B, void* out, void* stream) {
  STX_CHECK_ARG(l && x_pred && x_mlp && out, "stx_layer_step: null pointer");
  return stx_layer_step_stages(l, x_pred, x_mlp, B, out, stream, STX_STAGE_ALL);
}

int stx_layer_set_lazy_cache(stx_layer_t* l, int lazy) {
  STX_CHECK_ARG(l, "stx_layer_set_lazy_cache: null layer");
  l->lazy = lazy != 0 && l->gather;
  return STX_OK;
}

int stx_layer_set_peer(stx_layer_t* l, stx_peer_t* peer) {
  STX_CHECK_ARG(l, "stx_layer_set_peer: null layer");
  if (peer) {
    STX_CHECK_ARG(peer->connected, "stx_layer_set_peer: connect the peer object first");
    STX_CHECK_ARG(peer->max_elems >= l->max_batch * l->cache->H,
                  "stx_layer_set_peer: max_elems=%lld is smaller than max_batch*H=%lld", static_cast<long long>(peer->max_elems),
                  static_cast<long long>(l->max_batch * l->cache->H));
  }
  l->peer = peer;
  return STX_OK;
}

int stx_layer_single_row_fused(stx_layer_t* l, int64_t B, int* fused_out) {
  STX_CHECK_ARG(l && fused_out, "stx_layer_single_row_fused: null pointer");
  *fused_out = single_row_fusable(l, B) ? 1 : 0;
  return STX_OK;
}

int stx_layer_mask_bits(stx_layer_t* l, const uint32_t** bits_out) {
  STX_CHECK_ARG(l && bits_out, "stx_layer_mask_bits: null pointer");
  *bits_out = l->bits;
  return STX_OK;
}

int stx_layer_step_host(stx_layer_t* l, const void* x_host, int64_t B, void* out_host, void* stream) {
  STX_CHECK_ARG(l && x_host && out_host, "stx_layer_step_host: null pointer");
  STX_CHECK_ARG(B > 0 && B <= l->max_batch, "stx_layer_step_host: B outside 1..max_batch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t bytes = static_cast<size_t>(B) * l->cache->H * dtype_size(l->cache->dtype);
  if (!l->x_stage) {
    const size_t cap = static_cast<size_t>(l->max_batch) * l->cache->H * dtype_size(l->cache->dtype);
    cudaError_t e = cudaMalloc(&l->x_stage, cap);
    if (e == cudaSuccess) e = cudaMalloc(&l->out_stage, cap);
    if (e != cudaSuccess) {
      set_error("stx_layer_step_host: staging allocation failed: %s", cudaGetErrorString(e));
      return STX_ERR_ALLOC;
    }
  }
  STX_CUDA(cudaMemcpyAsync(l->x_stage, x_host, bytes, cudaMemcpyHostToDevice, s));
  int rc = stx_layer_step(l, l->x_stage, l->x_stage, B, l->out_stage, stream);
  if (rc != STX_OK) return rc;
  STX_CUDA(cudaMemcpyAsync(out_host, l->out_stage, bytes, cudaMemcpyDeviceToHost, s));
  STX_CUDA(cudaStreamSynchronize(s));
  return STX_OK;
}

int stx_stack_destroy(stx_stack_t* s) {
  if (!s) return STX_OK;
  if (s->exec) cudaGraphExecDestroy(s->exec);
  if (s->graph) cudaGraphDestroy(s->graph);
  for (cudaEvent_t ev : s->events) cudaEventDestroy(ev);
  for (void* p : s->b1_scratch) cudaFree(p);
  cudaFree(s->upkeep_args);
  cudaFree(s->status_ptrs);
  cudaFree(s->status_dev);
  if (s->status_host) cudaFreeHost(s->status_host);
  cudaFree(s->x_in);
  cudaFree(s->out);
  delete s;
  return STX_OK;
}

// A single row through layers that all take the one-kernel path of the threshold rule and share
// their shapes: the whole stack runs as ONE persistent kernel per group of layers
// (stx_stack_b1.cu); the cache upkeep of every layer (index plan, row copies) forks off behind the
// group's kernel, one branch per layer, and joins at the end of the step.
static bool stack_persistent_wanted(const stx_stack* s, unsigned stages) {
  const unsigned need = STX_STAGE_PREDICT | STX_STAGE_MLP;
  if (s->B != 1 || (stages & need) != need) return false;
  const stx_layer* l0 = s->layers[0];
  const stx_cache* c0 = l0->cache;
  // which of the two persistent kernels will run decides how large I may be
  const char* st = getenv("STX_STACK_STRICT");
  const bool strict = st && atoi(st) != 0;
  const int64_t gsz = std::min<int64_t>(static_cast<int64_t>(s->layers.size()), STACK_B1_MAX_LAYERS);
  const bool flow = !strict && !(l0->peer && l0->peer->world > 1 && gsz * c0->H > l0->peer->max_elems);
  if (!stack_b1_supported(c0->H, c0->I, l0->r, c0->has_gate, c0->dtype, flow)) return false;
  for (const stx_layer* l : s->layers) {
    const stx_cache* c = l->cache;
    if (!single_row_fusable(l, 1) || l->peer != l0->peer || c->I != c0->I || c->has_gate != c0->has_gate || l->r != l0->r) return false;
  }
  return true;
}

// Layers per launch of the persistent kernel: STX_STACK_GROUP in the environment (1..40), default
// all layers in one launch.  Smaller groups let the cache upkeep of a group overlap the next group.
static int64_t stack_group_size(int64_t L) {
  int64_t g = std::min<int64_t>(L, STACK_B1_MAX_LAYERS);
  if (const char* e = getenv("STX_STACK_GROUP")) {
    const long v = strtol(e, nullptr, 10);
    if (v >= 1 && v <= STACK_B1_MAX_LAYERS) g = std::min<int64_t>(g, v);
  }
  return g;
}

// Last nodes of a step's graph: the layers' error bits -> one word -> pinned host memory.
static int capture_status(stx_stack* s, cudaStream_t cs) {
  k_stack_status<<<1, 32, 0, cs>>>(s->status_ptrs, static_cast<int>(s->layers.size()), s->status_dev);
  STX_LAUNCH_CHECK("k_stack_status");
  STX_CUDA(cudaMemcpyAsync(s->status_host, s->status_dev, sizeof(int), cudaMemcpyDeviceToHost, cs));
  return STX_OK;
}

static int capture_persistent(stx_stack* s, unsigned stages, cudaStream_t cs, std::vector<cudaStream_t>& sides) {
  const int64_t L = static_cast<int64_t>(s->layers.size());
  const size_t xbytes = static_cast<size_t>(s->H) * s->es;
  const stx_layer* l0 = s->layers[0];
  const int64_t gsz = stack_group_size(L);
  const bool strict = getenv("STX_STACK_STRICT") && atoi(getenv("STX_STACK_STRICT")) != 0;
  const bool upkeep = (stages & (STX_STAGE_PLAN | STX_STAGE_COPY)) != 0;
  size_t ev = 0;
  std::vector<bool> forked((L + gsz - 1) / gsz, false);
  for (int64_t g0 = 0, gi = 0; g0 < L; g0 += gsz, ++gi) {
    const int64_t n = std::min<int64_t>(gsz, L - g0);
    StackB1Args a = {};
    for (int64_t i = 0; i < n; ++i) {
      stx_layer* l = s->layers[g0 + i];
      stx_cache* c = l->cache;
      StackLayerDesc& d = a.layer[i];
      d.cat = c->pool_cat;
      d.A = l->A;
      d.Bm = l->Bm;
      d.bits = l->bits;
      d.out = static_cast<char*>(s->out) + (g0 + i) * xbytes;
      d.status = c->state + ST_STATUS;
      d.tau = l->param;
      d.act = l->act;
    }
    a.x = s->x_in;
    a.L = static_cast<int>(n);
    a.H = static_cast<int>(s->H);
    a.I = static_cast<int>(l0->cache->I);
    a.r = static_cast<int>(l0->r);
    a.has_gate = l0->cache->has_gate;
    a.strict = strict ? 1 : 0;
    a.peer = PeerArgs{};
    a.peer.world = 1;
    if (l0->peer && l0->peer->world > 1) {
      if (!peer_args(l0->peer, &a.peer)) {
        set_error("stx_stack_create: the layers' peer object is not connected");
        return STX_ERR_INVALID_ARG;
      }
      if (s->H > l0->peer->max_elems) {
        set_error("stx_stack_create: H=%lld exceeds the peer object's max_elems", static_cast<long long>(s->H));
        return STX_ERR_INVALID_ARG;
      }
    }
    // where it has the room, the flow kernel keeps the caches up to date itself (plans, then row copies)
    const unsigned both = STX_STAGE_PLAN | STX_STAGE_COPY;
    const bool inside = (stages & both) == both && s->upkeep_args && stack_flow_upkeep_inside(a, l0->cache->dtype);
    a.upkeep = inside ? s->upkeep_args + g0 : nullptr;
    int rc = stack_b1_forward(a, s->b1_scratch[gi], l0->cache->dtype, cs);
    if (rc != STX_OK) return rc;
    if (inside) {
      for (int64_t i = 0; i < n; ++i)
        if (s->layers[g0 + i]->lazy) s->layers[g0 + i]->cache->lazy_used = true;
      continue;
    }
    if (!upkeep) continue;
    // the masks of the group exist now: one branch per layer
    forked[gi] = true;
    STX_CUDA(cudaEventRecord(s->events[ev], cs));
    const cudaEvent_t fork_ev = s->events[ev++];
    for (int64_t i = 0; i < n; ++i) {
      stx_layer* l = s->layers[g0 + i];
      cudaStream_t side = sides[g0 + i];
      STX_CUDA(cudaStreamWaitEvent(side, fork_ev, 0));
      if (stages & STX_STAGE_PLAN) {
        rc = cache_plan(l->cache, l->bits, side, l->lazy);
        if (rc != STX_OK) return rc;
      }
      if ((stages & STX_STAGE_COPY) && !l->lazy) {
        rc = cache_copy_rows(l->cache, side);
        if (rc != STX_OK) return rc;
      }
    }
  }
  for (int64_t i = 0; i < L; ++i) {  // join the branches of the groups that forked
    if (!forked[i / gsz]) continue;
    STX_CUDA(cudaEventRecord(s->events[ev], sides[i]));
    STX_CUDA(cudaStreamWaitEvent(cs, s->events[ev++], 0));
  }
  return STX_OK;
}

int stx_stack_create(stx_stack_t** out, stx_layer_t* const* layers, int64_t L, int64_t B) {
  return stx_stack_create_stages(out, layers, L, B, STX_STAGE_ALL);
}

int stx_stack_create_stages(stx_stack_t** out, stx_layer_t* const* layers, int64_t L, int64_t B, unsigned stages) {
  STX_CHECK_ARG(out, "stx_stack_create: out is null");
  *out = nullptr;
  STX_CHECK_ARG(layers && L > 0 && B > 0, "stx_stack_create: bad argument");
  for (int64_t i = 0; i < L; ++i) {
    STX_CHECK_ARG(layers[i], "stx_stack_create: layer %lld is null", static_cast<long long>(i));
    STX_CHECK_ARG(layers[i]->cache->H == layers[0]->cache->H && layers[i]->cache->dtype == layers[0]->cache->dtype,
                  "stx_stack_create: all layers must share H and dtype");
    STX_CHECK_ARG(B <= layers[i]->max_batch, "stx_stack_create: B exceeds layer %lld max_batch", static_cast<long long>(i));
  }
  stx_stack* s = new (std::nothrow) stx_stack();
  if (!s) {
    set_error("stx_stack_create: out of host memory");
    return STX_ERR_ALLOC;
  }
  s->layers.assign(layers, layers + L);
  s->B = B;
  s->H = layers[0]->cache->H;
  s->es = dtype_size(layers[0]->cache->dtype);
  const size_t xbytes = static_cast<size_t>(B) * s->H * s->es;
  cudaError_t e = cudaMalloc(&s->x_in, xbytes);
  if (e == cudaSuccess) e = cudaMalloc(&s->out, xbytes * L);
  if (e == cudaSuccess) e = cudaMemset(s->x_in, 0, xbytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&s->status_ptrs), sizeof(int*) * L);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&s->status_dev), sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(s->status_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&s->status_host), sizeof(int));
  if (e == cudaSuccess) {
    *s->status_host = 0;
    std::vector<int*> hp(L);
    for (int64_t i = 0; i < L; ++i) hp[i] = layers[i]->cache->state + ST_STATUS;
    e = cudaMemcpy(s->status_ptrs, hp.data(), sizeof(int*) * L, cudaMemcpyHostToDevice);
  }
  if (e != cudaSuccess) {
    set_error("stx_stack_create: device allocation failed: %s", cudaGetErrorString(e));
    stx_stack_destroy(s);
    return STX_ERR_ALLOC;
  }
  // Capture the L steps (nothing executes during capture).  The critical path (predictor ->
  // sparse MLP, layer after layer) stays on one stream; each layer's cache maintenance forks
  // off after its predictor onto a side stream and everything joins at the end of the step.
  // The maintenance itself uses two side streams: index plans on one, row copies on the other.
  cudaStream_t cs = nullptr, side = nullptr, side2 = nullptr;
  e = cudaStreamCreateWithFlags(&cs, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&side2, cudaStreamNonBlocking);
  for (int64_t i = 0; i < 2 * L + 2 && e == cudaSuccess; ++i) {
    cudaEvent_t ev = nullptr;
    e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e == cudaSuccess) s->events.push_back(ev);
  }
  if (e != cudaSuccess) {
    if (cs) cudaStreamDestroy(cs);
    if (side) cudaStreamDestroy(side);
    if (side2) cudaStreamDestroy(side2);
    stx_stack_destroy(s);
    return cuda_fail(e, "stx_stack_create: stream/event creation");
  }
  int rc = STX_OK;
  s->persistent = stack_persistent_wanted(s, stages);
  std::vector<cudaStream_t> sides;
  if (s->persistent) {
    const int64_t gsz = stack_group_size(L);
    for (int64_t g0 = 0; g0 < L && e == cudaSuccess; g0 += gsz) {
      const size_t bytes = stack_b1_scratch_bytes(std::min<int64_t>(gsz, L - g0), s->H, s->layers[0]->r);
      void* p = nullptr;
      e = cudaMalloc(&p, bytes);
      if (e == cudaSuccess) {
        s->b1_scratch.push_back(p);
        e = cudaMemset(p, 0, bytes);
      }
    }
    for (int64_t i = 0; i < L && e == cudaSuccess; ++i) {
      cudaStream_t st = nullptr;
      e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
      if (e == cudaSuccess) sides.push_back(st);
    }
    for (int64_t i = 0; i < L && e == cudaSuccess && rc == STX_OK; ++i) rc = cache_ensure_cat(s->layers[i]->cache, nullptr);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&s->upkeep_args), sizeof(UpkeepArgs) * L);
    if (e == cudaSuccess) {
      std::vector<UpkeepArgs> hu(L);
      for (int64_t i = 0; i < L; ++i) {
        const stx_cache* c = s->layers[i]->cache;
        UpkeepArgs& u = hu[i];
        u = UpkeepArgs{};
        u.cur_bits = c->cur_bits, u.active = c->active, u.pos_of = c->pos_of, u.lists = c->lists, u.jobs = c->jobs;
        u.state = c->state, u.stale = c->stale, u.lazy = s->layers[i]->lazy ? 1 : 0;
        if (c->has_gate) {
          u.pool[0] = c->pool_gate, u.pool[1] = c->pool_up, u.pool[2] = c->pool_down;
          u.pk[0] = c->pk_gate, u.pk[1] = c->pk_up, u.pk[2] = c->pk_down;
        } else {
          u.pool[0] = c->pool_up, u.pool[1] = c->pool_down;
          u.pk[0] = c->pk_up, u.pk[1] = c->pk_down;
        }
      }
      e = cudaMemcpy(s->upkeep_args, hu.data(), sizeof(UpkeepArgs) * L, cudaMemcpyHostToDevice);
    }
    if (e == cudaSuccess) e = cudaDeviceSynchronize();  // cleared counters and per-neuron pools are in place before the first launch
    if (e == cudaSuccess && rc == STX_OK) e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeRelaxed);
    if (e == cudaSuccess && rc == STX_OK) {
      rc = capture_persistent(s, stages, cs, sides);
      if (rc == STX_OK) rc = capture_status(s, cs);
      cudaError_t e2 = cudaStreamEndCapture(cs, &s->graph);
      if (rc == STX_OK && e2 != cudaSuccess) e = e2;
    }
    for (cudaStream_t st : sides) cudaStreamDestroy(st);
  } else {
  e = cudaStreamBeginCapture(cs, cudaStreamCaptureModeRelaxed);
  if (e == cudaSuccess) {
    bool forked = false, used2 = false;
    for (int64_t i = 0; i < L && rc == STX_OK; ++i) {
      stx_layer* l = s->layers[i];
      rc = layer_step_streams(l, s->x_in, s->x_in, B, static_cast<char*>(s->out) + i * xbytes, cs, side, s->events[i], stages,
                              side2, s->events[L + 1 + i], &used2);
      const bool big = l->cache->pk_gate && !single_row_fusable(l, B) &&
                       prefill_wanted(B, l->cache->H, l->cache->I, l->cache->dtype, l->cache->has_gate);
      forked = forked || (l->gather && !big && (stages & (STX_STAGE_PLAN | STX_STAGE_COPY)));
    }
    if (rc == STX_OK && forked) {  // join
      cudaError_t ej = cudaEventRecord(s->events[L], side);
      if (ej == cudaSuccess) ej = cudaStreamWaitEvent(cs, s->events[L], 0);
      if (ej == cudaSuccess && used2) {
        ej = cudaEventRecord(s->events[2 * L + 1], side2);
        if (ej == cudaSuccess) ej = cudaStreamWaitEvent(cs, s->events[2 * L + 1], 0);
      }
      if (ej != cudaSuccess) e = ej;
    }
    if (rc == STX_OK && e == cudaSuccess) rc = capture_status(s, cs);
    cudaError_t e2 = cudaStreamEndCapture(cs, &s->graph);
    if (rc == STX_OK && e == cudaSuccess && e2 != cudaSuccess) e = e2;
  }
  }
  if (e == cudaSuccess && rc == STX_OK) e = cudaGraphInstantiate(&s->exec, s->graph, 0);
  cudaStreamDestroy(cs);
  cudaStreamDestroy(side);
  cudaStreamDestroy(side2);
  if (rc != STX_OK) {
    stx_stack_destroy(s);
    return rc;
  }
  if (e != cudaSuccess) {
    stx_stack_destroy(s);
    return cuda_fail(e, "stx_stack_create: graph capture/instantiate");
  }
  size_t n = 0;
  if (cudaGraphGetNodes(s->graph, nullptr, &n) == cudaSuccess && n > 0) {
    std::vector<cudaGraphNode_t> nodes(n);
    if (cudaGraphGetNodes(s->graph, nodes.data(), &n) == cudaSuccess) {
      for (size_t i = 0; i < n; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++s->kernel_nodes;
      }
    }
  }
  *out = s;
  return STX_OK;
}

int stx_stack_buffers(stx_stack_t* s, void** x_in_out, void** out_out) {
  STX_CHECK_ARG(s, "stx_stack_buffers: null stack");
  if (x_in_out) *x_in_out = s->x_in;
  if (out_out) *out_out = s->out;
  return STX_OK;
}

// A step whose kernels gave up on a bounded wait (or skipped an access after a failed bounds check) has
// produced garbage.  The graph's last node leaves the error bits in pinned memory; the next call sees them
// without synchronising and refuses to go on.
static int stack_check_status(const stx_stack* s) {
  const int st = *reinterpret_cast<volatile int*>(s->status_host);
  if (st & DEV_TIMEOUT) {
    set_error("stx_stack_step: a bounded wait expired in an earlier step of this stack (device status 0x%x); its outputs are invalid", st);
    return STX_ERR_TIMEOUT;
  }
  if (st & DEV_BAD_INDEX) {
    set_error("stx_stack_step: a device bounds check failed in an earlier step of this stack (device status 0x%x)", st);
    return STX_ERR_INVALID_ARG;
  }
  return STX_OK;
}

int stx_stack_step(stx_stack_t* s, const void* x, void* out, void* stream) {
  STX_CHECK_ARG(s, "stx_stack_step: null stack");
  if (int rc = stack_check_status(s)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xbytes = static_cast<size_t>(s->B) * s->H * s->es;
  if (x && x != s->x_in) STX_CUDA(cudaMemcpyAsync(s->x_in, x, xbytes, cudaMemcpyDeviceToDevice, st));
  STX_CUDA(cudaGraphLaunch(s->exec, st));
  if (out && out != s->out)
    STX_CUDA(cudaMemcpyAsync(out, s->out, xbytes * s->layers.size(), cudaMemcpyDeviceToDevice, st));
  return STX_OK;
}

int stx_stack_step_host(stx_stack_t* s, const void* x_host, void* out_host, void* stream) {
  STX_CHECK_ARG(s && x_host && out_host, "stx_stack_step_host: null pointer");
  if (int rc = stack_check_status(s)) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t xbytes = static_cast<size_t>(s->B) * s->H * s->es;
  STX_CUDA(cudaMemcpyAsync(s->x_in, x_host, xbytes, cudaMemcpyHostToDevice, st));
  STX_CUDA(cudaGraphLaunch(s->exec, st));
  STX_CUDA(cudaMemcpyAsync(out_host, s->out, xbytes * s->layers.size(), cudaMemcpyDeviceToHost, st));
  STX_CUDA(cudaStreamSynchronize(st));
  return STX_OK;
}

int stx_stack_launches_per_step(stx_stack_t* s, int64_t* n_out) {
  STX_CHECK_ARG(s && n_out, "stx_stack_launches_per_step: null pointer");
  *n_out = s->kernel_nodes;
  return STX_OK;
}

}  // extern "C"
