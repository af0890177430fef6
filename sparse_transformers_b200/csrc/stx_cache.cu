// Device-resident differential weight cache.
//
// Behavioural contract (what a caller of the reference's WeightCache observes,
// sparse_transformers/csrc/weight_cache.h:229-359): after update(mask) the packed row j of
// gate/up/down belongs to neuron active[j], where `active` evolves from the previous order
// by (1) pairing the i-th removed neuron with the i-th added neuron (both ascending) and
// overwriting the removed neuron's slot, (2) appending surplus additions in ascending
// order, (3) deleting surplus removals in ascending order, each by moving the current last
// row into the hole.  Here the *index plan* (active / pos_of / list of rewritten slots) is
// computed by one thread block, and the data movement is a separate, fully parallel pass
// that rewrites every changed slot j from the full pool row of neuron active[j].  Because
// a packed row is by definition pool[active[j]], no packed->packed move is ever needed.
#include "stx_cache.cuh"
#include "stx_cache_plan.cuh"

#include <algorithm>
#include <new>

namespace stx {

__global__ void __launch_bounds__(PLAN_THREADS, 1)
k_cache_plan(const uint32_t* __restrict__ new_bits, uint32_t* __restrict__ cur_bits,
             int32_t* __restrict__ active, int32_t* __restrict__ pos_of, int32_t* __restrict__ lists,
             int32_t* __restrict__ jobs, int32_t* __restrict__ state, uint32_t* __restrict__ stale, int lazy, int I) {
  extern __shared__ int32_t sm[];
  plan_block(new_bits, cur_bits, active, pos_of, lists, jobs, state, stale, lazy, I, sm);
}

// One warp per (job, matrix): packed[m][pos] = pool[m][active[pos]], 16-byte vectors.
__global__ void __launch_bounds__(128)
k_cache_copy_rows(const int32_t* __restrict__ jobs, const int32_t* __restrict__ active,
                  const int32_t* __restrict__ state, const void* pool0, const void* pool1,
                  const void* pool2, void* pk0, void* pk1, void* pk2, int nmat, int vec_per_row, int I) {
  const int njobs = state[ST_NJOBS];
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int units = njobs * nmat;
  for (int u = warp; u < units; u += nwarps) {
    const int job = u / nmat, m = u - job * nmat;
    const int pos = jobs[job];
    if (pos < 0 || pos >= I) continue;
    const int src = active[pos];
    if (src < 0 || src >= I) continue;
    const uint4* sp = reinterpret_cast<const uint4*>(m == 0 ? pool0 : (m == 1 ? pool1 : pool2)) +
                      static_cast<size_t>(src) * vec_per_row;
    uint4* dp = reinterpret_cast<uint4*>(m == 0 ? pk0 : (m == 1 ? pk1 : pk2)) +
                static_cast<size_t>(pos) * vec_per_row;
    int c = lane;
    for (; c + 96 < vec_per_row; c += 128) {
      uint4 v0 = ld_stream16(sp + c), v1 = ld_stream16(sp + c + 32), v2 = ld_stream16(sp + c + 64),
            v3 = ld_stream16(sp + c + 96);
      st16(dp + c, v0);
      st16(dp + c + 32, v1);
      st16(dp + c + 64, v2);
      st16(dp + c + 96, v3);
    }
    for (; c < vec_per_row; c += 32) st16(dp + c, ld_stream16(sp + c));
  }
}

// [R,C] -> [C,R] for 2- or 4-byte elements (32x32 tiles through shared memory).
template <typename E>
__global__ void __launch_bounds__(256) k_transpose(const E* __restrict__ in, E* __restrict__ out, int R, int C) {
  __shared__ E tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int k = ty; k < 32; k += 8) {
    const int r = r0 + k, c = c0 + tx;
    if (r < R && c < C) tile[k][tx] = in[static_cast<size_t>(r) * C + c];
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, r = r0 + tx;
    if (r < R && c < C) out[static_cast<size_t>(c) * R + r] = tile[tx][k];
  }
}

__global__ void k_bytes_to_bits(const uint8_t* __restrict__ bytes, uint32_t* __restrict__ bits, int I) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool on = (i < I) && bytes[i] != 0;
  const uint32_t w = __ballot_sync(0xffffffffu, on);
  if ((threadIdx.x & 31) == 0 && i < I) bits[i >> 5] = w;
}

__global__ void k_bits_to_bytes(const uint32_t* __restrict__ bits, uint8_t* __restrict__ bytes, int I) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < I) bytes[i] = (bits[i >> 5] >> (i & 31)) & 1u;
}

// concat[0:K] = packed gate[0:K]; concat[K:2K] = packed up[0:K]  (K read on the device)
__global__ void __launch_bounds__(256)
k_concat(const uint4* __restrict__ pg, const uint4* __restrict__ pu, uint4* __restrict__ out,
         const int32_t* __restrict__ state, int vec_per_row, int has_gate) {
  const size_t n = static_cast<size_t>(state[ST_K]) * vec_per_row;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (has_gate) {
      out[i] = ld_stream16(pg + i);
      out[n + i] = ld_stream16(pu + i);
    } else {
      out[i] = ld_stream16(pu + i);
    }
  }
}

__global__ void k_fill_i32(int32_t* p, int32_t v, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}

static size_t plan_smem_bytes(int64_t I) { return plan_smem_words(I) * sizeof(int32_t); }

int cache_plan(stx_cache* c, const uint32_t* bits, cudaStream_t s, bool lazy) {
  static bool attr_set[64] = {};
  int dev = 0;
  STX_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_cache_plan, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(plan_smem_bytes(MAX_I))));
    attr_set[dev] = true;
  }
  // two mask words per thread at most; small index spaces use fewer threads (cheaper barriers)
  const int W = static_cast<int>((c->I + 31) / 32);
  const int threads = W <= 256 ? 256 : (W <= 512 ? 512 : PLAN_THREADS);
  k_cache_plan<<<1, threads, plan_smem_bytes(c->I), s>>>(bits, c->cur_bits, c->active, c->pos_of, c->lists, c->jobs,
                                                        c->state, c->stale, lazy ? 1 : 0, static_cast<int>(c->I));
  STX_LAUNCH_CHECK("k_cache_plan");
  if (lazy) c->lazy_used = true;
  return STX_OK;
}

// Turns the stale bitmap into the job list (slots below K, ascending) and clears it.
__global__ void __launch_bounds__(1024, 1)
k_stale_to_jobs(uint32_t* __restrict__ stale, int32_t* __restrict__ jobs, int32_t* __restrict__ state, int I) {
  __shared__ Int2 s_ws[32];
  __shared__ Int2 s_tot;
  const int W = (I + 31) >> 5;
  const int t = threadIdx.x;
  const int WPT = (W + blockDim.x - 1) / blockDim.x;
  const int K = state[ST_K];
  uint32_t dw[2] = {0, 0};
  Int2 jc{0, 0};
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    if (w < W) {
      uint32_t d = stale[w];
      stale[w] = 0u;
      const int lo = w * 32;
      if (lo >= K) d = 0u;
      else if (K - lo < 32) d &= (1u << (K - lo)) - 1u;
      dw[k] = d;
      jc.x += __popc(d);
    }
  }
  Int2 joff = block_excl_scan2(jc, &s_tot, s_ws);
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    uint32_t d = dw[k];
    while (d) {
      jobs[joff.x++] = w * 32 + __ffs(d) - 1;
      d &= d - 1;
    }
  }
  if (t == 0) state[ST_NJOBS] = s_tot.x;
}

// Brings the packed rows up to date after lazy plans.  A cache that has ever been planned
// lazily (possibly inside a captured graph that is replayed later) is flushed on every call.
int cache_flush(stx_cache* c, cudaStream_t s) {
  if (!c->lazy_used) return STX_OK;
  k_stale_to_jobs<<<1, 1024, 0, s>>>(c->stale, c->jobs, c->state, static_cast<int>(c->I));
  STX_LAUNCH_CHECK("k_stale_to_jobs");
  return cache_copy_rows(c, s);
}

int cache_copy_rows(stx_cache* c, cudaStream_t s) {
  const int nmat = c->has_gate ? 3 : 2;
  const int vec = static_cast<int>(c->row_bytes / 16);
  // small blocks with few registers: they fit next to the MLP kernels' CTAs when the cache is
  // maintained on a side stream
  const int grid = num_sms() * 4;
  if (c->has_gate) {
    k_cache_copy_rows<<<grid, 128, 0, s>>>(c->jobs, c->active, c->state, c->pool_gate, c->pool_up,
                                          c->pool_down, c->pk_gate, c->pk_up, c->pk_down, nmat, vec,
                                          static_cast<int>(c->I));
  } else {
    k_cache_copy_rows<<<grid, 128, 0, s>>>(c->jobs, c->active, c->state, c->pool_up, c->pool_down, nullptr,
                                          c->pk_up, c->pk_down, nullptr, nmat, vec, static_cast<int>(c->I));
  }
  STX_LAUNCH_CHECK("k_cache_copy_rows");
  return STX_OK;
}

int cache_update_bits(stx_cache* c, const uint32_t* bits, cudaStream_t s) {
  int rc = cache_flush(c, s);  // rows left stale by earlier lazy plans come first
  if (rc != STX_OK) return rc;
  rc = cache_plan(c, bits, s, false);
  if (rc != STX_OK) return rc;
  return cache_copy_rows(c, s);
}

// cat[n] = [gate[n] | up[n] | down[n]] (nmat rows of vec 16-byte vectors each)
__global__ void __launch_bounds__(256)
k_interleave_rows(const uint4* __restrict__ p0, const uint4* __restrict__ p1, const uint4* __restrict__ p2,
                  uint4* __restrict__ cat, int nmat, int vec, size_t total) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t rec = static_cast<size_t>(nmat) * vec;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t n = i / rec, o = i - n * rec;
    const int m = static_cast<int>(o / vec);
    const size_t v = o - static_cast<size_t>(m) * vec;
    const uint4* src = m == 0 ? p0 : (m == 1 ? p1 : p2);
    cat[i] = ld_stream16(src + n * vec + v);
  }
}

int cache_ensure_cat(stx_cache* c, cudaStream_t s) {
  if (c->pool_cat) return STX_OK;
  const int nmat = c->has_gate ? 3 : 2;
  const size_t bytes = static_cast<size_t>(c->I) * nmat * c->row_bytes;
  cudaError_t e = cudaMalloc(&c->pool_cat, bytes);
  if (e != cudaSuccess) {
    c->pool_cat = nullptr;
    set_error("weight cache: allocating the per-neuron pool (%zu bytes) failed: %s", bytes, cudaGetErrorString(e));
    return STX_ERR_ALLOC;
  }
  const int vec = static_cast<int>(c->row_bytes / 16);
  const size_t total = static_cast<size_t>(c->I) * nmat * vec;
  const uint4* p0 = static_cast<const uint4*>(c->has_gate ? c->pool_gate : c->pool_up);
  const uint4* p1 = static_cast<const uint4*>(c->has_gate ? c->pool_up : c->pool_down);
  const uint4* p2 = static_cast<const uint4*>(c->has_gate ? c->pool_down : nullptr);
  k_interleave_rows<<<num_sms() * 8, 256, 0, s>>>(p0, p1, p2, static_cast<uint4*>(c->pool_cat), nmat, vec, total);
  STX_LAUNCH_CHECK("k_interleave_rows");
  return STX_OK;
}

int cache_read_state(stx_cache* c, cudaStream_t s) {
  STX_CUDA(cudaMemcpyAsync(c->host_state, c->state, ST_COUNT * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
  STX_CUDA(cudaStreamSynchronize(s));
  return STX_OK;
}

}  // namespace stx

using namespace stx;

extern "C" {

int stx_cache_bytes(int64_t I, int64_t H, int dtype, int has_gate, unsigned flags, size_t* bytes_out) {
  STX_CHECK_ARG(bytes_out, "stx_cache_bytes: bytes_out is null");
  STX_CHECK_ARG(I > 0 && H > 0, "stx_cache_bytes: I and H must be positive");
  const size_t mat = static_cast<size_t>(I) * H * dtype_size(dtype);
  const int nmat = has_gate ? 3 : 2;
  size_t total = mat /*pool_down*/ + nmat * mat /*packed*/;
  if (!(flags & STX_CACHE_ALIAS_GATE_UP)) total += (nmat - 1) * mat;
  total += static_cast<size_t>(I) * 5 * sizeof(int32_t) + 2 * ((I + 31) / 32) * sizeof(uint32_t) +
           ST_COUNT * sizeof(int32_t);
  *bytes_out = total;
  return STX_OK;
}

int stx_cache_destroy(stx_cache_t* c) {
  if (!c) return STX_OK;
  cudaFree(c->own_gate);
  cudaFree(c->own_up);
  cudaFree(c->pool_cat);
  cudaFree(c->pool_down);
  if (c->pk_gate)
    cudaFree(c->pk_gate);  // pk_up lives in the same allocation
  else
    cudaFree(c->pk_up);
  cudaFree(c->pk_down);
  cudaFree(c->concat);
  cudaFree(c->active);
  cudaFree(c->pos_of);
  cudaFree(c->lists);
  cudaFree(c->jobs);
  cudaFree(c->cur_bits);
  cudaFree(c->tmp_bits);
  cudaFree(c->stale);
  cudaFree(c->state);
  if (c->host_state) cudaFreeHost(c->host_state);
  delete c;
  return STX_OK;
}

#define STX_ALLOC(ptr, bytes)                                                                   \
  do {                                                                                          \
    cudaError_t e__ = cudaMalloc(reinterpret_cast<void**>(&(ptr)), (bytes));                    \
    if (e__ != cudaSuccess) {                                                                   \
      set_error("stx_cache_create: cudaMalloc(%zu bytes) failed: %s", static_cast<size_t>(bytes), \
                cudaGetErrorString(e__));                                                       \
      stx_cache_destroy(c);                                                                     \
      return STX_ERR_ALLOC;                                                                     \
    }                                                                                           \
  } while (0)

int stx_cache_create(stx_cache_t** out, int64_t I, int64_t H, int dtype, int has_gate, const void* gate_w,
                     const void* up_w, const void* down_w, const uint8_t* init_mask_bytes, unsigned flags,
                     void* stream) {
  STX_CHECK_ARG(out, "stx_cache_create: out is null");
  *out = nullptr;
  STX_CHECK_ARG(I > 0 && H > 0, "stx_cache_create: I and H must be positive");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_cache_create: bad dtype %d", dtype);
  STX_CHECK_ARG(up_w && down_w, "stx_cache_create: up_w/down_w is null");
  STX_CHECK_ARG(!has_gate || gate_w, "stx_cache_create: has_gate set but gate_w is null");
  if (I > MAX_I) {
    set_error("stx_cache_create: I=%lld exceeds the supported maximum %d", static_cast<long long>(I), MAX_I);
    return STX_ERR_TOO_LARGE;
  }
  const size_t es = dtype_size(dtype);
  if ((H * es) % 16 != 0) {
    set_error("stx_cache_create: row size H*elem (%lld bytes) must be a multiple of 16", static_cast<long long>(H * es));
    return STX_ERR_UNSUPPORTED;
  }
  const bool alias = (flags & STX_CACHE_ALIAS_GATE_UP) != 0;
  if (alias && ((reinterpret_cast<uintptr_t>(up_w) & 15) || (has_gate && (reinterpret_cast<uintptr_t>(gate_w) & 15)))) {
    set_error("stx_cache_create: aliased gate/up buffers must be 16-byte aligned");
    return STX_ERR_INVALID_ARG;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  stx_cache* c = new (std::nothrow) stx_cache();
  if (!c) {
    set_error("stx_cache_create: out of host memory");
    return STX_ERR_ALLOC;
  }
  c->I = I;
  c->H = H;
  c->dtype = dtype;
  c->has_gate = has_gate ? 1 : 0;
  c->flags = flags;
  c->row_bytes = static_cast<size_t>(H) * es;
  cudaGetDevice(&c->device);
  const size_t mat = static_cast<size_t>(I) * c->row_bytes;
  const size_t W = static_cast<size_t>((I + 31) / 32);

  STX_ALLOC(c->pool_down, mat);
  // packed gate and up rows share one allocation, gate first: [pk_gate ; pk_up] is the concat
  // weight of a cache whose I slots are all in use, which the tensor-core path reads directly
  if (has_gate) {
    STX_ALLOC(c->pk_gate, 2 * mat);
    c->pk_up = static_cast<char*>(c->pk_gate) + mat;
  } else {
    STX_ALLOC(c->pk_up, mat);
  }
  STX_ALLOC(c->pk_down, mat);
  if (!alias) {
    STX_ALLOC(c->own_up, mat);
    if (has_gate) STX_ALLOC(c->own_gate, mat);
  }
  STX_ALLOC(c->active, I * sizeof(int32_t));
  STX_ALLOC(c->pos_of, I * sizeof(int32_t));
  STX_ALLOC(c->lists, 2 * I * sizeof(int32_t));
  STX_ALLOC(c->jobs, I * sizeof(int32_t));
  STX_ALLOC(c->cur_bits, W * sizeof(uint32_t));
  STX_ALLOC(c->tmp_bits, W * sizeof(uint32_t));
  STX_ALLOC(c->stale, W * sizeof(uint32_t));
  STX_ALLOC(c->state, ST_COUNT * sizeof(int32_t));
  if (cudaMallocHost(reinterpret_cast<void**>(&c->host_state), ST_COUNT * sizeof(int32_t)) != cudaSuccess) {
    set_error("stx_cache_create: cudaMallocHost failed");
    stx_cache_destroy(c);
    return STX_ERR_ALLOC;
  }

  // pools (weight_cache.h:199-220): gate/up verbatim, down transposed [H,I] -> [I,H]
  cudaError_t e = cudaSuccess;
  if (alias) {
    c->pool_up = up_w;
    c->pool_gate = has_gate ? gate_w : nullptr;
  } else {
    e = cudaMemcpyAsync(c->own_up, up_w, mat, cudaMemcpyDeviceToDevice, s);
    if (e == cudaSuccess && has_gate) e = cudaMemcpyAsync(c->own_gate, gate_w, mat, cudaMemcpyDeviceToDevice, s);
    c->pool_up = c->own_up;
    c->pool_gate = c->own_gate;
  }
  if (e == cudaSuccess) {
    dim3 grid(static_cast<unsigned>((I + 31) / 32), static_cast<unsigned>((H + 31) / 32));
    if (es == 4)
      k_transpose<uint32_t><<<grid, 256, 0, s>>>(static_cast<const uint32_t*>(down_w),
                                                static_cast<uint32_t*>(c->pool_down), static_cast<int>(H),
                                                static_cast<int>(I));
    else
      k_transpose<uint16_t><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(down_w),
                                                static_cast<uint16_t*>(c->pool_down), static_cast<int>(H),
                                                static_cast<int>(I));
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemsetAsync(c->cur_bits, 0, W * sizeof(uint32_t), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(c->stale, 0, W * sizeof(uint32_t), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(c->state, 0, ST_COUNT * sizeof(int32_t), s);
  if (e == cudaSuccess) e = cudaMemsetAsync(c->pos_of, 0xff, I * sizeof(int32_t), s);  // -1
  if (e == cudaSuccess) e = cudaMemsetAsync(c->active, 0xff, I * sizeof(int32_t), s);
  if (e != cudaSuccess) {
    int rc = cuda_fail(e, "stx_cache_create: initialisation");
    stx_cache_destroy(c);
    return rc;
  }
  if (init_mask_bytes) {
    int rc = stx_cache_update(c, init_mask_bytes, stream);
    if (rc != STX_OK) {
      stx_cache_destroy(c);
      return rc;
    }
  }
  *out = c;
  return STX_OK;
}

int stx_mask_bytes_to_bits(const uint8_t* bytes, int64_t I, uint32_t* bits_out, void* stream) {
  STX_CHECK_ARG(bytes && bits_out && I > 0, "stx_mask_bytes_to_bits: bad argument");
  const int threads = 256;
  const int blocks = static_cast<int>((I + threads - 1) / threads);
  k_bytes_to_bits<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(bytes, bits_out, static_cast<int>(I));
  STX_LAUNCH_CHECK("k_bytes_to_bits");
  return STX_OK;
}

int stx_mask_bits_to_bytes(const uint32_t* bits, int64_t I, uint8_t* bytes_out, void* stream) {
  STX_CHECK_ARG(bits && bytes_out && I > 0, "stx_mask_bits_to_bytes: bad argument");
  const int threads = 256;
  const int blocks = static_cast<int>((I + threads - 1) / threads);
  k_bits_to_bytes<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(bits, bytes_out, static_cast<int>(I));
  STX_LAUNCH_CHECK("k_bits_to_bytes");
  return STX_OK;
}

int stx_cache_update(stx_cache_t* c, const uint8_t* mask_bytes, void* stream) {
  STX_CHECK_ARG(c && mask_bytes, "stx_cache_update: null argument");
  int rc = stx_mask_bytes_to_bits(mask_bytes, c->I, c->tmp_bits, stream);
  if (rc != STX_OK) return rc;
  return cache_update_bits(c, c->tmp_bits, static_cast<cudaStream_t>(stream));
}

int stx_cache_update_bits(stx_cache_t* c, const uint32_t* mask_bits, void* stream) {
  STX_CHECK_ARG(c && mask_bits, "stx_cache_update_bits: null argument");
  return cache_update_bits(c, mask_bits, static_cast<cudaStream_t>(stream));
}

static int state_to_status(const stx_cache* c) {
  const int32_t* h = c->host_state;
  if (h[ST_STATUS] & DEV_BAD_INDEX) {
    set_error("weight cache: a device bounds check failed (status 0x%x)", h[ST_STATUS]);
    return STX_ERR_INVALID_ARG;
  }
  if (h[ST_K] == 0 && (h[ST_STATUS] & DEV_NO_ACTIVE)) {
    set_error("No active weights");
    return STX_ERR_NO_ACTIVE;
  }
  if (!h[ST_VALID]) {
    set_error("Cache is not valid");
    return STX_ERR_CACHE_INVALID;
  }
  return STX_OK;
}

int stx_cache_num_active(stx_cache_t* c, int64_t* k_out, void* stream) {
  STX_CHECK_ARG(c && k_out, "stx_cache_num_active: null argument");
  int rc = cache_read_state(c, static_cast<cudaStream_t>(stream));
  if (rc != STX_OK) return rc;
  *k_out = c->host_state[ST_K];
  return state_to_status(c);
}

int stx_cache_concat_weight(stx_cache_t* c, void** ptr_out, int64_t* rows_out, void* stream) {
  STX_CHECK_ARG(c && ptr_out && rows_out, "stx_cache_concat_weight: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = cache_flush(c, s);
  if (rc != STX_OK) return rc;
  rc = cache_read_state(c, s);
  if (rc != STX_OK) return rc;
  rc = state_to_status(c);
  if (rc != STX_OK) return rc;
  const int64_t K = c->host_state[ST_K];
  if (!c->concat) {
    const size_t bytes = static_cast<size_t>(c->has_gate ? 2 : 1) * c->I * c->row_bytes;
    cudaError_t e = cudaMalloc(&c->concat, bytes);
    if (e != cudaSuccess) {
      c->concat = nullptr;
      set_error("stx_cache_concat_weight: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
      return STX_ERR_ALLOC;
    }
    c->concat_epoch = -1;
  }
  if (c->concat_epoch != c->host_state[ST_EPOCH]) {
    const int vec = static_cast<int>(c->row_bytes / 16);
    k_concat<<<num_sms() * 4, 256, 0, s>>>(static_cast<const uint4*>(c->pk_gate), static_cast<const uint4*>(c->pk_up),
                                          static_cast<uint4*>(c->concat), c->state, vec, c->has_gate);
    STX_LAUNCH_CHECK("k_concat");
    c->concat_epoch = c->host_state[ST_EPOCH];
  }
  *ptr_out = c->concat;
  *rows_out = c->has_gate ? 2 * K : K;
  return STX_OK;
}

int stx_cache_active_down(stx_cache_t* c, void** ptr_out, int64_t* k_out, void* stream) {
  STX_CHECK_ARG(c && ptr_out && k_out, "stx_cache_active_down: null argument");
  int rc = cache_flush(c, static_cast<cudaStream_t>(stream));
  if (rc != STX_OK) return rc;
  rc = cache_read_state(c, static_cast<cudaStream_t>(stream));
  if (rc != STX_OK) return rc;
  rc = state_to_status(c);
  if (rc != STX_OK) return rc;
  *ptr_out = c->pk_down;
  *k_out = c->host_state[ST_K];
  return STX_OK;
}

int stx_cache_flush(stx_cache_t* c, void* stream) {
  STX_CHECK_ARG(c, "stx_cache_flush: null cache");
  return cache_flush(c, static_cast<cudaStream_t>(stream));
}

int stx_cache_packed_ptrs(stx_cache_t* c, void** gate_out, void** up_out, void** down_out,
                          const int32_t** k_dev_out) {
  STX_CHECK_ARG(c, "stx_cache_packed_ptrs: null cache");
  if (gate_out) *gate_out = c->pk_gate;
  if (up_out) *up_out = c->pk_up;
  if (down_out) *down_out = c->pk_down;
  if (k_dev_out) *k_dev_out = c->state + ST_K;
  return STX_OK;
}

int stx_cache_active_indices(stx_cache_t* c, int32_t* host_out, int64_t cap, int64_t* k_out, void* stream) {
  STX_CHECK_ARG(c && k_out, "stx_cache_active_indices: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = cache_read_state(c, s);
  if (rc != STX_OK) return rc;
  const int64_t K = c->host_state[ST_K];
  *k_out = K;
  if (host_out && K > 0) {
    STX_CHECK_ARG(cap >= K, "stx_cache_active_indices: capacity %lld < K=%lld", static_cast<long long>(cap),
                  static_cast<long long>(K));
    STX_CUDA(cudaMemcpyAsync(host_out, c->active, K * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    STX_CUDA(cudaStreamSynchronize(s));
  }
  return STX_OK;
}

int stx_cache_last_update_stats(stx_cache_t* c, int64_t* added, int64_t* removed, int64_t* rows_copied, void* stream) {
  STX_CHECK_ARG(c, "stx_cache_last_update_stats: null cache");
  int rc = cache_read_state(c, static_cast<cudaStream_t>(stream));
  if (rc != STX_OK) return rc;
  if (added) *added = c->host_state[ST_ADDED];
  if (removed) *removed = c->host_state[ST_REMOVED];
  if (rows_copied) *rows_copied = c->host_state[ST_NJOBS];
  return STX_OK;
}

}  // extern "C"
