// Sparse gated MLP over packed active rows (decode-sized batches).
//
//   out[b,:] = sum_j act(x[b]·gate[j]) * (x[b]·up[j]) * down[j,:]        j = 0..K-1
//
// gate/up/down rows are the packed rows of the active neurons (one contiguous H-row per
// neuron in each matrix), so every byte that is read is useful and every read is a
// 16-byte coalesced vector.  Replaces sparse_mlp_forward_cpu (sparse_mlp_op.cpp:79-192),
// the unfinished CUDA kernels (sparse_mlp_cuda.cu:28-88) and the two matmuls the models
// actually run (src/modeling_skip.py:114-117).
//
// k_mlp_fused: persistent blocks, each owning a contiguous range of neurons.
//   phase A  one warp per neuron: both dot products with x (shared memory), warp-shuffle
//            reduction, activation and product in registers -> a[j,b] in shared memory
//   phase B  one thread per 16-byte column chunk: acc[b,chunk] += a[j,b] * down[j,chunk]
//            over the block's neurons -> the block's partial output [B,H] (fp32) in the scratch
//   the last block to finish adds the partial outputs in block order (deterministic, no atomics on
//   data) and converts to the output dtype.  The partial outputs live where the scratch has room for
//   them - the accumulator region and the a[K][B] region of the streaming kernels - and the launcher
//   takes no more blocks than fit there.
#include "stx_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

namespace stx {

struct MlpArgs {
  const void* x;
  const void* gate;
  const void* up;
  const void* down;
  void* combined;        // optional [B, 2K] (or [B,K]) in dtype
  void* out;             // [B,H] in dtype
  float* out_acc;        // [B,H] fp32: partial output of block 0 (zero on exit)
  float* part_rest;      // [gridDim.x - 1][B,H] fp32: partial outputs of the other blocks
  unsigned* counter;     // zero on entry, zero on exit
  const int32_t* K_dev;  // device K (may be null -> K_host)
  int K_host;
  int up_after_gate;     // 1: up rows start K rows after `gate` (concat layout, device K)
  int B, H, act, has_gate, a_cap;
};

template <typename T, int NB>
__global__ void __launch_bounds__(256, 2) k_mlp_fused(const MlpArgs p) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* x_s = reinterpret_cast<T*>(smem_raw);                                   // [NB][H]
  float* a_s = reinterpret_cast<float*>(smem_raw + sizeof(T) * NB * p.H);    // [a_cap][NB]
  __shared__ int s_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int H = p.H, nchunk = H / V;
  const int K = p.K_dev ? *p.K_dev : p.K_host;
  const T* gate = static_cast<const T*>(p.gate);
  const T* up = static_cast<const T*>(p.up);
  if (p.up_after_gate) up = gate + static_cast<size_t>(K) * H;
  const T* down = static_cast<const T*>(p.down);
  T* combined = static_cast<T*>(p.combined);
  const int ldc = p.has_gate ? 2 * K : K;

  // contiguous, balanced neuron range of this block
  const int base = K / gridDim.x, rem = K % gridDim.x;
  const int j0 = blockIdx.x * base + min(static_cast<int>(blockIdx.x), rem);
  int j1 = j0 + base + (static_cast<int>(blockIdx.x) < rem ? 1 : 0);
  if (j1 - j0 > p.a_cap) j1 = j0 + p.a_cap;  // cannot happen for K <= capacity; never index past a_s

  for (int b0 = 0; b0 < p.B; b0 += NB) {
    const int nb = min(NB, p.B - b0);
    if (j1 > j0) {
      // stage the x tile
      const uint4* xg = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + static_cast<size_t>(b0) * H);
      uint4* xs4 = reinterpret_cast<uint4*>(x_s);
      for (int i = tid; i < nb * nchunk; i += blockDim.x) xs4[i] = xg[i];
      for (int i = nb * nchunk + tid; i < NB * nchunk; i += blockDim.x) xs4[i] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();

    // ---- phase A
    for (int j = j0 + warp; j < j1; j += nwarps) {
      float ag[NB], au[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) ag[b] = au[b] = 0.f;
      const T* grow = gate + static_cast<size_t>(j) * H;
      const T* urow = up + static_cast<size_t>(j) * H;
      for (int c0 = lane; c0 < nchunk; c0 += 128) {
        uint4 gv[4], uv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + 32 * u;
          if (c < nchunk) {
            uv[u] = ld_stream16(urow + c * V);
            if (p.has_gate) gv[u] = ld_stream16(grow + c * V);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + 32 * u;
          if (c < nchunk) {
            float wu[V], wg[V];
            Unpack<T>::run(uv[u], wu);
            if (p.has_gate) Unpack<T>::run(gv[u], wg);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              float xv[V];
              Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + b * H + c * V), xv);
#pragma unroll
              for (int v = 0; v < V; ++v) {
                au[b] = fmaf(xv[v], wu[v], au[b]);
                if (p.has_gate) ag[b] = fmaf(xv[v], wg[v], ag[b]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float u = warp_sum_xor(au[b]);
        float a;
        if (p.has_gate) {
          const float g = warp_sum_xor(ag[b]);
          a = apply_act(p.act, g) * u;
        } else {
          a = apply_act(p.act, u);
        }
        if (lane == 0) {
          a_s[(j - j0) * NB + b] = a;
          if (combined && b < nb) {
            combined[static_cast<size_t>(b0 + b) * ldc + j] = DT<T>::from_f(a);
            if (p.has_gate) combined[static_cast<size_t>(b0 + b) * ldc + K + j] = DT<T>::from_f(u);
          }
        }
      }
    }
    __syncthreads();

    // ---- phase B
    if (j1 > j0) {
      for (int c = tid; c < nchunk; c += blockDim.x) {
        float acc[NB][V];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
          for (int v = 0; v < V; ++v) acc[b][v] = 0.f;
        const T* dcol = down + c * V;
        int j = j0;
        for (; j + 4 <= j1; j += 4) {
          uint4 dv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) dv[u] = ld_stream16(dcol + static_cast<size_t>(j + u) * H);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float wd[V];
            Unpack<T>::run(dv[u], wd);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
              const float a = a_s[(j + u - j0) * NB + b];
#pragma unroll
              for (int v = 0; v < V; ++v) acc[b][v] = fmaf(a, wd[v], acc[b][v]);
            }
          }
        }
        for (; j < j1; ++j) {
          float wd[V];
          Unpack<T>::run(ld_stream16(dcol + static_cast<size_t>(j) * H), wd);
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            const float a = a_s[(j - j0) * NB + b];
#pragma unroll
            for (int v = 0; v < V; ++v) acc[b][v] = fmaf(a, wd[v], acc[b][v]);
          }
        }
        float* mine = blockIdx.x == 0 ? p.out_acc : p.part_rest + static_cast<size_t>(blockIdx.x - 1) * p.B * H;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if (b < nb) {
            float* dst = mine + static_cast<size_t>(b0 + b) * H + c * V;
#pragma unroll
            for (int v = 0; v < V; v += 4) *reinterpret_cast<float4*>(dst + v) = make_float4(acc[b][v], acc[b][v + 1], acc[b][v + 2], acc[b][v + 3]);
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- the last block adds the partial outputs of the blocks that had neurons (the first min(gridDim.x, K)), in
  //      block order, and converts
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned ticket = atomicAdd(p.counter, 1u);
    s_last = (ticket == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    T* out = static_cast<T*>(p.out);
    const int n4 = p.B * H / 4;
    const int nact = min(static_cast<int>(gridDim.x), K);
    const float4* first = reinterpret_cast<const float4*>(p.out_acc);
    const float4* rest = reinterpret_cast<const float4*>(p.part_rest);
    for (int i = tid; i < n4; i += blockDim.x) {
      float4 v = nact > 0 ? __ldcg(first + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int blk = 1; blk < nact; ++blk) {
        const float4 u = __ldcg(rest + static_cast<size_t>(blk - 1) * n4 + i);
        v.x += u.x;
        v.y += u.y;
        v.z += u.z;
        v.w += u.w;
      }
      out[4 * i + 0] = DT<T>::from_f(v.x);
      out[4 * i + 1] = DT<T>::from_f(v.y);
      out[4 * i + 2] = DT<T>::from_f(v.z);
      out[4 * i + 3] = DT<T>::from_f(v.w);
      // the accumulator region is handed back zeroed, as callers of the scratch may expect of its head
      reinterpret_cast<float4*>(p.out_acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (tid == 0) *p.counter = 0u;
  }
}

template <typename T, int NB>
static int launch_fused(const MlpArgs& a, int grid, int threads, cudaStream_t s) {
  const size_t smem = sizeof(T) * NB * a.H + sizeof(float) * NB * a.a_cap;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_mlp_fused<T, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_set[dev] = true;
  }
  if (smem > 200 * 1024) {
    set_error("sparse MLP: shared-memory tile of %zu bytes exceeds 200 KiB (H too large)", smem);
    return STX_ERR_TOO_LARGE;
  }
  k_mlp_fused<T, NB><<<grid, threads, smem, s>>>(a);
  STX_LAUNCH_CHECK("k_mlp_fused");
  return STX_OK;
}

template <typename T>
static int dispatch_nb(MlpArgs& a, int grid, int threads, cudaStream_t s) {
  if (a.B == 1) return launch_fused<T, 1>(a, grid, threads, s);
  if (a.B == 2) return launch_fused<T, 2>(a, grid, threads, s);
  return launch_fused<T, 4>(a, grid, threads, s);
}

struct GatherSpec {
  const uint32_t* mask_bits;
  int32_t* idx;
  int32_t* count;
  int I;
};
int mlp_forward_tma(const void* x, int64_t B, int64_t H, const void* gate, const void* up, const void* down,
                    const int32_t* K_dev, int64_t K_host, const GatherSpec* gs, void* out, void* combined, int act,
                    int has_gate, int dtype, void* scratch, float* partial, int* status, unsigned parts,
                    cudaStream_t s);

size_t prefill_scratch_bytes(int64_t B, int64_t H, int64_t K);
bool prefill_wanted(int64_t B, int64_t H, int64_t K, int dtype, int has_gate);
int prefill_forward(const void* x, int64_t B, int64_t H, const void* concat, const void* down_packed, int64_t K,
                    void* out, void* combined, int act, int dtype, void* scratch, int* status, const int* k_dev,
                    cudaStream_t s);

constexpr int64_t PARTIAL_ROWS = 256;  // per-CTA partial output vectors of the batch-1 kernel (>= SM count)

// without the batch-1 partial vectors: what the built-in scratch of the no-alloc entry point holds
static size_t decode_scratch_bytes_min(int64_t B, int64_t H, int64_t K) {
  // [counter | fp32 accumulator B*H (kept zero) | 256 | fp32 a[K][B]]
  return 256 + align_up(static_cast<size_t>(B) * H * sizeof(float), 256) + 256 +
         align_up(static_cast<size_t>(B) * std::max<int64_t>(K, 1) * sizeof(float), 256);
}
static size_t decode_scratch_bytes(int64_t B, int64_t H, int64_t K) {
  return decode_scratch_bytes_min(B, H, K) + (B == 1 ? align_up(static_cast<size_t>(PARTIAL_ROWS) * H * sizeof(float), 256) : 0);
}

// Scratch of the tensor-core path inside a buffer that stx_mlp_scratch_bytes(B', H, K) sized, B' >= B >= STX_GEMM_MIN_ROWS.
void* mlp_prefill_region(void* scratch, int64_t B, int64_t H, int64_t K) {
  return static_cast<char*>(scratch) + decode_scratch_bytes(B, H, K);
}

// Per-CTA partial output vectors of the batch-1 kernel inside a scratch buffer that
// stx_mlp_scratch_bytes(1, H, K_cap) sized; nullptr when the device has too many SMs for it.
float* b1_partial_region(void* scratch, int64_t H, int64_t K_cap) {
  if (num_sms() > PARTIAL_ROWS) return nullptr;
  return reinterpret_cast<float*>(static_cast<char*>(scratch) + decode_scratch_bytes_min(1, H, K_cap));
}

// Shared by the op entry point and the fused layer step.  Gather mode (mask_bits != null,
// streaming kernels only): gate/up/down are full [I,H] pools and the rows are those of the set
// mask bits; idx_out [I] / count_out receive the list of active neuron ids and its length.
int mlp_forward(const void* x, int64_t B, int64_t H, const void* gate, const void* up, const void* down,
                const int32_t* K_dev, int64_t K_host, int64_t K_cap, int up_after_gate, void* out, void* combined,
                int act, int has_gate, int dtype, void* scratch, int* status, unsigned parts,
                const uint32_t* mask_bits, int32_t* idx_out, int32_t* count_out, bool scratch_has_partial,
                cudaStream_t s) {
  const bool row_idx = mask_bits != nullptr;
  GatherSpec gs{mask_bits, idx_out, count_out, static_cast<int>(K_cap)};
  if (!up_after_gate) {
    // the streaming kernels keep a[K][B] behind the (always zero) accumulator region
    void* a_region = static_cast<char*>(scratch) + align_up(static_cast<size_t>(B) * H * sizeof(float), 256);
    float* partial = nullptr;
    if (scratch_has_partial && B == 1) partial = b1_partial_region(scratch, H, K_cap);
    const int rc = mlp_forward_tma(x, B, H, gate, up, down, K_dev, K_host, row_idx ? &gs : nullptr, out, combined, act,
                                   has_gate, dtype, a_region, partial, status, parts, s);
    if (rc != STX_ERR_UNSUPPORTED) return rc;
  }
  if (row_idx) {
    set_error("sparse MLP: the gather path needs a row size of at least 512 bytes");
    return STX_ERR_UNSUPPORTED;
  }
  if (!(parts & 1u)) return STX_OK;  // the fused kernel below cannot be split: it runs as the first part
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  const int nchunk = static_cast<int>(H / V);
  MlpArgs a;
  a.x = x;
  a.gate = gate;
  a.up = up;
  a.down = down;
  a.combined = combined;
  a.out = out;
  a.out_acc = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256);
  a.counter = static_cast<unsigned*>(scratch);
  a.K_dev = K_dev;
  a.K_host = static_cast<int>(K_host);
  a.up_after_gate = up_after_gate;
  a.B = static_cast<int>(B);
  a.H = static_cast<int>(H);
  a.act = act;
  a.has_gate = has_gate;
  const int slots = (nchunk + 255) / 256;
  int threads = (nchunk + slots - 1) / slots;
  threads = std::min(256, std::max(64, (threads + 31) / 32 * 32));
  int grid = num_sms() * 2;
  if (!K_dev) grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(grid, K_host)));
  // one partial output per block: block 0 in the accumulator region, the others in the a[K][B] region behind it
  // (scratch layout: 256 | fp32 [B,H] | 256 | fp32 a[K][B], see decode_scratch_bytes_min)
  const size_t acc_bytes = static_cast<size_t>(B) * H * sizeof(float);
  const size_t a_bytes = align_up(static_cast<size_t>(B) * std::max<int64_t>(K_cap, 1) * sizeof(float), 256);
  grid = static_cast<int>(std::min<size_t>(static_cast<size_t>(grid), 1 + a_bytes / acc_bytes));
  a.part_rest = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256 + align_up(acc_bytes, 256) + 256);
  a.a_cap = static_cast<int>((K_cap + grid - 1) / grid);
  switch (dtype) {
    case STX_F32: return dispatch_nb<float>(a, grid, threads, s);
    case STX_F16: return dispatch_nb<__half>(a, grid, threads, s);
    default: return dispatch_nb<__nv_bfloat16>(a, grid, threads, s);
  }
}

}  // namespace stx

using namespace stx;

namespace stx {
int sparse_mlp_forward_check(const void* x, int64_t B, int64_t H, const void* concat_w, const void* down_packed, int64_t K,
                             void* down_buf, int act, int dtype, const void* scratch);
int sparse_mlp_forward_impl(const void* x, int64_t B, int64_t H, const void* concat_w, const void* down_packed,
                            int64_t K, void* down_buf, void* combined_buf, int act, int has_gate, int dtype,
                            void* scratch, bool scratch_has_partial, void* stream);
}

extern "C" {

int stx_mlp_scratch_bytes(int64_t B, int64_t H, int64_t K, size_t* bytes_out) {
  STX_CHECK_ARG(bytes_out && B > 0 && H > 0 && K >= 0, "stx_mlp_scratch_bytes: bad argument");
  // decode kernels' regions, then (row blocks of 9 and more) the tensor-core path's
  // activation matrix and transposed down weight
  *bytes_out = decode_scratch_bytes(B, H, K) + (B >= STX_GEMM_MIN_ROWS ? prefill_scratch_bytes(B, H, K) : 0);
  return STX_OK;
}

int stx_sparse_mlp_forward(const void* x, int64_t B, int64_t H, const void* concat_w, const void* down_packed,
                           int64_t K, void* down_buf, void* combined_buf, int act, int has_gate, int dtype,
                           void* scratch, void* stream) {
  return stx::sparse_mlp_forward_impl(x, B, H, concat_w, down_packed, K, down_buf, combined_buf, act, has_gate, dtype,
                                      scratch, true, stream);
}

}  // extern "C"

namespace stx {
// Argument checks shared by the two entry points (nothing is enqueued before they pass).
int sparse_mlp_forward_check(const void* x, int64_t B, int64_t H, const void* concat_w, const void* down_packed, int64_t K,
                             void* down_buf, int act, int dtype, const void* scratch) {
  STX_CHECK_ARG(x && concat_w && down_packed && down_buf && scratch, "stx_sparse_mlp_forward: null pointer");
  STX_CHECK_ARG(B > 0 && H > 0 && K >= 0, "stx_sparse_mlp_forward: bad sizes B=%lld H=%lld K=%lld",
                static_cast<long long>(B), static_cast<long long>(H), static_cast<long long>(K));
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_sparse_mlp_forward: bad dtype %d", dtype);
  STX_CHECK_ARG(act >= STX_ACT_RELU && act <= STX_ACT_GELU, "stx_sparse_mlp_forward: bad activation %d", act);
  const size_t es = dtype_size(dtype);
  if ((H * es) % 16 != 0) {
    set_error("stx_sparse_mlp_forward: H*elem must be a multiple of 16 bytes");
    return STX_ERR_UNSUPPORTED;
  }
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(concat_w) |
                       reinterpret_cast<uintptr_t>(down_packed) | reinterpret_cast<uintptr_t>(scratch);
  STX_CHECK_ARG((al & 15) == 0, "stx_sparse_mlp_forward: x, concat_w, down_packed and scratch must be 16-byte aligned");
  return STX_OK;
}

// scratch_has_partial: the scratch was sized by stx_mlp_scratch_bytes (true) or is the smaller
// built-in array of the no-alloc entry point (false: batch 1 keeps the two-kernel path).
int sparse_mlp_forward_impl(const void* x, int64_t B, int64_t H, const void* concat_w, const void* down_packed,
                            int64_t K, void* down_buf, void* combined_buf, int act, int has_gate, int dtype,
                            void* scratch, bool scratch_has_partial, void* stream) {
  const int chk = sparse_mlp_forward_check(x, B, H, concat_w, down_packed, K, down_buf, act, dtype, scratch);
  if (chk != STX_OK) return chk;
  const size_t es = dtype_size(dtype);
  // the built-in scratch of the no-alloc entry point (scratch_has_partial == false) has no room for the
  // tensor-core path's buffers: its row blocks stay on the streaming kernels
  if (scratch_has_partial && prefill_wanted(B, H, K, dtype, has_gate)) {
    // row blocks: the gathered weights form a dense contraction -> tcgen05 GEMMs
    return prefill_forward(x, B, H, concat_w, down_packed, K, down_buf, combined_buf, act, dtype,
                           static_cast<char*>(scratch) + decode_scratch_bytes(B, H, K), nullptr, nullptr,
                           static_cast<cudaStream_t>(stream));
  }
  const char* cw = static_cast<const char*>(concat_w);
  const void* gate = has_gate ? cw : nullptr;
  const void* up = has_gate ? cw + static_cast<size_t>(K) * H * es : cw;
  return mlp_forward(x, B, H, gate, up, down_packed, nullptr, K, std::max<int64_t>(K, 1), 0, down_buf, combined_buf, act,
                     has_gate ? 1 : 0, dtype, scratch, nullptr, 3u, nullptr, nullptr, nullptr, scratch_has_partial,
                     static_cast<cudaStream_t>(stream));
}
}  // namespace stx

// ---------------------------------------------------------------------------------------
// Allocation-free variant of stx_sparse_mlp_forward.
//
// Some hosts of this library are not allowed to allocate device memory at all: a serving
// process that reserves its whole HBM budget at start-up and forbids later cudaMalloc calls
// (they serialise the device and can fail under memory pressure), or a plugin that is handed
// raw device pointers by an engine that owns the allocator and cannot lend it out.  Such a
// caller has nowhere to get the scratch buffer that stx_sparse_mlp_forward asks for, so this
// entry point brings its own: a fixed array in device global memory that is part of the
// loaded library image.  Every GPU that loads libstx.so holds the array (about 256 KiB)
// until the process exits.
//
// Limits and rules:
//   * B * (H + K) must not exceed STX_NOALLOC_MAX_ELEMS (65536) elements; larger calls are
//     refused with STX_ERR_TOO_LARGE.
//   * The first call on each device looks up the array's device address (once per device,
//     with that device current).  Make that first call outside any stream capture.
//   * All calls on a device share the one array.  It still holds whatever the previous call
//     left there, so each call clears the part it uses before launching; two calls whose
//     GPU work overlaps (different streams, or different host threads) race on it and give
//     wrong results.  Keep calls on one stream, or otherwise ordered.
//   * No cudaMalloc, cudaFree or other allocating routine is called.
constexpr int64_t STX_NOALLOC_MAX_ELEMS = 65536;
constexpr size_t NOALLOC_BYTES = 1024 + static_cast<size_t>(STX_NOALLOC_MAX_ELEMS) * sizeof(float);

// In host code this name is only a handle for the runtime, never a device address: the
// address a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];
// stands in for the scratch pointer in the argument checks that run before the array's address is looked up
alignas(256) static const unsigned char g_noalloc_host_tag[16] = {};

namespace stx {

// Device address of the array on the current device; looked up once per device.  The table is read
// and written with atomics, so host threads that race on a device's first call all end up with the
// same value (the lookup is idempotent).
static int noalloc_scratch_ptr(void** out) {
  static std::atomic<void*> ptrs[64] = {};
  int dev = 0;
  STX_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    set_error("stx_sparse_mlp_forward_noalloc: device index %d not supported", dev);
    return STX_ERR_UNSUPPORTED;
  }
  void* p = ptrs[dev].load(std::memory_order_acquire);
  if (!p) {
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_scratch)");
    if (!p) {
      set_error("stx_sparse_mlp_forward_noalloc: the scratch array has no device address");
      return STX_ERR_CUDA;
    }
    ptrs[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return STX_OK;
}

}  // namespace stx

extern "C" int stx_sparse_mlp_forward_noalloc(const void* x, int64_t B, int64_t H, const void* concat_w,
                                              const void* down_packed, int64_t K, void* down_buf, void* combined_buf,
                                              int act, int has_gate, int dtype, void* stream) {
  STX_CHECK_ARG(B > 0 && H > 0 && K >= 0, "stx_sparse_mlp_forward_noalloc: bad sizes B=%lld H=%lld K=%lld",
                static_cast<long long>(B), static_cast<long long>(H), static_cast<long long>(K));
  const size_t need = decode_scratch_bytes_min(B, H, K);
  if (need > NOALLOC_BYTES) {
    set_error("stx_sparse_mlp_forward_noalloc: B*(H+K) = %lld exceeds the built-in scratch of %lld elements; "
              "use stx_sparse_mlp_forward with a caller-provided scratch buffer",
              static_cast<long long>(B * (H + K)), static_cast<long long>(STX_NOALLOC_MAX_ELEMS));
    return STX_ERR_TOO_LARGE;
  }
  // every argument check comes before the shared array is touched: a refused call enqueues nothing
  int rc = stx::sparse_mlp_forward_check(x, B, H, concat_w, down_packed, K, down_buf, act, dtype, g_noalloc_host_tag);
  if (rc != STX_OK) return rc;
  void* scratch = nullptr;
  rc = noalloc_scratch_ptr(&scratch);
  if (rc != STX_OK) return rc;
  // the array keeps the previous call's contents: clear the counter and the accumulator
  const size_t used = 256 + align_up(static_cast<size_t>(B) * H * sizeof(float), 256);
  STX_CUDA(cudaMemsetAsync(scratch, 0, used, static_cast<cudaStream_t>(stream)));
  return stx::sparse_mlp_forward_impl(x, B, H, concat_w, down_packed, K, down_buf, combined_buf, act, has_gate, dtype,
                                      scratch, false, stream);
}
