// Per-row selection rules that need a whole score row, and the approximate top-k threshold.
//
//   statistical_topk  src/modeling_skip.py:197-202  scores > mean + std_pop * z   (per row)
//   topk              src/modeling_skip.py:208-211  scatter True at scores.topk(k)
//   approx_topk_threshold  sparse_transformers/csrc/approx_topk.h:10-87
//
// One block of 1024 threads per batch row; the per-row masks are OR-ed into the output bit
// words (mask.any(dim=0), src/modeling_skip.py:214).  All three are reproducible bit for bit
// by the CPU restatement (oracle/stx_oracle.c): exact k-th element by radix select, ties at
// the k-th value taken in ascending index order, and a fixed double-precision summation order
// for the mean and variance (1024 interleaved partial sums; XOR butterfly inside each group
// of 32 consecutive partials, then the 32 group sums added in ascending order).
#include "stx_common.cuh"

#include <algorithm>

namespace stx {

constexpr int SEL_THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {  // ascending float order -> ascending uint order
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// Sum over the block in the documented order; every thread gets the result.
__device__ __forceinline__ double block_sum_fixed(double v, double* s_w /*[32]*/, double* s_out) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if (lane == 0) s_w[wid] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
    for (int w = 0; w < 32; ++w) s += s_w[w];
    *s_out = s;
  }
  __syncthreads();
  const double r = *s_out;
  __syncthreads();
  return r;
}

// k-th largest (k >= 1) of n keys produced by key_at(i), exact, by 4 radix passes of 8 bits.
// All threads of the block must call it; returns the key.  s_hist: 256 ints; s_pick: 2 ints.
template <typename KeyAt>
__device__ __forceinline__ uint32_t block_kth_largest(KeyAt key_at, int n, int k, int* s_hist, int* s_pick) {
  uint32_t prefix = 0u, mask = 0u;
  int kk = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const uint32_t key = key_at(i);
      if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, b = 255;
      for (; b > 0; --b) {
        if (acc + s_hist[b] >= kk) break;
        acc += s_hist[b];
      }
      s_pick[0] = b;
      s_pick[1] = kk - acc;
    }
    __syncthreads();
    prefix |= static_cast<uint32_t>(s_pick[0]) << shift;
    mask |= 255u << shift;
    kk = s_pick[1];
    __syncthreads();
  }
  return prefix;
}

template <typename T>
__global__ void __launch_bounds__(SEL_THREADS)
k_mask_statistical(const T* __restrict__ scores, int I, float z, uint32_t* __restrict__ bits, float* __restrict__ cutoff_out) {
  __shared__ double s_w[32];
  __shared__ double s_out;
  const T* s = scores + static_cast<size_t>(blockIdx.x) * I;
  const int t = threadIdx.x;
  double a = 0.0;
  for (int i = t; i < I; i += SEL_THREADS) a += static_cast<double>(DT<T>::to_f(s[i]));
  const double mean_d = block_sum_fixed(a, s_w, &s_out) / static_cast<double>(I);
  a = 0.0;
  for (int i = t; i < I; i += SEL_THREADS) {
    const double d = static_cast<double>(DT<T>::to_f(s[i])) - mean_d;
    a += d * d;
  }
  const double var_d = block_sum_fixed(a, s_w, &s_out) / static_cast<double>(I);
  // rounding points of the reference's tensor arithmetic in the scores' dtype
  const float mean_r = DT<T>::round_f(static_cast<float>(mean_d));
  const float std_r = DT<T>::round_f(static_cast<float>(sqrt(var_d)));
  const float z_r = DT<T>::round_f(z);
  const float prod = DT<T>::round_f(__fmul_rn(std_r, z_r));
  const float cutoff = DT<T>::round_f(__fadd_rn(mean_r, prod));
  if (t == 0 && cutoff_out) cutoff_out[blockIdx.x] = cutoff;
  const int W = (I + 31) >> 5;
  for (int w = t; w < W; w += SEL_THREADS) {
    uint32_t word = 0u;
    const int n = min(32, I - w * 32);
    for (int b = 0; b < n; ++b)
      if (DT<T>::to_f(s[w * 32 + b]) > cutoff) word |= 1u << b;
    if (word) atomicOr(&bits[w], word);
  }
}

template <typename T>
__global__ void __launch_bounds__(SEL_THREADS)
k_mask_topk(const T* __restrict__ scores, int I, int k, uint32_t* __restrict__ bits) {
  __shared__ int s_hist[256];
  __shared__ int s_pick[2];
  __shared__ int s_wsum[32];
  __shared__ int s_above;
  const T* s = scores + static_cast<size_t>(blockIdx.x) * I;
  const int t = threadIdx.x, lane = t & 31, wid = t >> 5;
  const uint32_t kth_key = block_kth_largest([&](int i) { return order_key(DT<T>::to_f(s[i])); }, I, k, s_hist, s_pick);
  const float kth = key_value(kth_key);
  // contiguous index ranges per thread keep the ascending order for the tie rule
  const int per = (I + SEL_THREADS - 1) / SEL_THREADS;
  const int lo = t * per, hi = min(I, lo + per);
  int above = 0, ties = 0;
  for (int i = lo; i < hi; ++i) {
    const float v = DT<T>::to_f(s[i]);
    above += v > kth;
    ties += v == kth;
  }
  if (t == 0) s_above = 0;
  __syncthreads();
  atomicAdd(&s_above, above);
  int inc = ties;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += v;
  }
  if (lane == 31) s_wsum[wid] = inc;
  __syncthreads();
  if (t == 0) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int v = s_wsum[w];
      s_wsum[w] = run;
      run += v;
    }
  }
  __syncthreads();
  int tie_rank = s_wsum[wid] + inc - ties;  // ties before this thread's range
  const int ties_wanted = k - s_above;
  for (int i = lo; i < hi; ++i) {
    const float v = DT<T>::to_f(s[i]);
    bool on = v > kth;
    if (v == kth) {
      on = tie_rank < ties_wanted;
      ++tie_rank;
    }
    if (on) atomicOr(&bits[i >> 5], 1u << (i & 31));
  }
}

// approx_topk.h:25-83.  Shared memory: 4 * width bucket keys.
template <typename T>
__global__ void __launch_bounds__(SEL_THREADS)
k_approx_topk(const T* __restrict__ scores, int I, int k, T* __restrict__ thr_out) {
  extern __shared__ uint32_t s_sk[];
  __shared__ int s_hist[256];
  __shared__ int s_pick[2];
  __shared__ int s_n;
  const T* s = scores + static_cast<size_t>(blockIdx.x) * I;
  const int t = threadIdx.x;
  const int S = 4;
  const int width = min(1024, I / 4);
  if (width <= 0) {
    if (t == 0) thr_out[blockIdx.x] = DT<T>::from_f(0.f);
    return;
  }
  const uint32_t neg_inf = order_key(-INFINITY);
  for (int i = t; i < S * width; i += SEL_THREADS) s_sk[i] = neg_inf;
  if (t == 0) s_n = 0;
  __syncthreads();
  for (int q = 0; q < S; ++q)
    for (int j = t; j < I; j += SEL_THREADS) {
      const long long key = static_cast<long long>(q) * I + j;  // std::hash<int64_t> is the identity
      const int pos = static_cast<int>(key % width);
      atomicMax(&s_sk[q * width + pos], order_key(DT<T>::to_f(s[j])));
    }
  __syncthreads();
  int mine = 0;
  for (int i = t; i < S * width; i += SEL_THREADS) mine += s_sk[i] != neg_inf;
  atomicAdd(&s_n, mine);
  __syncthreads();
  const int n = s_n;
  if (n == 0) {
    if (t == 0) thr_out[blockIdx.x] = DT<T>::from_f(0.f);
    return;
  }
  long long sketch_k = static_cast<long long>(k) * n / I;
  if (sketch_k < 1) sketch_k = 1;
  if (sketch_k > n) sketch_k = n;
  // the excluded -inf buckets sort last, so the rank among all buckets is the same
  const uint32_t key = block_kth_largest([&](int i) { return s_sk[i]; }, S * width, static_cast<int>(sketch_k), s_hist, s_pick);
  if (t == 0) thr_out[blockIdx.x] = DT<T>::from_f(__fmul_rn(key_value(key), 0.9f));
}

int mask_from_scores(const void* scores, int64_t B, int64_t I, int dtype, int method, float param,
                     uint32_t* bits_out, void* scratch, cudaStream_t s) {
  (void)scratch;
  const size_t W = static_cast<size_t>((I + 31) / 32);
  STX_CUDA(cudaMemsetAsync(bits_out, 0, W * sizeof(uint32_t), s));
  const unsigned grid = static_cast<unsigned>(B);
  if (method == STX_MASK_STATISTICAL) {
    switch (dtype) {
      case STX_F32:
        k_mask_statistical<float><<<grid, SEL_THREADS, 0, s>>>(static_cast<const float*>(scores), static_cast<int>(I), param, bits_out, nullptr);
        break;
      case STX_F16:
        k_mask_statistical<__half><<<grid, SEL_THREADS, 0, s>>>(static_cast<const __half*>(scores), static_cast<int>(I), param, bits_out, nullptr);
        break;
      default:
        k_mask_statistical<__nv_bfloat16><<<grid, SEL_THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(scores), static_cast<int>(I), param, bits_out, nullptr);
        break;
    }
    STX_LAUNCH_CHECK("k_mask_statistical");
    return STX_OK;
  }
  if (method == STX_MASK_TOPK) {
    int k = static_cast<int>(param);
    if (k < 1 || k > I) {
      set_error("topk rule: k=%d outside 1..%lld", k, static_cast<long long>(I));
      return STX_ERR_INVALID_ARG;
    }
    switch (dtype) {
      case STX_F32:
        k_mask_topk<float><<<grid, SEL_THREADS, 0, s>>>(static_cast<const float*>(scores), static_cast<int>(I), k, bits_out);
        break;
      case STX_F16:
        k_mask_topk<__half><<<grid, SEL_THREADS, 0, s>>>(static_cast<const __half*>(scores), static_cast<int>(I), k, bits_out);
        break;
      default:
        k_mask_topk<__nv_bfloat16><<<grid, SEL_THREADS, 0, s>>>(static_cast<const __nv_bfloat16*>(scores), static_cast<int>(I), k, bits_out);
        break;
    }
    STX_LAUNCH_CHECK("k_mask_topk");
    return STX_OK;
  }
  set_error("mask rule %d needs no score pass", method);
  return STX_ERR_INVALID_ARG;
}

}  // namespace stx

using namespace stx;

extern "C" {

int stx_approx_topk_scratch_bytes(int64_t B, int64_t I, size_t* bytes_out) {
  STX_CHECK_ARG(bytes_out && B > 0 && I > 0, "stx_approx_topk_scratch_bytes: bad argument");
  *bytes_out = 256;  // the kernel works in shared memory; kept for interface stability
  return STX_OK;
}

int stx_approx_topk_threshold(const void* scores, int64_t B, int64_t I, int64_t k, int dtype, void* threshold_out,
                              void* scratch, void* stream) {
  (void)scratch;
  STX_CHECK_ARG(scores && threshold_out, "stx_approx_topk_threshold: null pointer");
  STX_CHECK_ARG(B > 0 && I > 0, "stx_approx_topk_threshold: sizes must be positive");
  STX_CHECK_ARG(k > 0, "k must be positive");
  STX_CHECK_ARG(k <= I, "k cannot be larger than feature size");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_approx_topk_threshold: bad dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int width = static_cast<int>(std::min<int64_t>(1024, I / 4));
  const size_t smem = static_cast<size_t>(4) * std::max(width, 1) * sizeof(uint32_t);
  const unsigned grid = static_cast<unsigned>(B);
  switch (dtype) {
    case STX_F32:
      k_approx_topk<float><<<grid, SEL_THREADS, smem, s>>>(static_cast<const float*>(scores), static_cast<int>(I), static_cast<int>(k), static_cast<float*>(threshold_out));
      break;
    case STX_F16:
      k_approx_topk<__half><<<grid, SEL_THREADS, smem, s>>>(static_cast<const __half*>(scores), static_cast<int>(I), static_cast<int>(k), static_cast<__half*>(threshold_out));
      break;
    default:
      k_approx_topk<__nv_bfloat16><<<grid, SEL_THREADS, smem, s>>>(static_cast<const __nv_bfloat16*>(scores), static_cast<int>(I), static_cast<int>(k), static_cast<__nv_bfloat16*>(threshold_out));
      break;
  }
  STX_LAUNCH_CHECK("k_approx_topk");
  return STX_OK;
}

}  // extern "C"
