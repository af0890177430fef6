// Decode-time glue of the LlamaSkip host around the sparse MLP (C ABI: stx_attn_decode,
// stx_add_rmsnorm): one query token against the KV cache, and residual add + RMSNorm.
//
//   k_attn_decode   grid = query heads.  A CTA rotates its q head and the k head of its group
//                   (rotate-half RoPE in fp32, rounded to the model dtype), appends k and v to
//                   the cache (the first head of each group writes), scores the keys 0..pos
//                   a warp per key with eight keys in flight, soft-maxes in fp32 and sums the
//                   values with 16-byte chunks of the head dimension across threads.  The position is read from device memory, so a
//                   captured CUDA graph can be replayed token after token.
//   k_add_rmsnorm   one CTA: h <- h + a (rounded to the model dtype), then
//                   x = round(h * rsqrt(mean(h^2) + eps)) * w, the order of operations of
//                   LlamaSkipRMSNorm (src/models/llama/modelling_llama_skip.py:39-44).
#include "stx_common.cuh"
#include "stx_tma.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <cooperative_groups.h>

namespace stx {

namespace cg = cooperative_groups;

constexpr int ATT_THREADS = 512;
constexpr int NORM_THREADS = 1024;

template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ void load(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x;
    b = v.y;
  }
};
template <> struct Pair<__half> {
  static __device__ __forceinline__ void load(const __half* p, float& a, float& b) {
    const float2 v = __half22float2(*reinterpret_cast<const __half2*>(p));
    a = v.x;
    b = v.y;
  }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float& a, float& b) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    a = v.x;
    b = v.y;
  }
};

// Block-wide max / sum over the block's threads; `red` has 32 floats.  Every thread gets the result.
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float o = __shfl_xor_sync(0xffffffffu, v, off);
    v = IS_MAX ? fmaxf(v, o) : v + o;
  }
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = IS_MAX ? -INFINITY : 0.f;
  for (int w = 0; w < nw; ++w) r = IS_MAX ? fmaxf(r, red[w]) : r + red[w];  // same order in every thread
  return r;
}

// `BYTES` consecutive bytes (4, 8, 16 or 32; aligned to min(BYTES, 16)) as 32-bit words.
template <int BYTES>
__device__ __forceinline__ void load_words(const void* p, uint32_t (&w)[BYTES / 4]) {
  if constexpr (BYTES == 4) {
    w[0] = *reinterpret_cast<const uint32_t*>(p);
  } else if constexpr (BYTES == 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    w[0] = v.x;
    w[1] = v.y;
  } else {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      const uint4 v = reinterpret_cast<const uint4*>(p)[i];
      w[4 * i] = v.x;
      w[4 * i + 1] = v.y;
      w[4 * i + 2] = v.z;
      w[4 * i + 3] = v.w;
    }
  }
}
// Word i of a row of T as floats: one element for fp32, two for the 16-bit types.
template <typename T> struct Words;
template <> struct Words<float> {
  static constexpr int EPW = 1;
  static __device__ __forceinline__ void run(uint32_t w, float* f) { f[0] = __uint_as_float(w); }
};
template <> struct Words<__half> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void run(uint32_t w, float* f) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w));
    f[0] = t.x;
    f[1] = t.y;
  }
};
template <> struct Words<__nv_bfloat16> {
  static constexpr int EPW = 2;
  static __device__ __forceinline__ void run(uint32_t w, float* f) {
    f[0] = __uint_as_float(w << 16);
    f[1] = __uint_as_float(w & 0xffff0000u);
  }
};

// Workspace of stx_attn_decode: one arrival counter per head (zero between launches), then per
// head and split the unnormalised value sum [HD], the split's score maximum and its sum of
// exponentials.
constexpr size_t ATT_COUNTER_BYTES = 4096;  // up to 1024 heads
__host__ __device__ inline int att_part_floats(int hd) { return hd + 2; }

// Grid (heads, splits): split s of a head takes an equal share of the cached keys (the last split
// also the token's own key), so that one query head is read by several SMs.  CL: the splits of a
// head form a thread-block cluster and split 0 merges the partial soft-maxes out of the others'
// shared memory; otherwise they meet in the workspace and the split that arrives last at the
// head's counter merges (a store, a fence, an atomic and a load more on the critical path).
// Shared memory (floats): q_s[HD] | kn_s[HD] | vn_s[HD] | red[32] | acc_s[NG][HD] | sc[keys of the split + 1]
template <typename T, int HD, bool CL>
__global__ void __launch_bounds__(ATT_THREADS) k_attn_decode(const T* __restrict__ qkv, const float* __restrict__ cos_t,
                                                              const float* __restrict__ sin_t,
                                                              const long long* __restrict__ pos_dev, T* k_cache, T* v_cache,
                                                              T* __restrict__ out, int nh, int nkv, long long max_len,
                                                              float scale, unsigned char* workspace) {
  constexpr int V = DT<T>::V;              // elements per 16 bytes
  constexpr int NW = ATT_THREADS / 32;
  constexpr int E = HD / 32;               // elements of a key row per lane
  constexpr int KB = E * sizeof(T);        // the same in bytes
  constexpr int TPR = HD / V;              // threads per value row (16 bytes each)
  constexpr int NG = ATT_THREADS / TPR;    // key groups of the value sum
  constexpr int U = 8;                     // keys a warp has in flight
  extern __shared__ float sm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* q_s = sm;
  float* kn_s = q_s + HD;
  float* vn_s = kn_s + HD;
  float* red = vn_s + HD;
  float* acc_s = red + 32;
  float* sc = acc_s + NG * HD;
  const long long pos = *pos_dev;
  if (pos < 0 || pos >= max_len) return;  // nothing sensible to do; the output is left as it was
  const int h = blockIdx.x;
  const int sp = blockIdx.y, NSP = gridDim.y;
  const int rep = nh / nkv;
  const int g = h / rep;
  T* kc = k_cache + static_cast<size_t>(g) * max_len * HD;
  T* vc = v_cache + static_cast<size_t>(g) * max_len * HD;
  const int chunk = (static_cast<int>(pos) + NSP - 1) / NSP;  // cached keys per split
  const int lo = min(sp * chunk, static_cast<int>(pos)), hi = min(lo + chunk, static_cast<int>(pos));
  const bool own = sp == NSP - 1;   // this split also scores the token's own key
  const T* ks = kc + static_cast<size_t>(lo) * HD;  // key j of the split is cached key lo + j
  const T* vs = vc + static_cast<size_t>(lo) * HD;
  const int n = hi - lo + 1;        // sc[n - 1] is the own key's slot (unused unless `own`)
  // The first batch of keys is requested before the rotation: it depends on the position only.
  uint32_t kw[U][KB / 4];
  auto load_keys = [&](int j0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + NW * u;
      if (j < n - 1) load_words<KB>(reinterpret_cast<const char*>(ks + static_cast<size_t>(j) * HD) + lane * KB, kw[u]);
    }
  };
  load_keys(warp);

  if (tid < HD) {
    constexpr int half = HD / 2;
    const int dp = tid < half ? tid + half : tid - half;
    const float sign = tid < half ? -1.f : 1.f;
    const float c = cos_t[pos * HD + tid], s = sin_t[pos * HD + tid];
    const T* qrow = qkv + static_cast<size_t>(h) * HD;
    const T* krow = qkv + static_cast<size_t>(nh + g) * HD;
    const T* vrow = qkv + static_cast<size_t>(nh + nkv + g) * HD;
    // x * cos + rotate_half(x) * sin: two rounded products, one rounded sum, then the model dtype
    const T qr = DT<T>::from_f(__fadd_rn(__fmul_rn(DT<T>::to_f(qrow[tid]), c), __fmul_rn(sign * DT<T>::to_f(qrow[dp]), s)));
    const T kr = DT<T>::from_f(__fadd_rn(__fmul_rn(DT<T>::to_f(krow[tid]), c), __fmul_rn(sign * DT<T>::to_f(krow[dp]), s)));
    const T vr = vrow[tid];
    q_s[tid] = DT<T>::to_f(qr);
    kn_s[tid] = DT<T>::to_f(kr);
    vn_s[tid] = DT<T>::to_f(vr);
    if (h == g * rep && sp == 0) {  // one writer per group; every head of the group uses its own copy in shared memory
      kc[pos * HD + tid] = kr;
      vc[pos * HD + tid] = vr;
    }
  }
  __syncthreads();

  // ---- scores: a warp per key, lane l holds elements [l*E, l*E + E); U keys in flight per warp
  float qf[E];
#pragma unroll
  for (int e = 0; e < E; ++e) qf[e] = q_s[lane * E + e];
  float lmax = -INFINITY;
  // the first batch of values, requested before the soft-max needs anything
  const int grp = tid / TPR, ch = tid - grp * TPR;
  uint4 raw[4];
  auto load_values = [&](int j0) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + NG * u;
      if (j < n - 1) raw[u] = *reinterpret_cast<const uint4*>(vs + static_cast<size_t>(j) * HD + ch * V);
    }
  };
  load_values(grp);
  for (int j0 = warp; j0 < n - 1; j0 += NW * U) {
    if (j0 != warp) load_keys(j0);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + NW * u;
      if (j < n - 1) {  // uniform over the warp
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < KB / 4; ++i) {
          float f[Words<T>::EPW];
          Words<T>::run(kw[u][i], f);
#pragma unroll
          for (int e = 0; e < Words<T>::EPW; ++e) dot = fmaf(qf[i * Words<T>::EPW + e], f[e], dot);
        }
        dot = warp_sum_xor(dot) * scale;
        if (lane == 0) sc[j] = dot;
        lmax = fmaxf(lmax, dot);
      }
    }
  }
  if (warp == 0 && own) {  // the key of this token
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < E; ++e) dot = fmaf(qf[e], kn_s[lane * E + e], dot);
    dot = warp_sum_xor(dot) * scale;
    if (lane == 0) sc[n - 1] = dot;
    lmax = fmaxf(lmax, dot);
  }
  const float m = block_reduce<true>(lmax, red);  // its barriers also publish sc
  const int nsc = own ? n : n - 1;
  float lsum = 0.f;
  for (int j = tid; j < nsc; j += ATT_THREADS) {
    const float p = __expf(sc[j] - m);
    sc[j] = p;
    lsum += p;
  }
  const float denom = block_reduce<false>(lsum, red);

  // ---- values: thread (grp, ch) sums p_j * v_j[16-byte chunk ch] over the keys j = grp, grp + NG, ...
  float acc[V];
#pragma unroll
  for (int v = 0; v < V; ++v) acc[v] = 0.f;
  for (int j0 = grp; j0 < n - 1; j0 += 4 * NG) {
    if (j0 != grp) load_values(j0);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + NG * u;
      if (j < n - 1) {
        float f[V];
        Unpack<T>::run(raw[u], f);
        const float p = sc[j];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = fmaf(p, f[v], acc[v]);
      }
    }
  }
  if (grp == 0 && own) {
    const float p = sc[n - 1];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = fmaf(p, vn_s[ch * V + v], acc[v]);
  }
#pragma unroll
  for (int v = 0; v < V; ++v) acc_s[grp * HD + ch * V + v] = acc[v];
  __syncthreads();
  if constexpr (CL) {
    // this split's unnormalised sum, maximum and sum of exponentials, where the cluster can read them
    if (tid < HD) {
      float s = 0.f;
      for (int k = 0; k < NG; ++k) s += acc_s[k * HD + tid];
      q_s[tid] = s;  // the query is not needed any more
    }
    if (tid == 0) {
      red[0] = m;
      red[1] = denom;
    }
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (sp == 0 && tid < HD) {
      float pm[8], pl[8], pa[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (k < NSP) {
          const float* rq = cluster.map_shared_rank(q_s, k);
          const float* rr = cluster.map_shared_rank(red, k);
          pm[k] = rr[0];
          pl[k] = rr[1];
          pa[k] = rq[tid];
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < NSP) M = fmaxf(M, pm[k]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if (k < NSP) {
          const float wgt = __expf(pm[k] - M);  // 0 for a split without keys (its maximum is -inf)
          num = fmaf(wgt, pa[k], num);
          den = fmaf(wgt, pl[k], den);
        }
      }
      out[static_cast<size_t>(h) * HD + tid] = DT<T>::from_f(num / den);
    }
    cluster.sync();  // nobody leaves while split 0 may still read its shared memory
    return;
  }
  int* counter = reinterpret_cast<int*>(workspace) + h;
  float* part = reinterpret_cast<float*>(workspace + ATT_COUNTER_BYTES) + static_cast<size_t>(h) * NSP * att_part_floats(HD);
  float* mine = part + static_cast<size_t>(sp) * att_part_floats(HD);
  if (tid < HD) {
    float s = 0.f;
    for (int k = 0; k < NG; ++k) s += acc_s[k * HD + tid];
    if (NSP == 1) {
      out[static_cast<size_t>(h) * HD + tid] = DT<T>::from_f(s / denom);
    } else {
      __stcg(mine + tid, s);
      if (tid == 0) {
        __stcg(mine + HD, m);
        __stcg(mine + HD + 1, denom);
      }
    }
  }
  if (NSP == 1) return;
  // ---- the split that arrives last merges: out = sum_s e^(m_s - M) acc_s / sum_s e^(m_s - M) l_s
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int t = atomicAdd(counter, 1);
    s_last = t == NSP - 1;
    if (s_last) *counter = 0;  // every other split has arrived: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid < HD) {
    float pm[8], pl[8], pa[8];  // all loads in flight together (at most 8 splits)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < NSP) {
        const float* pk = part + k * att_part_floats(HD);
        pm[k] = __ldcg(pk + HD);
        pl[k] = __ldcg(pk + HD + 1);
        pa[k] = __ldcg(pk + tid);
      }
    }
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < NSP) M = fmaxf(M, pm[k]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < NSP) {
        const float wgt = __expf(pm[k] - M);  // 0 for a split without keys (its maximum is -inf)
        num = fmaf(wgt, pa[k], num);
        den = fmaf(wgt, pl[k], den);
      }
    }
    out[static_cast<size_t>(h) * HD + tid] = DT<T>::from_f(num / den);
  }
}

// h_out = round(h + a) (a may be null: h_out = h, nothing written unless write_h), then
// x = round(h_out * rsqrt(mean(h_out^2) + eps)) * w.  Thread t owns elements t, t + blockDim.x, ...
// (at most MAXPT of them, kept in registers).  `store_x(i, value)` receives x.
constexpr int NORM_MAX_H = 8192;
template <int MAXPT> struct NormRegs {
  float v[MAXPT], wv[MAXPT];
};
// Part 1: the loads (and the add).  Kernels that also stream bulk copies call this BEFORE they
// request the copies: small loads issued behind hundreds of KB of bulk traffic of the same SM
// come back only when that traffic has drained.
template <typename T, int MAXPT>
__device__ __forceinline__ void norm_load(const T* h, const T* __restrict__ a, const T* __restrict__ w, int H,
                                          NormRegs<MAXPT>& r) {
  const int tid = threadIdx.x, nt = blockDim.x;
#pragma unroll
  for (int k = 0; k < MAXPT; ++k) {
    const int i = tid + k * nt;
    r.v[k] = 0.f;
    r.wv[k] = 0.f;
    if (i < H) {
      r.v[k] = DT<T>::to_f(h[i]);
      if (a) r.v[k] = DT<T>::round_f(r.v[k] + DT<T>::to_f(a[i]));
      r.wv[k] = DT<T>::to_f(w[i]);
    }
  }
}
// Part 2: h_out, the sum of squares, x.
template <typename T, int MAXPT, typename StoreX>
__device__ __forceinline__ void norm_finish(const NormRegs<MAXPT>& r, float eps, T* h_out, int H, float* red, StoreX store_x) {
  const int tid = threadIdx.x, nt = blockDim.x;
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXPT; ++k) {
    const int i = tid + k * nt;
    if (i < H && h_out) h_out[i] = DT<T>::from_f(r.v[k]);
    ss = fmaf(r.v[k], r.v[k], ss);
  }
  const float tot = block_reduce<false>(ss, red);
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
  for (int k = 0; k < MAXPT; ++k) {
    const int i = tid + k * nt;
    if (i < H) store_x(i, DT<T>::from_f(DT<T>::round_f(r.v[k] * inv) * r.wv[k]));
  }
}
template <typename T, int MAXPT, typename StoreX>
__device__ __forceinline__ void add_rmsnorm_block(const T* h, const T* __restrict__ a, const T* __restrict__ w, float eps,
                                                  T* h_out, int H, float* red, StoreX store_x) {
  NormRegs<MAXPT> r;
  norm_load<T, MAXPT>(h, a, w, H, r);
  norm_finish<T, MAXPT>(r, eps, h_out, H, red, store_x);
}

template <typename T>
__global__ void __launch_bounds__(NORM_THREADS) k_add_rmsnorm(const T* h, const T* __restrict__ a, const T* __restrict__ w,
                                                               float eps, T* h_out, T* __restrict__ x_out, int H) {
  __shared__ float red[32];
  add_rmsnorm_block<T, NORM_MAX_H / NORM_THREADS>(h, a, w, eps, a ? h_out : nullptr, H, red, [&](int i, T x) { x_out[i] = x; });
}

// y[n] = W[n,:] . x for a row-major W [N,H], with x either given (w_norm == null: x = h) or made
// on the fly as x = RMSNorm(h + a) * w_norm in every CTA (the vector is a few KB; recomputing it
// costs less than a kernel boundary).  CTA 0 also writes h + a to h_out and x to x_out (either
// may be null).  h_out must not alias h: other CTAs still read h.  A warp per output row, 16-byte
// loads, two batches of eight per lane in flight, the first of them while the norm is computed.
constexpr int GEMV_THREADS = 512;
constexpr int GEMV_BATCH = 8;  // 16-byte loads per lane and item
template <typename T>
__global__ void __launch_bounds__(GEMV_THREADS) k_norm_gemv(const T* __restrict__ h, const T* __restrict__ a,
                                                             const T* __restrict__ w_norm, float eps,
                                                             const T* __restrict__ W, T* __restrict__ y, T* h_out,
                                                             T* x_out, int H, int N) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(128) unsigned char gsm[];
  T* x_s = reinterpret_cast<T*>(gsm);
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = H / V;
  const int wpg = (GEMV_THREADS / 32) * gridDim.x;  // warps in the grid
  const int row0 = blockIdx.x * (GEMV_THREADS / 32) + warp;
  // A warp's work is a sequence of items: item it = (its row number it / nb, batch it % nb of that
  // row), a batch being GEMV_BATCH x 32 consecutive 16-byte chunks.  Two items are in flight.
  const int nb = (nchunk + 32 * GEMV_BATCH - 1) / (32 * GEMV_BATCH);
  const int nrows = row0 < N ? (N - 1 - row0) / wpg + 1 : 0;
  const int nitems = nrows * nb;
  auto load_item = [&](int it, uint4 (&buf)[GEMV_BATCH]) {
    const int r = it / nb, bi = it - r * nb;
    const uint4* wr = reinterpret_cast<const uint4*>(W + static_cast<size_t>(row0 + r * wpg) * H) + bi * 32 * GEMV_BATCH + lane;
    const int left = nchunk - bi * 32 * GEMV_BATCH - lane;
#pragma unroll
    for (int i = 0; i < GEMV_BATCH; ++i)
      if (32 * i < left) buf[i] = ld_stream16(wr + 32 * i);
  };
  float acc0 = 0.f, acc1 = 0.f;
  auto compute_item = [&](int it, const uint4 (&buf)[GEMV_BATCH]) {
    const int r = it / nb, bi = it - r * nb;
    const uint4* xs = reinterpret_cast<const uint4*>(x_s) + bi * 32 * GEMV_BATCH + lane;
    const int left = nchunk - bi * 32 * GEMV_BATCH - lane;
#pragma unroll
    for (int i = 0; i < GEMV_BATCH; ++i) {
      if (32 * i < left) {
        float wf[V], xf[V];
        Unpack<T>::run(buf[i], wf);
        Unpack<T>::run(xs[32 * i], xf);
        float t = 0.f;
#pragma unroll
        for (int v = 0; v < V; ++v) t = fmaf(xf[v], wf[v], t);
        if (i & 1) acc1 += t; else acc0 += t;
      }
    }
    if (bi == nb - 1) {  // the row is complete
      const float dot = warp_sum_xor(acc0 + acc1);
      if (lane == 0) y[row0 + r * wpg] = DT<T>::from_f(dot);
      acc0 = 0.f;
      acc1 = 0.f;
    }
  };
  uint4 bufa[GEMV_BATCH], bufb[GEMV_BATCH];
  if (nitems > 0) load_item(0, bufa);  // in flight while the norm is computed
  if (w_norm) {
    const bool first = blockIdx.x == 0;
    add_rmsnorm_block<T, NORM_MAX_H / GEMV_THREADS>(h, a, w_norm, eps, first ? h_out : nullptr, H, red, [&](int i, T x) {
      x_s[i] = x;
      if (first && x_out) x_out[i] = x;
    });
  } else {
    for (int i = tid; i < nchunk; i += GEMV_THREADS) reinterpret_cast<uint4*>(x_s)[i] = reinterpret_cast<const uint4*>(h)[i];
  }
  __syncthreads();
  for (int it = 0; it < nitems; it += 2) {
    if (it + 1 < nitems) load_item(it + 1, bufb);
    compute_item(it, bufa);
    if (it + 2 < nitems) load_item(it + 2, bufa);
    if (it + 1 < nitems) compute_item(it + 1, bufb);
  }
}

// The same product when the CTA's share of W fits in shared memory (N * H elements over one CTA
// per SM, e.g. a 5120 x 3072 fp16 projection: 35 rows, 215 KB): every row is requested by a bulk
// copy before anything else happens, so the whole matrix is in flight while the norm is
// computed, and each warp then reads its rows from shared memory.
// Dynamic shared memory: [0,128) one mbarrier per warp | x_s [H] | rows [rows_per_cta][H].
template <typename T>
__global__ void __launch_bounds__(GEMV_THREADS) k_norm_gemv_tma(const T* __restrict__ h, const T* __restrict__ a,
                                                                 const T* __restrict__ w_norm, float eps,
                                                                 const T* __restrict__ W, T* __restrict__ y, T* h_out,
                                                                 T* x_out, int H, int N, int rows_per_cta) {
  constexpr int V = DT<T>::V;
  constexpr int NW = GEMV_THREADS / 32;
  extern __shared__ __align__(128) unsigned char gsm[];
  __shared__ float red[32];
  uint64_t* bar = reinterpret_cast<uint64_t*>(gsm);
  T* x_s = reinterpret_cast<T*>(gsm + 128);
  const size_t row_bytes = static_cast<size_t>(H) * sizeof(T);
  unsigned char* rows = gsm + 128 + (row_bytes + 127) / 128 * 128;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nchunk = H / V;
  const int r0 = blockIdx.x * rows_per_cta;
  const int nr = max(0, min(rows_per_cta, N - r0));
  const int mine = warp < nr ? (nr - 1 - warp) / NW + 1 : 0;  // local rows warp, warp + NW, ...
  if (tid == 0) {
    for (int w = 0; w < NW; ++w) mbar_init(&bar[w], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // the small loads of the prologue go first: behind the bulk copies they would come back last
  constexpr int MAXPT = NORM_MAX_H / GEMV_THREADS;
  NormRegs<MAXPT> nr_regs;
  uint4 xr[MAXPT / 4 + 1];
  if (w_norm) {
    norm_load<T, MAXPT>(h, a, w_norm, H, nr_regs);
  } else {
#pragma unroll
    for (int k = 0; k < MAXPT / 4 + 1; ++k)
      if (tid + k * GEMV_THREADS < nchunk) xr[k] = reinterpret_cast<const uint4*>(h)[tid + k * GEMV_THREADS];
  }
  if (mine > 0) {
    if (lane == 0) mbar_expect_tx(&bar[warp], static_cast<uint32_t>(mine * row_bytes));
    __syncwarp();
    for (int k = lane; k < mine; k += 32) {
      const int lr = warp + k * NW;
      bulk_load(rows + static_cast<size_t>(lr) * row_bytes, W + static_cast<size_t>(r0 + lr) * H, static_cast<uint32_t>(row_bytes),
                &bar[warp]);
    }
  }
  if (w_norm) {
    const bool first = blockIdx.x == 0;
    norm_finish<T, MAXPT>(nr_regs, eps, first ? h_out : nullptr, H, red, [&](int i, T x) {
      x_s[i] = x;
      if (first && x_out) x_out[i] = x;
    });
  } else {
#pragma unroll
    for (int k = 0; k < MAXPT / 4 + 1; ++k)
      if (tid + k * GEMV_THREADS < nchunk) reinterpret_cast<uint4*>(x_s)[tid + k * GEMV_THREADS] = xr[k];
  }
  __syncthreads();
  if (mine == 0) return;
  const bool ok = mbar_wait_bounded(&bar[warp], 0);
  for (int k = 0; k < mine; ++k) {
    const int lr = warp + k * NW;
    const uint4* wr = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(lr) * row_bytes);
    float acc0 = 0.f, acc1 = 0.f;
    int c = lane;
    for (; c + 32 < nchunk; c += 64) {
      float w0[V], w1[V], x0[V], x1[V];
      Unpack<T>::run(wr[c], w0);
      Unpack<T>::run(wr[c + 32], w1);
      Unpack<T>::run(reinterpret_cast<const uint4*>(x_s)[c], x0);
      Unpack<T>::run(reinterpret_cast<const uint4*>(x_s)[c + 32], x1);
#pragma unroll
      for (int v = 0; v < V; ++v) {
        acc0 = fmaf(x0[v], w0[v], acc0);
        acc1 = fmaf(x1[v], w1[v], acc1);
      }
    }
    for (; c < nchunk; c += 32) {
      float w0[V], x0[V];
      Unpack<T>::run(wr[c], w0);
      Unpack<T>::run(reinterpret_cast<const uint4*>(x_s)[c], x0);
#pragma unroll
      for (int v = 0; v < V; ++v) acc0 = fmaf(x0[v], w0[v], acc0);
    }
    const float dot = warp_sum_xor(acc0 + acc1);
    // a copy that did not arrive within the wait limit must not pass for a result
    if (lane == 0) y[r0 + lr] = DT<T>::from_f(ok ? dot : __int_as_float(0x7fc00000));
  }
}

template <typename T>
static int launch_norm_gemv(const void* h, const void* a, const void* w_norm, float eps, const void* W, void* y, void* h_out,
                            void* x_out, int H, int N, cudaStream_t s) {
  const int warps = GEMV_THREADS / 32;
  const int sms = num_sms();
  // A CTA of this size needs an SM to itself; a few SMs are left to kernels that run beside it on
  // other streams (the weight cache's upkeep), or one CTA would wait for a second wave.
  const int target = std::max(1, sms - 4);
  const int rows_per_cta = (N + target - 1) / target;
  const size_t row_bytes = static_cast<size_t>(H) * sizeof(T);
  const size_t smem_tma = 128 + (row_bytes + 127) / 128 * 128 + static_cast<size_t>(rows_per_cta) * row_bytes;
  const size_t budget = 227 * 1024 - 1024;  // per-block limit less the kernel's static shared memory
  if (smem_tma <= budget) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      STX_CUDA(cudaFuncSetAttribute(k_norm_gemv_tma<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(budget)));
      attr_set[dev] = true;
    }
    const unsigned grid = static_cast<unsigned>((N + rows_per_cta - 1) / rows_per_cta);
    k_norm_gemv_tma<T><<<grid, GEMV_THREADS, smem_tma, s>>>(static_cast<const T*>(h), static_cast<const T*>(a),
                                                            static_cast<const T*>(w_norm), eps, static_cast<const T*>(W),
                                                            static_cast<T*>(y), static_cast<T*>(h_out), static_cast<T*>(x_out), H,
                                                            N, rows_per_cta);
  } else {
    const int want = (N + warps - 1) / warps;
    const unsigned grid = static_cast<unsigned>(std::min(want, sms));  // one CTA per SM: the norm is made once per CTA
    k_norm_gemv<T><<<grid, GEMV_THREADS, row_bytes, s>>>(static_cast<const T*>(h), static_cast<const T*>(a),
                                                         static_cast<const T*>(w_norm), eps, static_cast<const T*>(W),
                                                         static_cast<T*>(y), static_cast<T*>(h_out), static_cast<T*>(x_out), H, N);
  }
  STX_LAUNCH_CHECK("k_norm_gemv");
  return STX_OK;
}

// Splits of the keys per head: enough CTAs to cover the SMs once, at most 8.
static int att_splits(int n_heads) { return std::max(1, std::min(8, (num_sms() + n_heads - 1) / n_heads)); }

}  // namespace stx

using namespace stx;

extern "C" {

int stx_attn_decode_workspace_bytes(int n_heads, int head_dim, int64_t* bytes_out) {
  STX_CHECK_ARG(bytes_out, "stx_attn_decode_workspace_bytes: null pointer");
  STX_CHECK_ARG(n_heads > 0 && n_heads <= 1024 && head_dim > 0, "stx_attn_decode_workspace_bytes: bad shape");
  *bytes_out = static_cast<int64_t>(ATT_COUNTER_BYTES + sizeof(float) * static_cast<size_t>(n_heads) * 8 * att_part_floats(head_dim));
  return STX_OK;
}

int stx_attn_decode(const void* qkv, const float* cos_table, const float* sin_table, const int64_t* pos_dev, void* k_cache,
                    void* v_cache, void* out, int n_heads, int n_kv_heads, int head_dim, int64_t max_len, int dtype,
                    void* workspace, void* stream) {
  STX_CHECK_ARG(qkv && cos_table && sin_table && pos_dev && k_cache && v_cache && out && workspace,
                "stx_attn_decode: null pointer");
  STX_CHECK_ARG(n_heads <= 1024, "stx_attn_decode: more than 1024 heads");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_attn_decode: bad dtype %d", dtype);
  STX_CHECK_ARG(head_dim == 64 || head_dim == 128 || head_dim == 256, "stx_attn_decode: head_dim %d is not 64, 128 or 256",
                head_dim);
  STX_CHECK_ARG(n_heads > 0 && n_kv_heads > 0 && n_heads % n_kv_heads == 0,
                "stx_attn_decode: %d query heads do not divide into %d key/value heads", n_heads, n_kv_heads);
  STX_CHECK_ARG(max_len > 0 && max_len <= 8192, "stx_attn_decode: max_len %lld outside 1..8192", static_cast<long long>(max_len));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int V = 16 / static_cast<int>(dtype_size(dtype));
  const int nsp = att_splits(n_heads);
  const size_t smem = sizeof(float) * (3 * head_dim + 32 + static_cast<size_t>(ATT_THREADS) * V +
                                       static_cast<size_t>((max_len + nsp - 1) / nsp + 1));
  const float scale = 1.0f / sqrtf(static_cast<float>(head_dim));
  const long long* pos = reinterpret_cast<const long long*>(pos_dev);
  const long long ml = max_len;
  static int use_cluster = -1;  // STX_ATTN_MERGE=workspace selects the merge through global memory (A/B measurements)
  if (use_cluster < 0) {
    const char* e = getenv("STX_ATTN_MERGE");
    use_cluster = (e && !strcmp(e, "workspace")) ? 0 : 1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_heads, nsp, 1);
  cfg.blockDim = dim3(ATT_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(nsp);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (use_cluster && nsp > 1) ? 1 : 0;
#define STX_ATT_LAUNCH_CL(T, HD, CL)                                                                                       \
  do {                                                                                                                     \
    if (smem > 48 * 1024)                                                                                                  \
      STX_CUDA(cudaFuncSetAttribute(k_attn_decode<T, HD, CL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));    \
    STX_CUDA(cudaLaunchKernelEx(&cfg, k_attn_decode<T, HD, CL>, static_cast<const T*>(qkv), cos_table, sin_table, pos,     \
                                static_cast<T*>(k_cache), static_cast<T*>(v_cache), static_cast<T*>(out), n_heads,         \
                                n_kv_heads, ml, scale, static_cast<unsigned char*>(workspace)));                           \
  } while (0)
#define STX_ATT_LAUNCH(T, HD)                                   \
  do {                                                          \
    if (cfg.numAttrs) STX_ATT_LAUNCH_CL(T, HD, true);           \
    else STX_ATT_LAUNCH_CL(T, HD, false);                       \
  } while (0)
#define STX_ATT_HD(T)                       \
  do {                                      \
    if (head_dim == 64) STX_ATT_LAUNCH(T, 64);        \
    else if (head_dim == 128) STX_ATT_LAUNCH(T, 128); \
    else STX_ATT_LAUNCH(T, 256);            \
  } while (0)
  switch (dtype) {
    case STX_F32: STX_ATT_HD(float); break;
    case STX_F16: STX_ATT_HD(__half); break;
    default: STX_ATT_HD(__nv_bfloat16); break;
  }
#undef STX_ATT_HD
#undef STX_ATT_LAUNCH
#undef STX_ATT_LAUNCH_CL
  STX_LAUNCH_CHECK("k_attn_decode");
  return STX_OK;
}

int stx_add_rmsnorm(const void* h, const void* a, const void* w, float eps, void* h_out, void* x_out, int64_t H, int dtype,
                    void* stream) {
  STX_CHECK_ARG(h && w && x_out, "stx_add_rmsnorm: null pointer");
  STX_CHECK_ARG(!a || h_out, "stx_add_rmsnorm: h_out is required when a is given");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_add_rmsnorm: bad dtype %d", dtype);
  STX_CHECK_ARG(H > 0 && H <= NORM_MAX_H, "stx_add_rmsnorm: H=%lld outside 1..%d", static_cast<long long>(H), NORM_MAX_H);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int Hi = static_cast<int>(H);
  switch (dtype) {
    case STX_F32:
      k_add_rmsnorm<float><<<1, NORM_THREADS, 0, s>>>(static_cast<const float*>(h), static_cast<const float*>(a),
                                                      static_cast<const float*>(w), eps, static_cast<float*>(h_out),
                                                      static_cast<float*>(x_out), Hi);
      break;
    case STX_F16:
      k_add_rmsnorm<__half><<<1, NORM_THREADS, 0, s>>>(static_cast<const __half*>(h), static_cast<const __half*>(a),
                                                       static_cast<const __half*>(w), eps, static_cast<__half*>(h_out),
                                                       static_cast<__half*>(x_out), Hi);
      break;
    default:
      k_add_rmsnorm<__nv_bfloat16><<<1, NORM_THREADS, 0, s>>>(
          static_cast<const __nv_bfloat16*>(h), static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(w), eps,
          static_cast<__nv_bfloat16*>(h_out), static_cast<__nv_bfloat16*>(x_out), Hi);
      break;
  }
  STX_LAUNCH_CHECK("k_add_rmsnorm");
  return STX_OK;
}

int stx_norm_gemv(const void* h, const void* a, const void* w_norm, float eps, const void* W, void* y, void* h_out,
                  void* x_out, int64_t H, int64_t N, int dtype, void* stream) {
  STX_CHECK_ARG(h && W && y, "stx_norm_gemv: null pointer");
  STX_CHECK_ARG(w_norm || (!a && !h_out && !x_out), "stx_norm_gemv: a, h_out and x_out need w_norm");
  STX_CHECK_ARG(!h_out || h_out != h, "stx_norm_gemv: h_out must not alias h");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_norm_gemv: bad dtype %d", dtype);
  const int64_t V = 16 / static_cast<int64_t>(dtype_size(dtype));
  STX_CHECK_ARG(H > 0 && H <= NORM_MAX_H && H % V == 0, "stx_norm_gemv: H=%lld must be a multiple of %lld, at most %d",
                static_cast<long long>(H), static_cast<long long>(V), NORM_MAX_H);
  STX_CHECK_ARG(N > 0 && N <= (1 << 30), "stx_norm_gemv: N=%lld out of range", static_cast<long long>(N));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int Hi = static_cast<int>(H), Ni = static_cast<int>(N);
  switch (dtype) {
    case STX_F32: return launch_norm_gemv<float>(h, a, w_norm, eps, W, y, h_out, x_out, Hi, Ni, s);
    case STX_F16: return launch_norm_gemv<__half>(h, a, w_norm, eps, W, y, h_out, x_out, Hi, Ni, s);
    default: return launch_norm_gemv<__nv_bfloat16>(h, a, w_norm, eps, W, y, h_out, x_out, Hi, Ni, s);
  }
}

}  // extern "C"
