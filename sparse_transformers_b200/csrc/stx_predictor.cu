// LoRA importance predictor -> per-row rule -> bit mask -> OR over the batch.
//
// Replaces FastLoRAProjection.forward (src/modeling_skip.py:52-53: scores = up(down(x)),
// two bias-free nn.Linear) and _compute_binary_mask (src/modeling_skip.py:204-214).
//
// Arithmetic contract (what makes the mask reproducible bit for bit by a CPU restatement):
//   t[b,k]  = round_dtype( sum_h x[b,h] * A[k,h] )      fp32 fused multiply-adds
//   s[b,i]  = round_dtype( sum_k t[b,k] * Bm[i,k] )     fp32 fused multiply-adds
// with a fixed summation order.  With V = 16 / sizeof(elem) elements per chunk:
//   t: NT = min(1024, ceil(H/V) rounded up to 32) partial sums; partial u adds chunks
//      u, u+NT, u+2NT, ... in ascending element order starting from +0.  Each group of 32
//      consecutive partials is combined by the butterfly p[l] += p[l^16]; ... ; p[l] += p[l^1];
//      the NT/32 group sums, padded with +0 to 32 values, are combined by the same butterfly.
//   s: 8 partial sums; partial g adds chunks g, g+8, ... likewise; butterfly over 4, 2, 1.
// Every thread issues all of its loads up front, so each kernel costs about one memory
// round trip.
#include "stx_common.cuh"

#include <algorithm>
#include <cmath>

namespace stx {

constexpr int PRED_BT = 8;  // batch rows accumulated per pass

__host__ __device__ inline int pred_t_threads(int H, int V) {
  const int nchunk = (H + V - 1) / V;
  const int nt = (nchunk + 31) / 32 * 32;
  return nt < 1024 ? nt : 1024;
}

// One block per (predictor row k, tile of PRED_BT batch rows); thread u owns chunks u, u+NT, ...
template <typename T>
__global__ void __launch_bounds__(1024)
k_pred_t(const T* __restrict__ x, const T* __restrict__ A, float* __restrict__ t_out, int B, int H, int r,
         uint32_t* __restrict__ zero_words, int n_zero) {
  constexpr int V = DT<T>::V;
  __shared__ float s_ws[32][PRED_BT];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const int k = blockIdx.x;
  const int nchunk = H / V;
  pdl_wait();
  pdl_launch_dependents();
  const T* arow = A + static_cast<size_t>(k) * H;
  // several batch groups OR their mask words together later: clear the words here, one kernel ahead
  if (zero_words && blockIdx.y == 0)
    for (int w = k * blockDim.x + tid; w < n_zero; w += r * blockDim.x) zero_words[w] = 0u;
  {
    const int b0 = blockIdx.y * PRED_BT;
    float acc[PRED_BT];
#pragma unroll
    for (int b = 0; b < PRED_BT; ++b) acc[b] = 0.f;
    const int nb = min(PRED_BT, B - b0);
    for (int c = tid; c < nchunk; c += blockDim.x) {
      float wa[V];
      Unpack<T>::run(ld_stream16(arow + c * V), wa);
#pragma unroll
      for (int b = 0; b < PRED_BT; ++b) {
        if (b < nb) {
          float xv[V];
          Unpack<T>::run(ld_cached16(x + static_cast<size_t>(b0 + b) * H + c * V), xv);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[b] = fmaf(xv[v], wa[v], acc[b]);
        }
      }
    }
#pragma unroll
    for (int b = 0; b < PRED_BT; ++b) {
      const float s = warp_sum_xor(acc[b]);
      if (lane == 0) s_ws[wid][b] = s;
    }
    __syncthreads();
    if (wid == 0) {
      for (int b = 0; b < nb; ++b) {
        const float s = warp_sum_xor(lane < nw ? s_ws[lane][b] : 0.f);
        if (lane == 0) t_out[static_cast<size_t>(b0 + b) * r + k] = DT<T>::round_f(s);
      }
    }
  }
}

// One block (256 threads) per (mask word, group of PRED_BT batch rows): 8 lanes cooperate on one
// neuron, 32 neurons per block.  Dynamic shared memory: the group's rows of t, fp32.  With more
// than one group the blocks OR their words into `bits` (zeroed by the launcher): the union over
// the batch does not depend on the order.
template <typename T>
__global__ void __launch_bounds__(256)
k_pred_scores(const float* __restrict__ t, const T* __restrict__ Bm, uint32_t* __restrict__ bits,
              T* __restrict__ scores_out, int B, int r, int I, float tau, int write_bits) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(16) float t_s[];
  __shared__ uint32_t s_nib[8];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int g = lane & 7;
  const int w = blockIdx.x;
  const int i = w * 32 + (tid >> 3);
  const bool i_ok = i < I;
  const bool vec_ok = (r % V) == 0 && ((reinterpret_cast<uintptr_t>(Bm) & 15) == 0);
  const int nchunk = (r + V - 1) / V;
  const T* brow = Bm + static_cast<size_t>(i_ok ? i : 0) * r;

  // weights first (they do not depend on the previous kernel), then the t tile
  constexpr int MAXC = 4;  // chunks held in registers per lane: r <= 8 * MAXC * V on the fast path
  float wv[MAXC][V];
  const bool in_regs = nchunk <= 8 * MAXC;
  if (in_regs) {
#pragma unroll
    for (int q = 0; q < MAXC; ++q) {
      const int c = g + 8 * q;
#pragma unroll
      for (int v = 0; v < V; ++v) wv[q][v] = 0.f;
      if (i_ok && c < nchunk) {
        if (vec_ok) {
          Unpack<T>::run(ld_stream16(brow + c * V), wv[q]);
        } else {
#pragma unroll
          for (int v = 0; v < V; ++v) wv[q][v] = (c * V + v < r) ? DT<T>::to_f(brow[c * V + v]) : 0.f;
        }
      }
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  const int bg0 = blockIdx.y * PRED_BT;          // first batch row of this block's group
  const int Bg = min(PRED_BT, B - bg0);           // rows in the group
  for (int k = tid; k < Bg * r; k += blockDim.x) t_s[k] = t[static_cast<size_t>(bg0) * r + k];
  __syncthreads();

  const float tau_r = DT<T>::round_f(tau);
  bool on = false;
  {
    const int b0 = 0;  // row index inside the group (t_s holds the group's rows only)
    float acc[PRED_BT];
#pragma unroll
    for (int b = 0; b < PRED_BT; ++b) acc[b] = 0.f;
    const int nb = Bg;
    if (i_ok) {
      if (in_regs) {
#pragma unroll
        for (int q = 0; q < MAXC; ++q) {
          const int c = g + 8 * q;
          if (c < nchunk) {
#pragma unroll
            for (int b = 0; b < PRED_BT; ++b) {
              if (b < nb) {
                const float* tb = t_s + (b0 + b) * r + c * V;
                if (vec_ok) {  // 16-byte shared-memory loads; the additions keep their order
#pragma unroll
                  for (int v4 = 0; v4 < V / 4; ++v4) {
                    const float4 tv = reinterpret_cast<const float4*>(tb)[v4];
                    acc[b] = fmaf(tv.x, wv[q][4 * v4], acc[b]);
                    acc[b] = fmaf(tv.y, wv[q][4 * v4 + 1], acc[b]);
                    acc[b] = fmaf(tv.z, wv[q][4 * v4 + 2], acc[b]);
                    acc[b] = fmaf(tv.w, wv[q][4 * v4 + 3], acc[b]);
                  }
                } else {
#pragma unroll
                  for (int v = 0; v < V; ++v)
                    if (c * V + v < r) acc[b] = fmaf(tb[v], wv[q][v], acc[b]);
                }
              }
            }
          }
        }
      } else {
        for (int c = g; c < nchunk; c += 8) {
          float wc[V];
          if (vec_ok) {
            Unpack<T>::run(ld_stream16(brow + c * V), wc);
          } else {
#pragma unroll
            for (int v = 0; v < V; ++v) wc[v] = (c * V + v < r) ? DT<T>::to_f(brow[c * V + v]) : 0.f;
          }
#pragma unroll
          for (int b = 0; b < PRED_BT; ++b) {
            if (b < nb) {
              const float* tb = t_s + (b0 + b) * r + c * V;
#pragma unroll
              for (int v = 0; v < V; ++v)
                if (vec_ok || c * V + v < r) acc[b] = fmaf(tb[v], wc[v], acc[b]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < PRED_BT; ++b) {
      float s = acc[b];
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if (b < nb) {
        const float sr = DT<T>::round_f(s);
        if (scores_out && g == 0 && i_ok) scores_out[static_cast<size_t>(bg0 + b) * I + i] = DT<T>::from_f(s);
        on = on || (sr >= tau_r);
      }
    }
  }
  const uint32_t bal = __ballot_sync(0xffffffffu, on && i_ok && g == 0);
  if (lane == 0) s_nib[wid] = (bal & 1u) | ((bal >> 7) & 2u) | ((bal >> 14) & 4u) | ((bal >> 21) & 8u);
  __syncthreads();
  if (write_bits && tid == 0) {
    uint32_t word = 0u;
#pragma unroll
    for (int q = 0; q < 8; ++q) word |= s_nib[q] << (4 * q);
    if (gridDim.y == 1)
      bits[w] = word;
    else if (word)
      atomicOr(&bits[w], word);
  }
}


// Row blocks of 16-bit weights under the threshold rule: the scores on the tensor pipe, the mask bit-exact.
//
// k_pred_scores fixes the order of the r multiply-adds of a score (eight partial sums per neuron, then a butterfly)
// because the mask has to match the reference bit for bit, and at 64 rows it is the longest kernel of a layer (117 M
// FMAs that wait for shared-memory operands).  Here a warp owns one mask word: two 16-neuron tiles against all rows,
// mma.sync m16n8k16 with fp32 accumulation - and next to every score s' the same product of the ABSOLUTE values,
// S = sum |t_k| |w_k|.  The exact score s (in the fixed order) and s' are both sums of the same exactly
// representable products, so |s' - s| <= r * 2^-20 * S with a wide margin, and the mask bit "round(s) >= tau" is
// "s above the midpoint m between tau and its predecessor in the model dtype".  Only a score within that bound
// of m is evaluated again in the fixed order (a few hundred of 64 x 14336); all others are decided by s'.
// Operand fragments are 16-byte chunks straight from global / shared memory: the k index of a product does not
// matter for a sum, so thread t takes the four k-pairs of its A and B fragments of two k16 steps from the same chunk.
template <typename T> struct MmaScores;
template <> struct MmaScores<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};
template <> struct MmaScores<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

constexpr int PSM_WARPS = 4;      // mask words per block
constexpr int PSM_MAX_SPANS = 8;  // r <= 256: a thread keeps 2 x r / 32 chunks of its two neurons in registers
constexpr int PSM_LIST = 64;      // scores of a warp that wait for their evaluation in the fixed order

// Dynamic shared memory: t in the model dtype, [Bpad][r + 8] (rows of 16 bytes more than r elements: the 16-byte
// fragment loads of eight rows then fall into different banks), Bpad = B rounded up to 8, rows >= B zero.
template <typename T>
__global__ void __launch_bounds__(PSM_WARPS * 32)
k_pred_scores_mma(const float* __restrict__ t, const T* __restrict__ Bm, uint32_t* __restrict__ bits, int B, int r, int I, float tau) {
  extern __shared__ __align__(16) unsigned char psm_raw[];
  T* t_s = reinterpret_cast<T*>(psm_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, tq = lane & 3;
  const int Bpad = (B + 7) & ~7, ts = r + 8, nspan = r >> 5;
  const int W = (I + 31) >> 5;
  const int w = blockIdx.x * PSM_WARPS + warp;
  const int i0 = w * 32;

  // weights first (they do not depend on the previous kernel): the chunks of this thread's four neurons
  uint4 alo[2][PSM_MAX_SPANS], ahi[2][PSM_MAX_SPANS];
  int ra[2], rb[2];
#pragma unroll
  for (int tt = 0; tt < 2; ++tt) {
    ra[tt] = i0 + 16 * tt + g;
    rb[tt] = ra[tt] + 8;
    const T* pa = Bm + static_cast<size_t>(min(ra[tt], I - 1)) * r;
    const T* pb = Bm + static_cast<size_t>(min(rb[tt], I - 1)) * r;
#pragma unroll
    for (int sp = 0; sp < PSM_MAX_SPANS; ++sp) {
      if (sp < nspan && w < W) {
        alo[tt][sp] = ld_stream16(pa + sp * 32 + tq * 8);
        ahi[tt][sp] = ld_stream16(pb + sp * 32 + tq * 8);
      } else {
        alo[tt][sp] = ahi[tt][sp] = make_uint4(0, 0, 0, 0);
      }
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  {
    // t holds values of the model dtype: the conversion is exact.  Four values per load, eight loads in flight.
    const int r4 = r >> 2, n4 = Bpad * r4;
    const float4* t4 = reinterpret_cast<const float4*>(t);
#pragma unroll 8
    for (int k = tid; k < n4; k += PSM_WARPS * 32) {
      const int b = k / r4, e = (k - b * r4) * 4;
      const float4 v = b < B ? __ldcg(t4 + k) : make_float4(0.f, 0.f, 0.f, 0.f);
      T* dst = t_s + b * ts + e;
      dst[0] = DT<T>::from_f(v.x);
      dst[1] = DT<T>::from_f(v.y);
      dst[2] = DT<T>::from_f(v.z);
      dst[3] = DT<T>::from_f(v.w);
    }
  }
  __syncthreads();
  if (w >= W) return;

  // "round(s) >= tau_r"  <=>  s above the midpoint between tau_r and its predecessor (ties: evaluated exactly)
  const float tau_r = DT<T>::round_f(tau);
  float mid;
  {
    T tv = DT<T>::from_f(tau_r);
    unsigned short u = *reinterpret_cast<unsigned short*>(&tv);
    if (tau_r > 0.f) u -= 1;
    else if (tau_r < 0.f) u += 1;
    else u = 0x8001;  // the largest value below zero
    const float pred = DT<T>::to_f(*reinterpret_cast<T*>(&u));
    mid = 0.5f * pred + 0.5f * tau_r;
  }
  const float eps_scale = static_cast<float>(r) * (1.0f / 1048576.0f);  // r * 2^-20

  // Scores too close to call wait in a list of the warp ((row << 8) | neuron inside the word) and are evaluated at
  // the end in the arithmetic order of k_pred_scores, four at a time: a group of eight lanes per score, lane g of
  // the group owns the chunks g, g + 8, ... of the r products, the eight partial sums meet by butterfly (xor 4, 2,
  // 1).  A neuron's bit is the OR over the rows, so a result only has to reach the word.
  __shared__ int s_unc[PSM_WARPS][PSM_LIST];
  int* unc = s_unc[warp];
  int n_unc = 0;
  uint32_t word = 0u;
  auto flush = [&]() {
    for (int k0 = 0; k0 < n_unc; k0 += 4) {
      const int grp = lane >> 3, gl = lane & 7;
      const bool have = k0 + grp < n_unc;
      const int e = have ? unc[k0 + grp] : 0;
      const int bq = e >> 8, il = e & 0xff;
      float acc = 0.f;
      if (have) {
        const T* wrow = Bm + static_cast<size_t>(i0 + il) * r;
        const T* tr = t_s + bq * ts;
        for (int c = gl; c < (r >> 3); c += 8) {
          float wv[8], tv[8];
          Unpack<T>::run(ld_stream16(wrow + c * 8), wv);
          Unpack<T>::run(*reinterpret_cast<const uint4*>(tr + c * 8), tv);
#pragma unroll
          for (int v = 0; v < 8; ++v) acc = fmaf(tv[v], wv[v], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      const bool res = have && DT<T>::round_f(acc) >= tau_r;
      const uint32_t rb4 = __ballot_sync(0xffffffffu, res && gl == 0);  // bits 0, 8, 16, 24: the four results
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int eq = __shfl_sync(0xffffffffu, e, q * 8);
        if ((rb4 >> (8 * q)) & 1u) word |= 1u << (eq & 0xff);
      }
    }
    n_unc = 0;
    __syncwarp();
  };

#pragma unroll
  for (int tt = 0; tt < 2; ++tt) {
    bool on_a = false, on_b = false;  // neuron ra / rb active for some row
    for (int cg0 = 0; cg0 < Bpad; cg0 += 16) {  // two groups of eight rows in flight
      float d[2][4], da[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < 4; ++j) d[h][j] = da[h][j] = 0.f;
      const bool two = cg0 + 8 < Bpad;
      const T* trow0 = t_s + (cg0 + g) * ts + tq * 8;
      const T* trow1 = t_s + ((two ? cg0 + 8 : cg0) + g) * ts + tq * 8;
#pragma unroll
      for (int sp = 0; sp < PSM_MAX_SPANS; ++sp) {
        if (sp < nspan) {
          const uint4 lo = alo[tt][sp], hi = ahi[tt][sp];
          const uint4 tb0 = *reinterpret_cast<const uint4*>(trow0 + sp * 32);
          const uint4 tb1 = *reinterpret_cast<const uint4*>(trow1 + sp * 32);
          constexpr uint32_t M = 0x7fff7fffu;
          MmaScores<T>::run(d[0], lo.x, hi.x, lo.y, hi.y, tb0.x, tb0.y);
          MmaScores<T>::run(d[1], lo.x, hi.x, lo.y, hi.y, tb1.x, tb1.y);
          MmaScores<T>::run(da[0], lo.x & M, hi.x & M, lo.y & M, hi.y & M, tb0.x & M, tb0.y & M);
          MmaScores<T>::run(da[1], lo.x & M, hi.x & M, lo.y & M, hi.y & M, tb1.x & M, tb1.y & M);
          MmaScores<T>::run(d[0], lo.z, hi.z, lo.w, hi.w, tb0.z, tb0.w);
          MmaScores<T>::run(d[1], lo.z, hi.z, lo.w, hi.w, tb1.z, tb1.w);
          MmaScores<T>::run(da[0], lo.z & M, hi.z & M, lo.w & M, hi.w & M, tb0.z & M, tb0.w & M);
          MmaScores<T>::run(da[1], lo.z & M, hi.z & M, lo.w & M, hi.w & M, tb1.z & M, tb1.w & M);
        }
      }
      // d[h][0], d[h][1]: neuron ra, rows cg + 2 tq, + 1;  d[h][2], d[h][3]: neuron rb, same rows
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int cg = cg0 + 8 * h;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int b = cg + 2 * tq + (j & 1);
          const int i = (j < 2) ? ra[tt] : rb[tt];
          const bool valid = (h == 0 || two) && b < B && i < I;
          const float eps = eps_scale * da[h][j];
          const bool on = valid && d[h][j] > mid + eps;
          const bool close = valid && !on && !(d[h][j] < mid - eps);
          const uint32_t um = __ballot_sync(0xffffffffu, close);
          if (um) {
            if (n_unc + __popc(um) > PSM_LIST) flush();
            if (close) unc[n_unc + __popc(um & ((1u << lane) - 1u))] = (b << 8) | (i - i0);
            n_unc += __popc(um);
            __syncwarp();
          }
          if (j < 2) on_a = on_a || on;
          else on_b = on_b || on;
        }
      }
    }
    // the four threads of a quad hold the rows of the same two neurons
    const uint32_t ba = __ballot_sync(0xffffffffu, on_a), bb = __ballot_sync(0xffffffffu, on_b);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if ((ba >> (4 * q)) & 0xfu) word |= 1u << (16 * tt + q);
      if ((bb >> (4 * q)) & 0xfu) word |= 1u << (16 * tt + 8 + q);
    }
  }
  flush();
  if (lane == 0) bits[w] = word;
}

template <typename T>
static int launch_scores_mma(const float* t_scratch, const void* Bm, uint32_t* bits, int64_t B, int64_t r, int64_t I, float tau,
                             size_t smem, cudaStream_t s) {
  const int64_t W = (I + 31) / 32;
  STX_CUDA(launch_pdl(k_pred_scores_mma<T>, dim3(static_cast<unsigned>((W + PSM_WARPS - 1) / PSM_WARPS)), dim3(PSM_WARPS * 32), smem, s,
                      t_scratch, static_cast<const T*>(Bm), bits, static_cast<int>(B), static_cast<int>(r), static_cast<int>(I), tau));
  return STX_OK;
}
template <>
int launch_scores_mma<float>(const float*, const void*, uint32_t*, int64_t, int64_t, int64_t, float, size_t, cudaStream_t) {
  return STX_ERR_UNSUPPORTED;
}

template <typename T>
static int launch_predict(const void* x, int64_t B, int64_t H, const void* A, int64_t r, const void* Bm,
                          int64_t I, float tau, uint32_t* bits, void* scores_out, float* t_scratch,
                          int write_bits, unsigned parts, cudaStream_t s) {
  const unsigned groups = static_cast<unsigned>((B + PRED_BT - 1) / PRED_BT);
  if (parts & 1u)
    STX_CUDA(launch_pdl(k_pred_t<T>, dim3(static_cast<unsigned>(r), groups), dim3(pred_t_threads(static_cast<int>(H), DT<T>::V)),
                        0, s, static_cast<const T*>(x), static_cast<const T*>(A), t_scratch, static_cast<int>(B),
                        static_cast<int>(H), static_cast<int>(r), (groups > 1 && write_bits && (parts & 2u)) ? bits : nullptr,
                        static_cast<int>((I + 31) / 32)));
  const int64_t W = (I + 31) / 32;
  const size_t smem = static_cast<size_t>(std::min<int64_t>(B, PRED_BT)) * r * sizeof(float);
  // row blocks of 16-bit weights under the threshold rule: scores on the tensor pipe (the mask stays bit-exact)
  const size_t smem_mma = static_cast<size_t>((B + 7) / 8 * 8) * (r + 8) * sizeof(T);
  if ((parts & 2u) && sizeof(T) == 2 && write_bits && !scores_out && B >= 9 && r % 32 == 0 && r <= 32 * PSM_MAX_SPANS &&
      smem_mma <= 48 * 1024 && std::isfinite(tau) && (reinterpret_cast<uintptr_t>(Bm) & 15) == 0)
    return launch_scores_mma<T>(t_scratch, Bm, bits, B, r, I, tau, smem_mma, s);
  if ((parts & 2u) && !(parts & 1u) && groups > 1 && write_bits) STX_CUDA(cudaMemsetAsync(bits, 0, W * sizeof(uint32_t), s));
  if (parts & 2u)
  STX_CUDA(launch_pdl(k_pred_scores<T>, dim3(static_cast<unsigned>(W), groups), dim3(256), smem, s, t_scratch,
                      static_cast<const T*>(Bm), bits, static_cast<T*>(scores_out), static_cast<int>(B),
                      static_cast<int>(r), static_cast<int>(I), tau, write_bits));
  
  return STX_OK;
}

// Implemented in stx_select.cu: per-row rules that need the whole score row.
int mask_from_scores(const void* scores, int64_t B, int64_t I, int dtype, int method, float param,
                     uint32_t* bits_out, void* scratch, cudaStream_t s);

// parts: bit 0 = t = A x, bit 1 = scores, threshold/selection and mask
int predict_mask(const void* x, int64_t B, int64_t H, const void* A, int64_t r, const void* Bm, int64_t I,
                 int dtype, int method, float param, uint32_t* bits, void* scores_out, void* scratch, unsigned parts,
                 cudaStream_t s) {
  float* t_scratch = static_cast<float*>(scratch);
  const int write_bits = method == STX_MASK_THRESHOLD ? 1 : 0;
  int rc;
  switch (dtype) {
    case STX_F32:
      rc = launch_predict<float>(x, B, H, A, r, Bm, I, param, bits, scores_out, t_scratch, write_bits, parts, s);
      break;
    case STX_F16:
      rc = launch_predict<__half>(x, B, H, A, r, Bm, I, param, bits, scores_out, t_scratch, write_bits, parts, s);
      break;
    default:
      rc = launch_predict<__nv_bfloat16>(x, B, H, A, r, Bm, I, param, bits, scores_out, t_scratch, write_bits, parts, s);
      break;
  }
  if (rc != STX_OK || method == STX_MASK_THRESHOLD || !(parts & 2u)) return rc;
  void* sel_scratch = static_cast<char*>(scratch) + align_up(static_cast<size_t>(B) * r * sizeof(float), 256);
  return mask_from_scores(scores_out, B, I, dtype, method, param, bits, sel_scratch, s);
}

}  // namespace stx

using namespace stx;

extern "C" {

int stx_predict_scratch_bytes(int64_t B, int64_t I, int64_t r, size_t* bytes_out) {
  STX_CHECK_ARG(bytes_out && B > 0 && I > 0 && r > 0, "stx_predict_scratch_bytes: bad argument");
  // t [B,r] fp32, then per-row selection scratch (B x 4 floats + B x ceil(I/32) words)
  *bytes_out = align_up(static_cast<size_t>(B) * r * sizeof(float), 256) +
               align_up(static_cast<size_t>(B) * (16 + ((I + 31) / 32) * sizeof(uint32_t)), 256);
  return STX_OK;
}

int stx_predict_mask(const void* x, int64_t B, int64_t H, const void* A, int64_t r, const void* Bm, int64_t I,
                     int dtype, int method, float param, uint32_t* mask_bits_out, void* scores_out, void* scratch,
                     void* stream) {
  STX_CHECK_ARG(x && A && Bm && mask_bits_out && scratch, "stx_predict_mask: null pointer");
  STX_CHECK_ARG(B > 0 && H > 0 && r > 0 && I > 0, "stx_predict_mask: sizes must be positive");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_predict_mask: bad dtype %d", dtype);
  STX_CHECK_ARG(method >= STX_MASK_THRESHOLD && method <= STX_MASK_STATISTICAL, "stx_predict_mask: bad method %d",
                method);
  STX_CHECK_ARG(method == STX_MASK_THRESHOLD || scores_out, "stx_predict_mask: this rule needs scores_out");
  if ((H * dtype_size(dtype)) % 16 != 0 || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(A) & 15)) {
    set_error("stx_predict_mask: x and A rows must be 16-byte aligned (H*elem %% 16 == 0)");
    return STX_ERR_UNSUPPORTED;
  }
  if (static_cast<size_t>(std::min<int64_t>(B, 8)) * r * sizeof(float) > 48 * 1024) {
    set_error("stx_predict_mask: min(B,8)*r=%lld exceeds the shared-memory tile (12288 values)",
              static_cast<long long>(std::min<int64_t>(B, 8) * r));
    return STX_ERR_TOO_LARGE;
  }
  return predict_mask(x, B, H, A, r, Bm, I, dtype, method, param, mask_bits_out, scores_out, scratch, 3u,
                      static_cast<cudaStream_t>(stream));
}

}  // extern "C"
