// One decode token (a single row) through a whole stack of sparse layers in ONE persistent kernel.
//
// The per-layer chain  t = A x  ->  scores, mask  ->  gather + gated MLP  ->  sum of partial outputs
// (FastLoRAProjection.forward + _compute_binary_mask + SkipMLP._forward_sparse_weight_cache,
// src/modeling_skip.py:52-53,204-214,114-117) costs three dependent launches per layer when every
// link is its own kernel, and each dependent launch boundary is 2.4-3.1 us on this GPU, more than
// most links take to compute.  Here the layers are a loop inside one kernel of one CTA per SM and
// the links are separated by grid-wide barriers on counters in global memory (about 1.2 us each).
//
// Work split.  The CTAs run as thread-block clusters of two ("pairs").  CTA c owns the mask bytes
// c, c + G, c + 2G, ... (8 neurons each), exactly like k_mlp_b1: it computes the predictor scores
// of its own neurons, in the arithmetic order of k_pred_scores, and writes their mask bytes.  The
// two CTAs of a pair then swap their lists of active neurons through distributed shared memory and
// BOTH work on every neuron of the pair, each on one half of the hidden dimension:
//   phase 1   CTA `rank` fetches columns [rank*H/2, (rank+1)*H/2) of the neuron's gate and up rows
//             (bulk copies global -> shared, mbarrier completion), forms the two half dot products
//             with its half of x and stores them in both CTAs' shared memory;
//   cluster barrier; both CTAs now hold every half sum and compute a = act(g0+g1) * (u0+u1);
//   phase 2   thread t adds a * down[neuron][its 16-byte chunk of the CTA's column half] over the
//             pair's neurons in list order (registers).
// Inside a pair the work is balanced by construction (each CTA streams exactly half of every row),
// and the two CTAs produce DISJOINT column halves of the pair's partial output, so no pair-level
// reduction is needed: the pair writes one fp32 vector [H] and the layer's output is the sum of
// the G/2 pair vectors in ascending pair order (deterministic, no atomics).
//
// Per layer and CTA:
//   [CTAs c < r]  t[c] = round(A[c] . x)       A's row waits in registers since the previous layer
//   barrier A     (r arrivals)                  every CTA then reads t (r floats)
//   scores -> mask bytes -> own list -> swap with the partner (cluster barrier)
//   bulk copies of up to S neurons x 3 half rows; phase 1; cluster barrier; phase 2; further
//   rounds of S neurons when the pair has more
//   pair partial -> global;  barrier B (G arrivals)
//   sum of the pair partials for the CTA's few output columns -> out[l]   (overlaps the next
//   layer's t, which does not depend on it: every layer of a stack reads the same x; with
//   `strict` a third barrier C orders that sum before the next layer's first instruction, the
//   order a model that feeds a layer's output forward would need)
// Weights of the next layer that the front end needs (a row of A, the CTA's slice of the predictor's
// up matrix) are loaded into registers one layer ahead: they do not depend on data.
//
// Every wait is bounded.  A grid barrier that expires sets DEV_TIMEOUT in the layer's status word
// and the CTA stops waiting on grid barriers for the rest of the launch (it falls through them), so
// the kernel always terminates; the cluster barriers are hardware barriers between two CTAs whose
// control flow never diverges.  The counters only grow; a launch derives its targets from a
// generation word that CTA 0 advances at the end, so a replayed CUDA graph needs no reset.
#include "stx_common.cuh"
#include "stx_tma.cuh"
#include "stx_stack_b1.cuh"

#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace cg = cooperative_groups;

namespace stx {

constexpr int SB1_THREADS = 512;
constexpr int SB1_MAX_SLOTS = 32;
constexpr int SB1_XL_STRIDE = 80;  // ints per rank in the list exchange: [0] count, [8..8+64) ids
constexpr int SB1_OFF_AS = 512;     // a_s [32] floats
constexpr int SB1_OFF_PD = 640;     // half sums [2 buffers][2 ranks][32 slots][2 quarters] float2
constexpr int SB1_OFF_XL = 2688;    // list exchange [2 ranks][SB1_XL_STRIDE] ints
constexpr int SB1_OFF_T = 3328;     // t of the layer in the score layout, <= 512 bytes
constexpr int SB1_HEADER = 3840;    // x follows, then the slots
constexpr uint32_t SB1_GRID_WAIT_LIMIT = 1u << 21;

// sync words (uint32): [0] generation, [32] barrier A count, [64] barrier B count, [96] barrier C count
constexpr int SB1_SYNC_GEN = 0, SB1_SYNC_A = 32, SB1_SYNC_B = 64, SB1_SYNC_C = 96;

__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until the counter has reached `target` (wrap-safe).  False when the limit expired.
__device__ __forceinline__ bool grid_wait(const uint32_t* ctr, uint32_t target) {
  for (uint32_t it = 0; it < SB1_GRID_WAIT_LIMIT; ++it) {
    if (static_cast<int32_t>(ld_acquire_u32(ctr) - target) >= 0) return true;
  }
  return false;
}

template <typename T>
__global__ void __launch_bounds__(SB1_THREADS, 1) k_stack_b1(const __grid_constant__ StackB1Args q) {
  constexpr int V = DT<T>::V;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_ws[32];
  __shared__ uint32_t s_nib[16];
  __shared__ uint8_t s_bytes[8];
  __shared__ int s_dead;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, c = blockIdx.x;
  const int rank = static_cast<int>(cluster.block_rank());
  const int pair = c >> 1, npairs = G >> 1;
  const int H = q.H, I = q.I, r = q.r, L = q.L, S = q.nslot;
  const int nchunk = H / V, hchunk = nchunk >> 1, qchunk = hchunk >> 1;
  const uint32_t hb = static_cast<uint32_t>(H / 2) * sizeof(T);  // bytes of a half row
  const int ngu = q.has_gate ? 2 : 1;
  const uint32_t slot_bytes = hb * (ngu + 1);

  uint64_t* bar_gu = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar_d = bar_gu + SB1_MAX_SLOTS;
  float* a_s = reinterpret_cast<float*>(smem + SB1_OFF_AS);
  float2* pd = reinterpret_cast<float2*>(smem + SB1_OFF_PD);
  int* xl = reinterpret_cast<int*>(smem + SB1_OFF_XL);
  float* t_s = reinterpret_cast<float*>(smem + SB1_OFF_T);
  T* x_s = reinterpret_cast<T*>(smem + SB1_HEADER);
  unsigned char* slots = smem + SB1_HEADER + (static_cast<size_t>(H) * sizeof(T) + 127) / 128 * 128;
  float2* pd_remote = cluster.map_shared_rank(pd, rank ^ 1);
  int* xl_remote = cluster.map_shared_rank(xl, rank ^ 1);

  if (tid == 0) {
    for (int w = 0; w < SB1_MAX_SLOTS; ++w) {
      mbar_init(&bar_gu[w], 1);
      mbar_init(&bar_d[w], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_dead = 0;
  }
  {
    const uint4* xg = reinterpret_cast<const uint4*>(q.x);
    uint4* xs4 = reinterpret_cast<uint4*>(x_s);
    for (int i = tid; i < nchunk; i += SB1_THREADS) xs4[i] = __ldcg(xg + i);
  }
  const uint32_t gen = __ldcg(q.sync + SB1_SYNC_GEN);
  cluster.sync();  // barriers initialised, x staged, the partner is running (its shared memory may be written)

  // ---- score geometry (one pass of 8 mask bytes per CTA; the launcher guarantees nby <= 8)
  const int rch = r / V, nc4 = (rch + 7) >> 3;  // nc4 <= 2
  const int NBY = (I + 7) >> 3;
  const int nby = NBY > c ? (NBY - 1 - c) / G + 1 : 0;
  const int g8 = tid & 7;
  const int kk = tid >> 6;                              // mask byte of the CTA this thread works on
  const int my_n = 8 * (c + G * kk) + ((tid >> 3) & 7);  // its neuron
  const bool n_ok = kk < nby && my_n < I;
  const int NT = min(1024, (nchunk + 31) / 32 * 32);    // virtual threads of the t reduction (as k_pred_t's block)

  // weights one layer ahead: a row of A (CTAs c < r), the CTA's slice of the predictor's up matrix
  uint4 areg[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  uint4 wraw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  auto load_a = [&](int l) {
    if (c < r) {
      const T* arow = static_cast<const T*>(q.layer[l].A) + static_cast<size_t>(c) * H;
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int v = tid + k * SB1_THREADS;
        if (v < nchunk) areg[k] = ld_stream16(arow + v * V);
      }
    }
  };
  auto load_w = [&](int l) {
    const T* Bm = static_cast<const T*>(q.layer[l].Bm);
#pragma unroll
    for (int c4 = 0; c4 < 2; ++c4) {
      const int ch = g8 + 8 * c4;
      wraw[c4] = make_uint4(0, 0, 0, 0);
      if (n_ok && ch < rch) wraw[c4] = ld_stream16(Bm + static_cast<size_t>(my_n) * r + ch * V);
    }
  };
  // t[c] of layer l in the summation order of k_pred_t (virtual thread v = one 16-byte chunk; butterfly
  // over each group of 32, then over the group sums), published with a release on barrier A's counter
  auto do_t = [&](int l) {
    if (c < r) {  // CTA-uniform
      float acc[2] = {0.f, 0.f};
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const int v = tid + k * SB1_THREADS;
        if (v < nchunk) {
          float wa[V], xv[V];
          Unpack<T>::run(areg[k], wa);
          Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + v * V), xv);
#pragma unroll
          for (int e = 0; e < V; ++e) acc[k] = fmaf(xv[e], wa[e], acc[k]);
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float s = warp_sum_xor(acc[k]);
        const int grp = warp + k * (SB1_THREADS / 32);
        if (lane == 0 && grp * 32 < NT) s_ws[grp] = s;
      }
      __syncthreads();
      if (warp == 0) {
        const float s = warp_sum_xor(lane < NT / 32 ? s_ws[lane] : 0.f);
        if (lane == 0) {
          q.t_buf[static_cast<size_t>(l) * r + c] = DT<T>::round_f(s);
          red_release_add(q.sync + SB1_SYNC_A, 1u);
        }
      }
      if (l + 1 < L) load_a(l + 1);
    }
  };
  // sum of the pair partials of layer l for this CTA's output columns, ascending pair order
  const int ncol4 = H / 4;
  const int cpc = (ncol4 + G - 1) / G;
  const int col0 = c * cpc;
  const int ncols = max(0, min(cpc, ncol4 - col0));
  auto do_reduce = [&](int l) {
    float4* s_red = reinterpret_cast<float4*>(slots);  // the slots are idle between two layers
    const float* part = q.partial + static_cast<size_t>(l & 1) * npairs * H;
    for (int i = tid; i < npairs * ncols; i += SB1_THREADS) {
      const int p = i / ncols, qq = i - p * ncols;
      s_red[p * cpc + qq] = __ldcg(reinterpret_cast<const float4*>(part + static_cast<size_t>(p) * H) + col0 + qq);
    }
    __syncthreads();
    if (tid < ncols * 4) {
      const int col = tid >> 2, comp = tid & 3;
      float s = 0.f;
      for (int p = 0; p < npairs; ++p) s += reinterpret_cast<const float*>(&s_red[p * cpc + col])[comp];
      static_cast<T*>(q.layer[l].out)[(col0 + col) * 4 + comp] = DT<T>::from_f(s);
    }
    __syncthreads();
  };
  auto grid_barrier_wait = [&](int word, uint32_t target, int l) {
    if (tid == 0 && !s_dead) {
      if (!grid_wait(q.sync + word, target)) {
        s_dead = 1;
        if (q.layer[l].status) atomicOr(q.layer[l].status, DEV_TIMEOUT);
      }
    }
    __syncthreads();
  };

  load_a(0);
  load_w(0);
  do_t(0);

  uint32_t ph_gu = 0u, ph_d = 0u;  // mbarrier phase parity per slot (same in every thread)
  bool timed_out = false;
  const int xoff = rank * (H / 2);  // first column of this CTA's half

  for (int l = 0; l < L; ++l) {
    const StackLayerDesc& ld = q.layer[l];
    const uint32_t seq = gen * static_cast<uint32_t>(L) + static_cast<uint32_t>(l) + 1u;
    // ---- barrier A: t of this layer is complete
    grid_barrier_wait(SB1_SYNC_A, seq * static_cast<uint32_t>(r), l);
    if (tid < r) {
      const int e = tid, ch = e / V, v = e - ch * V;
      t_s[(((ch >> 3) * (V / 4) + (v >> 2)) * 8 + (ch & 7)) * 4 + (v & 3)] = __ldcg(q.t_buf + static_cast<size_t>(l) * r + e);
    }
    __syncthreads();

    // ---- scores of the CTA's own neurons (arithmetic of k_pred_scores), mask bytes, own list
    {
      const float tau_r = DT<T>::round_f(ld.tau);
      float sc = 0.f;
#pragma unroll
      for (int c4 = 0; c4 < 2; ++c4) {
        const int ch = g8 + 8 * c4;
        if (c4 < nc4 && ch < rch) {
          float w[V];
          Unpack<T>::run(wraw[c4], w);
          const float4* tb = reinterpret_cast<const float4*>(t_s) + (c4 * (V / 4)) * 8 + g8;
#pragma unroll
          for (int v4 = 0; v4 < V / 4; ++v4) {
            const float4 tv = tb[v4 * 8];
            sc = fmaf(tv.x, w[4 * v4], sc);
            sc = fmaf(tv.y, w[4 * v4 + 1], sc);
            sc = fmaf(tv.z, w[4 * v4 + 2], sc);
            sc = fmaf(tv.w, w[4 * v4 + 3], sc);
          }
        }
      }
      sc += __shfl_xor_sync(0xffffffffu, sc, 4);
      sc += __shfl_xor_sync(0xffffffffu, sc, 2);
      sc += __shfl_xor_sync(0xffffffffu, sc, 1);
      const bool on = n_ok && DT<T>::round_f(sc) >= tau_r;
      const uint32_t bal = __ballot_sync(0xffffffffu, on && g8 == 0);
      if (lane == 0) s_nib[warp] = (bal & 1u) | ((bal >> 7) & 2u) | ((bal >> 14) & 4u) | ((bal >> 21) & 8u);
      if (l + 1 < L) load_w(l + 1);  // this register set is free again
      __syncthreads();
      if (warp == 0) {
        // lane k < 8: mask byte k of the CTA; the CTA's active neurons in ascending order go to both
        // CTAs of the pair (own shared memory and the partner's)
        uint32_t byte = 0u;
        if (lane < 8 && lane < nby) {
          byte = s_nib[2 * lane] | (s_nib[2 * lane + 1] << 4);
          reinterpret_cast<uint8_t*>(ld.bits)[c + G * lane] = static_cast<uint8_t>(byte);
        }
        const int cnt = __popc(byte);
        int inc = cnt;
#pragma unroll
        for (int off = 1; off < 8; off <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, inc, off);
          if (lane >= off) inc += v;
        }
        int pos = inc - cnt;
        int* mine = xl + rank * SB1_XL_STRIDE;
        int* theirs = xl_remote + rank * SB1_XL_STRIDE;
        while (byte) {
          const int n = 8 * (c + G * lane) + __ffs(byte) - 1;
          byte &= byte - 1;
          mine[8 + pos] = n;
          theirs[8 + pos] = n;
          ++pos;
        }
        const int total = __shfl_sync(0xffffffffu, inc, 7);
        if (lane == 0) {
          mine[0] = total;
          theirs[0] = total;
        }
      }
    }
    cluster.sync();  // both lists are in both CTAs
    const int n0 = xl[0], n1 = xl[SB1_XL_STRIDE];
    const int n = n0 + n1;
    auto neuron = [&](int j) { return j < n0 ? xl[8 + j] : xl[SB1_XL_STRIDE + 8 + (j - n0)]; };

    const char* gsrc = static_cast<const char*>(ld.gate) + static_cast<size_t>(xoff) * sizeof(T);
    const char* usrc = static_cast<const char*>(ld.up) + static_cast<size_t>(xoff) * sizeof(T);
    const char* dsrc = static_cast<const char*>(ld.down) + static_cast<size_t>(xoff) * sizeof(T);
    const size_t row_bytes = static_cast<size_t>(H) * sizeof(T);
    // slot s <- neuron j: gate and up halves on bar_gu[s], the down half on bar_d[s]
    auto issue_gu = [&](int s, int j) {
      unsigned char* dst = slots + static_cast<size_t>(s) * slot_bytes;
      const size_t off = static_cast<size_t>(neuron(j)) * row_bytes;
      mbar_expect_tx(&bar_gu[s], hb * ngu);
      if (q.has_gate) bulk_load(dst, gsrc + off, hb, &bar_gu[s]);
      bulk_load(dst + (q.has_gate ? hb : 0), usrc + off, hb, &bar_gu[s]);
    };
    auto issue_d = [&](int s, int j) {
      unsigned char* dst = slots + static_cast<size_t>(s) * slot_bytes + static_cast<size_t>(ngu) * hb;
      mbar_expect_tx(&bar_d[s], hb);
      bulk_load(dst, dsrc + static_cast<size_t>(neuron(j)) * row_bytes, hb, &bar_d[s]);
    };
    if (lane == 0) {
      // the slots were last touched through the generic proxy (phase 2, the staging of the output sum)
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      for (int s = warp; s < min(S, n); s += SB1_THREADS / 32) {
        issue_gu(s, s);
        issue_d(s, s);
      }
    }

    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;

    const int nrounds = (n + S - 1) / S;
    for (int rd = 0; rd < nrounds; ++rd) {
      const int base = rd * S;
      const int nvalid = min(S, n - base);
      float2* pd_mine = pd + (rd & 1) * (2 * SB1_MAX_SLOTS * 2);
      float2* pd_theirs = pd_remote + (rd & 1) * (2 * SB1_MAX_SLOTS * 2);
      // ---- phase 1: a task is one quarter row pair (slot, quarter): tasks in slot order over the warps
      for (int task = warp; task < 2 * nvalid; task += SB1_THREADS / 32) {
        const int s = task >> 1, sub = task & 1;
        if (!mbar_wait_bounded(&bar_gu[s], (ph_gu >> s) & 1u)) timed_out = true;
        const unsigned char* sl = slots + static_cast<size_t>(s) * slot_bytes;
        const T* grow = reinterpret_cast<const T*>(sl) + sub * (H / 4);
        const T* urow = reinterpret_cast<const T*>(sl + (q.has_gate ? hb : 0)) + sub * (H / 4);
        const T* xrow = x_s + xoff + sub * (H / 4);
        float ag = 0.f, au = 0.f;
        for (int ch = lane; ch < qchunk; ch += 32) {
          float wu[V], wg[V], xv[V];
          Unpack<T>::run(*reinterpret_cast<const uint4*>(urow + ch * V), wu);
          Unpack<T>::run(*reinterpret_cast<const uint4*>(xrow + ch * V), xv);
          float su = 0.f, sg = 0.f;
          if (q.has_gate) {
            Unpack<T>::run(*reinterpret_cast<const uint4*>(grow + ch * V), wg);
#pragma unroll
            for (int v = 0; v < V; ++v) sg = fmaf(xv[v], wg[v], sg);
          }
#pragma unroll
          for (int v = 0; v < V; ++v) su = fmaf(xv[v], wu[v], su);
          au += su;
          ag += sg;
        }
        const float u = warp_sum_xor(au);
        const float gs = q.has_gate ? warp_sum_xor(ag) : 0.f;
        if (lane == 0) {
          const int idx = (rank * SB1_MAX_SLOTS + s) * 2 + sub;
          pd_mine[idx] = make_float2(gs, u);
          pd_theirs[idx] = make_float2(gs, u);
        }
      }
      cluster.sync();  // every half sum of the round is in both CTAs; the gate/up parts of the slots are free
      if (tid < nvalid) {
        const float2 p00 = pd_mine[(0 * SB1_MAX_SLOTS + tid) * 2], p01 = pd_mine[(0 * SB1_MAX_SLOTS + tid) * 2 + 1];
        const float2 p10 = pd_mine[(1 * SB1_MAX_SLOTS + tid) * 2], p11 = pd_mine[(1 * SB1_MAX_SLOTS + tid) * 2 + 1];
        const float gsum = (p00.x + p01.x) + (p10.x + p11.x);
        const float usum = (p00.y + p01.y) + (p10.y + p11.y);
        a_s[tid] = q.has_gate ? apply_act(ld.act, gsum) * usum : apply_act(ld.act, usum);
      }
      if (lane == 0 && base + S < n) {  // next round's gate/up halves into the freed parts
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        for (int s = warp; s < min(S, n - base - S); s += SB1_THREADS / 32) issue_gu(s, base + S + s);
      }
      __syncthreads();  // a_s complete
      // ---- phase 2: thread t < hchunk owns one 16-byte chunk of the CTA's column half
      if (tid < hchunk) {
        for (int s = 0; s < nvalid; ++s) {
          if (!mbar_wait_bounded(&bar_d[s], (ph_d >> s) & 1u)) timed_out = true;
          const float a = a_s[s];
          const T* drow = reinterpret_cast<const T*>(slots + static_cast<size_t>(s) * slot_bytes + static_cast<size_t>(ngu) * hb);
          float wd[V];
          Unpack<T>::run(*reinterpret_cast<const uint4*>(drow + tid * V), wd);
#pragma unroll
          for (int v = 0; v < V; ++v) acc[v] = fmaf(a, wd[v], acc[v]);
        }
      }
      const uint32_t used = nvalid >= 32 ? 0xffffffffu : ((1u << nvalid) - 1u);
      ph_gu ^= used;
      ph_d ^= used;
      if (rd + 1 < nrounds) {
        __syncthreads();  // every thread is done with a_s and the down halves of this round
        if (lane == 0) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          for (int s = warp; s < min(S, n - base - S); s += SB1_THREADS / 32) issue_d(s, base + S + s);
        }
      }
    }

    // ---- pair partial: this CTA's column half
    if (tid < hchunk) {
      float* dst = q.partial + (static_cast<size_t>(l & 1) * npairs + pair) * H + xoff + tid * V;
#pragma unroll
      for (int v = 0; v < V; v += 4) *reinterpret_cast<float4*>(dst + v) = make_float4(acc[v], acc[v + 1], acc[v + 2], acc[v + 3]);
    }
    __syncthreads();
    if (tid == 0) red_release_add(q.sync + SB1_SYNC_B, 1u);
    // ---- barrier B: all pair partials of this layer are complete
    grid_barrier_wait(SB1_SYNC_B, seq * static_cast<uint32_t>(G), l);
    if (q.strict) {
      do_reduce(l);
      if (tid == 0) red_release_add(q.sync + SB1_SYNC_C, 1u);
      grid_barrier_wait(SB1_SYNC_C, seq * static_cast<uint32_t>(G), l);
      if (l + 1 < L) do_t(l + 1);
    } else {
      if (l + 1 < L) do_t(l + 1);
      do_reduce(l);
    }
  }
  if (timed_out && q.layer[0].status) atomicOr(q.layer[0].status, DEV_TIMEOUT);
  if (c == 0 && tid == 0) q.sync[SB1_SYNC_GEN] = gen + 1u;
  cluster.sync();  // no CTA exits while its partner may still address its shared memory
}

// ------------------------------------------------------------------------------------------ host

// STX_STACK_KERNEL=layers keeps a single-row stack on the per-layer kernels (k_pred_t, k_mlp_b1,
// k_partial_reduce); read when a stack is created.
static bool stack_b1_enabled() {
  const char* e = getenv("STX_STACK_KERNEL");
  return !(e && !strcmp(e, "layers"));
}

template <typename T>
static size_t sb1_smem_budget() {
  static size_t budget = 0;
  if (!budget) {
    cudaFuncAttributes fa;
    size_t stat = 1024;
    if (cudaFuncGetAttributes(&fa, k_stack_b1<T>) == cudaSuccess) stat = fa.sharedSizeBytes;
    budget = 227 * 1024 - (stat + 127) / 128 * 128;
  }
  return budget;
}

template <typename T>
static int sb1_slots(int H, int has_gate) {
  const size_t hb = static_cast<size_t>(H / 2) * sizeof(T);
  const size_t fixed = SB1_HEADER + (static_cast<size_t>(H) * sizeof(T) + 127) / 128 * 128;
  const size_t budget = sb1_smem_budget<T>();
  if (budget < fixed + 8 * hb * (has_gate ? 3 : 2)) return 0;
  return static_cast<int>(std::min<size_t>(SB1_MAX_SLOTS, (budget - fixed) / (hb * (has_gate ? 3 : 2))));
}

static int sb1_slots_dt(int H, int has_gate, int dtype) {
  switch (dtype) {
    case STX_F32: return sb1_slots<float>(H, has_gate);
    case STX_F16: return sb1_slots<__half>(H, has_gate);
    default: return sb1_slots<__nv_bfloat16>(H, has_gate);
  }
}

int stack_b1_grid() {
  const int sms = num_sms();
  return sms - (sms & 1);
}

bool stack_b1_supported(int64_t H, int64_t I, int64_t r, int has_gate, int dtype) {
  if (!stack_b1_enabled()) return false;
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  const int G = stack_b1_grid();
  if (G < 2 || H % (4 * V) != 0 || H / V > 2 * SB1_THREADS || H / V < 64) return false;  // quarter rows of whole chunks
  if (r % V != 0 || r / V > 16 || r > G || r > SB1_THREADS) return false;
  if (((I + 7) / 8 + G - 1) / G > 8) return false;  // one pass of 8 mask bytes per CTA
  if ((H / 4 + G - 1) / G * 4 > SB1_THREADS) return false;
  const int S = sb1_slots_dt(static_cast<int>(H), has_gate, dtype);
  // the reduction stages G/2 x cpc float4 in the slot space
  const size_t red_bytes = static_cast<size_t>(G / 2) * ((H / 4 + G - 1) / G) * 16;
  const size_t slot_bytes = static_cast<size_t>(H / 2) * es * (has_gate ? 3 : 2);
  return S >= 8 && red_bytes <= static_cast<size_t>(S) * slot_bytes;
}

size_t stack_b1_scratch_bytes(int64_t L, int64_t H, int64_t r) {
  // sync words | t [L][r] | partial [2][G/2][H]
  return 512 + align_up(static_cast<size_t>(L) * r * 4, 256) + static_cast<size_t>(2) * (stack_b1_grid() / 2) * H * 4;
}

template <typename T>
static int launch_stack_b1(StackB1Args& a, cudaStream_t s) {
  const int G = stack_b1_grid();
  a.nslot = sb1_slots<T>(a.H, a.has_gate);
  const size_t smem = SB1_HEADER + (static_cast<size_t>(a.H) * sizeof(T) + 127) / 128 * 128 +
                      static_cast<size_t>(a.nslot) * (a.H / 2) * sizeof(T) * (a.has_gate ? 3 : 2);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_stack_b1<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb1_smem_budget<T>())));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(SB1_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: they wait on one another
  at[1].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 2;
  STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_b1<T>, a));
  return STX_OK;
}

int stack_b1_forward(StackB1Args& a, void* scratch, int dtype, cudaStream_t s) {
  char* p = static_cast<char*>(scratch);
  a.sync = reinterpret_cast<uint32_t*>(p);
  a.t_buf = reinterpret_cast<float*>(p + 512);
  a.partial = reinterpret_cast<float*>(p + 512 + align_up(static_cast<size_t>(a.L) * a.r * 4, 256));
  switch (dtype) {
    case STX_F32: return launch_stack_b1<float>(a, s);
    case STX_F16: return launch_stack_b1<__half>(a, s);
    default: return launch_stack_b1<__nv_bfloat16>(a, s);
  }
}

}  // namespace stx
