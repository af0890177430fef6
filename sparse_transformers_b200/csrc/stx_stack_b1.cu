// One decode token (a single row) through a whole stack of sparse layers in ONE persistent kernel.
//
// The per-layer chain  t = A x  ->  scores, mask  ->  gather + gated MLP  ->  sum of partial outputs
// (FastLoRAProjection.forward + _compute_binary_mask + SkipMLP._forward_sparse_weight_cache,
// src/modeling_skip.py:52-53,204-214,114-117) costs three dependent launches per layer when every
// link is its own kernel, and each dependent launch boundary is 2.4-3.1 us on this GPU, more than
// most links take to compute.  Here the layers are a loop inside one kernel of one CTA per SM and
// the links are separated by grid-wide barriers on counters in global memory (about 1.2 us each).
//
// Per layer l and CTA c (G CTAs):
//   scores     CTA c owns the mask bytes c, c + G, c + 2G, ... (8 neurons each): scores of those
//              neurons from t(l) in the arithmetic order of k_pred_scores, threshold, mask bytes to
//              the layer's mask words in global memory
//   barrier M  the whole mask of the layer exists.  Every CTA reads it (I/8 bytes), counts the K set
//              bits and takes the neurons of ranks [c*K/G, (c+1)*K/G): the CTAs' shares differ by at
//              most one neuron, whatever the mask looks like
//   stream     one bulk copy (global -> shared, mbarrier completion) per neuron brings its gate, up
//              and down row, which the cache keeps as one contiguous record; up to S neurons at once,
//              all requested before anything is consumed
//   the CTA consumes its neurons four at a time, as their copies land:
//   phase 1    a task is a quarter of a neuron's gate and up row against the matching quarter of x
//              (kept in registers): 16 tasks, one per warp; a = act(sum g) * (sum u)
//   phase 2    thread j adds a * down_row[16-byte chunk j] for the four neurons (registers)
//              the four slots are then free for the CTA's neurons beyond the S it could request at once
//   the CTA's partial output vector -> global (fp32);  barrier B
//   out[l] = sum of the G partial vectors in a fixed order, each CTA a few columns (deterministic, no
//              atomics); it runs while the rows of the next layer are on their way
// t(l) = round(A(l) x) is formed by the CTAs c < r, one value each, in the summation order of k_pred_t,
// from a row of A that waits in registers since the previous layer (weights do not depend on data;
// the CTA's slice of the predictor's up matrix is prefetched the same way).
//
// Order between layers.  Every layer of a stack reads the same x (the contract of stx_stack_step),
// so by default t(l+1) is formed while layer l streams and out[l] is summed while layer l+1 waits
// for its mask: two barriers per layer (M, B).  With `strict` nothing of layer l+1 starts before
// out[l] is complete - B(l), sum, barrier C, t(l+1), barrier A, scores(l+1) ... : the order a model
// needs that feeds a layer's output forward; four barriers per layer.
//
// Sharded over several GPUs (every rank owns a slice of the neurons and runs this kernel on it), the output
// sum of a layer ends with the all-reduce over the ranks through peer memory (stx_peer.cuh): each CTA pushes
// the fp32 sums of its few columns into every peer's exchange buffer, adds what the peers pushed in rank
// order and writes the columns.  In the default order this sits behind the next layer's row stream, so the
// NVLink round trip is off the critical path.
//
// Every wait is bounded.  A grid barrier that expires sets DEV_TIMEOUT in the layer's status word
// and the CTA stops waiting on grid barriers for the rest of the launch (it falls through them), so
// the kernel always terminates.  The counters only grow; a launch derives its targets from a
// generation word that CTA 0 advances at the end, so a replayed CUDA graph needs no reset.  The
// launch is cooperative: all CTAs are co-resident, which the barriers need.
#include "stx_common.cuh"
#include "stx_tma.cuh"
#include "stx_stack_b1.cuh"
#include "stx_stack_dev.cuh"
#include "stx_cache_plan.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace stx {

// PASS: 16-byte column chunks per thread (1: H / V <= 512, 2: up to 1024)
template <typename T, int PASS>
__global__ void __launch_bounds__(SB1_THREADS, 1) k_stack_b1(const __grid_constant__ StackB1Args q) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float s_ws[32];
  __shared__ uint32_t s_nib[16];
  __shared__ int s_wsum[SB1_WARPS];
  __shared__ int s_total;
  __shared__ int s_dead;
  __shared__ __align__(16) float s_part[SB1_WARPS][32];  // output sum: per-warp partial sums of the CTA's columns

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, c = blockIdx.x;
  const int H = q.H, I = q.I, r = q.r, L = q.L, S = q.nslot;
  const int nchunk = H / V, qchunk = nchunk >> 2;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const int ngu = q.has_gate ? 2 : 1;
  const uint32_t slot_bytes = row_bytes * (ngu + 1);
  const bool strict = q.strict != 0;

  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);  // one per slot
  float* a_s = reinterpret_cast<float*>(smem + SB1_OFF_AS);
  float2* pd = reinterpret_cast<float2*>(smem + SB1_OFF_PD);
  float* t_s = reinterpret_cast<float*>(smem + SB1_OFF_T);
  int* s_my = reinterpret_cast<int*>(smem + SB1_OFF_MY);
  T* x_s = reinterpret_cast<T*>(smem + SB1_HEADER);
  unsigned char* slots = smem + SB1_HEADER + (static_cast<size_t>(row_bytes) + 127) / 128 * 128;

  if (tid == 0) {
    for (int w = 0; w < SB1_MAX_SLOTS; ++w) {
      mbar_init(&bar[w], 1);
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
  // exchange number of the peer object before this launch; layer l is exchange peer_epoch0 + l + 1
  const int peer_epoch0 = q.peer.world > 1 ? *reinterpret_cast<volatile int*>(q.peer.ctl) : 0;
  __syncthreads();
  // phase 1: warp w always works on quarter w & 3 of a row; its lanes' chunks of x stay in registers
  const int sub = warp & 3;
  uint4 xq[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int ch = lane + 32 * k;
    xq[k] = ch < (nchunk >> 2) ? reinterpret_cast<const uint4*>(x_s)[sub * (nchunk >> 2) + ch] : make_uint4(0, 0, 0, 0);
  }

  // ---- score geometry (one pass of 8 mask bytes per CTA; the launcher guarantees nby <= 8)
  const int rch = r / V, nc4 = (rch + 7) >> 3;  // nc4 <= 2
  const int NBY = (I + 7) >> 3;
  const int nby = NBY > c ? (NBY - 1 - c) / G + 1 : 0;
  const int g8 = tid & 7;
  const int kk = tid >> 6;                               // mask byte of the CTA this thread works on
  const int my_n = 8 * (c + G * kk) + ((tid >> 3) & 7);  // its neuron
  const bool n_ok = kk < nby && my_n < I;
  const int NT = min(1024, (nchunk + 31) / 32 * 32);     // virtual threads of the t reduction (as k_pred_t's block)
  const int W = (I + 31) >> 5;                           // mask words
  const int WPT = (W + SB1_THREADS - 1) / SB1_THREADS;   // <= 4

  // weights a little ahead of their use (they do not depend on data): a row of A (CTAs c < r) is requested
  // before the wait for the mask and used after the rows are requested; the CTA's slice of the predictor's
  // up matrix is requested before barrier B and used right after it.  Neither stays in registers while the
  // rows are consumed.
  uint4 areg[PASS];
#pragma unroll
  for (int k = 0; k < PASS; ++k) areg[k] = make_uint4(0, 0, 0, 0);
  uint4 wraw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  auto load_a = [&](int l) {
    if (c < r) {
      const T* arow = static_cast<const T*>(q.layer[l].A) + static_cast<size_t>(c) * H;
#pragma unroll
      for (int k = 0; k < PASS; ++k) {
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
  // over each group of 32, then over the group sums).  Thread 0 stores it; the same thread's next
  // release on a barrier counter publishes it.  Contains a block barrier (c < r is CTA-uniform).
  auto do_t = [&](int l) {
    if (c < r) {
      float acc[PASS];
#pragma unroll
      for (int k = 0; k < PASS; ++k) {
        acc[k] = 0.f;
        const int v = tid + k * SB1_THREADS;
        // same bits as convert + fmaf in element order (the order of k_pred_t)
        if (v < nchunk) acc[k] = MixDot<T>::run(areg[k], *reinterpret_cast<const uint4*>(x_s + v * V), 0.f);
      }
#pragma unroll
      for (int k = 0; k < PASS; ++k) {
        const float s = warp_sum_xor(acc[k]);
        const int grp = warp + k * SB1_WARPS;
        if (lane == 0 && grp * 32 < NT) s_ws[grp] = s;
      }
      __syncthreads();
      if (warp == 0) {
        const float s = warp_sum_xor(lane < NT / 32 ? s_ws[lane] : 0.f);
        if (lane == 0) q.t_buf[static_cast<size_t>(l) * r + c] = DT<T>::round_f(s);
      }
    }
  };
  // out[l] = sum of the CTAs' partial vectors for this CTA's columns (cpc float4 columns, cpc <= 8) in a
  // fixed order: a lane adds up to three vectors, the four lanes of a column meet by butterfly, the 16
  // warp sums are added in warp order.  All loads are in flight at once; needs no staging space.
  const int ncol4 = H / 4;
  const int cpc = (ncol4 + G - 1) / G;
  const int col0 = c * cpc;
  const int ncols = max(0, min(cpc, ncol4 - col0));
  // lane = (vector group ps = lane >> 3, float4 column lane & 7); vector p = warp * 4 + ps + 64 k, k < 3
  float4 rv[3];
  const int rcol = lane & 7, rps = lane >> 3;
  auto reduce_load = [&](int l) {  // all loads in flight at once; nothing waits for them here
    const float* part = q.partial + static_cast<size_t>(l & 1) * G * H;
#pragma unroll
    for (int k = 0; k < 3; ++k) {
      const int p = warp * 4 + rps + 64 * k;
      rv[k] = (rcol < ncols && p < G) ? __ldcg(reinterpret_cast<const float4*>(part + static_cast<size_t>(p) * H) + col0 + rcol)
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  };
  auto reduce_sum = [&](int l) {  // contains a block barrier
    float4 sum = rv[0];
#pragma unroll
    for (int k = 1; k < 3; ++k) {
      sum.x += rv[k].x;
      sum.y += rv[k].y;
      sum.z += rv[k].z;
      sum.w += rv[k].w;
    }
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {  // the four vector groups of the warp
      sum.x += __shfl_xor_sync(0xffffffffu, sum.x, off);
      sum.y += __shfl_xor_sync(0xffffffffu, sum.y, off);
      sum.z += __shfl_xor_sync(0xffffffffu, sum.z, off);
      sum.w += __shfl_xor_sync(0xffffffffu, sum.w, off);
    }
    if (rps == 0) *reinterpret_cast<float4*>(&s_part[warp][rcol * 4]) = sum;
    __syncthreads();
    if (tid < ncols * 4) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SB1_WARPS; ++w) t += s_part[w][tid];
      if (q.peer.world > 1) {  // sum over the shards: push to every peer, add what they pushed, in rank order
        const int epoch = peer_epoch0 + l + 1;
        bool lost = false;
        peer_push(q.peer, epoch, col0 * 4 + tid, t);
        t = peer_collect(q.peer, epoch, col0 * 4 + tid, t, &lost);
        if (lost) {
          atomicOr(q.peer.ctl + 2, DEV_TIMEOUT);
          if (q.layer[l].status) atomicOr(q.layer[l].status, DEV_TIMEOUT);
        }
      }
      static_cast<T*>(q.layer[l].out)[col0 * 4 + tid] = DT<T>::from_f(t);
    }
  };
  auto barrier_arrive = [&](int word) {  // everything this CTA wrote before is published
    __syncthreads();
    if (tid == 0) red_release_add(q.sync + word, 1u);
  };
  auto barrier_wait = [&](int word, uint32_t target, int l) {
    if (tid == 0 && !s_dead) {
      if (!grid_wait(q.sync + word, target, grid_wait_limit(q.peer.world))) {
        s_dead = 1;
        if (q.layer[l].status) atomicOr(q.layer[l].status, DEV_TIMEOUT);
      }
    }
    __syncthreads();
  };

  load_a(0);
  load_w(0);
  do_t(0);
  barrier_arrive(SB1_SYNC_A);
  barrier_wait(SB1_SYNC_A, (strict ? gen * static_cast<uint32_t>(L) + 1u : gen + 1u) * static_cast<uint32_t>(G), 0);

  uint32_t ph = 0u;  // mbarrier phase parity per slot (same in every thread)
  bool timed_out = false;

  for (int l = 0; l < L; ++l) {
    const StackLayerDesc& ld = q.layer[l];
    const uint32_t seq = gen * static_cast<uint32_t>(L) + static_cast<uint32_t>(l) + 1u;
    // ---- t of this layer is complete and visible
    if (tid < r) {
      const int e = tid, ch = e / V, v = e - ch * V;
      t_s[(((ch >> 3) * (V / 4) + (v >> 2)) * 8 + (ch & 7)) * 4 + (v & 3)] = __ldcg(q.t_buf + static_cast<size_t>(l) * r + e);
    }
    __syncthreads();

    // ---- scores of the CTA's own neurons (arithmetic of k_pred_scores) -> mask bytes
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
      __syncthreads();
      if (tid < 8 && tid < nby)
        reinterpret_cast<uint8_t*>(ld.bits)[c + G * tid] = static_cast<uint8_t>(s_nib[2 * tid] | (s_nib[2 * tid + 1] << 4));
    }
    barrier_arrive(SB1_SYNC_M);
    // requested now, used after the rows are requested: the partial vectors of the previous layer, A's row
    if (!strict && l > 0) reduce_load(l - 1);
    if (!strict && l + 1 < L) load_a(l + 1);
    // ---- barrier M: the layer's mask is complete
    barrier_wait(SB1_SYNC_M, seq * static_cast<uint32_t>(G), l);

    // ---- the CTA's share of the active neurons: ranks [c*K/G, (c+1)*K/G) of the set bits
    int nloc;
    {
      uint32_t wv[4];
      int cnt = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int w = tid * WPT + k;
        wv[k] = (k < WPT && w < W) ? __ldcg(ld.bits + w) : 0u;
        cnt += __popc(wv[k]);
      }
      int inc = cnt;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += v;
      }
      if (lane == 31) s_wsum[warp] = inc;
      __syncthreads();
      if (warp == 0) {
        const int v = lane < SB1_WARPS ? s_wsum[lane] : 0;
        int winc = v;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int u = __shfl_up_sync(0xffffffffu, winc, off);
          if (lane >= off) winc += u;
        }
        if (lane < SB1_WARPS) s_wsum[lane] = winc - v;
        if (lane == 31) s_total = winc;
      }
      __syncthreads();
      const int K = s_total;
      const int lo = static_cast<int>(static_cast<long long>(c) * K / G);
      const int hi = static_cast<int>(static_cast<long long>(c + 1) * K / G);
      nloc = min(hi - lo, SB1_MY_CAP);
      int rho = s_wsum[warp] + inc - cnt;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t b = wv[k];
        const int w = tid * WPT + k;
        if (rho + __popc(b) > lo && rho < hi) {
          while (b) {
            const int n = w * 32 + __ffs(b) - 1;
            b &= b - 1;
            if (rho >= lo && rho - lo < nloc) s_my[rho - lo] = n;
            ++rho;
          }
        } else {
          rho += __popc(b);
        }
      }
      __syncthreads();
    }

    const char* csrc = static_cast<const char*>(ld.cat);
    // slot s <- local neuron j: its whole record (gate, up and down row) with one bulk copy
    auto issue = [&](int s, int j) {
      mbar_expect_tx(&bar[s], slot_bytes);
      bulk_load(slots + static_cast<size_t>(s) * slot_bytes, csrc + static_cast<size_t>(s_my[j]) * slot_bytes, slot_bytes, &bar[s]);
    };
    // One lane per slot.  The slots were last READ (generic proxy, phase 2 of the previous layer, several
    // block barriers ago); the copies only write them, so no proxy fence is needed here.
    if (warp == 0 && lane < min((S >> 2) << 2, nloc)) issue(lane, lane);
    // while the rows are on their way: t of the next layer, the output sum of the previous one
    if (!strict && l + 1 < L) do_t(l + 1);
    if (!strict && l > 0) reduce_sum(l - 1);

    float acc[PASS][V];
#pragma unroll
    for (int k = 0; k < PASS; ++k)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[k][v] = 0.f;

    // The CTA walks its neurons in groups of four: 16 tasks (neuron, quarter of the row) = one per warp.
    // Group g sits in slots 4 * (g % nsg) ..; its slots are re-used by group g + nsg the moment it is done,
    // so a CTA with more neurons than slots pays no extra round trip unless it has very many.
    const int nsg = S >> 2;  // slot groups
    const int ngroups = (nloc + 3) >> 2;
    const int gi = warp >> 2;  // this warp's neuron within a group (its quarter is sub = warp & 3)
    for (int g = 0; g < ngroups; ++g) {
      const int s0 = (g % nsg) * 4;
      const int nv = min(4, nloc - 4 * g);
      float2* pdg = pd + (g & 1) * 16;
      // ---- phase 1
      if (gi < nv) {
        const int sl_i = s0 + gi;
        if (!mbar_wait_bounded(&bar[sl_i], (ph >> sl_i) & 1u)) timed_out = true;
        const unsigned char* sl = slots + static_cast<size_t>(sl_i) * slot_bytes;
        const uint4* grow = reinterpret_cast<const uint4*>(sl) + sub * qchunk;
        const uint4* urow = reinterpret_cast<const uint4*>(sl + (q.has_gate ? row_bytes : 0)) + sub * qchunk;
        float ag0 = 0.f, ag1 = 0.f, au0 = 0.f, au1 = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // the chunks whose x sits in registers
          const int ch = lane + 32 * k;
          if (ch < qchunk) {
            if (k & 1) au1 = MixDot<T>::run(urow[ch], xq[k], au1);
            else au0 = MixDot<T>::run(urow[ch], xq[k], au0);
            if (q.has_gate) {
              if (k & 1) ag1 = MixDot<T>::run(grow[ch], xq[k], ag1);
              else ag0 = MixDot<T>::run(grow[ch], xq[k], ag0);
            }
          }
          if (k == 1) asm volatile("" ::: "memory");  // two chunk pairs in flight, not four (registers)
        }
        for (int ch = lane + 128; ch < qchunk; ch += 32) {  // rows longer than 512 chunks: x from shared memory
          const uint4 xv = reinterpret_cast<const uint4*>(x_s)[sub * qchunk + ch];
          au0 = MixDot<T>::run(urow[ch], xv, au0);
          if (q.has_gate) ag0 = MixDot<T>::run(grow[ch], xv, ag0);
        }
        const float u = warp_sum_xor(au0 + au1);
        const float gs = q.has_gate ? warp_sum_xor(ag0 + ag1) : 0.f;
        if (lane == 0) pdg[gi * 4 + sub] = make_float2(gs, u);
      }
      __syncthreads();  // the quarter sums of the group are there (and its rows have arrived)
      if (tid < nv) {
        const float2 p0 = pdg[tid * 4], p1 = pdg[tid * 4 + 1], p2 = pdg[tid * 4 + 2], p3 = pdg[tid * 4 + 3];
        const float gsum = (p0.x + p1.x) + (p2.x + p3.x);
        const float usum = (p0.y + p1.y) + (p2.y + p3.y);
        a_s[(g & 1) * 4 + tid] = q.has_gate ? apply_act(ld.act, gsum) * usum : apply_act(ld.act, usum);
      }
      __syncthreads();  // a of the group
      // ---- phase 2: thread j owns the 16-byte column chunks j, j + 512
#pragma unroll
      for (int k = 0; k < PASS; ++k) {
        const int cc = tid + k * SB1_THREADS;
        if (cc < nchunk) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (i < nv) {
              const float a = a_s[(g & 1) * 4 + i];
              const T* drow = reinterpret_cast<const T*>(slots + static_cast<size_t>(s0 + i) * slot_bytes + static_cast<size_t>(ngu) * row_bytes);
              float wd[V];
              Unpack<T>::run(*reinterpret_cast<const uint4*>(drow + cc * V), wd);
#pragma unroll
              for (int v = 0; v < V; ++v) acc[k][v] = fmaf(a, wd[v], acc[k][v]);
            }
          }
        }
      }
      ph ^= ((1u << nv) - 1u) << s0;
      if (4 * (g + nsg) < nloc) {  // CTA-uniform: the group's slots take the neurons of group g + nsg
        __syncthreads();           // every thread is done with them
        if (warp == 0 && lane < min(4, nloc - 4 * (g + nsg))) {
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          issue(s0 + lane, 4 * (g + nsg) + lane);
        }
      }
    }

    // ---- the CTA's partial output vector
    {
      float* dst = q.partial + (static_cast<size_t>(l & 1) * G + c) * H;
#pragma unroll
      for (int k = 0; k < PASS; ++k) {
        const int cc = tid + k * SB1_THREADS;
        if (cc < nchunk) {
#pragma unroll
          for (int v = 0; v < V; v += 4)
            *reinterpret_cast<float4*>(dst + cc * V + v) = make_float4(acc[k][v], acc[k][v + 1], acc[k][v + 2], acc[k][v + 3]);
        }
      }
    }
    if (l + 1 < L) load_w(l + 1);
    barrier_arrive(SB1_SYNC_B);  // also publishes t of the next layer (default order)
    // ---- barrier B: all partial vectors of this layer are complete
    barrier_wait(SB1_SYNC_B, seq * static_cast<uint32_t>(G), l);
    if (strict) {
      if (l + 1 < L) load_a(l + 1);
      reduce_load(l);
      reduce_sum(l);
      barrier_arrive(SB1_SYNC_C);
      barrier_wait(SB1_SYNC_C, seq * static_cast<uint32_t>(G), l);
      if (l + 1 < L) {
        do_t(l + 1);
        barrier_arrive(SB1_SYNC_A);
        barrier_wait(SB1_SYNC_A, (seq + 1u) * static_cast<uint32_t>(G), l);
      }
    }
  }
  if (!strict) {
    reduce_load(L - 1);
    reduce_sum(L - 1);
  }
  if (timed_out && q.layer[0].status) atomicOr(q.layer[0].status, DEV_TIMEOUT);
  if (c == 0 && tid == 0) q.sync[SB1_SYNC_GEN] = gen + 1u;
  if (q.peer.world > 1) {
    // the launch's last CTA advances the peer object's exchange number (every CTA read it at the start, and
    // every CTA is past its last exchange when it arrives here)
    __syncthreads();
    if (tid == 0 && atomicAdd(reinterpret_cast<unsigned*>(q.peer.ctl + 1), 1u) == gridDim.x - 1) {
      q.peer.ctl[1] = 0;
      *reinterpret_cast<volatile int*>(q.peer.ctl) = peer_epoch0 + L;
    }
  }
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
    if (cudaFuncGetAttributes(&fa, k_stack_b1<T, 2>) == cudaSuccess) stat = fa.sharedSizeBytes;
    budget = 227 * 1024 - (stat + 127) / 128 * 128;
  }
  return budget;
}

static size_t sb1_fixed_bytes(int H, size_t es) { return SB1_HEADER + (static_cast<size_t>(H) * es + 127) / 128 * 128; }

template <typename T>
static int sb1_slots(int H, int has_gate) {
  const size_t slot = static_cast<size_t>(H) * sizeof(T) * (has_gate ? 3 : 2);
  const size_t fixed = sb1_fixed_bytes(H, sizeof(T));
  const size_t budget = sb1_smem_budget<T>();
  if (budget < fixed + 4 * slot) return 0;
  return static_cast<int>(std::min<size_t>(SB1_MAX_SLOTS, (budget - fixed) / slot));
}

static int sb1_slots_dt(int H, int has_gate, int dtype) {
  switch (dtype) {
    case STX_F32: return sb1_slots<float>(H, has_gate);
    case STX_F16: return sb1_slots<__half>(H, has_gate);
    default: return sb1_slots<__nv_bfloat16>(H, has_gate);
  }
}

static int stack_b1_grid() { return num_sms(); }

static bool stack_flow_enabled();

bool stack_b1_supported(int64_t H, int64_t I, int64_t r, int has_gate, int dtype, bool flow) {
  if (!stack_b1_enabled()) return false;
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  const int G = stack_b1_grid();
  if (G < 2 || H % (4 * V) != 0 || H / V > SB1_MAX_PASS * SB1_THREADS || H / V < 64) return false;  // quarter rows of whole chunks
  if (r % V != 0 || r / V > 16 || r > G || r > SB1_THREADS) return false;
  if (((I + 7) / 8 + G - 1) / G > (flow && stack_flow_enabled() ? 8 * FLOW_MAX_PASSES : 8)) return false;  // passes of 8 mask bytes per CTA
  if ((I + 31) / 32 > 4 * SB1_THREADS) return false;        // four mask words per thread
  if ((I + G - 1) / G > SB1_MY_CAP) return false;           // the CTA's list of a layer
  if ((H / 4 + G - 1) / G > 8 || G > 192) return false;  // the output sum: <= 8 float4 columns per CTA, <= 3 x 64 vectors
  return sb1_slots_dt(static_cast<int>(H), has_gate, dtype) >= 4;
}

size_t stack_b1_scratch_bytes(int64_t L, int64_t H, int64_t r) {
  // sync words | t [L][r] | partial [max(L, 2)][G][H] (the layer-by-layer kernel uses two of them)
  return 1024 + align_up(static_cast<size_t>(L) * r * 4, 256) + static_cast<size_t>(std::max<int64_t>(L, 2)) * stack_b1_grid() * H * 4;
}

// STX_STACK_ORDER=layerwise keeps the layer-by-layer kernel also where the layers could flow (read when a
// stack's graph is captured).
static bool stack_flow_enabled() {
  const char* e = getenv("STX_STACK_ORDER");
  return !(e && !strcmp(e, "layerwise"));
}

// Layers that do not feed one another flow (stx_stack_flow.cu).  Sharded, every layer needs its own place in the
// peer object's exchange buffer.
static bool stack_flow_selected(const StackB1Args& a) {
  return !a.strict && stack_flow_enabled() && (a.peer.world <= 1 || static_cast<long long>(a.L) * a.H <= a.peer.max_elems);
}

// STX_STACK_UPKEEP=kernels keeps the index plans and row copies of the layers' caches in kernels of their own
// behind the flow kernel (read when a stack's graph is captured).
bool stack_flow_upkeep_inside(const StackB1Args& a, int dtype) {
  const char* e = getenv("STX_STACK_UPKEEP");
  if (e && !strcmp(e, "kernels")) return false;
  if (!stack_flow_selected(a) || a.L > stack_b1_grid() || (a.I + 31) / 32 > 2 * SB1_THREADS) return false;
  const size_t slot = static_cast<size_t>(a.H) * dtype_size(dtype) * (a.has_gate ? 3 : 2);
  return plan_smem_words(a.I) * sizeof(int32_t) <= static_cast<size_t>(sb1_slots_dt(a.H, a.has_gate, dtype)) * slot;
}

template <typename T>
static int launch_stack_b1(StackB1Args& a, int dtype, cudaStream_t s) {
  const int G = stack_b1_grid();
  a.nslot = sb1_slots<T>(a.H, a.has_gate);
  const size_t smem = sb1_fixed_bytes(a.H, sizeof(T)) + static_cast<size_t>(a.nslot) * a.H * sizeof(T) * (a.has_gate ? 3 : 2);
  if (stack_flow_selected(a)) return stack_flow_launch(a, dtype, smem, sb1_smem_budget<T>(), s);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_stack_b1<T, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb1_smem_budget<T>())));
    STX_CUDA(cudaFuncSetAttribute(k_stack_b1<T, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sb1_smem_budget<T>())));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G);
  cfg.blockDim = dim3(SB1_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident: they wait on one another
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  if (a.H / DT<T>::V <= SB1_THREADS)
    STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_b1<T, 1>, a));
  else
    STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_b1<T, 2>, a));
  return STX_OK;
}

int stack_b1_forward(StackB1Args& a, void* scratch, int dtype, cudaStream_t s) {
  char* p = static_cast<char*>(scratch);
  a.sync = reinterpret_cast<uint32_t*>(p);
  a.t_buf = reinterpret_cast<float*>(p + 1024);
  a.partial = reinterpret_cast<float*>(p + 1024 + align_up(static_cast<size_t>(a.L) * a.r * 4, 256));
  switch (dtype) {
    case STX_F32: return launch_stack_b1<float>(a, dtype, s);
    case STX_F16: return launch_stack_b1<__half>(a, dtype, s);
    default: return launch_stack_b1<__nv_bfloat16>(a, dtype, s);
  }
}

}  // namespace stx
