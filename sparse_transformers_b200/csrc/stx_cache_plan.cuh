// The upkeep of the differential weight cache as device functions: the index plan of one cache by one thread
// block (the plan kernel of stx_cache.cu is a thin wrapper around it) and the copy of one packed row by one warp.
// The flow kernel of single-row stacks (stx_stack_flow.cu) runs both inside its own launch.
#pragma once

#include "stx_cache.cuh"

namespace stx {

constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MFAST = 2048;     // surplus removals replayed from shared memory
constexpr int PLAN_LIST_CAP = 4096;  // added / removed ids kept in shared memory
constexpr int MAX_I = 65536;      // 2 mask words per plan thread

struct Int2 {
  int x, y;
};

// Exclusive scan of two counters over the block (thread order).  Ends with a barrier.
__device__ __forceinline__ Int2 block_excl_scan2(Int2 v, Int2* total, Int2* warp_sums) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  Int2 inc = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    int a = __shfl_up_sync(0xffffffffu, inc.x, off);
    int b = __shfl_up_sync(0xffffffffu, inc.y, off);
    if (lane >= off) {
      inc.x += a;
      inc.y += b;
    }
  }
  if (lane == 31) warp_sums[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    Int2 w = lane < static_cast<int>(blockDim.x >> 5) ? warp_sums[lane] : Int2{0, 0};
    Int2 winc = w;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int a = __shfl_up_sync(0xffffffffu, winc.x, off);
      int b = __shfl_up_sync(0xffffffffu, winc.y, off);
      if (lane >= off) {
        winc.x += a;
        winc.y += b;
      }
    }
    warp_sums[lane] = Int2{winc.x - w.x, winc.y - w.y};
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  Int2 base = warp_sums[wid];
  Int2 r{base.x + inc.x - v.x, base.y + inc.y - v.y};
  __syncthreads();
  return r;
}

// One block of PLAN_THREADS threads.  Dynamic shared memory (int32 words):
//   s_rem[W] s_remoff[W] s_dirty[W] | s_added[CAP] s_removed[CAP] s_rpos[CAP] | s_tail[MFAST]
//
// Common case (both diff lists fit PLAN_LIST_CAP, surplus removals fit PLAN_MFAST): the lists
// live in shared memory and the kernel makes two dependent trips to global memory — (1) mask
// words and K, (2) pos_of of every removed neuron plus the tail of `active` — everything
// else is shared-memory work and fire-and-forget stores.  Otherwise a generic path keeps the
// lists in global memory.
// All threads of the block call it (blockDim.x a multiple of 32, at most 2 mask words per thread); `sm` is the
// block's work space of plan_smem_words(I) words.  Ends without a block barrier.
__device__ __forceinline__ void plan_block(const uint32_t* __restrict__ new_bits, uint32_t* __restrict__ cur_bits,
                                           int32_t* __restrict__ active, int32_t* __restrict__ pos_of, int32_t* __restrict__ lists,
                                           int32_t* __restrict__ jobs, int32_t* __restrict__ state, uint32_t* __restrict__ stale, int lazy,
                                           int I, int32_t* sm) {
  __shared__ Int2 s_ws[32];
  __shared__ Int2 s_tot;
  __shared__ int s_knew, s_slow;

  const int W = (I + 31) >> 5;
  uint32_t* s_rem = reinterpret_cast<uint32_t*>(sm);
  int32_t* s_remoff = sm + W;
  uint32_t* s_dirty = reinterpret_cast<uint32_t*>(sm + 2 * W);
  int32_t* s_added = sm + 3 * W;
  int32_t* s_removed = s_added + PLAN_LIST_CAP;
  int32_t* s_rpos = s_removed + PLAN_LIST_CAP;
  int32_t* s_tail = s_rpos + PLAN_LIST_CAP;

  const int t = threadIdx.x;
  const int NT = blockDim.x;
  const int WPT = (W + NT - 1) / NT;  // <= 2 by construction of the launch

  // ---- 1. diff words (weight_cache.h:84-110: added = new & ~old, removed = old & ~new)
  const int K0 = state[ST_K];
  uint32_t nbw[2] = {0, 0}, aw[2] = {0, 0}, rw[2] = {0, 0};
  Int2 cnt{0, 0};
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    if (w < W) {
      uint32_t nb = new_bits[w];
      const uint32_t ob = cur_bits[w];
      if (w == W - 1 && (I & 31)) nb &= (1u << (I & 31)) - 1u;
      nbw[k] = nb;
      aw[k] = nb & ~ob;
      rw[k] = ob & ~nb;
      s_rem[w] = rw[k];
      s_dirty[w] = 0u;
      cnt.x += __popc(aw[k]);
      cnt.y += __popc(rw[k]);
    }
  }
  if (t == 0) s_slow = 0;
  Int2 off = block_excl_scan2(cnt, &s_tot, s_ws);
  const int na = s_tot.x, nr = s_tot.y;

  if (na == 0 && nr == 0) {  // unchanged mask: the reference returns before touching anything
    if (t == 0) {
      state[ST_NJOBS] = 0;
      state[ST_ADDED] = 0;
      state[ST_REMOVED] = 0;
    }
    return;
  }
  const int pairs = min(na, nr);
  const int m = nr > na ? nr - na : 0;   // surplus removals
  const int n1 = K0 - m;                 // size after phase 3 when every removal is found
  const bool fast = na <= PLAN_LIST_CAP && nr <= PLAN_LIST_CAP && m <= PLAN_MFAST && n1 >= 0;
  int32_t* added = fast ? s_added : lists;
  int32_t* removed = fast ? s_removed : lists + I;

  // ---- 2. ascending id lists (torch::nonzero order)
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    if (w < W) {
      s_remoff[w] = off.y;
      uint32_t a = aw[k], r = rw[k];
      while (a) {
        const int b = __ffs(a) - 1;
        added[off.x++] = w * 32 + b;
        a &= a - 1;
      }
      while (r) {
        const int b = __ffs(r) - 1;
        removed[off.y++] = w * 32 + b;
        r &= r - 1;
      }
    }
  }
  __syncthreads();

  int Knew = K0;
  if (fast) {
    // ---- one round of reads: position of every removed neuron, and the tail of `active`
    for (int i = t; i < nr; i += NT) {
      const int p = pos_of[s_removed[i]];
      s_rpos[i] = p;
      if (p < 0) s_slow = 1;  // inconsistent state (only after a NO_ACTIVE error): generic replay
    }
    for (int i = t; i < m; i += NT) s_tail[i] = active[n1 + i];
    __syncthreads();
    // ---- phase 1: i-th removed slot receives the i-th added neuron (weight_cache.h:248-277)
    for (int i = t; i < pairs; i += NT) {
      const int r = s_removed[i], a = s_added[i];
      const int p = s_rpos[i];
      if (p >= 0) {
        active[p] = a;
        pos_of[a] = p;
        pos_of[r] = -1;
        atomicOr(&s_dirty[p >> 5], 1u << (p & 31));
        if (m > 0 && p >= n1) s_tail[p - n1] = a;  // keep the shared-memory copy of the tail current
      }
    }
    if (na > nr) {
      // ---- phase 2: append surplus additions in ascending order (weight_cache.h:280-307)
      const int extra = na - nr;
      for (int i = t; i < extra; i += NT) {
        const int a = s_added[pairs + i];
        const int p = K0 + i;
        if (p < I) {
          active[p] = a;
          pos_of[a] = p;
          atomicOr(&s_dirty[p >> 5], 1u << (p & 31));
        }
      }
      Knew = min(K0 + extra, I);
    }
    __syncthreads();
    if (m > 0) {
      // ---- phase 3: surplus removals, ascending, each filled by the then-last row
      //      (weight_cache.h:310-353).  Sequential by definition; one thread replays it on
      //      indices only.  Every row it can move lives in the tail [n1, K0).
      if (t == 0) {
        int n = K0;
        if (!s_slow) {
          for (int i = 0; i < m; ++i) {
            const int e = s_removed[pairs + i];
            const int p = s_rpos[pairs + i];
            const int last = n - 1;
            if (p != last) {
              const int x = s_tail[last - n1];
              if (p >= n1) {
                s_tail[p - n1] = x;
              } else {
                active[p] = x;
                s_dirty[p >> 5] |= 1u << (p & 31);
              }
              pos_of[x] = p;
              const uint32_t rwd = s_rem[x >> 5];
              if ((rwd >> (x & 31)) & 1u) {  // x itself is removed later: track where it now sits
                const int idx = s_remoff[x >> 5] + __popc(rwd & ((1u << (x & 31)) - 1u));
                if (idx > pairs + i && idx < nr) s_rpos[idx] = p;
              }
            }
            pos_of[e] = -1;
            --n;
          }
        } else {
          for (int i = 0; i < m; ++i) {
            const int e = s_removed[pairs + i];
            const int p = pos_of[e];
            if (p < 0) continue;  // not cached: the reference skips it
            const int last = n - 1;
            if (p != last) {
              const int x = active[last];
              active[p] = x;
              pos_of[x] = p;
              s_dirty[p >> 5] |= 1u << (p & 31);
            }
            pos_of[e] = -1;
            --n;
          }
        }
        s_knew = n;
      }
      __syncthreads();
      Knew = s_knew;
    }
  } else {
    // ---------------------------------------------------------------- generic path (global lists)
    for (int i = t; i < pairs; i += NT) {
      const int r = removed[i], a = added[i];
      const int p = pos_of[r];
      if (p >= 0) {
        active[p] = a;
        pos_of[a] = p;
        pos_of[r] = -1;
        atomicOr(&s_dirty[p >> 5], 1u << (p & 31));
      }
    }
    __syncthreads();
    if (na > nr) {
      const int extra = na - nr;
      for (int i = t; i < extra; i += NT) {
        const int a = added[pairs + i];
        const int p = K0 + i;
        if (p < I) {
          active[p] = a;
          pos_of[a] = p;
          atomicOr(&s_dirty[p >> 5], 1u << (p & 31));
        }
      }
      Knew = min(K0 + extra, I);
    } else if (nr > na) {
      if (t == 0) {
        int n = K0;
        for (int i = 0; i < m; ++i) {
          const int e = removed[pairs + i];
          const int p = pos_of[e];
          if (p < 0) continue;
          const int last = n - 1;
          if (p != last) {
            const int x = active[last];
            active[p] = x;
            pos_of[x] = p;
            s_dirty[p >> 5] |= 1u << (p & 31);
          }
          pos_of[e] = -1;
          --n;
        }
        s_knew = n;
      }
      __syncthreads();
      Knew = s_knew;
    }
    __syncthreads();
  }

  // ---- 4. rewritten slots below the new K, ascending.  Lazy mode only remembers them in
  //         the cache's stale bitmap; the rows are brought up to date when somebody reads them.
  Int2 jc{0, 0};
  uint32_t dw[2] = {0, 0};
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    if (w < W) {
      uint32_t d = s_dirty[w];
      if (lazy) {
        if (d) stale[w] |= d;
        d = 0u;
      }
      const int lo = w * 32;
      if (lo >= Knew) d = 0u;
      else if (Knew - lo < 32) d &= (1u << (Knew - lo)) - 1u;
      dw[k] = d;
      jc.x += __popc(d);
    }
  }
  Int2 joff = block_excl_scan2(jc, &s_tot, s_ws);
  for (int k = 0; k < WPT; ++k) {
    const int w = t * WPT + k;
    uint32_t d = dw[k];
    while (d) {
      const int b = __ffs(d) - 1;
      jobs[joff.x++] = w * 32 + b;
      d &= d - 1;
    }
  }

  // ---- 5. commit
  if (Knew > 0) {
    for (int k = 0; k < WPT; ++k) {
      const int w = t * WPT + k;
      if (w < W) cur_bits[w] = nbw[k];
    }
  }
  if (t == 0) {
    state[ST_K] = Knew;
    state[ST_ADDED] = na;
    state[ST_REMOVED] = nr;
    if (Knew > 0) {
      state[ST_NJOBS] = s_tot.x;
      state[ST_VALID] = 1;
      state[ST_EPOCH] = state[ST_EPOCH] + 1;
    } else {
      // the reference throws "No active weights" here, before it records the new mask
      state[ST_NJOBS] = 0;
      state[ST_STATUS] = state[ST_STATUS] | DEV_NO_ACTIVE;
    }
  }
}


__host__ __device__ inline size_t plan_smem_words(int64_t I) {
  const int64_t W = (I + 31) / 32;
  return static_cast<size_t>(3 * W + 3 * PLAN_LIST_CAP + PLAN_MFAST);
}

// What another kernel needs to keep one cache up to date: the plan's arrays, and where the rows live.
struct UpkeepArgs {
  uint32_t* cur_bits;
  int32_t* active;
  int32_t* pos_of;
  int32_t* lists;
  int32_t* jobs;
  int32_t* state;
  uint32_t* stale;
  const void* pool[3];  // gate | up | down rows of all neurons ([up | down] without a gate)
  void* pk[3];          // the packed rows
  int lazy;             // plan only: the rewritten slots go to the stale bitmap
};

}  // namespace stx
