// One decode token (a single row) through a stack of sparse layers as ONE persistent kernel whose row stream
// never stops: the predictors of ALL layers first, then the active rows of layer after layer without a grid
// barrier in between.
//
// stx_stack_step feeds every layer of the stack the same x (its contract), so nothing a layer computes is
// an input of another layer.  The layer-by-layer kernel (stx_stack_b1.cu) still pays, per layer, two grid
// barriers and a round trip to HBM during which no row is in flight: 15 us per layer of which the rows
// need 5.  Here:
//   phase T   t(l) = round(A(l) x) for all layers: L * r dot products, one per warp, spread over all CTAs,
//             in the summation order of k_pred_t;                                             grid barrier
//   phase S   for every layer the CTA's 8 mask bytes: scores in the arithmetic order of k_pred_scores,
//             threshold, mask bytes to the layer's mask words.  t of all layers sits in shared memory, the
//             CTA's slice of the predictor's up matrix is requested four layers ahead, and the loop over the
//             layers contains no block barrier;                                               grid barrier
//   phase R   the layers are dealt to groups of CTAs (flow_groups below); a CTA walks the layers of its group.  Per
//             layer it scans the mask (its words were requested a layer earlier), takes its share of the set
//             bits by rank and consumes those neurons four at a time from shared-memory slots (one bulk copy
//             per neuron record, mbarrier completion) exactly as the layer-by-layer kernel does.  The slots are
//             a ring over ALL its layers: a group of four slots that has been consumed takes the CTA's next
//             group of neurons, which may belong to its next layer, so rows never stop streaming.  The CTA's
//             partial output vector of a layer goes to its own place in global memory (fp32);
//   plan      (with the cache upkeep inside the launch) CTA l < L then runs the index plan of layer l's weight
//             cache, with a smaller share of the rows to have the time;                       grid barrier
//   phase O   out[l] = sum of the layer's partial vectors in a fixed order: a warp per layer, a lane adds every
//             fourth vector of a float4 column, the four lanes of a column meet by butterfly (deterministic,
//             no atomics).  Sharded over several GPUs the warp pushes its sums to every peer's exchange
//             buffer (stx_peer.cuh), every layer in its own place, and collects all layers afterwards: the
//             NVLink round trip is paid once per token, not once per layer.
//   phase C   (cache upkeep inside the launch) the rows of every slot the plans rewrote, all layers at once, by
//             bulk copies through row buffers in the idle slot area.
// A model that feeds out[l] forward into layer l+1 cannot use this order: the layer-by-layer kernel with
// `strict` is the one for it.
//
// Every wait is bounded (grid barriers, mbarriers, peer words); an expired wait sets DEV_TIMEOUT in a
// layer's status word and the kernel falls through, so it always terminates.  The barrier counters only
// grow; a launch derives its targets from a generation word that CTA 0 advances at the end, so a replayed
// CUDA graph needs no reset.  The launch is cooperative: all CTAs are co-resident, which the barriers need.
#include "stx_common.cuh"
#include "stx_tma.cuh"
#include "stx_stack_b1.cuh"
#include "stx_stack_dev.cuh"
#include "stx_cache_plan.cuh"

namespace stx {

constexpr int FLOW_AHEAD = 4;         // layers whose predictor slices a thread has requested ahead of the one it scores
constexpr int FLOW_PLAN_WEIGHT = 11;  // share of a CTA that also runs an index plan, in sixteenths of a full share
constexpr int FLOW_LIST_CAP = 256;  // neurons of one CTA per layer (two lists of 16-bit ids fill 2 x 512 bytes of the header)

// Layers are dealt to `ng` groups of CTAs (CTA c is in group c % ng and works on the layers l with l % ng equal to
// its group): a layer's neurons then spread over G / ng CTAs, each with ng times as many neurons of a quarter of
// the layers - the same work, but a layer leaves G / ng partial vectors instead of G, and the per-layer overhead
// of a CTA (scan, list, partial vector) is paid L / ng times.  ng is the largest of 4, 2, 1 that divides L and
// keeps a CTA's share of a full mask within its list.
__host__ __device__ inline int flow_groups(int L, int G, int I) {
  for (int n = 4; n >= 2; n >>= 1)
    if (L % n == 0 && G / n >= 1 && (I + G / n - 1) / (G / n) <= FLOW_LIST_CAP) return n;
  return 1;
}

// NP: passes in which a CTA scores its mask bytes of a layer, eight bytes per pass (1: ceil(ceil(I / 8) / G) <= 8)
template <typename T, int PASS, int NP>
__global__ void __launch_bounds__(SB1_THREADS, 1) k_stack_flow(const __grid_constant__ StackB1Args q) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ int s_wsum[SB1_WARPS];
  __shared__ int s_total;
  __shared__ int s_dead;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, c = blockIdx.x;
  const int H = q.H, I = q.I, r = q.r, L = q.L, S = q.nslot;
  const int nchunk = H / V, qchunk = nchunk >> 2;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const int ngu = q.has_gate ? 2 : 1;
  const uint32_t slot_bytes = row_bytes * (ngu + 1);

  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);  // one per slot
  uint64_t* bar2 = reinterpret_cast<uint64_t*>(smem + 128);  // sixteen more for the row buffers of phase C
  float* a_s = reinterpret_cast<float*>(smem + SB1_OFF_AS);
  float2* pd = reinterpret_cast<float2*>(smem + SB1_OFF_PD);
  // the CTA's neurons of a layer (16-bit ids, FLOW_LIST_CAP of them), two buffers used in turn
  uint16_t* list_even = reinterpret_cast<uint16_t*>(smem + SB1_OFF_MY);
  uint16_t* list_odd = reinterpret_cast<uint16_t*>(smem + SB1_OFF_T);
  T* x_s = reinterpret_cast<T*>(smem + SB1_HEADER);
  unsigned char* slots = smem + SB1_HEADER + (static_cast<size_t>(row_bytes) + 127) / 128 * 128;

  if (tid == 0) {
    for (int w = 0; w < SB1_MAX_SLOTS; ++w) {
      mbar_init(&bar[w], 1);
      mbar_init(&bar2[w], 1);
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
  const int peer_epoch0 = q.peer.world > 1 ? *reinterpret_cast<volatile int*>(q.peer.ctl) : 0;
  __syncthreads();
  bool timed_out = false;

  auto barrier_arrive = [&](int word) {  // everything this CTA wrote before is published
    __syncthreads();
    if (tid == 0) red_release_add(q.sync + word, 1u);
  };
  auto barrier_wait = [&](int word) {
    if (tid == 0 && !s_dead) {
      if (!grid_wait(q.sync + word, (gen + 1u) * static_cast<uint32_t>(G), grid_wait_limit(q.peer.world))) {
        s_dead = 1;
        if (q.layer[0].status) atomicOr(q.layer[0].status, DEV_TIMEOUT);
      }
    }
    __syncthreads();
  };

  // ---- score geometry: CTA c owns the mask bytes c, c + G, ... (nby of them; the launcher guarantees
  // nby <= 8 * FLOW_MAX_PASSES); a pass of the 512 threads scores 8 of them (64 neurons x 8 lanes)
  const int rch = r / V, nc4 = (rch + 7) >> 3;  // nc4 <= 2
  const int NBY = (I + 7) >> 3;
  const int nby = NBY > c ? (NBY - 1 - c) / G + 1 : 0;
  const int g8 = tid & 7;
  const int kk = tid >> 6;  // mask byte of a pass this thread works on
  // this thread's neuron in pass p, or -1
  auto neuron_of = [&](int p) {
    const int by = kk + 8 * p;
    const int n = 8 * (c + G * by) + ((tid >> 3) & 7);
    return (by < nby && n < I) ? n : -1;
  };
  const int NT = min(1024, (nchunk + 31) / 32 * 32);     // virtual threads of the t reduction (as k_pred_t's block)
  const int W = (I + 31) >> 5;                           // mask words
  const int WPT = (W + SB1_THREADS - 1) / SB1_THREADS;   // <= 4

  // the CTA's slice of the predictor's up matrix, FLOW_AHEAD layers ahead (weights do not depend on data: the
  // first ones are on their way while t is formed)
  // An item of phase S is (layer, pass): item it = l * NP + p.
  const int nitem = L * NP;
  uint4 wq[FLOW_AHEAD][2];
  auto load_w = [&](int it, uint4 (&dst)[2]) {
    const int l = it / NP, n = neuron_of(it - l * NP);
    const T* Bm = static_cast<const T*>(q.layer[l].Bm);
#pragma unroll
    for (int c4 = 0; c4 < 2; ++c4) {
      const int ch = g8 + 8 * c4;
      dst[c4] = make_uint4(0, 0, 0, 0);
      if (n >= 0 && ch < rch) dst[c4] = ld_stream16(Bm + static_cast<size_t>(n) * r + ch * V);
    }
  };
#pragma unroll
  for (int u = 0; u < FLOW_AHEAD; ++u) {
    wq[u][0] = wq[u][1] = make_uint4(0, 0, 0, 0);
    if (u < nitem) load_w(u, wq[u]);
  }

  // ================================================================== phase T: t of every layer
  // Task (l, k) = row k of A(l) against x, one warp each.  Virtual thread v of k_pred_t owns the 16-byte chunk
  // v; its block adds the chunk sums by butterfly inside each group of 32 and then over the group sums.  A warp
  // reproduces that: group g's butterfly leaves the group sum in every lane, lane g keeps it, and a last
  // butterfly over the lanes adds the group sums.
  {
    const int ntask = L * r, NTG = NT >> 5;
    for (int task = c + G * warp; task < ntask; task += G * SB1_WARPS) {
      const int l = task / r, k = task - l * r;
      const T* arow = static_cast<const T*>(q.layer[l].A) + static_cast<size_t>(k) * H;
      float mine = 0.f;
      for (int g0 = 0; g0 < NTG; g0 += 8) {  // eight chunks per lane in flight
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int ch = (g0 + u) * 32 + lane;
          w[u] = (g0 + u < NTG && ch < nchunk) ? ld_stream16(arow + ch * V) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (g0 + u < NTG) {
            const int ch = (g0 + u) * 32 + lane;
            float p = 0.f;
            if (ch < nchunk) p = MixDot<T>::run(w[u], *reinterpret_cast<const uint4*>(x_s + ch * V), 0.f);
            p = warp_sum_xor(p);
            if (lane == g0 + u) mine = p;
          }
        }
      }
      const float s = warp_sum_xor(lane < NTG ? mine : 0.f);
      if (lane == 0) q.t_buf[task] = DT<T>::round_f(s);
    }
  }
  barrier_arrive(SB1_SYNC_FT);
  barrier_wait(SB1_SYNC_FT);

  // ================================================================== phase S: the masks of every layer
  // t of all layers goes to shared memory once (the slot area is idle until phase R), in the layout the score
  // loop reads; the loop over the layers then needs no block barrier: a warp's four mask nibbles per layer are
  // collected in shared memory and the CTA's mask bytes of all layers are written in one pass at the end.
  {
    float* t_all = reinterpret_cast<float*>(slots);                                           // [L][128]
    uint32_t* nib_all = reinterpret_cast<uint32_t*>(slots + STACK_B1_MAX_LAYERS * 512);       // [L * NP][16]
    for (int i = tid; i < L * r; i += SB1_THREADS) {
      const int l = i / r, e = i - l * r;
      const int ch = e / V, v = e - ch * V;
      t_all[l * 128 + (((ch >> 3) * (V / 4) + (v >> 2)) * 8 + (ch & 7)) * 4 + (v & 3)] = __ldcg(q.t_buf + i);
    }
    __syncthreads();
    for (int it0 = 0; it0 < nitem; it0 += FLOW_AHEAD) {
#pragma unroll
      for (int u = 0; u < FLOW_AHEAD; ++u) {
        const int it = it0 + u;
        if (it < nitem) {
          const int l = it / NP;
          const bool n_ok = neuron_of(it - l * NP) >= 0;
          const float tau_r = DT<T>::round_f(q.layer[l].tau);
          float sc = 0.f;
#pragma unroll
          for (int c4 = 0; c4 < 2; ++c4) {
            const int ch = g8 + 8 * c4;
            if (c4 < nc4 && ch < rch) {
              float w[V];
              Unpack<T>::run(wq[u][c4], w);
              const float4* tb = reinterpret_cast<const float4*>(t_all + l * 128) + (c4 * (V / 4)) * 8 + g8;
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
          if (it + FLOW_AHEAD < nitem) load_w(it + FLOW_AHEAD, wq[u]);
          sc += __shfl_xor_sync(0xffffffffu, sc, 4);
          sc += __shfl_xor_sync(0xffffffffu, sc, 2);
          sc += __shfl_xor_sync(0xffffffffu, sc, 1);
          const bool on = n_ok && DT<T>::round_f(sc) >= tau_r;
          const uint32_t bal = __ballot_sync(0xffffffffu, on && g8 == 0);
          if (lane == 0) nib_all[it * 16 + warp] = (bal & 1u) | ((bal >> 7) & 2u) | ((bal >> 14) & 4u) | ((bal >> 21) & 8u);
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < nitem * 8; i += SB1_THREADS) {
      const int it = i >> 3, j = i & 7;
      const int l = it / NP, by = j + 8 * (it - l * NP);
      if (by < nby)
        reinterpret_cast<uint8_t*>(q.layer[l].bits)[c + G * by] = static_cast<uint8_t>(nib_all[it * 16 + 2 * j] | (nib_all[it * 16 + 2 * j + 1] << 4));
    }
  }
  // t and the nibbles were written to the slot area with ordinary stores; the bulk copies of phase R write the same
  // bytes through the async proxy
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  barrier_arrive(SB1_SYNC_FM);
  barrier_wait(SB1_SYNC_FM);

  // ================================================================== phase R: the rows, layer after layer
  // phase 1: warp w always works on quarter w & 3 of a row; its lanes' chunks of x stay in registers
  const int sub = warp & 3, gi = warp >> 2;
  uint4 xq[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int ch = lane + 32 * k;
    xq[k] = ch < qchunk ? reinterpret_cast<const uint4*>(x_s)[sub * qchunk + ch] : make_uint4(0, 0, 0, 0);
  }
  const int ng = flow_groups(L, G, I);
  const int gq = c % ng, mem = c / ng;           // this CTA's group and its place in it
  const int Gg = (G - gq + ng - 1) / ng;          // CTAs of the group
  const int GgMax = (G + ng - 1) / ng;            // partial vectors kept per layer
  const int nl = gq < L ? (L - gq + ng - 1) / ng : 0;  // layers of this CTA: gq, gq + ng, ...
  auto layer_of = [&](int j) { return gq + j * ng; };
  // CTAs c < L plan layer c's cache behind their rows: in a group these are its first Pm CTAs
  const int Pm = q.upkeep != nullptr ? min(Gg, max(0, (min(L, G) - gq + ng - 1) / ng)) : 0;
  auto load_words = [&](int l, uint32_t (&wv)[4]) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int w = tid * WPT + k;
      wv[k] = (k < WPT && w < W) ? __ldcg(q.layer[l].bits + w) : 0u;
    }
  };
  // The CTA's share of the active neurons of its j-th layer, ranks [s*K/Gg, (s+1)*K/Gg) of the set bits (s: its
  // share number in the group), into `dst`.  Returns their number.  Contains block barriers (three; the last one
  // publishes the list).
  auto build_list = [&](const uint32_t (&wv)[4], uint16_t* dst, int j) {
    int cnt = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) cnt += __popc(wv[k]);
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
    // Which shares are one neuron larger is a fixed pattern in the share number: the CTAs take the shares
    // rotated by the layer count, so that nobody collects the extra neuron of every layer.
    // The CTAs that run an index plan afterwards (the first Pm of the group) take FLOW_PLAN_WEIGHT sixteenths
    // of a share; in share order they are the cyclic interval [rot, rot + Pm).
    const int K = s_total;
    const int rot = (j * 5) % Gg;
    const int share = (mem + rot) % Gg;
    auto weight_below = [&](int p) {  // sum of the weights of the shares 0 .. p-1
      const int b = rot + Pm;
      const int planners = b <= Gg ? min(max(p - rot, 0), Pm) : min(p, b - Gg) + max(p - rot, 0);
      return 16 * p - (16 - FLOW_PLAN_WEIGHT) * planners;
    };
    const int wtot = 16 * Gg - (16 - FLOW_PLAN_WEIGHT) * Pm;
    const int lo = static_cast<int>(static_cast<long long>(K) * weight_below(share) / wtot);
    const int hi = static_cast<int>(static_cast<long long>(K) * weight_below(share + 1) / wtot);
    const int n = min(hi - lo, FLOW_LIST_CAP);
    int rho = s_wsum[warp] + inc - cnt;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      uint32_t b = wv[k];
      const int w = tid * WPT + k;
      if (rho + __popc(b) > lo && rho < hi) {
        while (b) {
          const int id = w * 32 + __ffs(b) - 1;
          b &= b - 1;
          if (rho >= lo && rho - lo < n) dst[rho - lo] = static_cast<uint16_t>(id);
          ++rho;
        }
      } else {
        rho += __popc(b);
      }
    }
    __syncthreads();
    return n;
  };

  // The slots are a ring of nsg groups of four.  Groups of neurons are numbered through all layers of the CTA:
  // group number i sits in slot group i % nsg.  n_cons groups have been consumed, n_issued requested; a slot
  // group may be requested again once every thread has passed a block barrier behind its last read (n_safe).
  // All of this is the same in every thread; warp 1 issues the copies.  jl, jg: the CTA's layer (counted in its
  // own layers) and the group of the next request.
  const int nsg = S >> 2;
  uint32_t ph = 0u;   // mbarrier phase parity per slot
  int n_cons = 0, n_issued = 0, n_safe = 0, sg_cons = 0, sg_issue = 0;
  int jl = 0, jg = 0;
  auto try_issue = [&](int j_cons, int n_c, int n_n, bool next_ok) {
    while (n_issued - n_safe < nsg) {
      if (jl == j_cons && jg * 4 >= n_c) {
        jl = j_cons + 1;
        jg = 0;
      }
      int n_of;
      if (jl == j_cons) n_of = n_c;
      else if (jl == j_cons + 1 && next_ok) n_of = n_n;
      else break;
      if (jg * 4 >= n_of) break;  // nothing more is known yet
      const int nv = min(4, n_of - 4 * jg);
      if (warp == 1 && lane < nv) {
        // the slot was only READ since its last copy, and every reader has passed a block barrier: no proxy fence
        const uint16_t* lst = (jl & 1) ? list_odd : list_even;
        const int s = sg_issue * 4 + lane;
        mbar_expect_tx(&bar[s], slot_bytes);
        bulk_load(slots + static_cast<size_t>(s) * slot_bytes,
                  static_cast<const char*>(q.layer[layer_of(jl)].cat) + static_cast<size_t>(lst[4 * jg + lane]) * slot_bytes, slot_bytes, &bar[s]);
      }
      ++jg;
      ++n_issued;
      sg_issue = sg_issue + 1 == nsg ? 0 : sg_issue + 1;
    }
  };

  uint32_t wnext[4] = {0u, 0u, 0u, 0u};
  int n_cur = 0, n_next = 0;
  if (nl > 0) {
    load_words(layer_of(0), wnext);
    n_cur = build_list(wnext, list_even, 0);
    if (nl > 1) load_words(layer_of(1), wnext);
  }

  for (int j = 0; j < nl; ++j) {
    const int l = layer_of(j);
    const StackLayerDesc& ld = q.layer[l];
    if (jl < j) {
      jl = j;
      jg = 0;
    }
    // the list of the CTA's next layer from the words requested a layer ago; then the words of the one after it
    const bool next_ok = j + 1 < nl;
    n_next = 0;
    if (next_ok) {
      n_next = build_list(wnext, ((j + 1) & 1) ? list_odd : list_even, j + 1);
      if (j + 2 < nl) load_words(layer_of(j + 2), wnext);
    } else {
      __syncthreads();
    }
    n_safe = n_cons;  // every thread has passed a block barrier since the last group was read
    try_issue(j, n_cur, n_next, next_ok);

    float acc[PASS][V];
#pragma unroll
    for (int k = 0; k < PASS; ++k)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[k][v] = 0.f;

    const int ngroups = (n_cur + 3) >> 2;
    for (int g = 0; g < ngroups; ++g) {
      const int s0 = sg_cons * 4;
      const int nv = min(4, n_cur - 4 * g);
      float2* pdg = pd + (g & 1) * 16;
      // ---- phase 1: a task is a quarter of a neuron's gate and up row against the matching quarter of x
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
      __syncthreads();  // the quarter sums of the group are there; every thread is done with the group before
      n_safe = n_cons;
      if (tid < nv) {
        const float2 p0 = pdg[tid * 4], p1 = pdg[tid * 4 + 1], p2 = pdg[tid * 4 + 2], p3 = pdg[tid * 4 + 3];
        const float gsum = (p0.x + p1.x) + (p2.x + p3.x);
        const float usum = (p0.y + p1.y) + (p2.y + p3.y);
        a_s[(g & 1) * 4 + tid] = q.has_gate ? apply_act(ld.act, gsum) * usum : apply_act(ld.act, usum);
      }
      try_issue(j, n_cur, n_next, next_ok);  // warp 1 requests while warp 0 forms a
      __syncthreads();  // a of the group
      // ---- phase 2: thread t owns the 16-byte column chunks t, t + 512
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
      ++n_cons;
      sg_cons = sg_cons + 1 == nsg ? 0 : sg_cons + 1;
      if (nsg == 1) {
        // Rows so long that a CTA holds a single group of four slots: the next group can only be requested into
        // the slots this one just left, so the request cannot wait for the next group's barrier.
        __syncthreads();
        n_safe = n_cons;
        try_issue(j, n_cur, n_next, next_ok);
      }
    }

    // ---- the CTA's partial output vector of the layer
    {
      float* dst = q.partial + (static_cast<size_t>(l) * GgMax + mem) * H;
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
    n_cur = n_next;
  }
  // ---- the index plan of layer c's weight cache (CTAs c < L; they took a smaller share of the rows to have the
  // time).  The masks are final since barrier FM; the plan's work space is the slot area, idle from here on.
  if (q.upkeep != nullptr && c < L) {
    __syncthreads();  // every thread is done with the slots
    const UpkeepArgs* ua = q.upkeep + c;
    plan_block(q.layer[c].bits, ua->cur_bits, ua->active, ua->pos_of, ua->lists, ua->jobs, ua->state, ua->stale, ua->lazy, I,
               reinterpret_cast<int32_t*>(slots));
    // the plan's work space becomes row buffers of phase C, which bulk copies write through the async proxy
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  barrier_arrive(SB1_SYNC_FP);
  barrier_wait(SB1_SYNC_FP);

  // ================================================================== phase O: out[l] = sum of the partial vectors
  // This CTA's columns: cpc float4 columns (<= 8).  Warp w sums layers w, w + 16, ...: lane = (vector group
  // ps = lane >> 3, column lane & 7) adds the vectors ps, ps + 4, ps + 8, ... of the layer's group in that order,
  // the four lanes of a column meet by butterfly.
  {
    const int ncol4 = H / 4;
    const int cpc = (ncol4 + G - 1) / G;
    const int col0 = c * cpc;
    const int ncols = max(0, min(cpc, ncol4 - col0));
    const int rcol = lane & 7, rps = lane >> 3;
    const bool sharded = q.peer.world > 1;
    const int epoch = peer_epoch0 + 1;
    float4 mine[(STACK_B1_MAX_LAYERS + SB1_WARPS - 1) / SB1_WARPS];
    int round = 0;
    for (int l = warp; l < L; l += SB1_WARPS, ++round) {
      const float* part = q.partial + static_cast<size_t>(l) * GgMax * H;
      const int nvec = (G - (l % ng) + ng - 1) / ng;  // CTAs of the layer's group
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      if (rcol < ncols) {
        for (int p0 = rps; p0 < nvec; p0 += 64) {  // sixteen vectors per lane in flight
          float4 v[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int p = p0 + 4 * u;
            v[u] = p < nvec ? __ldcg(reinterpret_cast<const float4*>(part + static_cast<size_t>(p) * H) + col0 + rcol) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            sum.x += v[u].x;
            sum.y += v[u].y;
            sum.z += v[u].z;
            sum.w += v[u].w;
          }
        }
      }
#pragma unroll
      for (int off = 8; off <= 16; off <<= 1) {
        sum.x += __shfl_xor_sync(0xffffffffu, sum.x, off);
        sum.y += __shfl_xor_sync(0xffffffffu, sum.y, off);
        sum.z += __shfl_xor_sync(0xffffffffu, sum.z, off);
        sum.w += __shfl_xor_sync(0xffffffffu, sum.w, off);
      }
      if (sharded) {  // lane rps carries element rps of the column's four
        const float own = rps == 0 ? sum.x : rps == 1 ? sum.y : rps == 2 ? sum.z : sum.w;
        if (rcol < ncols) peer_push(q.peer, epoch, static_cast<long long>(l) * H + (col0 + rcol) * 4 + rps, own);
      }
#pragma unroll
      for (int k = 0; k < static_cast<int>(sizeof(mine) / sizeof(mine[0])); ++k)
        if (k == round) mine[k] = sum;
    }
    round = 0;
    for (int l = warp; l < L; l += SB1_WARPS, ++round) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int k = 0; k < static_cast<int>(sizeof(mine) / sizeof(mine[0])); ++k)
        if (k == round) sum = mine[k];
      float own = rps == 0 ? sum.x : rps == 1 ? sum.y : rps == 2 ? sum.z : sum.w;
      if (rcol < ncols) {
        if (sharded) {  // add what the peers pushed, in rank order
          bool lost = false;
          own = peer_collect(q.peer, epoch, static_cast<long long>(l) * H + (col0 + rcol) * 4 + rps, own, &lost);
          if (lost) {
            atomicOr(q.peer.ctl + 2, DEV_TIMEOUT);
            if (q.layer[l].status) atomicOr(q.layer[l].status, DEV_TIMEOUT);
          }
        }
        static_cast<T*>(q.layer[l].out)[(col0 + rcol) * 4 + rps] = DT<T>::from_f(own);
      }
    }
  }

  // ================================================================== phase C: the rewritten rows of every cache
  // packed[m][pos] = pool[m][active[pos]] for every slot the plans listed (k_cache_copy_rows's work), all layers
  // at once.  A unit is (layer, listed slot, matrix) = one row; the units are dealt round robin to the CTAs.  A
  // CTA first looks up source and destination of up to 512 of its units, one per thread (two dependent loads,
  // issued while nothing else is in flight: behind bulk traffic such a load waits microseconds), then moves the
  // rows through NB row buffers in the idle slot area, one bulk copy in and one out per row.  Each buffer has an
  // owner thread, two per warp, so that the requests of a round do not queue behind one another in one warp.
  if (q.upkeep != nullptr) {
    struct RowJob {
      const char* sp;
      char* dp;  // null: nothing to copy
    };
    const int nrows = S * (ngu + 1);
    const size_t tail_bytes = STACK_B1_MAX_LAYERS * sizeof(UpkeepArgs) + 48 * sizeof(int) + SB1_THREADS * sizeof(RowJob);
    const int reserve = static_cast<int>((tail_bytes + row_bytes - 1) / row_bytes);
    const int NB = min(2 * SB1_WARPS, nrows - reserve);
    unsigned char* tail = slots + static_cast<size_t>(nrows - reserve) * row_bytes;
    UpkeepArgs* ua_s = reinterpret_cast<UpkeepArgs*>(tail);                                                   // [L]
    int* pre = reinterpret_cast<int*>(tail + STACK_B1_MAX_LAYERS * sizeof(UpkeepArgs));                       // [L + 1] units before layer l
    RowJob* table = reinterpret_cast<RowJob*>(tail + STACK_B1_MAX_LAYERS * sizeof(UpkeepArgs) + 48 * sizeof(int));  // [512]
    __syncthreads();
    for (int i = tid; i < L * static_cast<int>(sizeof(UpkeepArgs) / 8); i += SB1_THREADS)
      reinterpret_cast<uint64_t*>(ua_s)[i] = reinterpret_cast<const uint64_t*>(q.upkeep)[i];
    __syncthreads();
    const int nmat = ngu + 1;
    if (tid < L) pre[tid + 1] = ua_s[tid].lazy ? 0 : max(0, min(__ldcg(ua_s[tid].state + ST_NJOBS), I)) * nmat;
    __syncthreads();
    if (tid == 0) {
      pre[0] = 0;
      for (int l = 0; l < L; ++l) pre[l + 1] += pre[l];
    }
    __syncthreads();
    const int total = pre[L];
    const int mine = total > c ? (total - c + G - 1) / G : 0;  // units c, c + G, c + 2G, ...
    const int b = warp * 2 + lane;                              // buffer of an owner thread (lanes 0 and 1)
    const bool owner = lane < 2 && b < NB;
    uint64_t* mb = b < SB1_MAX_SLOTS ? &bar[b] : bar2 + ((b - SB1_MAX_SLOTS) & (SB1_MAX_SLOTS - 1));
    uint32_t par = b < SB1_MAX_SLOTS ? (ph >> b) & 1u : 0u;
    unsigned char* buf = slots + static_cast<size_t>(owner ? b : 0) * row_bytes;
    for (int k0 = 0; k0 < mine && NB > 0; k0 += SB1_THREADS) {
      RowJob rj{nullptr, nullptr};
      if (k0 + tid < mine) {
        const int u = (k0 + tid) * G + c;
        int lyr = 0;
        while (lyr + 1 < L && pre[lyr + 1] <= u) ++lyr;
        const int v = u - pre[lyr];
        const int job = v / nmat, m = v - job * nmat;
        const int pos = __ldcg(ua_s[lyr].jobs + job);
        if (pos >= 0 && pos < I) {
          const int src = __ldcg(ua_s[lyr].active + pos);
          if (src >= 0 && src < I) {
            rj.sp = static_cast<const char*>(ua_s[lyr].pool[m]) + static_cast<size_t>(src) * row_bytes;
            rj.dp = static_cast<char*>(ua_s[lyr].pk[m]) + static_cast<size_t>(pos) * row_bytes;
          }
        }
      }
      table[tid] = rj;
      __syncthreads();
      if (owner) {
        const int n = min(SB1_THREADS, mine - k0);
        for (int k = b; k < n; k += NB) {
          const RowJob w = table[k];
          if (w.dp == nullptr) continue;
          mbar_expect_tx(mb, row_bytes);
          bulk_load(buf, w.sp, row_bytes, mb);
          if (!mbar_wait_bounded(mb, par)) {  // the row never arrived: report it, write nothing, stop
            timed_out = true;
            break;
          }
          par ^= 1u;
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(w.dp), "r"(smem_u32(buf)), "r"(row_bytes) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the buffer may be overwritten
        }
      }
      __syncthreads();
    }
    if (owner) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  if (timed_out && q.layer[0].status) atomicOr(q.layer[0].status, DEV_TIMEOUT);
  if (c == 0 && tid == 0) q.sync[SB1_SYNC_GEN] = gen + 1u;
  if (q.peer.world > 1) {
    // the launch's last CTA advances the peer object's exchange number (every CTA read it at the start, and
    // every CTA is past its exchanges when it arrives here)
    __syncthreads();
    if (tid == 0 && atomicAdd(reinterpret_cast<unsigned*>(q.peer.ctl + 1), 1u) == gridDim.x - 1) {
      q.peer.ctl[1] = 0;
      *reinterpret_cast<volatile int*>(q.peer.ctl) = peer_epoch0 + 1;
    }
  }
}

template <typename T>
static int launch_stack_flow(const StackB1Args& a, size_t smem, size_t smem_limit, cudaStream_t s) {
  const int G = num_sms();
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_stack_flow<T, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_limit)));
    STX_CUDA(cudaFuncSetAttribute(k_stack_flow<T, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_limit)));
    STX_CUDA(cudaFuncSetAttribute(k_stack_flow<T, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_limit)));
    STX_CUDA(cudaFuncSetAttribute(k_stack_flow<T, 2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_limit)));
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
  const bool one = a.H / DT<T>::V <= SB1_THREADS;
  const bool single = ((a.I + 7) / 8 + G - 1) / G <= 8;  // one pass of eight mask bytes per CTA and layer
  static_assert(FLOW_MAX_PASSES == 2, "two instantiations of the pass count");
  if (single) {
    if (one) STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_flow<T, 1, 1>, a));
    else STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_flow<T, 2, 1>, a));
  } else {
    if (one) STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_flow<T, 1, 2>, a));
    else STX_CUDA(cudaLaunchKernelEx(&cfg, k_stack_flow<T, 2, 2>, a));
  }
  return STX_OK;
}

int stack_flow_launch(const StackB1Args& a, int dtype, size_t smem, size_t smem_limit, cudaStream_t s) {
  switch (dtype) {
    case STX_F32: return launch_stack_flow<float>(a, smem, smem_limit, s);
    case STX_F16: return launch_stack_flow<__half>(a, smem, smem_limit, s);
    default: return launch_stack_flow<__nv_bfloat16>(a, smem, smem_limit, s);
  }
}

}  // namespace stx
