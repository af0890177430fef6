// Sparse gated MLP for 1..8 rows as ONE kernel per layer: predictor scores of the CTA's own neurons, mask bytes,
// row gather and the whole MLP (k_mlp_b1: one row; k_mlp_bn: 2..8 rows of 16-bit gated weights with both
// projections on the tensor pipe), then the sum of the per-CTA partial vectors (k_partial_reduce,
// k_partial_reduce4), which also carries the all-reduce of sharded layers.
#include "stx_mlp_stream.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace stx {

// ------------------------------------------------------------------------------------------
// Batch 1: gate/up, activation and the down projection of a neuron in one pass.
//
// k_mlp_b1: a CTA owns S "slots" (one per warp w < S); a slot holds the gate, up and down
// row of one neuron, fetched by bulk copies the moment the CTA knows its neurons.  With
// S * gridDim.x >= K (the usual case) every byte the kernel reads is in flight from the start.
//   phase 1  warp w: gate/up dot products of its neuron against x -> a = act(g) * u -> a_s[w]
//   phase 2  all threads: thread t owns the 16-byte column chunks t, t + blockDim.x, ... and adds
//            a_s[slot] * down_row[slot][chunk] over the slots in ascending order (registers)
// A second round (K > S * gridDim.x) re-fills a slot's gate/up part right after phase 1 and its
// down part after phase 2.  At the end each thread writes its columns of the CTA's partial
// output vector; k_partial_reduce adds the per-CTA vectors in ascending CTA order:
// deterministic, no atomics, nothing to re-zero.  One launch that streams gate, up and down
// rows pays the launch, listing and first-byte latency once instead of twice.
constexpr int B1_MAX_SLOTS = 16;
constexpr int B1_MAX_PASS = 2;    // column chunks per thread: H / V <= 2 * 512
constexpr int B1_HEADER = 512;    // [0,256) 2 x 16 mbarriers | [256,320) a_s

struct MlpB1Args {
  GateUpArgs g;          // x, gate, up, combined, gather spec, K, H, act, has_gate; nwarps = slots S
  const void* down;
  float* partial;        // [gridDim.x][H]
  // Predictor back half inside the kernel (Bm != nullptr): scores of the CTA's own neurons from
  // t = A x (fp32 [r], written by the preceding kernel), threshold, mask bytes to `bits`.
  const float* t;
  const void* Bm;        // [I][r]
  uint32_t* bits;        // mask words of the layer (written bytewise)
  int r;
  float tau;
  int* xchg;             // k_mlp_bn: count/id exchange between the CTAs (BN_XCHG_BYTES, zero before the first launch) or null
};

// With the predictor's back half fused in, CTA c owns mask bytes c, c + G, c + 2G, ... (8
// neurons each): it needs nobody else's scores to know which of its rows to fetch, so the
// mask never makes a round trip through global memory on the critical path.  The price is
// balance: the CTAs' active counts differ (binomially) instead of by at most one.
//
// Measured alternative, not kept: letting the CTAs publish their counts and hand their excess
// to lighter CTAs (a deterministic plan from the exchanged counts) balanced the work, but the
// exchange's small messages queue behind the bulk row traffic of the same SM and the two
// round trips cost more than the imbalance they removed.
constexpr int B1_MAX_BYTES = 24;   // mask bytes per CTA: ceil(ceil(I / 8) / G) <= 24 (192 neurons)
constexpr int B1_LIST_CAP = 192;

// Shared-memory footprint of t for the fused predictor back half: B rows, stored so that the eight
// lanes of a neuron read one contiguous 128-byte line per load: [b][c4][v4][g][4 floats] for chunk
// c = g + 8*c4 and elements 4*v4 .. 4*v4+3 of the chunk (V elements per chunk, ceil(r/V/8) groups c4).
__host__ __device__ inline size_t pred_t_smem_bytes(int B, int r, int V) {
  return r > 0 ? static_cast<size_t>(B) * ((r / V + 7) / 8) * 8 * V * sizeof(float) : 0;
}

// Predictor back half for the calling CTA's neurons (mask bytes blockIdx.x, + gridDim.x, ...),
// all 512 threads.  Same arithmetic as k_pred_scores: 8 lanes per neuron, lane g takes the
// 16-byte chunks g, g + 8, ... of the r-long row in order, then a butterfly over the 8 lanes
// (4, 2, 1); the mask bit is the OR over the B rows.  The CTA's slice of the up matrix is loaded
// BEFORE the dependency wait (weights do not depend on the preceding kernel); the function
// contains the kernel's griddepcontrol wait.  t_s: shared fp32 [B][r].  Writes the mask bytes to
// `bits` and the CTA's active neurons, ascending, to s_my; returns their number.
template <typename T>
__device__ __forceinline__ int cta_scores_and_list(const T* __restrict__ Bm, const float* __restrict__ t_gl, float* t_s, int B,
                                                   int r, int I, float tau, uint32_t* bits, int32_t* s_my, uint32_t* s_nib,
                                                   uint8_t* s_bytes, int* s_nlocal) {
  constexpr int V = DT<T>::V;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x;
  const int rch = r / V;  // <= 32
  const int nc4 = (rch + 7) >> 3;
  const int NBY = (I + 7) >> 3;
  const int nby = NBY > static_cast<int>(blockIdx.x) ? (NBY - 1 - static_cast<int>(blockIdx.x)) / G + 1 : 0;
  const int g = tid & 7;
  // Two register sets of weights: a pass computes from one set while the loads of the next pass
  // into the other set are in flight (the first set is loaded before the dependency wait).
  float wv0[4][V], wv1[4][V];
  bool ok0 = false, ok1 = false;
  auto load_w = [&](int pass, float (&w)[4][V], bool& ok) {
    const int kk = pass * 8 + (tid >> 6);
    const int n = 8 * (static_cast<int>(blockIdx.x) + G * kk) + ((tid >> 3) & 7);
    ok = kk < nby && n < I;
#pragma unroll
    for (int c4 = 0; c4 < 4; ++c4) {
      const int c = g + 8 * c4;
#pragma unroll
      for (int v = 0; v < V; ++v) w[c4][v] = 0.f;
      if (ok && c < rch) Unpack<T>::run(ld_stream16(Bm + static_cast<size_t>(n) * r + c * V), w[c4]);
    }
  };
  load_w(0, wv0, ok0);
  pdl_wait();
  pdl_launch_dependents();
  if (8 < nby) load_w(1, wv1, ok1);
  for (int k = tid; k < B * r; k += blockDim.x) {
    const int b = k / r, e = k - b * r, c = e / V, v = e - c * V;
    t_s[(((b * nc4 + (c >> 3)) * (V / 4) + (v >> 2)) * 8 + (c & 7)) * 4 + (v & 3)] = __ldcg(t_gl + k);
  }
  __syncthreads();
  const float tau_r = DT<T>::round_f(tau);
  constexpr int SB = 8;  // batch rows whose chains run side by side (each row's own order is unchanged)
  auto run_pass = [&](int pass, float (&w)[4][V], bool& ok) {
    bool on = false;
    for (int b0 = 0; b0 < B; b0 += SB) {
      float sc[SB];
#pragma unroll
      for (int b = 0; b < SB; ++b) sc[b] = 0.f;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const int c = g + 8 * c4;
        if (c < rch) {
#pragma unroll
          for (int b = 0; b < SB; ++b) {
            if (b0 + b < B) {
              // elements 4*v4 .. of chunk c of row b0+b: one 128-byte line per (row, c4, v4) for the 8 lanes of a neuron
              const float4* tb = reinterpret_cast<const float4*>(t_s) + (((b0 + b) * nc4 + c4) * (V / 4)) * 8 + g;
#pragma unroll
              for (int v4 = 0; v4 < V / 4; ++v4) {
                const float4 tv = tb[v4 * 8];
                sc[b] = fmaf(tv.x, w[c4][4 * v4], sc[b]);
                sc[b] = fmaf(tv.y, w[c4][4 * v4 + 1], sc[b]);
                sc[b] = fmaf(tv.z, w[c4][4 * v4 + 2], sc[b]);
                sc[b] = fmaf(tv.w, w[c4][4 * v4 + 3], sc[b]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int b = 0; b < SB; ++b) {
        float t = sc[b];
        t += __shfl_xor_sync(0xffffffffu, t, 4);
        t += __shfl_xor_sync(0xffffffffu, t, 2);
        t += __shfl_xor_sync(0xffffffffu, t, 1);
        on = on || (b0 + b < B && DT<T>::round_f(t) >= tau_r);
      }
    }
    on = on && ok;
    if ((pass + 2) * 8 < nby) load_w(pass + 2, w, ok);  // this set is free again
    const uint32_t bal = __ballot_sync(0xffffffffu, on && g == 0);
    if (lane == 0) s_nib[warp] = (bal & 1u) | ((bal >> 7) & 2u) | ((bal >> 14) & 4u) | ((bal >> 21) & 8u);
    __syncthreads();
    if (tid < 8 && pass * 8 + tid < nby) {
      const uint32_t byte = s_nib[2 * tid] | (s_nib[2 * tid + 1] << 4);
      s_bytes[pass * 8 + tid] = static_cast<uint8_t>(byte);
      reinterpret_cast<uint8_t*>(bits)[blockIdx.x + G * (pass * 8 + tid)] = static_cast<uint8_t>(byte);
    }
    __syncthreads();
  };
  for (int pass = 0; pass * 8 < nby; pass += 2) {
    run_pass(pass, wv0, ok0);
    if ((pass + 1) * 8 < nby) run_pass(pass + 1, wv1, ok1);
  }
  if (warp == 0) {  // the CTA's active neurons in ascending order
    int carry = 0;
    for (int base = 0; base < nby; base += 32) {
      const int kk = base + lane;
      uint32_t byte = kk < nby ? s_bytes[kk] : 0u;
      const int cnt = __popc(byte);
      int inc = cnt;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += v;
      }
      int pos = carry + inc - cnt;
      while (byte) {
        const int n = 8 * (static_cast<int>(blockIdx.x) + G * kk) + __ffs(byte) - 1;
        byte &= byte - 1;
        if (pos < B1_LIST_CAP) s_my[pos] = n;
        ++pos;
      }
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) *s_nlocal = min(carry, B1_LIST_CAP);
  }
  __syncthreads();
  return *s_nlocal;
}

template <typename T>
__global__ void __launch_bounds__(512, 1) k_mlp_b1(const MlpB1Args q) {
  constexpr int V = DT<T>::V;
  const GateUpArgs& p = q.g;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int S = p.nwarps;
  const int H = p.H, nchunk = H / V;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const int ngu = p.has_gate ? 2 : 1;

  uint64_t* bar_gu = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar_d = bar_gu + B1_MAX_SLOTS;
  float* a_s = reinterpret_cast<float*>(smem + 256);
  // [B1_HEADER, +t_bytes): t of the fused predictor back half
  const size_t t_bytes = q.Bm ? pred_t_smem_bytes(1, q.r, V) : 0;
  T* x_s = reinterpret_cast<T*>(smem + B1_HEADER + t_bytes);
  const size_t x_bytes = (sizeof(T) * H + 127) / 128 * 128;
  unsigned char* gu_bufs = smem + B1_HEADER + t_bytes + x_bytes;
  unsigned char* d_bufs = gu_bufs + static_cast<size_t>(S) * ngu * row_bytes;
  unsigned char* my_gu = gu_bufs + static_cast<size_t>(warp) * ngu * row_bytes;

  __shared__ int32_t s_my[GATHER_MY_CAP];
  __shared__ uint32_t s_nib[16];
  __shared__ uint8_t s_bytes[B1_MAX_BYTES];
  __shared__ int s_nlocal;
  const char* gsrc = static_cast<const char*>(p.gate);
  const char* usrc = static_cast<const char*>(p.up);
  const char* dsrc = static_cast<const char*>(q.down);
  const bool fused = q.Bm != nullptr;
  T* combined = fused ? nullptr : static_cast<T*>(p.combined);
  const bool gather = fused || p.mask_bits != nullptr;
  const int G = gridDim.x;

  if (tid == 0) {
    for (int w = 0; w < S; ++w) {
      mbar_init(&bar_gu[w], 1);
      mbar_init(&bar_d[w], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  int K = 0, nlocal = 0;
  if (fused) {
    nlocal = cta_scores_and_list<T>(static_cast<const T*>(q.Bm), q.t, reinterpret_cast<float*>(smem + B1_HEADER), 1, q.r, p.I,
                                    q.tau, q.bits, s_my, s_nib, s_bytes, &s_nlocal);
  } else {
    pdl_wait();
    pdl_launch_dependents();
    K = gather ? cta_list_active(p.mask_bits, p.I, 1, s_my, p.idx_out, p.count_out) : (p.K_dev ? *p.K_dev : p.K_host);
    if (!gather) __syncthreads();
    nlocal = K > static_cast<int>(blockIdx.x) ? (K - 1 - static_cast<int>(blockIdx.x)) / G + 1 : 0;
  }

  // local neuron s (rank blockIdx.x + G*s) -> slot s % S; called by lane 0 of warp s % S
  auto row_of = [&](int s) { return gather ? s_my[s] : static_cast<int>(blockIdx.x) + G * s; };
  auto issue_gu = [&](int s) {
    mbar_expect_tx(&bar_gu[warp], row_bytes * ngu);
    const size_t off = static_cast<size_t>(row_of(s)) * row_bytes;
    if (p.has_gate) bulk_load(my_gu, gsrc + off, row_bytes, &bar_gu[warp]);
    bulk_load(my_gu + (p.has_gate ? row_bytes : 0), usrc + off, row_bytes, &bar_gu[warp]);
  };
  auto issue_d = [&](int s) {
    mbar_expect_tx(&bar_d[warp], row_bytes);
    bulk_load(d_bufs + static_cast<size_t>(warp) * row_bytes, dsrc + static_cast<size_t>(row_of(s)) * row_bytes, row_bytes,
              &bar_d[warp]);
  };
  if (warp < S && lane == 0 && warp < nlocal) {  // the rows stream in while x is staged
    issue_gu(warp);
    issue_d(warp);
  }
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    uint4* xs4 = reinterpret_cast<uint4*>(x_s);
    for (int i = tid; i < nchunk; i += blockDim.x) xs4[i] = xg[i];
  }
  __syncthreads();

  bool timed_out = false;
  float acc[B1_MAX_PASS][V];
#pragma unroll
  for (int k = 0; k < B1_MAX_PASS; ++k)
#pragma unroll
    for (int v = 0; v < V; ++v) acc[k][v] = 0.f;

  const int nrounds = (nlocal + S - 1) / S;
  for (int r = 0; r < nrounds; ++r) {
    const uint32_t parity = static_cast<uint32_t>(r) & 1u;
    const int s = warp + r * S;
    if (warp < S && s < nlocal) {
      const int j = static_cast<int>(blockIdx.x) + G * s;  // rank of this neuron
      if (!mbar_wait_bounded(&bar_gu[warp], parity)) timed_out = true;
      const T* grow = reinterpret_cast<const T*>(my_gu);
      const T* urow = reinterpret_cast<const T*>(my_gu + (p.has_gate ? row_bytes : 0));
      float ag = 0.f, au = 0.f;
      int c = lane;
      for (; c + 32 < nchunk; c += 64) {  // two chunks per iteration: independent chains
        float wu0[V], wu1[V], wg0[V], wg1[V], x0[V], x1[V];
        Unpack<T>::run(*reinterpret_cast<const uint4*>(urow + c * V), wu0);
        Unpack<T>::run(*reinterpret_cast<const uint4*>(urow + (c + 32) * V), wu1);
        Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + c * V), x0);
        Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + (c + 32) * V), x1);
        float su0 = 0.f, su1 = 0.f, sg0 = 0.f, sg1 = 0.f;
        if (p.has_gate) {
          Unpack<T>::run(*reinterpret_cast<const uint4*>(grow + c * V), wg0);
          Unpack<T>::run(*reinterpret_cast<const uint4*>(grow + (c + 32) * V), wg1);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) {
          su0 = fmaf(x0[v], wu0[v], su0);
          su1 = fmaf(x1[v], wu1[v], su1);
          if (p.has_gate) {
            sg0 = fmaf(x0[v], wg0[v], sg0);
            sg1 = fmaf(x1[v], wg1[v], sg1);
          }
        }
        au += su0 + su1;
        ag += sg0 + sg1;
      }
      for (; c < nchunk; c += 32) {
        float wu[V], wg[V], xv[V];
        Unpack<T>::run(*reinterpret_cast<const uint4*>(urow + c * V), wu);
        Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + c * V), xv);
        if (p.has_gate) Unpack<T>::run(*reinterpret_cast<const uint4*>(grow + c * V), wg);
        float su = 0.f, sg = 0.f;
#pragma unroll
        for (int v = 0; v < V; ++v) {
          su = fmaf(xv[v], wu[v], su);
          if (p.has_gate) sg = fmaf(xv[v], wg[v], sg);
        }
        au += su;
        ag += sg;
      }
      const float u = warp_sum_xor(au);
      const float gsum = p.has_gate ? warp_sum_xor(ag) : 0.f;
      const float a = p.has_gate ? apply_act(p.act, gsum) * u : apply_act(p.act, u);
      if (lane == 0) {
        a_s[warp] = a;
        if (combined) {
          combined[j] = DT<T>::from_f(a);
          if (p.has_gate) combined[K + j] = DT<T>::from_f(u);
        }
      }
      __syncwarp();
      if (lane == 0 && s + S < nlocal) {  // the gate/up part of the slot is free again
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue_gu(s + S);
      }
    }
    __syncthreads();  // a_s of this round complete

    const int nvalid = min(S, nlocal - r * S);
    if (tid < nchunk) {
      for (int slot = 0; slot < nvalid; ++slot) {
        if (!mbar_wait_bounded(&bar_d[slot], parity)) timed_out = true;
        const float a = a_s[slot];
        const T* drow = reinterpret_cast<const T*>(d_bufs + static_cast<size_t>(slot) * row_bytes);
#pragma unroll
        for (int k = 0; k < B1_MAX_PASS; ++k) {
          const int cc = tid + k * static_cast<int>(blockDim.x);
          if (cc < nchunk) {
            float wd[V];
            Unpack<T>::run(*reinterpret_cast<const uint4*>(drow + cc * V), wd);
#pragma unroll
            for (int v = 0; v < V; ++v) acc[k][v] = fmaf(a, wd[v], acc[k][v]);
          }
        }
      }
    }
    if (r + 1 < nrounds) {
      __syncthreads();  // every thread is done with a_s and the down rows of this round
      if (warp < S && lane == 0 && s + S < nlocal) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue_d(s + S);
      }
    }
  }
  if (timed_out && p.status) atomicOr(p.status, DEV_TIMEOUT);

  float* dst = q.partial + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
  for (int k = 0; k < B1_MAX_PASS; ++k) {
    const int cc = tid + k * static_cast<int>(blockDim.x);
    if (cc < nchunk) {
#pragma unroll
      for (int v = 0; v < V; v += 4)
        *reinterpret_cast<float4*>(dst + cc * V + v) = make_float4(acc[k][v], acc[k][v + 1], acc[k][v + 2], acc[k][v + 3]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// 2..8 rows, 16-bit weights, gated: the same one-kernel structure as k_mlp_b1 (scores of the CTA's
// own neurons -> mask bytes -> bulk copies of gate/up/down rows -> MLP -> per-CTA partial [B][H]),
// with the gate/up dot products on the tensor pipe.
//
// The CTA walks its neurons TN (<= 8) at a time.  Three shared-memory buffers hold one such tile:
//   X  the first halves (columns 0 .. H/2) of the TN gate and up rows
//   Y  their second halves
//   Z  the TN down rows
//   phase 1a/1b  A tile of mma.m16n8k16 = the 2*TN gate/up rows (neuron e in tile rows 2e, 2e+1),
//                B tile = x^T (8 batch columns); each of the 16 warps owns a sixteenth of each half
//                of H and keeps its accumulators in registers from X to Y; the sixteen partial
//                sums meet in shared memory and are added in warp order -> a[e][b] = act(g) * u
//   phase 2      also an mma: D[h][b] += down^T[h][e] * a[e][b] with m = 16 columns of H, n = the 8
//                batch rows, k = the (up to) 8 neurons of the tile (m16n8k8).  Warp w owns columns
//                w*H/16 .. and keeps its H/16 x 8 outputs in registers; the A fragments come
//                transposed out of the down rows with ldmatrix.trans; a is rounded to the model
//                dtype for the B fragment (as the reference's own activations are).
// A buffer is re-filled with the next tile's rows as soon as its phase is over, so two of the three
// are in flight or ready while the third is being read.  Filling all 16 tile rows matters: the
// kernel's instruction stream is dominated by the fragment loads of x (64 KB per tile pass) and the
// mma issue, both per tile, not per neuron.
// Rows of x and of the weights sit 64 bytes apart from a multiple of 128 so that the fragment
// loads of different rows fall into different banks.
// Balance.  A CTA's share of the active neurons is binomial; with tens of neurons per CTA the
// heaviest CTA would finish a quarter later than the mean.  So every CTA publishes its count and
// its list in global memory right after listing, starts on its first tile, and meanwhile reads
// everybody's counts: CTAs above the cap Tk = ceil(K / G) hand the tail of their list to CTAs
// below it, in ascending CTA order.  The plan is a pure function of the counts (deterministic);
// every published word carries the launch's epoch, so no fence orders the stores and a reader
// polls the word itself (bounded).  The exchange rides behind the first tile's loads.
constexpr int BN_XCHG_COUNTS = 64;   // int offsets inside the exchange buffer: [0] epoch
constexpr int BN_XCHG_IDS = BN_XCHG_COUNTS + 256;
constexpr size_t BN_XCHG_BYTES = sizeof(int) * BN_XCHG_IDS + sizeof(int2) * 256 * B1_LIST_CAP;
constexpr int BN_MAX_GRID = 160;
constexpr uint32_t BN_POLL_LIMIT = 1u << 20;

constexpr int BN_MAX = 8;
constexpr int BN_TN_MAX = 8;
constexpr int BN_MT_MAX = 16;  // m-tiles of 16 columns per warp: H <= 16 * 16 * 16
constexpr int BN_HEADER = 1024;                // [0,64) 3 mbarriers | [256,512) a_s [8 neurons][8 rows of the batch]
constexpr int BN_RED_BYTES = 16 * 16 * 8 * 4;  // [warp][tile row][batch] fp32

template <typename T>
__global__ void __launch_bounds__(512, 1) k_mlp_bn(const MlpB1Args q) {
  constexpr int V = DT<T>::V;
  static_assert(sizeof(T) == 2, "16-bit weights only");
  const GateUpArgs& p = q.g;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int TN = p.nwarps, B = p.B;
  const int H = p.H, nchunk = H / V;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t half_bytes = row_bytes / 2;
  const uint32_t rstride = row_bytes + 64, hstride = half_bytes + 64;
  const uint32_t zstride = row_bytes + 16;  // down rows 16 bytes off a multiple of 128: conflict-free ldmatrix

  uint64_t* bar_x = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar_y = bar_x + 1;
  uint64_t* bar_z = bar_x + 2;
  uint32_t* a_pk = reinterpret_cast<uint32_t*>(smem + 256);  // [neuron pair][batch row]: (a[2k][b], a[2k+1][b]) in the model dtype
  const size_t t_bytes = pred_t_smem_bytes(B, q.r, V);
  float* t_s = reinterpret_cast<float*>(smem + BN_HEADER);
  float* red_s = reinterpret_cast<float*>(smem + BN_HEADER + t_bytes);
  unsigned char* x_s = smem + BN_HEADER + t_bytes + BN_RED_BYTES;        // 8 rows of rstride
  unsigned char* X = x_s + static_cast<size_t>(BN_MAX) * rstride;         // [TN][gate, up] half rows of hstride
  unsigned char* Y = X + static_cast<size_t>(TN) * 2 * hstride;
  unsigned char* Z = Y + static_cast<size_t>(TN) * 2 * hstride;           // [TN] rows of zstride

  __shared__ int32_t s_my[GATHER_MY_CAP];
  __shared__ uint32_t s_nib[16];
  __shared__ uint8_t s_bytes[B1_MAX_BYTES];
  __shared__ int s_nlocal;
  const char* gsrc = static_cast<const char*>(p.gate);
  const char* usrc = static_cast<const char*>(p.up);
  const char* dsrc = static_cast<const char*>(q.down);

  if (tid == 0) {
    mbar_init(bar_x, 1);
    mbar_init(bar_y, 1);
    mbar_init(bar_z, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int G = gridDim.x;
  const bool balance = q.xchg != nullptr && G <= BN_MAX_GRID;
  __shared__ int s_epoch, s_plan[4];
  // the exchange's epoch was written by this layer's previous launch: read it ahead of everything
  // (the barriers inside the front-end make it visible to all threads)
  if (balance && tid == 0) s_epoch = *reinterpret_cast<volatile int*>(q.xchg);
  int nlocal = cta_scores_and_list<T>(static_cast<const T*>(q.Bm), q.t, t_s, B, q.r, p.I, q.tau, q.bits, s_my, s_nib,
                                      s_bytes, &s_nlocal);
  int niter = (nlocal + TN - 1) / TN;
  int epoch = 0;
  const int n_own = nlocal;
  if (balance) {  // publish the count and the list
    epoch = static_cast<int>(static_cast<unsigned>(s_epoch) + 1u);
    if (tid == 0)
      *reinterpret_cast<volatile int*>(q.xchg + BN_XCHG_COUNTS + blockIdx.x) = ((epoch & 0x1fffff) << 10) | n_own;
    if (tid < n_own) {
      int2* dst = reinterpret_cast<int2*>(q.xchg + BN_XCHG_IDS) + blockIdx.x * B1_LIST_CAP + tid;
      asm volatile("st.relaxed.gpu.global.v2.s32 [%0], {%1,%2};" ::"l"(dst), "r"(s_my[tid]), "r"(epoch) : "memory");
    }
  }

  // One warp fills a buffer with the rows of tile j (warp 0: X, warp 1: Y, warp 2: Z): lane 0 arms
  // the barrier with the byte count, then lane e issues the copies of neuron e, so the issue cost
  // of a dozen bulk copies does not sit on one thread between two block-wide barriers.
  auto fill = [&](int which, int j) {
    if (j >= niter || warp != which) return;
    const int nv = min(TN, nlocal - j * TN);
    uint64_t* bar = which == 0 ? bar_x : (which == 1 ? bar_y : bar_z);
    if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(nv) * (which < 2 ? 2 * half_bytes : row_bytes));
    __syncwarp();
    if (lane < nv) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const int e = lane;
      const size_t row = static_cast<size_t>(s_my[j * TN + e]) * row_bytes;
      if (which < 2) {
        unsigned char* buf = which == 0 ? X : Y;
        const size_t col = which == 0 ? 0 : half_bytes;
        bulk_load(buf + static_cast<size_t>(2 * e) * hstride, gsrc + row + col, half_bytes, bar);
        bulk_load(buf + static_cast<size_t>(2 * e + 1) * hstride, usrc + row + col, half_bytes, bar);
      } else {
        bulk_load(Z + static_cast<size_t>(e) * zstride, dsrc + row, row_bytes, bar);
      }
    }
  };
  // the first tile is this CTA's own in any case when it is full; a short list may still grow
  const bool early = !balance || n_own >= TN;
  if (early) {
    fill(0, 0);
    fill(1, 0);
  }
  if (early && niter > 0 && nlocal < TN) {
    // a short only tile: the unused down rows are multiplied by a = 0, so they must hold finite numbers
    for (int i = tid; i < TN * static_cast<int>(zstride / 16); i += blockDim.x)
      reinterpret_cast<uint4*>(Z)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }
  if (early) fill(2, 0);
  for (int i = tid; i < BN_MAX * nchunk; i += blockDim.x) {  // rows beyond B are zero
    const int b = i / nchunk, c = i - b * nchunk;
    const uint4 v = b < B ? ld_cached16(static_cast<const T*>(p.x) + static_cast<size_t>(b) * H + c * V) : make_uint4(0, 0, 0, 0);
    *reinterpret_cast<uint4*>(x_s + static_cast<size_t>(b) * rstride + c * 16) = v;
  }
  bool timed_out = false;
  if (balance) {
    // ---- everybody's counts (bounded wait; 16-byte loads: one request per line of the count array)
    int* xc = q.xchg;
    const int tag = epoch & 0x1fffff;
    int* s_cnt = s_my + B1_LIST_CAP;        // [BN_MAX_GRID]
    int* s_exE = s_cnt + BN_MAX_GRID;       // [BN_MAX_GRID] exclusive prefix of the excess counts
    if (tid * 4 < G) {
      int v[4] = {0, 0, 0, 0};
      bool got = false;
      for (uint32_t it = 0; it < BN_POLL_LIMIT; ++it) {
        asm volatile("ld.relaxed.gpu.global.v4.s32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                     : "l"(xc + BN_XCHG_COUNTS + tid * 4)
                     : "memory");
        got = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) got = got && (tid * 4 + i >= G || (v[i] >> 10) == tag);
        if (got) break;
        __nanosleep(100);
      }
      if (!got) timed_out = true;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (tid * 4 + i < G) s_cnt[tid * 4 + i] = got ? (v[i] & 1023) : 0;
    }
    const int any_timeout = __syncthreads_or(timed_out ? 1 : 0);
    if (warp == 0) {
      int total = 0;
      for (int c = lane; c < G; c += 32) total += s_cnt[c];
      total = __reduce_add_sync(0xffffffffu, total);
      const int Tk = max(TN, (total + G - 1) / G);  // cap: nobody keeps more than this
      int E = 0;
      for (int c = lane; c < G; c += 32) E += max(0, s_cnt[c] - Tk);
      E = __reduce_add_sync(0xffffffffu, E);
      // exclusive prefixes over CTAs in ascending order: excess (everybody needs all), room (this CTA's)
      int carry_e = 0, carry_s = 0, my_P = 0;
      for (int base = 0; base < G; base += 32) {
        const int c = base + lane;
        const int n = c < G ? s_cnt[c] : 0;
        const int ex = c < G ? max(0, n - Tk) : 0;
        const int sp = c < G ? max(0, Tk - n) : 0;
        int ie = ex, is = sp;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
          const int ve = __shfl_up_sync(0xffffffffu, ie, off);
          const int vs = __shfl_up_sync(0xffffffffu, is, off);
          if (lane >= off) {
            ie += ve;
            is += vs;
          }
        }
        if (c < G) s_exE[c] = carry_e + ie - ex;
        if (c == static_cast<int>(blockIdx.x)) my_P = carry_s + is - sp;
        carry_e += __shfl_sync(0xffffffffu, ie, 31);
        carry_s += __shfl_sync(0xffffffffu, is, 31);
      }
      my_P = __reduce_add_sync(0xffffffffu, my_P);  // one lane holds it
      if (lane == 0) {
        s_plan[0] = min(n_own, Tk);                        // neurons this CTA keeps
        s_plan[1] = max(0, min(Tk - n_own, E - my_P));     // neurons it takes over
        s_plan[2] = my_P;
        s_plan[3] = Tk;
      }
    }
    __syncthreads();
    if (!any_timeout) {
      const int keep = s_plan[0], take = s_plan[1], my_P = s_plan[2], Tk = s_plan[3];
      if (tid < take) {
        const int o = my_P + tid;  // index of the excess neuron this thread resolves
        int src = 0;
        for (int c = 0; c < G; ++c)
          if (s_exE[c] <= o) src = c;  // the last CTA whose prefix is <= o owns excess neuron o
        const int2* idp = reinterpret_cast<const int2*>(xc + BN_XCHG_IDS) + src * B1_LIST_CAP + Tk + (o - s_exE[src]);
        int id = 0, ep = 0;
        bool got = false;
        for (uint32_t it = 0; it < BN_POLL_LIMIT && !got; ++it) {
          asm volatile("ld.relaxed.gpu.global.v2.s32 {%0,%1}, [%2];" : "=r"(id), "=r"(ep) : "l"(idp) : "memory");
          got = ep == epoch;
          if (!got) __nanosleep(100);
        }
        if (!got) timed_out = true;
        s_my[keep + tid] = got ? id : 0;
      }
      nlocal = keep + take;
      niter = (nlocal + TN - 1) / TN;
    }
    // every CTA has published, hence read the epoch: advance it for the next launch
    if (blockIdx.x == 0 && tid == 0) *reinterpret_cast<volatile int*>(xc) = epoch;
    __syncthreads();
    if (!early) {
      if (niter > 0 && nlocal < TN) {  // as above: unused down rows must hold finite numbers
        for (int i = tid; i < TN * static_cast<int>(zstride / 16); i += blockDim.x)
          reinterpret_cast<uint4*>(Z)[i] = make_uint4(0, 0, 0, 0);
        __syncthreads();
      }
      fill(0, 0);
      fill(1, 0);
      fill(2, 0);
    }
  }
  __syncthreads();

  // outputs of this warp: m-tile mt = columns warp*H/16 + 16*mt .., fragment rows gq / gq + 8, batch 2tq / 2tq + 1
  float dacc[BN_MT_MAX][4];
#pragma unroll
  for (int mt = 0; mt < BN_MT_MAX; ++mt)
#pragma unroll
    for (int k = 0; k < 4; ++k) dacc[mt][k] = 0.f;
  const int MT = H / 256;  // m-tiles per warp (even)

  const int nwh = H / 64;  // windows (32 consecutive k = 64 bytes) per half row
  const int w_lo = (nwh * warp) / 16, w_hi = (nwh * (warp + 1)) / 16;  // this warp's share of each half
  for (int it = 0; it < niter; ++it) {
    const uint32_t parity = static_cast<uint32_t>(it) & 1u;
    const int nv = min(TN, nlocal - it * TN);
    // tile rows of this lane: gq (neuron gq >> 1) and gq + 8 (neuron 4 + (gq >> 1)); gate even, up odd
    const bool lo_on = gq < 2 * nv, hi_on = gq + 8 < 2 * nv;
    float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!mbar_wait_bounded(half == 0 ? bar_x : bar_y, parity)) timed_out = true;
      const unsigned char* buf = half == 0 ? X : Y;
      const unsigned char* arow_lo = buf + static_cast<size_t>(lo_on ? gq : 0) * hstride + tq * 16;
      const unsigned char* arow_hi = buf + static_cast<size_t>(hi_on ? gq + 8 : 0) * hstride + tq * 16;
      const unsigned char* xrow = x_s + static_cast<size_t>(gq) * rstride + static_cast<size_t>(half) * half_bytes + tq * 16;
      for (int w = w_lo; w < w_hi; ++w) {
        uint4 al = make_uint4(0, 0, 0, 0), ah = al;
        if (lo_on) al = *reinterpret_cast<const uint4*>(arow_lo + static_cast<size_t>(w) * 64);
        if (hi_on) ah = *reinterpret_cast<const uint4*>(arow_hi + static_cast<size_t>(w) * 64);
        const uint4 xv = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(w) * 64);
        MmaOp<T>::run16(d0, al.x, ah.x, al.y, ah.y, xv.x, xv.y);
        MmaOp<T>::run16(d1, al.z, ah.z, al.w, ah.w, xv.z, xv.w);
      }
      if (half == 1) {
        // lane (gq, tq): tile rows gq and gq + 8, batch columns 2tq and 2tq+1
        float* dst = red_s + (warp * 16 + gq) * 8 + 2 * tq;  // [warp][tile row][batch]
        dst[0] = d0[0] + d1[0];
        dst[1] = d0[1] + d1[1];
        dst[64] = d0[2] + d1[2];
        dst[65] = d0[3] + d1[3];
      }
      __syncthreads();  // nobody reads this half of the tile any more (half 1: the partial sums are complete)
      fill(half, it + 1);
    }
    if (tid < 64) {  // neuron e = tid >> 3 of the tile (a = 0 beyond the tile's last neuron), batch row b
      const int e = tid >> 3, b = tid & 7;
      float a = 0.f;
      if (e < nv) {
        const float* src = red_s + (2 * e) * 8 + b;  // [warp 0][row 2e][b]; the up row follows
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int k16 = 0; k16 < 16; ++k16) {
          g += src[k16 * 128];
          u += src[k16 * 128 + 8];
        }
        a = apply_act(p.act, g) * u;
      }
      const float a_next = __shfl_down_sync(0xffffffffu, a, 8);  // neuron e + 1, same batch row
      if ((e & 1) == 0) a_pk[(e >> 1) * 8 + b] = MmaK8<T>::pack(a, a_next);
    }
    __syncthreads();  // a_pk complete
    // ---- phase 2
    if (!mbar_wait_bounded(bar_z, parity)) timed_out = true;
    {
      const uint32_t bfrag = a_pk[tq * 8 + gq];  // B[k = 2tq, 2tq+1][n = gq]
      // ldmatrix row of this lane: neuron lane & 7 (a missing row of a short buffer reads row 0, its a is 0),
      // 8-column group lane >> 3 of the 32 columns of an m-tile pair
      const int zr = (lane & 7) < TN ? (lane & 7) : 0;
      const unsigned char* zrow = Z + static_cast<size_t>(zr) * zstride + (static_cast<size_t>(warp) * (H / 16) + (lane >> 3) * 8) * 2;
#pragma unroll
      for (int mp = 0; mp < BN_MT_MAX / 2; ++mp) {
        if (2 * mp < MT) {
          uint32_t af[4];
          ldmatrix_x4_trans(af, zrow + static_cast<size_t>(mp) * 64);
          MmaK8<T>::run(dacc[2 * mp], af[0], af[1], bfrag);
          MmaK8<T>::run(dacc[2 * mp + 1], af[2], af[3], bfrag);
        }
      }
    }
    if (it + 1 < niter) {
      __syncthreads();  // every thread is done with a_pk and the down rows of this tile
      fill(2, it + 1);
    }
  }
  if (timed_out && p.status) atomicOr(p.status, DEV_TIMEOUT);
  {
    float* dst = q.partial + static_cast<size_t>(blockIdx.x) * B * H + static_cast<size_t>(warp) * (H / 16) + gq;
    const int b0 = 2 * tq, b1 = 2 * tq + 1;
#pragma unroll
    for (int mt = 0; mt < BN_MT_MAX; ++mt) {
      if (mt < MT) {
        if (b0 < B) {
          dst[static_cast<size_t>(b0) * H + mt * 16] = dacc[mt][0];
          dst[static_cast<size_t>(b0) * H + mt * 16 + 8] = dacc[mt][2];
        }
        if (b1 < B) {
          dst[static_cast<size_t>(b1) * H + mt * 16] = dacc[mt][1];
          dst[static_cast<size_t>(b1) * H + mt * 16 + 8] = dacc[mt][3];
        }
      }
    }
  }
}

// out[h] = sum_c partial[c][h], c ascending.  Block: 32 columns x 32 groups of CTAs; a group
// adds a contiguous range of CTAs in order, then the groups are added in order.  With peers
// (pa.world > 1: the layer is one shard of several GPUs) the column sums are then exchanged
// over peer memory and added in rank order before the output is written: the all-reduce of the
// sharded down projection costs no extra launch.
template <typename T>
__global__ void __launch_bounds__(1024) k_partial_reduce(const float* __restrict__ partial, int G, int H, T* __restrict__ out,
                                                         const __grid_constant__ PeerArgs pa) {
  __shared__ float s_r[32][33];
  const int hc = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int h = blockIdx.x * 32 + hc;
  const int per = (G + 31) / 32;
  const int c0 = grp * per, c1 = min(G, c0 + per);
  pdl_wait();
  pdl_launch_dependents();
  const bool shared = pa.world > 1;
  const int epoch = shared ? peer_epoch_begin(pa) : 0;
  float sum = 0.f;
  if (h < H) {
#pragma unroll 8
    for (int c = c0; c < c1; ++c) sum += __ldcg(partial + static_cast<size_t>(c) * H + h);
  }
  s_r[grp][hc] = sum;
  __syncthreads();
  if (grp == 0 && h < H) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < 32; ++g) t += s_r[g][hc];
    if (shared) {
      bool timed_out = false;
      peer_push(pa, epoch, h, t);
      t = peer_collect(pa, epoch, h, t, &timed_out);
      if (timed_out) atomicOr(pa.ctl + 2, DEV_TIMEOUT);
    }
    out[h] = DT<T>::from_f(t);
  }
  if (shared) peer_epoch_end(pa, epoch);
}

// Same sum for long vectors (several rows): a thread owns 4 consecutive columns (16-byte loads),
// a block 128 columns x 32 groups of CTAs.  n must be a multiple of 128.
template <typename T>
__global__ void __launch_bounds__(1024) k_partial_reduce4(const float* __restrict__ partial, int G, int n, T* __restrict__ out,
                                                          const __grid_constant__ PeerArgs pa) {
  __shared__ float4 s_r[32][33];
  const int qc = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const int h = (blockIdx.x * 32 + qc) * 4;
  const int per = (G + 31) / 32;
  const int c0 = grp * per, c1 = min(G, c0 + per);
  pdl_wait();
  pdl_launch_dependents();
  const bool shared = pa.world > 1;
  const int epoch = shared ? peer_epoch_begin(pa) : 0;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
  for (int c = c0; c < c1; ++c) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + static_cast<size_t>(c) * n + h));
    sum.x += v.x;
    sum.y += v.y;
    sum.z += v.z;
    sum.w += v.w;
  }
  s_r[grp][qc] = sum;
  __syncthreads();
  if (grp == 0) {
    float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int g = 0; g < 32; ++g) {
      const float4 v = s_r[g][qc];
      t[0] += v.x;
      t[1] += v.y;
      t[2] += v.z;
      t[3] += v.w;
    }
    if (shared) {
      bool timed_out = false;
#pragma unroll
      for (int k = 0; k < 4; ++k) peer_push(pa, epoch, h + k, t[k]);
#pragma unroll
      for (int k = 0; k < 4; ++k) t[k] = peer_collect(pa, epoch, h + k, t[k], &timed_out);
      if (timed_out) atomicOr(pa.ctl + 2, DEV_TIMEOUT);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) out[h + k] = DT<T>::from_f(t[k]);
  }
  if (shared) peer_epoch_end(pa, epoch);
}


// ------------------------------------------------------------------------------------------ host

// Batch-1 fused path: parts bit 0 = k_mlp_b1, bit 1 = k_partial_reduce.
// Dynamic shared memory a k_mlp_b1 CTA may use: the 227 KB per-block limit less the kernel's
// static shared memory.
template <typename T>
static size_t b1_smem_budget() {
  static size_t budget = 0;
  if (!budget) {
    cudaFuncAttributes fa;
    size_t stat = 4096;
    if (cudaFuncGetAttributes(&fa, k_mlp_b1<T>) == cudaSuccess) stat = fa.sharedSizeBytes;
    budget = 227 * 1024 - (stat + 127) / 128 * 128;
  }
  return budget;
}

// slots per CTA for row length H (r: predictor rank when its back half is fused in, else 0),
// or 0 when the kernel does not fit the shape
template <typename T>
static int b1_slots(int H, int has_gate, int r) {
  const size_t row_bytes = static_cast<size_t>(H) * sizeof(T);
  const size_t x_bytes = (row_bytes + 127) / 128 * 128 + pred_t_smem_bytes(1, r, DT<T>::V);
  const int nmat = has_gate ? 3 : 2;
  const size_t budget = b1_smem_budget<T>();
  if (H / DT<T>::V > B1_MAX_PASS * 512 || budget < B1_HEADER + x_bytes) return 0;
  const size_t sl = (budget - B1_HEADER - x_bytes) / (nmat * row_bytes);
  return sl < 8 ? 0 : static_cast<int>(std::min<size_t>(B1_MAX_SLOTS, sl));
}

struct B1Pred {  // predictor back half fused into k_mlp_b1 (Bm == nullptr: not fused)
  PeerArgs peer = {};  // world > 1: k_partial_reduce ends with the all-reduce over the shards
  int* xchg = nullptr;
  const float* t = nullptr;
  const void* Bm = nullptr;
  uint32_t* bits = nullptr;
  int r = 0;
  float tau = 0.f;
};

template <typename T>
static int launch_b1(const GateUpArgs& g, const void* down, float* partial, void* out, int grid, unsigned parts,
                     const B1Pred& pr, cudaStream_t s) {
  const size_t row_bytes = static_cast<size_t>(g.H) * sizeof(T);
  const int nmat = g.has_gate ? 3 : 2;
  const size_t x_bytes = (row_bytes + 127) / 128 * 128 + pred_t_smem_bytes(1, pr.r, DT<T>::V);
  MlpB1Args q;
  q.g = g;
  q.g.nwarps = b1_slots<T>(g.H, g.has_gate, pr.r);
  q.down = down;
  q.partial = partial;
  q.t = pr.t;
  q.Bm = pr.Bm;
  q.bits = pr.bits;
  q.r = pr.r;
  q.tau = pr.tau;
  q.xchg = nullptr;
  const size_t smem = B1_HEADER + x_bytes + static_cast<size_t>(q.g.nwarps) * nmat * row_bytes;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_mlp_b1<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(b1_smem_budget<T>())));
    attr_set[dev] = true;
  }
  if (parts & 1u) STX_CUDA(launch_pdl(k_mlp_b1<T>, dim3(grid), dim3(512), smem, s, q));
  if (parts & 2u)
    STX_CUDA(launch_pdl(k_partial_reduce<T>, dim3((g.H + 31) / 32), dim3(1024), 0, s, static_cast<const float*>(partial),
                        grid, g.H, static_cast<T*>(out), pr.peer));
  return STX_OK;
}

// ---- k_mlp_bn (2..8 rows)
template <typename T>
static size_t bn_smem_budget() {
  static size_t budget = 0;
  if (!budget) {
    cudaFuncAttributes fa;
    size_t stat = 4096;
    if (cudaFuncGetAttributes(&fa, k_mlp_bn<T>) == cudaSuccess) stat = fa.sharedSizeBytes;
    budget = 227 * 1024 - (stat + 127) / 128 * 128;
  }
  return budget;
}

// bytes in front of the slots / slots per CTA (0: the kernel does not fit the shape)
static size_t bn_fixed_bytes(int H, int B, int r) {
  return BN_HEADER + pred_t_smem_bytes(B, r, 8) + BN_RED_BYTES +
         static_cast<size_t>(BN_MAX) * (static_cast<size_t>(H) * 2 + 64);
}
// shared memory per neuron of a tile: four half rows (gate/up x two halves) and the down row
static size_t bn_neuron_bytes(int H) { return 4 * (static_cast<size_t>(H) + 64) + static_cast<size_t>(H) * 2 + 16; }
// neurons per tile (0: the kernel does not fit the shape)
template <typename T>
static int bn_slots(int H, int B, int r) {
  const size_t fixed = bn_fixed_bytes(H, B, r), budget = bn_smem_budget<T>();
  if (H % 512 != 0 || H > 256 * BN_MT_MAX || budget < fixed + 2 * bn_neuron_bytes(H)) return 0;
  return static_cast<int>(std::min<size_t>(BN_TN_MAX, (budget - fixed) / bn_neuron_bytes(H)));
}

template <typename T>
static int launch_bn(const GateUpArgs& g, const void* down, float* partial, void* out, int grid, unsigned parts,
                     const B1Pred& pr, cudaStream_t s) {
  MlpB1Args q;
  q.g = g;
  q.g.nwarps = bn_slots<T>(g.H, g.B, pr.r);
  q.down = down;
  q.partial = partial;
  q.t = pr.t;
  q.Bm = pr.Bm;
  q.bits = pr.bits;
  q.r = pr.r;
  q.tau = pr.tau;
  q.xchg = pr.xchg;
  const size_t smem = bn_fixed_bytes(g.H, g.B, pr.r) + static_cast<size_t>(q.g.nwarps) * bn_neuron_bytes(g.H);
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_mlp_bn<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(bn_smem_budget<T>())));
    attr_set[dev] = true;
  }
  if (parts & 1u) STX_CUDA(launch_pdl(k_mlp_bn<T>, dim3(grid), dim3(512), smem, s, q));
  if (parts & 2u) {
    const int n = g.B * g.H;  // the partials of a CTA are one vector [B][H]
    if (n % 128 == 0)
      STX_CUDA(launch_pdl(k_partial_reduce4<T>, dim3(n / 128), dim3(1024), 0, s, static_cast<const float*>(partial), grid, n,
                          static_cast<T*>(out), pr.peer));
    else
      STX_CUDA(launch_pdl(k_partial_reduce<T>, dim3((n + 31) / 32), dim3(1024), 0, s, static_cast<const float*>(partial), grid,
                          n, static_cast<T*>(out), pr.peer));
  }
  return STX_OK;
}

static int b1_slots_dt(int H, int has_gate, int dtype, int r) {
  switch (dtype) {
    case STX_F32: return b1_slots<float>(H, has_gate, r);
    case STX_F16: return b1_slots<__half>(H, has_gate, r);
    default: return b1_slots<__nv_bfloat16>(H, has_gate, r);
  }
}


int mlp_row_slots(int H, int has_gate, int dtype, int r) { return b1_slots_dt(H, has_gate, dtype, r); }

int mlp_row_launch(const GateUpArgs& a, const void* down, float* partial, void* out, int grid, unsigned parts, int dtype,
                   cudaStream_t s) {
  switch (dtype) {
    case STX_F32: return launch_b1<float>(a, down, partial, out, grid, parts, B1Pred(), s);
    case STX_F16: return launch_b1<__half>(a, down, partial, out, grid, parts, B1Pred(), s);
    default: return launch_b1<__nv_bfloat16>(a, down, partial, out, grid, parts, B1Pred(), s);
  }
}

// One row through a layer whose mask comes from the threshold rule: the predictor's back half,
// the gather and the whole MLP in k_mlp_b1, then k_partial_reduce.  parts bit 0 / bit 1 select
// the two kernels.  `t` holds A x (fp32 [r]) written earlier on the same stream.
size_t layer_bn_xchg_bytes() { return BN_XCHG_BYTES; }

// Few partial vectors (a split contraction): one thread per 4 columns adds them in order.
template <typename T>
__global__ void __launch_bounds__(256) k_partial_sum_few(const float* __restrict__ partial, int G, int n, T* __restrict__ out) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  pdl_wait();
  pdl_launch_dependents();
  if (i >= n) return;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int g = 0; g < G; ++g) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(partial + static_cast<size_t>(g) * n + i));
    s.x += v.x;
    s.y += v.y;
    s.z += v.z;
    s.w += v.w;
  }
  out[i] = DT<T>::from_f(s.x);
  out[i + 1] = DT<T>::from_f(s.y);
  out[i + 2] = DT<T>::from_f(s.z);
  out[i + 3] = DT<T>::from_f(s.w);
}

// out[i] = sum over g < G of partial[g][i] in ascending g (n a multiple of 128), model dtype.
int partial_sum(const float* partial, int G, int64_t n, void* out, int dtype, cudaStream_t s) {
  STX_CHECK_ARG(n % 128 == 0 && n / 128 < (1ll << 31), "partial_sum: n must be a multiple of 128");
  if (G <= 16) {
    const int nn = static_cast<int>(n);
    const dim3 grid(static_cast<unsigned>((n / 4 + 255) / 256));
    switch (dtype) {
      case STX_F32: STX_CUDA(launch_pdl(k_partial_sum_few<float>, grid, dim3(256), 0, s, partial, G, nn, static_cast<float*>(out))); break;
      case STX_F16: STX_CUDA(launch_pdl(k_partial_sum_few<__half>, grid, dim3(256), 0, s, partial, G, nn, static_cast<__half*>(out))); break;
      default:
        STX_CUDA(launch_pdl(k_partial_sum_few<__nv_bfloat16>, grid, dim3(256), 0, s, partial, G, nn, static_cast<__nv_bfloat16*>(out)));
        break;
    }
    return STX_OK;
  }
  const PeerArgs none = {};
  const int nn = static_cast<int>(n);
  switch (dtype) {
    case STX_F32: STX_CUDA(launch_pdl(k_partial_reduce4<float>, dim3(nn / 128), dim3(1024), 0, s, partial, G, nn, static_cast<float*>(out), none)); break;
    case STX_F16: STX_CUDA(launch_pdl(k_partial_reduce4<__half>, dim3(nn / 128), dim3(1024), 0, s, partial, G, nn, static_cast<__half*>(out), none)); break;
    default:
      STX_CUDA(launch_pdl(k_partial_reduce4<__nv_bfloat16>, dim3(nn / 128), dim3(1024), 0, s, partial, G, nn,
                          static_cast<__nv_bfloat16*>(out), none));
      break;
  }
  return STX_OK;
}

bool layer_b1_supported(int64_t B, int64_t H, int64_t I, int64_t r, int has_gate, int dtype, const void* gate,
                        const void* up, const void* down, const void* Bm) {
  if (B < 1 || B > BN_MAX) return false;
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  if ((H * es) % 16 != 0 || H / V < 32 || r % V != 0 || r / V > 32 || H > (1 << 20) || I > (1 << 24))
    return false;
  const uintptr_t al = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                       reinterpret_cast<uintptr_t>(down) | reinterpret_cast<uintptr_t>(Bm);
  if (al & 15) return false;
  const int grid = std::max(1, num_sms() - 1);
  if (((I + 7) / 8 + grid - 1) / grid > B1_MAX_BYTES) return false;
  if (B == 1) return b1_slots_dt(static_cast<int>(H), has_gate, dtype, static_cast<int>(r)) > 0;
  if (!has_gate || dtype == STX_F32 || B * r * 4 > 16 * 1024) return false;
  return (dtype == STX_F16 ? bn_slots<__half>(static_cast<int>(H), static_cast<int>(B), static_cast<int>(r))
                           : bn_slots<__nv_bfloat16>(static_cast<int>(H), static_cast<int>(B), static_cast<int>(r))) >= 2;
}

int layer_b1_forward(const void* x, int64_t B, int64_t H, int64_t I, const void* gate, const void* up, const void* down,
                     const float* t, const void* Bm, int64_t r, float tau, uint32_t* bits, void* out, int act,
                     int has_gate, int dtype, float* partial, int* xchg, int* status, unsigned parts, const stx_peer* peer,
                     cudaStream_t s) {
  GateUpArgs a;
  a.x = x;
  a.gate = gate;
  a.up = up;
  a.combined = nullptr;
  a.a_out = nullptr;
  a.status = status;
  a.K_dev = nullptr;
  a.mask_bits = nullptr;
  a.idx_out = nullptr;
  a.count_out = nullptr;
  a.I = static_cast<int>(I);
  a.K_host = 0;
  a.B = static_cast<int>(B);
  a.H = static_cast<int>(H);
  a.act = act;
  a.has_gate = has_gate;
  a.nwarps = 0;
  B1Pred pr;
  pr.t = t;
  pr.Bm = Bm;
  pr.bits = bits;
  pr.r = static_cast<int>(r);
  pr.tau = tau;
  pr.xchg = xchg;
  if (peer && peer->world > 1) {
    if (!peer_args(peer, &pr.peer)) {
      set_error("stx_layer_step: the layer's peer object is not connected");
      return STX_ERR_INVALID_ARG;
    }
    if (B * H > peer->max_elems) {
      set_error("stx_layer_step: H=%lld exceeds the peer object's max_elems", static_cast<long long>(H));
      return STX_ERR_INVALID_ARG;
    }
  }
  const int grid = std::max(1, num_sms() - 1);
  switch (dtype) {
    case STX_F32: return launch_b1<float>(a, down, partial, out, grid, parts, pr, s);
    case STX_F16:
      return B == 1 ? launch_b1<__half>(a, down, partial, out, grid, parts, pr, s)
                    : launch_bn<__half>(a, down, partial, out, grid, parts, pr, s);
    default:
      return B == 1 ? launch_b1<__nv_bfloat16>(a, down, partial, out, grid, parts, pr, s)
                    : launch_bn<__nv_bfloat16>(a, down, partial, out, grid, parts, pr, s);
  }
}


}  // namespace stx
