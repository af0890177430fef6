// Sparse gated MLP for decode batches, two kernels over packed rows or a mask-listed gather: k_gateup_tma /
// k_gateup_mma, then k_down_rows.  Any dtype, gated or not.
//
//   a[j,b]   = act(x[b]·gate[j]) * (x[b]·up[j])      (K active neurons)
//   out[b,:] = sum_j a[j,b] * down[j,:]
//
// k_gateup_tma: one persistent CTA per SM owns a contiguous range of neurons.  Every warp is
// its own producer and consumer: lane 0 issues two 1-D bulk async copies (cp.async.bulk
// global -> shared, completion counted on the warp's mbarrier) that bring the gate row and the
// up row of the warp's next neuron into the warp's private shared-memory buffer; the warp then
// computes both dot products with x (shared memory) from that buffer, reduces them with a
// shuffle butterfly and writes a[j,:].  Warps never synchronise with each other inside the
// loop, so with K/148 neurons per SM and up to 16 warps, all rows of a 20 %-dense layer are in
// flight at once and the kernel costs about one memory round trip plus the stream time.
//
// k_down_rows: the packed down rows are split over a (column slab, row range) grid; the CTAs
// of one column slab form a thread-block cluster and add their partial sums through
// distributed shared memory in rank order, so the result is written once, in the output
// dtype, deterministically, with no global atomics and no scratch to re-zero.  A slab is 256
// bytes wide (sixteen 16-byte chunks), which keeps DRAM bursts long.
//
// Every wait on an mbarrier is bounded: when the limit is hit the kernel records
// DEV_TIMEOUT in the status word and carries on with the same control flow (the result is
// then garbage, but no thread is left waiting and the context stays usable).
#include "stx_mlp_stream.cuh"

#include <cooperative_groups.h>

namespace cg = cooperative_groups;

namespace stx {

template <typename T, int NB>
__global__ void __launch_bounds__(512, 1) k_gateup_tma(const GateUpArgs p) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int NWp = p.nwarps;
  const int H = p.H, nchunk = H / V;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const int nmat = p.has_gate ? 2 : 1;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  T* x_s = reinterpret_cast<T*>(smem + 256);
  const size_t x_bytes = (sizeof(T) * NB * H + 127) / 128 * 128;
  unsigned char* mybuf = smem + 256 + x_bytes + static_cast<size_t>(warp) * nmat * row_bytes;
  uint64_t* mybar = &bars[warp];

  __shared__ int32_t s_my[GATHER_MY_CAP];
  const char* gsrc = static_cast<const char*>(p.gate);
  const char* usrc = static_cast<const char*>(p.up);
  T* combined = static_cast<T*>(p.combined);
  const bool gather = p.mask_bits != nullptr;
  const int G = gridDim.x;

  if (tid == 0) {
    for (int w = 0; w < NWp; ++w) mbar_init(&bars[w], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();  // everything above is set-up; from here on the predecessor's results are read
  pdl_launch_dependents();
  // the list of active rows (gather mode) or K (packed mode); also orders the barrier init
  const int K = gather ? cta_list_active(p.mask_bits, p.I, 1, s_my, p.idx_out, p.count_out)
                       : (p.K_dev ? *p.K_dev : p.K_host);
  if (!gather) __syncthreads();
  const int ldc = p.has_gate ? 2 * K : K;
  const int nlocal = K > static_cast<int>(blockIdx.x) ? (K - 1 - static_cast<int>(blockIdx.x)) / G + 1 : 0;

  auto issue = [&](int q) {  // q: local slot; rank = blockIdx.x + G*q
    mbar_expect_tx(mybar, row_bytes * nmat);
    const int row = gather ? s_my[q] : static_cast<int>(blockIdx.x) + G * q;
    const size_t off = static_cast<size_t>(row) * row_bytes;
    if (p.has_gate) bulk_load(mybuf, gsrc + off, row_bytes, mybar);
    bulk_load(mybuf + (p.has_gate ? row_bytes : 0), usrc + off, row_bytes, mybar);
  };

  bool timed_out = false;
  uint32_t phase = 0;
  const int nbt = (p.B + NB - 1) / NB;
  for (int bt = 0; bt < nbt; ++bt) {
    const int b0 = bt * NB;
    const int nb = min(NB, p.B - b0);
    int q = warp;
    if (lane == 0 && q < nlocal) issue(q);  // the first rows stream in while x is staged
    if (bt > 0) __syncthreads();            // everyone done with the previous x tile
    {
      const uint4* xg = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + static_cast<size_t>(b0) * H);
      uint4* xs4 = reinterpret_cast<uint4*>(x_s);
      for (int i = tid; i < NB * nchunk; i += blockDim.x) xs4[i] = i < nb * nchunk ? xg[i] : make_uint4(0, 0, 0, 0);
    }
    __syncthreads();

    for (; q < nlocal; q += NWp) {
      const int j = static_cast<int>(blockIdx.x) + G * q;  // rank of this row
      if (!mbar_wait_bounded(mybar, phase)) timed_out = true;
      phase ^= 1u;
      const T* grow = reinterpret_cast<const T*>(mybuf);
      const T* urow = reinterpret_cast<const T*>(mybuf + (p.has_gate ? row_bytes : 0));
      float ag[NB], au[NB];
#pragma unroll
      for (int b = 0; b < NB; ++b) ag[b] = au[b] = 0.f;
      int c = lane;
      for (; c + 32 < nchunk; c += 64) {  // two chunks per iteration: independent chains
        const uint4 u0 = *reinterpret_cast<const uint4*>(urow + c * V);
        const uint4 u1 = *reinterpret_cast<const uint4*>(urow + (c + 32) * V);
        uint4 g0 = make_uint4(0, 0, 0, 0), g1 = g0;
        if (p.has_gate) {
          g0 = *reinterpret_cast<const uint4*>(grow + c * V);
          g1 = *reinterpret_cast<const uint4*>(grow + (c + 32) * V);
        }
        float wu0[V], wu1[V], wg0[V], wg1[V];
        Unpack<T>::run(u0, wu0);
        Unpack<T>::run(u1, wu1);
        Unpack<T>::run(g0, wg0);
        Unpack<T>::run(g1, wg1);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float x0[V], x1[V];
          Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + b * H + c * V), x0);
          Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + b * H + (c + 32) * V), x1);
          float su0 = 0.f, su1 = 0.f, sg0 = 0.f, sg1 = 0.f;
#pragma unroll
          for (int v = 0; v < V; ++v) {
            su0 = fmaf(x0[v], wu0[v], su0);
            su1 = fmaf(x1[v], wu1[v], su1);
            if (p.has_gate) {
              sg0 = fmaf(x0[v], wg0[v], sg0);
              sg1 = fmaf(x1[v], wg1[v], sg1);
            }
          }
          au[b] += su0 + su1;
          ag[b] += sg0 + sg1;
        }
      }
      for (; c < nchunk; c += 32) {
        float wu[V], wg[V];
        Unpack<T>::run(*reinterpret_cast<const uint4*>(urow + c * V), wu);
        if (p.has_gate) Unpack<T>::run(*reinterpret_cast<const uint4*>(grow + c * V), wg);
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float xv[V];
          Unpack<T>::run(*reinterpret_cast<const uint4*>(x_s + b * H + c * V), xv);
          float su = 0.f, sg = 0.f;
#pragma unroll
          for (int v = 0; v < V; ++v) {
            su = fmaf(xv[v], wu[v], su);
            if (p.has_gate) sg = fmaf(xv[v], wg[v], sg);
          }
          au[b] += su;
          ag[b] += sg;
        }
      }
      // the buffer is free again: fetch the next neuron's rows before the reduction
      __syncwarp();
      if (lane == 0 && q + NWp < nlocal) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(q + NWp);
      }
      float a_mine = 0.f, u_mine = 0.f;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const float u = warp_sum_xor(au[b]);
        const float gsum = p.has_gate ? warp_sum_xor(ag[b]) : 0.f;
        if (lane == b) {
          u_mine = u;
          a_mine = p.has_gate ? apply_act(p.act, gsum) * u : apply_act(p.act, u);
        }
      }
      if (lane < nb) {
        p.a_out[static_cast<size_t>(j) * p.B + b0 + lane] = a_mine;
        if (combined) {
          combined[static_cast<size_t>(b0 + lane) * ldc + j] = DT<T>::from_f(a_mine);
          if (p.has_gate) combined[static_cast<size_t>(b0 + lane) * ldc + K + j] = DT<T>::from_f(u_mine);
        }
      }
    }
  }
  if (timed_out && p.status && lane == 0) atomicOr(p.status, DEV_TIMEOUT);
}



// Shared-memory layout (dynamic): [0,256) mbarriers | x_s [min(B,8)][H*2 + 64] | bufs [nwarps][4][H*2 + 64]
template <typename T>
__global__ void __launch_bounds__(512, 1) k_gateup_mma(const GateUpArgs p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;  // fragment row (and batch column of B) / k-slot group
  const int NWp = p.nwarps;
  const int H = p.H;
  const int nwin = H / 32;                  // a window = 32 consecutive k = 4 chunks of 16 bytes
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t row_stride = row_bytes + 64;
  const int TR = p.has_gate ? 2 : 4;        // neurons per tile

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  unsigned char* x_s = smem + 256;
  const int xrows = min(p.B, 8);
  unsigned char* mybuf = smem + 256 + xrows * static_cast<size_t>(row_stride) +
                         static_cast<size_t>(warp) * MMA_TILE_ROWS * row_stride;
  uint64_t* mybar = &bars[warp];

  __shared__ int32_t s_my[GATHER_MY_CAP];
  const char* gsrc = static_cast<const char*>(p.gate);
  const char* usrc = static_cast<const char*>(p.up);
  T* combined = static_cast<T*>(p.combined);
  const bool gather = p.mask_bits != nullptr;
  const int G = gridDim.x;

  if (tid == 0) {
    for (int w = 0; w < NWp; ++w) mbar_init(&bars[w], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  pdl_launch_dependents();
  const int K = gather ? cta_list_active(p.mask_bits, p.I, TR, s_my, p.idx_out, p.count_out)
                       : (p.K_dev ? *p.K_dev : p.K_host);
  if (!gather) __syncthreads();
  const int ldc = p.has_gate ? 2 * K : K;
  const int ntile_all = (K + TR - 1) / TR;  // tile t belongs to CTA t % G, local slot t / G
  const int nlocal = ntile_all > static_cast<int>(blockIdx.x) ? (ntile_all - 1 - static_cast<int>(blockIdx.x)) / G + 1 : 0;

  auto issue = [&](int q) {
    const int r0 = (static_cast<int>(blockIdx.x) + G * q) * TR;
    const int nr = min(TR, K - r0);
    mbar_expect_tx(mybar, static_cast<uint32_t>(nr) * row_bytes * (p.has_gate ? 2 : 1));
    for (int i = 0; i < nr; ++i) {
      const int row = gather ? s_my[q * TR + i] : r0 + i;
      const size_t off = static_cast<size_t>(row) * row_bytes;
      if (p.has_gate) {
        bulk_load(mybuf + static_cast<size_t>(i) * row_stride, gsrc + off, row_bytes, mybar);
        bulk_load(mybuf + static_cast<size_t>(TR + i) * row_stride, usrc + off, row_bytes, mybar);
      } else {
        bulk_load(mybuf + static_cast<size_t>(i) * row_stride, usrc + off, row_bytes, mybar);
      }
    }
  };

  bool timed_out = false;
  uint32_t phase = 0;
  const int nbt = (p.B + 7) / 8;
  for (int bt = 0; bt < nbt; ++bt) {
    const int b0 = bt * 8;
    const int nb = min(8, p.B - b0);
    int q = warp;
    if (lane == 0 && q < nlocal) issue(q);  // first rows stream in while x is staged
    if (bt > 0) __syncthreads();
    for (int i = tid; i < nb * (H / 8); i += blockDim.x) {
      const int b = i / (H / 8), c = i % (H / 8);
      *reinterpret_cast<uint4*>(x_s + static_cast<size_t>(b) * row_stride + c * 16) =
          ld_cached16(static_cast<const T*>(p.x) + static_cast<size_t>(b0 + b) * H + c * 8);
    }
    __syncthreads();

    const unsigned char* arow = mybuf + static_cast<size_t>(gq < MMA_TILE_ROWS ? gq : 0) * row_stride + tq * 16;
    const bool x_on = gq < nb;  // batch columns beyond the tile multiply by zero
    const unsigned char* xrow = x_s + static_cast<size_t>(x_on ? gq : 0) * row_stride + tq * 16;
    for (; q < nlocal; q += NWp) {
      const int r0 = (static_cast<int>(blockIdx.x) + G * q) * TR;
      const int nr = min(TR, K - r0);
      if (!mbar_wait_bounded(mybar, phase)) timed_out = true;
      phase ^= 1u;
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
      float d2[4] = {0.f, 0.f, 0.f, 0.f}, d3[4] = {0.f, 0.f, 0.f, 0.f};
      int w = 0;
      for (; w + 1 < nwin; w += 2) {
        uint4 a0 = make_uint4(0, 0, 0, 0), a1 = a0;
        if (gq < MMA_TILE_ROWS) {
          a0 = *reinterpret_cast<const uint4*>(arow + static_cast<size_t>(w) * 64);
          a1 = *reinterpret_cast<const uint4*>(arow + static_cast<size_t>(w + 1) * 64);
        }
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
        if (x_on) {
          x0 = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(w) * 64);
          x1 = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(w + 1) * 64);
        }
        MmaOp<T>::run(d0, a0.x, a0.y, x0.x, x0.y);
        MmaOp<T>::run(d1, a0.z, a0.w, x0.z, x0.w);
        MmaOp<T>::run(d2, a1.x, a1.y, x1.x, x1.y);
        MmaOp<T>::run(d3, a1.z, a1.w, x1.z, x1.w);
      }
      for (; w < nwin; ++w) {
        uint4 a0 = make_uint4(0, 0, 0, 0);
        if (gq < MMA_TILE_ROWS) a0 = *reinterpret_cast<const uint4*>(arow + static_cast<size_t>(w) * 64);
        uint4 x0 = make_uint4(0, 0, 0, 0);
        if (x_on) x0 = *reinterpret_cast<const uint4*>(xrow + static_cast<size_t>(w) * 64);
        MmaOp<T>::run(d0, a0.x, a0.y, x0.x, x0.y);
        MmaOp<T>::run(d1, a0.z, a0.w, x0.z, x0.w);
      }
      // the buffer is free again: fetch this warp's next tile before the epilogue
      __syncwarp();
      if (lane == 0 && q + NWp < nlocal) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(q + NWp);
      }
      // lane (gq,tq): tile row gq, batch columns 2tq and 2tq+1
      const float s0 = (d0[0] + d1[0]) + (d2[0] + d3[0]);
      const float s1 = (d0[1] + d1[1]) + (d2[1] + d3[1]);
      const int c0 = 2 * tq, c1 = 2 * tq + 1;
      if (p.has_gate) {
        // rows 0,1 = gate of neurons r0, r0+1; rows 2,3 = their up rows (8 lanes further)
        const float u0 = __shfl_down_sync(0xffffffffu, s0, 8);
        const float u1 = __shfl_down_sync(0xffffffffu, s1, 8);
        if (gq < nr) {
          const int j = r0 + gq;
          const float a0 = apply_act(p.act, s0) * u0, a1 = apply_act(p.act, s1) * u1;
          if (c0 < nb) {
            p.a_out[static_cast<size_t>(j) * p.B + b0 + c0] = a0;
            if (combined) {
              combined[static_cast<size_t>(b0 + c0) * ldc + j] = DT<T>::from_f(a0);
              combined[static_cast<size_t>(b0 + c0) * ldc + K + j] = DT<T>::from_f(u0);
            }
          }
          if (c1 < nb) {
            p.a_out[static_cast<size_t>(j) * p.B + b0 + c1] = a1;
            if (combined) {
              combined[static_cast<size_t>(b0 + c1) * ldc + j] = DT<T>::from_f(a1);
              combined[static_cast<size_t>(b0 + c1) * ldc + K + j] = DT<T>::from_f(u1);
            }
          }
        }
      } else if (gq < nr) {
        const int j = r0 + gq;
        const float a0 = apply_act(p.act, s0), a1 = apply_act(p.act, s1);
        if (c0 < nb) {
          p.a_out[static_cast<size_t>(j) * p.B + b0 + c0] = a0;
          if (combined) combined[static_cast<size_t>(b0 + c0) * ldc + j] = DT<T>::from_f(a0);
        }
        if (c1 < nb) {
          p.a_out[static_cast<size_t>(j) * p.B + b0 + c1] = a1;
          if (combined) combined[static_cast<size_t>(b0 + c1) * ldc + j] = DT<T>::from_f(a1);
        }
      }
    }
  }
  if (timed_out && p.status && lane == 0) atomicOr(p.status, DEV_TIMEOUT);
}

// Grid (nslab, CS), cluster (1, CS, 1): CTA (sx, sy) owns the 256-byte column slab sx and the
// ranks j = sy (mod CS).  Thread t: chunk sx*16 + (t & 15), ranks sy + CS*((t >> 4) + 32*k).
// In gather mode rank j is row row_idx[j] of the full pool; the index and K are loaded
// together, so the row loads are two dependent trips away from the kernel start.
// Reduction order: the two row lanes of a warp, then the 16 warps ascending, then the
// cluster ranks ascending.
constexpr int DOWN_THREADS = 512;
constexpr int DOWN_MAXCS = 8;

template <typename T, int NB>
__global__ void __launch_bounds__(DOWN_THREADS, 2) k_down_rows(const DownArgs p) {
  constexpr int V = DT<T>::V;
  constexpr int DOWN_UNROLL = NB == 1 ? 8 : (NB == 2 ? 4 : 2);
  extern __shared__ __align__(16) float dsm[];
  float* red_s = dsm;                                    // [16 warps][16 chunks][NB][V]
  float* clu_s = dsm + 16 * 16 * NB * V;                 // [CS][16 chunks][NB][V]  (used on rank 0)
  cg::cluster_group cluster = cg::this_cluster();
  const int CS = gridDim.y;
  const int rank = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cl = tid & 15, rl = tid >> 4;
  const int H = p.H, nchunk = H / V;
  const int c = blockIdx.x * 16 + cl;
  const bool c_ok = c < nchunk;
  pdl_wait();
  pdl_launch_dependents();
  const int K = p.K_dev ? *p.K_dev : p.K_host;
  const T* dcol = static_cast<const T*>(p.down) + (c_ok ? c : 0) * V;
  float* clu0 = cluster.map_shared_rank(clu_s, 0);

  for (int b0 = 0; b0 < p.B; b0 += NB) {
    const int nb = min(NB, p.B - b0);
    float acc[NB][V];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[b][v] = 0.f;
    if (c_ok) {
      const int nrl = K > rank ? (K - 1 - rank) / CS + 1 : 0;  // ranks of this CTA: rank + CS*l, l < nrl
      for (int l0 = rl; l0 < nrl; l0 += 32 * DOWN_UNROLL) {
        uint4 dv[DOWN_UNROLL];
        float av[DOWN_UNROLL][NB];
        int rows[DOWN_UNROLL];
#pragma unroll
        for (int u = 0; u < DOWN_UNROLL; ++u) {
          const int jj = rank + CS * (l0 + 32 * u);
          rows[u] = (l0 + 32 * u < nrl) ? (p.row_idx ? p.row_idx[jj] : jj) : -1;
        }
#pragma unroll
        for (int u = 0; u < DOWN_UNROLL; ++u) {
          const int jj = rank + CS * (l0 + 32 * u);
          dv[u] = make_uint4(0, 0, 0, 0);
          if (rows[u] >= 0) dv[u] = ld_stream16(dcol + static_cast<size_t>(rows[u]) * H);
#pragma unroll
          for (int b = 0; b < NB; ++b) av[u][b] = (rows[u] >= 0 && b < nb) ? p.a[static_cast<size_t>(jj) * p.B + b0 + b] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < DOWN_UNROLL; ++u) {
          float wd[V];
          Unpack<T>::run(dv[u], wd);
#pragma unroll
          for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int v = 0; v < V; ++v) acc[b][v] = fmaf(av[u][b], wd[v], acc[b][v]);
        }
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int v = 0; v < V; ++v) {
        const float s = acc[b][v] + __shfl_xor_sync(0xffffffffu, acc[b][v], 16);
        if (lane < 16) red_s[((warp * 16 + cl) * NB + b) * V + v] = s;
      }
    __syncthreads();
    // CTA partial for its slab: 16 chunks x NB x V values, each summed over the 16 warps
    for (int i = tid; i < 16 * NB * V; i += DOWN_THREADS) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 16; ++w) s += red_s[w * 16 * NB * V + i];
      clu0[rank * 16 * NB * V + i] = s;  // distributed shared memory of cluster rank 0
    }
    cluster.sync();
    if (rank == 0) {
      for (int i = tid; i < 16 * NB * V; i += DOWN_THREADS) {
        const int v = i % V, b = (i / V) % NB, cc = i / (V * NB);
        const int col_chunk = blockIdx.x * 16 + cc;
        if (b < nb && col_chunk < nchunk) {
          float s = 0.f;
          for (int r = 0; r < CS; ++r) s += clu_s[r * 16 * NB * V + i];
          static_cast<T*>(p.out)[static_cast<size_t>(b0 + b) * H + col_chunk * V + v] = DT<T>::from_f(s);
        }
      }
    }
    cluster.sync();  // rank 0's buffer may be overwritten by the next batch tile only now
  }
}


// ------------------------------------------------------------------------------------------ host


template <typename T, int NB>
static int launch_gateup(const GateUpArgs& a, int grid, size_t smem, cudaStream_t s) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_gateup_tma<T, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(TMA_SMEM_BUDGET + 4096)));
    attr_set[dev] = true;
  }
  STX_CUDA(launch_pdl(k_gateup_tma<T, NB>, dim3(grid), dim3(a.nwarps * 32), smem, s, a));
  return STX_OK;
}

template <typename T>
static int launch_gateup_mma(const GateUpArgs& a, int grid, size_t smem, cudaStream_t s) {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_gateup_mma<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(TMA_SMEM_BUDGET + 4096)));
    attr_set[dev] = true;
  }
  STX_CUDA(launch_pdl(k_gateup_mma<T>, dim3(grid), dim3(a.nwarps * 32), smem, s, a));
  return STX_OK;
}
template <>
int launch_gateup_mma<float>(const GateUpArgs&, int, size_t, cudaStream_t) {
  return STX_ERR_UNSUPPORTED;
}

// The tensor-pipe kernel pays off once several batch rows share one pass over the weights;
// at batch 1-3 the FMA-pipe kernel measured faster.
static bool use_mma_path(int B) { return B >= 4; }

template <typename T, int NB>
static int launch_down(const DownArgs& d, cudaStream_t s) {
  constexpr int V = DT<T>::V;
  const int nchunk = d.H / V;
  const int nslab = (nchunk + 15) / 16;
  int cs = 1;  // largest power of two that keeps at most two CTAs per SM
  while (cs * 2 <= DOWN_MAXCS && nslab * cs * 2 <= 2 * num_sms()) cs *= 2;
  const size_t smem = sizeof(float) * (16 * 16 + DOWN_MAXCS * 16) * NB * V;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_down_rows<T, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nslab, cs, 1);
  cfg.blockDim = dim3(DOWN_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = cs;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  STX_CUDA(cudaLaunchKernelEx(&cfg, k_down_rows<T, NB>, d));
  return STX_OK;
}

template <typename T, int NB>
static int launch_both(const GateUpArgs& g, int grid, size_t smem, const DownArgs& d, unsigned parts, cudaStream_t s) {
  if (parts & 1u) {
    int rc = STX_ERR_UNSUPPORTED;
    if (sizeof(T) == 2 && (g.H % 32) == 0 && use_mma_path(g.B)) {
      // tensor-pipe kernel: 4-row tiles with padded rows, x tile of 8 padded rows
      const size_t stride = static_cast<size_t>(g.H) * sizeof(T) + 64;
      const size_t fixed = 256 + static_cast<size_t>(std::min(g.B, 8)) * stride;
      if (fixed + 2 * MMA_TILE_ROWS * stride <= TMA_SMEM_BUDGET) {
        GateUpArgs m = g;
        m.nwarps = static_cast<int>(std::min<size_t>(16, (TMA_SMEM_BUDGET - fixed) / (MMA_TILE_ROWS * stride)));
        rc = launch_gateup_mma<T>(m, g.mask_bits ? std::max(1, num_sms() - 1) : num_sms(),
                                  fixed + static_cast<size_t>(m.nwarps) * MMA_TILE_ROWS * stride, s);
      }
    }
    if (rc == STX_ERR_UNSUPPORTED) rc = launch_gateup<T, NB>(g, grid, smem, s);
    if (rc != STX_OK) return rc;
  }
  if (parts & 2u) {
    constexpr int NBD = NB > 4 ? 4 : NB;  // the down kernel walks batches of at most 4
    int rc = launch_down<T, NBD>(d, s);
    if (rc != STX_OK) return rc;
  }
  return STX_OK;
}


template <typename T>
static int dispatch_nb(const GateUpArgs& g, int nb, int grid, size_t smem, const DownArgs& d, unsigned parts,
                       cudaStream_t s) {
  switch (nb) {
    case 1: return launch_both<T, 1>(g, grid, smem, d, parts, s);
    case 2: return launch_both<T, 2>(g, grid, smem, d, parts, s);
    case 4: return launch_both<T, 4>(g, grid, smem, d, parts, s);
    default: return launch_both<T, 8>(g, grid, smem, d, parts, s);
  }
}

// Returns STX_ERR_UNSUPPORTED (without setting an error text) when the shape does not fit
// these kernels; the caller then uses the plain-load kernel.

int mlp_batch_launch(const GateUpArgs& g, int nb, int grid, size_t smem, const DownArgs& d, unsigned parts, int dtype,
                     cudaStream_t s) {
  switch (dtype) {
    case STX_F32: return dispatch_nb<float>(g, nb, grid, smem, d, parts, s);
    case STX_F16: return dispatch_nb<__half>(g, nb, grid, smem, d, parts, s);
    default: return dispatch_nb<__nv_bfloat16>(g, nb, grid, smem, d, parts, s);
  }
}

}  // namespace stx
