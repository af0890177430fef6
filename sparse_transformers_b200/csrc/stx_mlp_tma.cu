// Sparse gated MLP over packed active rows, decode batches — two streaming kernels.
//
//   a[j,b]   = act(x[b]·gate[j]) * (x[b]·up[j])            k_gateup_tma   (K neurons)
//   out[b,:] = sum_j a[j,b] * down[j,:]                    k_down_slab
//
// k_gateup_tma: one persistent CTA per SM owns a contiguous range of neurons and walks it in
// tiles of R neurons.  A producer warp streams each tile's gate and up rows (two contiguous
// ranges of the packed pools) into a ring of shared-memory stages with 1-D bulk async copies
// (cp.async.bulk global -> shared, completion counted on an mbarrier), so (S-1) stages of
// loads are in flight per SM without occupying registers.  Consumer warp (r, part) computes
// the dot products of x with its part of gate row r and up row r from shared memory, reduces
// them with a shuffle butterfly and stores two partial sums; the last warp to finish a
// neuron adds the parts in a fixed order, applies the activation and writes a[j,:].  There
// is no CTA-wide barrier in the loop: warps are only coupled through the stage ring.
//
// k_down_slab: CTA c owns two 16-byte column chunks (one 32-byte sector per row) of the
// output and walks all K packed down rows for them, so no partial sums ever cross CTAs: the
// result is written once, in the output dtype, in a fixed summation order (deterministic),
// with no atomics and no scratch to re-zero.
//
// Every wait on an mbarrier is bounded: when the limit is hit the kernel records
// DEV_TIMEOUT in the status word and carries on with the same control flow (the result is
// then garbage, but no thread is left waiting and the context stays usable).
#include "stx_common.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace stx {

struct GateUpArgs {
  const void* x;
  const void* gate;
  const void* up;
  void* combined;        // optional [B,2K] / [B,K] in dtype
  float* a_out;          // [K][B] fp32
  int* status;           // optional device status word
  const int32_t* K_dev;
  int K_host;
  int B, H, act, has_gate;
  int R, S;              // neurons per tile, stages
  int nconsumer;         // consumer threads (multiple of 32)
  uint32_t stage_bytes;  // R * nmat * row_bytes
};

struct DownArgs {
  const float* a;        // [K][B]
  const void* down;      // packed [K][H]
  void* out;             // [B][H] dtype
  const int32_t* K_dev;
  int K_host;
  int B, H;
};

constexpr uint32_t MBAR_WAIT_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false when the limit expired.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t it = 0; it < MBAR_WAIT_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 128) __nanosleep(64);
  }
  return false;
}
// 1-D bulk copy global -> this CTA's shared memory; completion bytes land on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void consumer_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

constexpr int GU_MAXR = 4;    // neurons per tile
constexpr int GU_MAXS = 8;    // ring stages
constexpr int GU_MAXP = 16;   // parts per neuron

// Shared-memory layout (dynamic):
//   [0, 256)   full[S], empty[S] mbarriers
//   cnt    [S][R] int                       arrival counters per (stage, neuron)
//   part_s [S][R][nparts][2][NB] float      partial dot products
//   x_s    [NB][H] T
//   stages [S][stage_bytes]                 (each: gate rows | up rows)
template <typename T, int NB>
__global__ void __launch_bounds__(544, 1) k_gateup_tma(const GateUpArgs p) {
  constexpr int V = DT<T>::V;
  extern __shared__ __align__(128) unsigned char smem[];

  const int tid = threadIdx.x;
  const int NT = p.nconsumer;
  const int H = p.H, nchunk = H / V;
  const int R = p.R, S = p.S;
  const int NW = NT >> 5, nparts = NW / R;
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const int nmat = p.has_gate ? 2 : 1;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + 16;
  int* cnt = reinterpret_cast<int*>(smem + 256);                                   // [S][R]
  float* part_base = reinterpret_cast<float*>(smem + 256 + 128);                   // [S][R][nparts][2][NB]
  const size_t part_bytes = (sizeof(float) * S * R * nparts * 2 * NB + 127) / 128 * 128;
  T* x_s = reinterpret_cast<T*>(smem + 256 + 128 + part_bytes);
  const size_t x_bytes = (sizeof(T) * NB * H + 127) / 128 * 128;
  unsigned char* stages = smem + 256 + 128 + part_bytes + x_bytes;

  const int K = p.K_dev ? *p.K_dev : p.K_host;
  const int base = K / gridDim.x, rem = K % gridDim.x;
  const int j0 = blockIdx.x * base + min(static_cast<int>(blockIdx.x), rem);
  const int j1 = j0 + base + (static_cast<int>(blockIdx.x) < rem ? 1 : 0);
  const int ntile = (j1 - j0 + R - 1) / R;
  const int nbt = (p.B + NB - 1) / NB;
  const int total = ntile * nbt;  // flat sequence of (batch tile, neuron tile)

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < S * R) cnt[tid] = 0;
  __syncthreads();

  bool timed_out = false;

  if (tid >= NT) {
    // ------------------------------------------------------------------ producer warp
    if (tid == NT) {
      const char* gsrc = static_cast<const char*>(p.gate);
      const char* usrc = static_cast<const char*>(p.up);
      for (int g = 0; g < total; ++g) {
        const int s = g % S;
        if (g >= S) {
          if (!mbar_wait_bounded(&empty[s], ((g / S) - 1) & 1)) timed_out = true;
        }
        const int it = g % ntile;
        const int r0 = j0 + it * R;
        const int nrows = min(R, j1 - r0);
        const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;
        unsigned char* st = stages + static_cast<size_t>(s) * p.stage_bytes;
        mbar_expect_tx(&full[s], bytes * nmat);
        const size_t off = static_cast<size_t>(r0) * row_bytes;
        if (p.has_gate) bulk_load(st, gsrc + off, bytes, &full[s]);
        bulk_load(st + (p.has_gate ? 1 : 0) * static_cast<size_t>(R) * row_bytes, usrc + off, bytes, &full[s]);
      }
      if (timed_out && p.status) atomicOr(p.status, DEV_TIMEOUT);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int lane = tid & 31, warp = tid >> 5;
  const int my_r = warp % R, my_part = warp / R;
  const bool a_active = my_part < nparts;          // warps beyond R*nparts only release stages
  const int cpp = (nchunk + nparts - 1) / nparts;  // chunks per part
  const int c_lo = my_part * cpp, c_hi = min(nchunk, c_lo + cpp);
  T* combined = static_cast<T*>(p.combined);
  const int ldc = p.has_gate ? 2 * K : K;

  int g = 0;
  for (int bt = 0; bt < nbt; ++bt) {
    const int b0 = bt * NB;
    const int nb = min(NB, p.B - b0);
    if (ntile > 0) {
      if (bt > 0) consumer_sync(NT);  // everyone done with the previous x tile
      const uint4* xg = reinterpret_cast<const uint4*>(static_cast<const T*>(p.x) + static_cast<size_t>(b0) * H);
      uint4* xs4 = reinterpret_cast<uint4*>(x_s);
      for (int i = tid; i < NB * nchunk; i += NT) xs4[i] = i < nb * nchunk ? xg[i] : make_uint4(0, 0, 0, 0);
      consumer_sync(NT);
    }

    for (int it = 0; it < ntile; ++it, ++g) {
      const int s = g % S;
      const int r0 = j0 + it * R;
      const int nrows = min(R, j1 - r0);
      const unsigned char* st = stages + static_cast<size_t>(s) * p.stage_bytes;
      const T* g_s = reinterpret_cast<const T*>(st);
      const T* u_s = reinterpret_cast<const T*>(st + (p.has_gate ? 1 : 0) * static_cast<size_t>(R) * row_bytes);
      if (!mbar_wait_bounded(&full[s], (g / S) & 1)) timed_out = true;

      if (a_active && my_r < nrows) {
        float ag[NB], au[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) ag[b] = au[b] = 0.f;
        const T* grow = g_s + static_cast<size_t>(my_r) * H;
        const T* urow = u_s + static_cast<size_t>(my_r) * H;
        int c = c_lo + lane;
        // two chunks per iteration: independent accumulation chains, loads issued together
        for (; c + 32 < c_hi; c += 64) {
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
        for (; c < c_hi; c += 32) {
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
        float* ps = part_base + (((s * R + my_r) * nparts + my_part) * 2) * NB;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const float u = warp_sum_xor(au[b]);
          const float gg = p.has_gate ? warp_sum_xor(ag[b]) : 0.f;
          if (lane == 0) {
            ps[b] = gg;
            ps[NB + b] = u;
          }
        }
        // last warp to finish neuron r adds the parts (fixed order) and publishes a[j,:]
        int last = 0;
        if (lane == 0) {
          __threadfence_block();
          last = (atomicAdd(&cnt[s * R + my_r], 1) == nparts - 1);
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence_block();
          if (lane < NB) {
            const int b = lane;
            float gsum = 0.f, usum = 0.f;
            const volatile float* pr = part_base + ((s * R + my_r) * nparts * 2) * NB;
            for (int q = 0; q < nparts; ++q) {
              gsum += pr[(q * 2) * NB + b];
              usum += pr[(q * 2 + 1) * NB + b];
            }
            const float a = p.has_gate ? apply_act(p.act, gsum) * usum : apply_act(p.act, usum);
            const int j = r0 + my_r;
            if (b < nb) {
              p.a_out[static_cast<size_t>(j) * p.B + b0 + b] = a;
              if (combined) {
                combined[static_cast<size_t>(b0 + b) * ldc + j] = DT<T>::from_f(a);
                if (p.has_gate) combined[static_cast<size_t>(b0 + b) * ldc + K + j] = DT<T>::from_f(usum);
              }
            }
          }
          if (lane == 0) cnt[s * R + my_r] = 0;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  if (timed_out && p.status && lane == 0) atomicOr(p.status, DEV_TIMEOUT);
}


// ------------------------------------------------------------------------------------------
// 16-bit weights: the dot products run on the tensor pipe (mma.sync m16n8k16, fp32
// accumulate), which multiplies fp16/bf16 operands exactly and needs no conversion
// instructions; on the FMA pipe the per-element conversions make the kernel issue-bound.
// The 8 batch columns of the MMA hold up to 8 rows of x, so batches up to 8 cost the same
// as batch 1.  Tile = 8 shared-memory rows: 4 gate + 4 up rows of 4 neurons (or 8 up rows
// without a gate); MMA rows 8..15 are fed zeros.  Warp w owns the k-windows w, w+16, ...
// (a window = 32 consecutive k); its x fragments stay in registers for the whole kernel.
// The summation over k is order-free, so each thread takes its A and B fragments from the
// same 16-byte chunk (k-slots are permuted identically on both sides) and rows are padded by
// 64 bytes in shared memory, which makes the 16-byte fragment loads conflict-free.
constexpr int MMA_MAXW = 16;  // windows per warp: H <= 16 warps * 16 * 32 = 8192

template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};

// Shared-memory layout (dynamic):
//   [0, 256)   full[S], empty[S] mbarriers; cnt[S] at +192
//   part_s [S][8 rows][16 parts][8 cols] float
//   stages [S][8][row_bytes + 64]
template <typename T>
__global__ void __launch_bounds__(544, 1) k_gateup_mma(const GateUpArgs p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int NW = 16, NT = NW * 32;
  const int tid = threadIdx.x;
  const int H = p.H, S = p.S;
  const int R = p.has_gate ? 4 : 8;  // neurons per tile
  const uint32_t row_bytes = static_cast<uint32_t>(H) * sizeof(T);
  const uint32_t row_stride = row_bytes + 64;
  const int nwin = H / 32;

  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + 8;
  int* cnt = reinterpret_cast<int*>(smem + 192);
  float* part_base = reinterpret_cast<float*>(smem + 256);
  unsigned char* stages = smem + 256 + static_cast<size_t>(S) * 8 * 16 * 8 * sizeof(float);

  const int K = p.K_dev ? *p.K_dev : p.K_host;
  const int base = K / gridDim.x, rem = K % gridDim.x;
  const int j0 = blockIdx.x * base + min(static_cast<int>(blockIdx.x), rem);
  const int j1 = j0 + base + (static_cast<int>(blockIdx.x) < rem ? 1 : 0);
  const int ntile = (j1 - j0 + R - 1) / R;
  const int nbt = (p.B + 7) / 8;
  const int total = ntile * nbt;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], NW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < S) cnt[tid] = 0;
  __syncthreads();

  bool timed_out = false;

  if (tid >= NT) {
    if (tid == NT) {
      const char* gsrc = static_cast<const char*>(p.gate);
      const char* usrc = static_cast<const char*>(p.up);
      for (int g = 0; g < total; ++g) {
        const int s = g % S;
        if (g >= S) {
          if (!mbar_wait_bounded(&empty[s], ((g / S) - 1) & 1)) timed_out = true;
        }
        const int it = g % ntile;
        const int r0 = j0 + it * R;
        const int nrows = min(R, j1 - r0);
        unsigned char* st = stages + static_cast<size_t>(s) * 8 * row_stride;
        mbar_expect_tx(&full[s], static_cast<uint32_t>(nrows) * row_bytes * (p.has_gate ? 2 : 1));
        for (int i = 0; i < nrows; ++i) {
          const size_t off = static_cast<size_t>(r0 + i) * row_bytes;
          if (p.has_gate) {
            bulk_load(st + static_cast<size_t>(i) * row_stride, gsrc + off, row_bytes, &full[s]);
            bulk_load(st + static_cast<size_t>(4 + i) * row_stride, usrc + off, row_bytes, &full[s]);
          } else {
            bulk_load(st + static_cast<size_t>(i) * row_stride, usrc + off, row_bytes, &full[s]);
          }
        }
      }
      if (timed_out && p.status) atomicOr(p.status, DEV_TIMEOUT);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  const int lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;  // fragment row / k-slot group
  T* combined = static_cast<T*>(p.combined);
  const int ldc = p.has_gate ? 2 * K : K;

  int g = 0;
  for (int bt = 0; bt < nbt; ++bt) {
    const int b0 = bt * 8;
    const int nb = min(8, p.B - b0);
    // x fragments of this warp's windows: batch row gq, chunk (4*window + tq)
    uint4 xf[MMA_MAXW];
#pragma unroll
    for (int q = 0; q < MMA_MAXW; ++q) {
      const int w = warp + NW * q;
      xf[q] = make_uint4(0, 0, 0, 0);
      if (w < nwin && gq < nb && ntile > 0)
        xf[q] = ld_cached16(static_cast<const T*>(p.x) + static_cast<size_t>(b0 + gq) * H + (4 * w + tq) * 8);
    }

    for (int it = 0; it < ntile; ++it, ++g) {
      const int s = g % S;
      const int r0 = j0 + it * R;
      const int nrows = min(R, j1 - r0);
      const unsigned char* st = stages + static_cast<size_t>(s) * 8 * row_stride;
      const unsigned char* arow = st + static_cast<size_t>(gq) * row_stride + tq * 16;
      if (!mbar_wait_bounded(&full[s], (g / S) & 1)) timed_out = true;

      float d[4] = {0.f, 0.f, 0.f, 0.f};
      float e[4] = {0.f, 0.f, 0.f, 0.f};  // second chain for instruction-level parallelism
#pragma unroll
      for (int q = 0; q < MMA_MAXW; ++q) {
        const int w = warp + NW * q;
        if (w < nwin) {
          const uint4 av = *reinterpret_cast<const uint4*>(arow + static_cast<size_t>(w) * 64);
          MmaOp<T>::run(d, av.x, av.y, xf[q].x, xf[q].y);
          MmaOp<T>::run(e, av.z, av.w, xf[q].z, xf[q].w);
        }
      }
      // lane (gq,tq): row gq, batch columns 2tq and 2tq+1
      float* ps = part_base + ((static_cast<size_t>(s) * 8 + gq) * 16 + warp) * 8 + 2 * tq;
      ps[0] = d[0] + e[0];
      ps[1] = d[1] + e[1];
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence_block();
        last = (atomicAdd(&cnt[s], 1) == NW - 1);
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence_block();
        // sum the 16 parts in ascending order: lane -> (row gq, cols 2tq, 2tq+1)
        const volatile float* pr = part_base + ((static_cast<size_t>(s) * 8 + gq) * 16) * 8 + 2 * tq;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int q = 0; q < NW; ++q) {
          s0 += pr[q * 8];
          s1 += pr[q * 8 + 1];
        }
        if (p.has_gate) {
          // rows 0..3 gate, rows 4..7 up of the same neurons: bring up sums to the gate lanes
          const float u0 = __shfl_down_sync(0xffffffffu, s0, 16);
          const float u1 = __shfl_down_sync(0xffffffffu, s1, 16);
          if (gq < 4 && gq < nrows) {
            const int j = r0 + gq;
            const float a0 = apply_act(p.act, s0) * u0, a1 = apply_act(p.act, s1) * u1;
            const int c0 = 2 * tq, c1 = 2 * tq + 1;
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
        } else if (gq < nrows) {
          const int j = r0 + gq;
          const float a0 = apply_act(p.act, s0), a1 = apply_act(p.act, s1);
          const int c0 = 2 * tq, c1 = 2 * tq + 1;
          if (c0 < nb) {
            p.a_out[static_cast<size_t>(j) * p.B + b0 + c0] = a0;
            if (combined) combined[static_cast<size_t>(b0 + c0) * ldc + j] = DT<T>::from_f(a0);
          }
          if (c1 < nb) {
            p.a_out[static_cast<size_t>(j) * p.B + b0 + c1] = a1;
            if (combined) combined[static_cast<size_t>(b0 + c1) * ldc + j] = DT<T>::from_f(a1);
          }
        }
        if (lane == 0) cnt[s] = 0;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }
  }
  if (timed_out && p.status && lane == 0) atomicOr(p.status, DEV_TIMEOUT);
}

// CTA c owns column chunks 2c and 2c+1 (32 bytes of every row).  Thread t: chunk 2c + (t&1),
// rows (t>>1), (t>>1)+256, ...; eight row loads (and their a values) are issued before the
// first use, so a CTA has 64 KB in flight and a 20 % dense layer needs one round trip.
// Reduction: shuffle butterfly over the 16 row lanes of a warp (xor 2,4,8,16), then the 16
// warps in ascending order.
constexpr int DOWN_THREADS = 512;
constexpr int DOWN_ROWS = DOWN_THREADS / 2;
constexpr int DOWN_UNROLL = 8;

template <typename T, int NB>
__global__ void __launch_bounds__(DOWN_THREADS) k_down_slab(const DownArgs p) {
  constexpr int V = DT<T>::V;
  __shared__ float red_s[DOWN_THREADS / 32][2][NB][V];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cid = tid & 1, rl = tid >> 1;
  const int H = p.H, nchunk = H / V;
  const int c = blockIdx.x * 2 + cid;
  const bool c_ok = c < nchunk;
  const int K = p.K_dev ? *p.K_dev : p.K_host;
  const T* dcol = static_cast<const T*>(p.down) + (c_ok ? c : 0) * V;

  for (int b0 = 0; b0 < p.B; b0 += NB) {
    const int nb = min(NB, p.B - b0);
    float acc[NB][V];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int v = 0; v < V; ++v) acc[b][v] = 0.f;
    if (c_ok) {
      for (int j = rl; j < K; j += DOWN_ROWS * DOWN_UNROLL) {
        uint4 dv[DOWN_UNROLL];
        float av[DOWN_UNROLL][NB];
#pragma unroll
        for (int u = 0; u < DOWN_UNROLL; ++u) {
          const int jj = j + DOWN_ROWS * u;
          dv[u] = make_uint4(0, 0, 0, 0);
          if (jj < K) dv[u] = ld_stream16(dcol + static_cast<size_t>(jj) * H);
#pragma unroll
          for (int b = 0; b < NB; ++b) av[u][b] = (jj < K && b < nb) ? p.a[static_cast<size_t>(jj) * p.B + b0 + b] : 0.f;
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
        float s = acc[b][v];
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 8);
        s += __shfl_xor_sync(0xffffffffu, s, 16);
        if (lane < 2) red_s[warp][lane][b][v] = s;
      }
    __syncthreads();
    // 2 chunks x NB rows x V elements results
    for (int i = tid; i < 2 * NB * V; i += blockDim.x) {
      const int v = i % V, b = (i / V) % NB, cc = i / (V * NB);
      const int col_chunk = blockIdx.x * 2 + cc;
      if (b < nb && col_chunk < nchunk) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < DOWN_THREADS / 32; ++w) s += red_s[w][cc][b][v];
        static_cast<T*>(p.out)[static_cast<size_t>(b0 + b) * H + col_chunk * V + v] = DT<T>::from_f(s);
      }
    }
    __syncthreads();
  }
}

constexpr size_t TMA_SMEM_BUDGET = 220 * 1024;

// STX_GATEUP=fma forces the FMA-pipe consumer for 16-bit types (A/B measurements).
static bool use_mma_path() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("STX_GATEUP");
    v = (e && !strcmp(e, "fma")) ? 0 : 1;
  }
  return v == 1;
}

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
  k_gateup_tma<T, NB><<<grid, a.nconsumer + 32, smem, s>>>(a);
  STX_LAUNCH_CHECK("k_gateup_tma");
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
  k_gateup_mma<T><<<grid, 16 * 32 + 32, smem, s>>>(a);
  STX_LAUNCH_CHECK("k_gateup_mma");
  return STX_OK;
}
template <>
int launch_gateup_mma<float>(const GateUpArgs&, int, size_t, cudaStream_t) {
  return STX_ERR_UNSUPPORTED;
}

template <typename T, int NB>
static int launch_both(const GateUpArgs& g, int grid, size_t smem, const DownArgs& d, unsigned parts, cudaStream_t s) {
  if (parts & 1u) {
    int rc = g.R == 0 ? launch_gateup_mma<T>(g, grid, smem, s) : launch_gateup<T, NB>(g, grid, smem, s);
    if (rc != STX_OK) return rc;
  }
  if (parts & 2u) {
    const int nchunk = d.H / DT<T>::V;
    k_down_slab<T, NB><<<(nchunk + 1) / 2, DOWN_THREADS, 0, s>>>(d);
    STX_LAUNCH_CHECK("k_down_slab");
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
// scratch: fp32 a[K][B] at offset 256.  parts: bit 0 = gate/up kernel, bit 1 = down kernel.
int mlp_forward_tma(const void* x, int64_t B, int64_t H, const void* gate, const void* up, const void* down,
                    const int32_t* K_dev, int64_t K_host, void* out, void* combined, int act, int has_gate, int dtype,
                    void* scratch, int* status, unsigned parts, cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  const int nchunk = static_cast<int>(H / V);
  if (nchunk < 32) return STX_ERR_UNSUPPORTED;
  const uintptr_t al = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(down);
  if (al & 15) return STX_ERR_UNSUPPORTED;
  const int NW = 16, NT = NW * 32;
  const int nb = B >= 8 ? 8 : (B >= 4 ? 4 : (B >= 2 ? 2 : 1));
  const int nmat = has_gate ? 2 : 1;
  const size_t row_bytes = static_cast<size_t>(H) * es;
  const size_t x_bytes = (es * nb * H + 127) / 128 * 128;
  int R = 0, S = 0;
  const bool use_mma = es == 2 && (H % 32) == 0 && H <= 16 * MMA_MAXW * 32 && use_mma_path();
  size_t mma_smem = 0;
  if (use_mma) {
    const size_t stage = 8 * (row_bytes + 64);
    for (int st = GU_MAXS; st >= 2; --st) {
      const size_t need = 256 + static_cast<size_t>(st) * 8 * 16 * 8 * sizeof(float) + st * stage;
      if (need <= TMA_SMEM_BUDGET) {
        S = st;
        mma_smem = need;
        break;
      }
    }
  }
  if (use_mma && S >= 2) {
    // R == 0 marks the tensor-pipe kernel; its tile height is fixed by has_gate
  } else
  for (int r = GU_MAXR; r >= 1; r >>= 1) {
    const size_t stage = static_cast<size_t>(r) * nmat * row_bytes;
    for (int st = GU_MAXS; st >= 2; --st) {
      const size_t part_bytes = (sizeof(float) * st * r * (NW / r) * 2 * nb + 127) / 128 * 128;
      if (256 + 128 + part_bytes + x_bytes + st * stage <= TMA_SMEM_BUDGET) {
        S = st;
        break;
      }
    }
    if (S >= 3 || (r == 1 && S >= 2)) {
      R = r;
      break;
    }
    S = 0;
  }
  const bool mma = use_mma && S >= 2 && R == 0;
  if (R == 0 && !mma) return STX_ERR_UNSUPPORTED;
  GateUpArgs a;
  a.x = x;
  a.gate = gate;
  a.up = up;
  a.combined = combined;
  a.a_out = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256);
  a.status = status;
  a.K_dev = K_dev;
  a.K_host = static_cast<int>(K_host);
  a.B = static_cast<int>(B);
  a.H = static_cast<int>(H);
  a.act = act;
  a.has_gate = has_gate;
  a.R = R;
  a.S = S;
  a.nconsumer = NT;
  a.stage_bytes = static_cast<uint32_t>(static_cast<size_t>(R) * nmat * row_bytes);
  size_t smem = mma_smem;
  if (!mma) {
    const size_t part_bytes = (sizeof(float) * S * R * (NW / R) * 2 * nb + 127) / 128 * 128;
    smem = 256 + 128 + part_bytes + x_bytes + static_cast<size_t>(S) * a.stage_bytes;
  }
  const int tile_r = mma ? (has_gate ? 4 : 8) : R;
  int grid = num_sms();
  if (!K_dev) grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(grid, (K_host + tile_r - 1) / tile_r)));
  DownArgs d;
  d.a = a.a_out;
  d.down = down;
  d.out = out;
  d.K_dev = K_dev;
  d.K_host = static_cast<int>(K_host);
  d.B = static_cast<int>(B);
  d.H = static_cast<int>(H);
  switch (dtype) {
    case STX_F32: return dispatch_nb<float>(a, nb, grid, smem, d, parts, s);
    case STX_F16: return dispatch_nb<__half>(a, nb, grid, smem, d, parts, s);
    default: return dispatch_nb<__nv_bfloat16>(a, nb, grid, smem, d, parts, s);
  }
}

}  // namespace stx
