// Shared by the streaming MLP kernels of decode batches: argument structs, the in-kernel listing of a mask's set
// bits, the mma.sync fragment helpers, and what the three translation units call of one another
// (stx_mlp_batch.cu: two kernels over packed or gathered rows; stx_mlp_row.cu: one-kernel paths for 1..8 rows;
// stx_mlp_tma.cu: the host dispatch between them).
#pragma once

#include "stx_common.cuh"
#include "stx_tma.cuh"
#include "stx_peer.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace stx {

constexpr size_t TMA_SMEM_BUDGET = 220 * 1024;

struct GateUpArgs {
  const void* x;
  const void* gate;
  const void* up;
  void* combined;        // optional [B,2K] / [B,K] in dtype
  float* a_out;          // [K][B] fp32
  int* status;           // optional device status word
  const int32_t* K_dev;
  // gather mode (mask_bits != null): the rows are those of the set mask bits, in ascending
  // order, taken from full [I,H] pools; every CTA lists the bits itself, CTA 0 also
  // publishes the list and its length for the down kernel
  const uint32_t* mask_bits;
  int32_t* idx_out;
  int32_t* count_out;
  int I;
  int K_host;
  int B, H, act, has_gate;
  int nwarps;
};

// Gather mode of the fused layer step: rows are the set bits of `mask_bits` in the full pools.
struct GatherSpec {
  const uint32_t* mask_bits;
  int32_t* idx;    // [I] out: active neuron ids, ascending
  int32_t* count;  // out: their number
  int I;
};

struct DownArgs {
  const float* a;        // [K][B]
  const void* down;      // packed [K][H]
  void* out;             // [B][H] dtype
  const int32_t* K_dev;
  const int32_t* row_idx;  // optional gather indices, as in GateUpArgs
  int K_host;
  int B, H;
};



constexpr int GATHER_MY_CAP = 512;  // per-CTA share of the active list: ceil(I / grid) + tile <= 512

// Lists the set bits of the mask in ascending order (rank rho = 0..K-1).  Bits are grouped in
// tiles of TR consecutive ranks; tile t belongs to CTA t % gridDim.x and lands in that CTA's
// s_my[(t / gridDim.x) * TR + rho % TR].  CTA 0 also writes the whole list and K to global
// memory.  All threads of the block must call it; returns K.  Ends with a barrier.
__device__ __forceinline__ int cta_list_active(const uint32_t* __restrict__ bits, int I, int TR, int32_t* s_my,
                                               int32_t* idx_out, int32_t* count_out) {
  __shared__ int s_wsum[32];
  __shared__ int s_total;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  const int W = (I + 31) >> 5;
  const int WPT = (W + blockDim.x - 1) / blockDim.x;
  uint32_t wv[8];  // W <= 2048 and at least 256 threads: WPT <= 8
  int cnt = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int w = tid * WPT + k;
    wv[k] = (k < WPT && w < W) ? __ldcg(bits + w) : 0u;
    cnt += __popc(wv[k]);
  }
  int inc = cnt;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, off);
    if (lane >= off) inc += v;
  }
  if (lane == 31) s_wsum[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    const int v = lane < nw ? s_wsum[lane] : 0;
    int winc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int u = __shfl_up_sync(0xffffffffu, winc, off);
      if (lane >= off) winc += u;
    }
    s_wsum[lane] = winc - v;
    if (lane == 31) s_total = winc;
  }
  __syncthreads();
  int rho = s_wsum[wid] + inc - cnt;
  const bool publish = blockIdx.x == 0 && idx_out != nullptr;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    uint32_t b = wv[k];
    const int w = tid * WPT + k;
    while (b) {
      const int n = w * 32 + __ffs(b) - 1;
      b &= b - 1;
      if (publish) idx_out[rho] = n;
      const int tile = rho / TR;
      if (tile % static_cast<int>(gridDim.x) == static_cast<int>(blockIdx.x)) {
        const int slot = (tile / static_cast<int>(gridDim.x)) * TR + rho % TR;
        if (slot < GATHER_MY_CAP) s_my[slot] = n;
      }
      ++rho;
    }
  }
  const int K = s_total;
  if (publish && tid == 0) *count_out = K;
  __syncthreads();
  return K;
}

// Shared-memory layout (dynamic): [0,256) mbarriers | x_s [NB][H] T | bufs [nwarps][nmat][H] T
// Rank rho (packed row, or rho-th active neuron) belongs to CTA rho % gridDim.x; inside the
// CTA, warp w takes its local slots w, w + nwarps, ...

// ------------------------------------------------------------------------------------------
// 16-bit weights: the dot products run on the tensor pipe (mma.sync m16n8k16, fp32
// accumulate).  It multiplies fp16/bf16 operands exactly and needs no conversion
// instructions (on the FMA pipe the per-element conversions make the kernel issue-bound),
// and its 8 batch columns hold up to 8 rows of x, so batches up to 8 cost the same as
// batch 1.  A warp's private buffer holds one tile of 4 rows: gate and up rows of 2 neurons
// (or the up rows of 4 neurons without a gate); MMA rows 4..15 are fed zeros.  The summation
// over k is order-free, so each thread takes its A and B fragments from the same 16-byte
// chunk (the k-slots are permuted identically on both sides); rows are padded by 64 bytes in
// shared memory, which makes the 16-byte fragment loads conflict-free.
template <typename T> struct MmaOp;
template <> struct MmaOp<__half> {
  // all 16 tile rows: a0/a2 = row g (k low/high pair), a1/a3 = row g + 8
  static __device__ __forceinline__ void run16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};
template <> struct MmaOp<__nv_bfloat16> {
  static __device__ __forceinline__ void run16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
  }
};

template <typename T> struct MmaK8;  // m16n8k8: A 16x8 (two registers), B 8x8 (one register)
template <> struct MmaK8<__half> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
template <> struct MmaK8<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0));
  }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
};
// Four 8x8 b16 matrices, transposed on the way into registers; lane l supplies the address of
// row l & 7 of matrix l >> 3.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(row_addr)));
}

constexpr int MMA_TILE_ROWS = 4;

// stx_mlp_batch.cu: gate/up kernel (parts bit 0) and down kernel (parts bit 1) for a batch tile of nb rows
int mlp_batch_launch(const GateUpArgs& g, int nb, int grid, size_t smem, const DownArgs& d, unsigned parts, int dtype,
                     cudaStream_t s);
// stx_mlp_row.cu: slots per CTA of k_mlp_b1 for rows of H elements (0: the kernel does not fit the shape), and the
// one-row path on packed or gathered rows without the predictor's back half (parts bit 0 = k_mlp_b1, bit 1 = k_partial_reduce)
int mlp_row_slots(int H, int has_gate, int dtype, int r);
int mlp_row_launch(const GateUpArgs& a, const void* down, float* partial, void* out, int grid, unsigned parts, int dtype,
                   cudaStream_t s);

}  // namespace stx
