// Sparse gated MLP over packed active rows for prefill-sized row blocks (hundreds of rows
// and more): here the gathered weights really form a dense contraction, so it runs on the
// 5th-generation tensor cores.
//
//   GEMM 1   [G | U] = X · [Wg ; Wu]^T      M = rows, N = K (twice), k = H
//            epilogue: A = act(G) * U  -> fp16/bf16 scratch [rows, K8] (and combined_buf)
//   GEMM 2   out = A · Wd                    M = rows, N = H, k = K
//            (Wd: the packed down rows, transposed once per call to [H, K8] so that both
//             operands of both GEMMs are K-major)
//
// One kernel, k_umma_gemm<T, MODE, MH>: per CTA MH (1 or 2) row halves of 128 and two 128-wide
// B tiles (MODE 0: gate and up rows of the same 128 neurons; MODE 1: 256 output columns), so a
// 64-wide k block of 64 KB feeds eight 128x128x16 MMAs; 64-wide k blocks.
//   warp 0      producer: TMA tiled loads (cp.async.bulk.tensor.2d, 128-byte swizzle) of the A
//               tile and one (MODE 1) or two (MODE 0: gate and up rows) B tiles into a ring of
//               shared-memory stages, completion on mbarriers
//   warp 1      allocates tensor memory and issues tcgen05.mma (cta_group::1, kind::f16,
//               M=128, N=128, K=16) from one elected lane; accumulators live in TMEM (128 or
//               256 columns); tcgen05.commit releases a stage / publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld 32 lanes x 32 columns at a time, activation and product
//               in registers, 16-byte stores
// Edges are handled by TMA zero fill on loads and by masked stores.  Every CTA loads its own tiles.
// Every mbarrier wait is bounded; on expiry the kernel records DEV_TIMEOUT and continues
// with the same control flow (the result is then garbage) so that TMEM is always freed.
#include "stx_common.cuh"

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace stx {

constexpr int PF_BM = 128, PF_BN = 128, PF_BK = 64;
constexpr int PF_THREADS = 192;
constexpr uint32_t PF_TILE_BYTES = PF_BM * PF_BK * 2;  // 16 KB per operand tile
constexpr uint32_t PF_WAIT_LIMIT = 1u << 22;

struct PfArgs {
  int M, N, Kd;        // output rows, output columns, contraction length
  int up_off;          // MODE 0: row offset of the up block inside the concat weight (= K)
  int stages;
  int stages_z;        // number of contraction splits (gridDim.z), 0/1 = none
  void* a_out;         // MODE 0: activations [M, lda] ; MODE 1: output [M, ldo]
  int ld_out;
  void* combined;      // MODE 0, optional: [M, 2K]
  int act;
  int* status;
  // Optional device-side count of valid rows of the packed weights (a weight cache's K): MODE 0
  // writes zero activations for columns >= *k_dev and skips tiles wholly beyond it; MODE 1 stops
  // its contraction at *k_dev (rounded up to a k-block, which MODE 0 filled with zeros).
  const int* k_dev;
  // Optional split of the contraction over gridDim.z CTAs: CTA z takes an equal share of the k-blocks
  // and writes its fp32 partial tile; the caller adds the partials.  MODE 1: part[z][M][ld_out].
  // MODE 0: part[z][M][2*ld_part], gate sums in columns [0, N), up sums in [ld_part, ld_part + N)
  // (the activation needs the complete sums, so it moves to the kernel that adds the partials).
  float* part;
  int ld_part;
};

__device__ __forceinline__ uint32_t pf_smem(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void pf_mbar_init(uint64_t* b, uint32_t n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pf_smem(b)), "r"(n) : "memory");
}
__device__ __forceinline__ void pf_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pf_smem(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool pf_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(pf_smem(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool pf_wait(uint64_t* b, uint32_t parity) {
  for (uint32_t it = 0; it < PF_WAIT_LIMIT; ++it) {
    if (pf_try_wait(b, parity)) return true;
    if (it > 1024) __nanosleep(64);
  }
  return false;
}
__device__ __forceinline__ void pf_tma_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          pf_smem(dst)),
      "l"(map), "r"(pf_smem(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t pf_smem_desc(const void* tile) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((pf_smem(tile) & 0x3ffffu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                           // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                           // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void pf_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void pf_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(pf_smem(bar)) : "memory");
}
__device__ __forceinline__ void pf_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Store n (<= 32) consecutive values of one row as T; 16-byte vectors when the address allows.
template <typename T>
__device__ __forceinline__ void pf_store_row(T* dst, const float* v, int n) {
  if (n == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __align__(16) T tmp[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) tmp[e] = DT<T>::from_f(v[q * 8 + e]);
      *reinterpret_cast<uint4*>(dst + q * 8) = *reinterpret_cast<const uint4*>(tmp);
    }
  } else {
    for (int e = 0; e < n; ++e) dst[e] = DT<T>::from_f(v[e]);
  }
}

// Dynamic shared memory (1024-byte aligned): stages x (A tile | B tile [| second B tile]);
// then full[stages], empty[stages], accum barrier, TMEM base address.
// DK: the device-side row count and the split of the contraction are compiled in (layer step on the
// packed cache); the plain operator call uses the variant without them.
template <typename T, int MODE, int MH, bool DK>
__global__ void __launch_bounds__(PF_THREADS, 1)
k_umma_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PfArgs p) {
  extern __shared__ unsigned char pf_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  constexpr uint32_t STAGE_BYTES = (MH + 2) * PF_TILE_BYTES;   // MH A tiles, 2 B tiles
  constexpr uint32_t TMEM_COLS = MH * 2 * PF_BN;               // accumulator (mh, nt) at column (2*mh + nt) * 128
  const int S = p.stages;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(S) * STAGE_BYTES);
  uint64_t* empty = full + S;
  uint64_t* accum = empty + S;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // MODE 0: row tiles vary fastest, so CTAs in flight share weight tiles and x (which fits L2)
  // is the re-read operand; MODE 1: column tiles vary fastest (the transposed down weight fits L2)
  const int n_idx = MODE == 0 ? blockIdx.y : blockIdx.x, m_idx = MODE == 0 ? blockIdx.x : blockIdx.y;
  const int n0 = n_idx * (MODE == 0 ? PF_BN : 2 * PF_BN), m0 = m_idx * (MH * PF_BM);
  const int k_valid = (DK && p.k_dev) ? *p.k_dev : 0x7fffffff;
  const int k_round = k_valid > 0x7fffff00 ? k_valid : (k_valid + PF_BK - 1) / PF_BK * PF_BK;
  if (DK && MODE == 0 && n0 >= k_round) return;  // nothing downstream reads these columns (uniform for the CTA)
  const int nkb_all = (min(p.Kd, MODE == 1 ? k_valid : p.Kd) + PF_BK - 1) / PF_BK;
  // this CTA's k-blocks [kb_lo, kb_lo + nkb)
  const int nz = DK ? static_cast<int>(gridDim.z) : 1, zi = DK ? static_cast<int>(blockIdx.z) : 0;
  const int kb_lo = (nkb_all * zi) / nz;
  const int nkb = (nkb_all * (zi + 1)) / nz - kb_lo;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      pf_mbar_init(&full[s], 1);
      pf_mbar_init(&empty[s], 1);
    }
    pf_mbar_init(accum, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // tensor memory: one warp allocates, the same warp frees
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(pf_smem(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  bool timed_out = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (kb >= S && !pf_wait(&empty[s], ((kb / S) - 1) & 1)) timed_out = true;
        unsigned char* st = smem + static_cast<size_t>(s) * STAGE_BYTES;
        pf_expect_tx(&full[s], STAGE_BYTES);
#pragma unroll
        for (int mh = 0; mh < MH; ++mh)
          pf_tma_2d(st + mh * PF_TILE_BYTES, &tmA, (kb_lo + kb) * PF_BK, m0 + mh * PF_BM, &full[s]);
        pf_tma_2d(st + MH * PF_TILE_BYTES, &tmB, (kb_lo + kb) * PF_BK, n0, &full[s]);
        pf_tma_2d(st + (MH + 1) * PF_TILE_BYTES, &tmB, (kb_lo + kb) * PF_BK, MODE == 0 ? p.up_off + n0 : n0 + PF_BN, &full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = f32, A/B = f16 or bf16, both K-major, N = 128, M = 128
      const uint32_t fmt = sizeof(T) == 2 && DT<T>::id == STX_BF16 ? 1u : 0u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(PF_BN >> 3) << 17) |
                             (static_cast<uint32_t>(PF_BM >> 4) << 24);
      for (int kb = 0; kb < nkb; ++kb) {
        const int s = kb % S;
        if (!pf_wait(&full[s], (kb / S) & 1)) timed_out = true;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* st = smem + static_cast<size_t>(s) * STAGE_BYTES;
        const uint64_t db0 = pf_smem_desc(st + MH * PF_TILE_BYTES), db1 = pf_smem_desc(st + (MH + 1) * PF_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < PF_BK / 16; ++kk) {
          const uint32_t acc = (kb | kk) != 0;
          const uint64_t adv = static_cast<uint64_t>(kk * 32 >> 4);  // 16 elements = 32 bytes along k
#pragma unroll
          for (int mh = 0; mh < MH; ++mh) {
            const uint64_t da = pf_smem_desc(st + mh * PF_TILE_BYTES) + adv;
            pf_mma(tmem_base + (2 * mh) * PF_BN, da, db0 + adv, idesc, acc);
            pf_mma(tmem_base + (2 * mh + 1) * PF_BN, da, db1 + adv, idesc, acc);
          }
        }
        pf_commit(&empty[s]);  // arrives when the MMAs that read this stage are done
      }
      pf_commit(accum);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int lg = warp & 3;                    // TMEM lane group this warp may read
    if (!pf_wait(accum, 0)) timed_out = true;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    T* out = static_cast<T*>(p.a_out);
    T* comb = static_cast<T*>(p.combined);
#pragma unroll 1
    for (int mh = 0; mh < MH; ++mh) {
      const int row = m0 + mh * PF_BM + lg * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lg * 32) << 16) + (2 * mh) * PF_BN;
      if (MODE == 0) {
#pragma unroll 1
        for (int c = 0; c < PF_BN; c += 32) {
          float g[32], u[32];
          pf_ld32(taddr + c, g);
          pf_ld32(taddr + PF_BN + c, u);
          const int col = n0 + c;
          const int n = min(32, p.N - col);
          if (DK && p.part) {  // split contraction: raw partial sums, the activation follows the sum
            if (row < p.M && n > 0) {
              float* dst = p.part + (static_cast<size_t>(zi) * p.M + row) * (2 * static_cast<size_t>(p.ld_part)) + col;
              for (int e = 0; e < n; ++e) {
                dst[e] = nkb > 0 ? g[e] : 0.f;
                dst[p.ld_part + e] = nkb > 0 ? u[e] : 0.f;
              }
            }
            continue;
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) g[e] = (!DK || col + e < k_valid) ? apply_act(p.act, g[e]) * u[e] : 0.f;
          if (row < p.M && n > 0) {
            if (out) pf_store_row<T>(out + static_cast<size_t>(row) * p.ld_out + col, g, n);
            if (comb) {
              pf_store_row<T>(comb + static_cast<size_t>(row) * (2 * p.N) + col, g, n);
              pf_store_row<T>(comb + static_cast<size_t>(row) * (2 * p.N) + p.N + col, u, n);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 2 * PF_BN; c += 32) {
          float g[32];
          pf_ld32(taddr + c, g);
          if (DK && nkb == 0) {  // empty contraction: the accumulator was never written
#pragma unroll
            for (int e = 0; e < 32; ++e) g[e] = 0.f;
          }
          const int col = n0 + c;
          const int n = min(32, p.N - col);
          if (row < p.M && n > 0) {
            if (DK && p.part) {
              float* dst = p.part + (static_cast<size_t>(zi) * p.M + row) * p.ld_out + col;
              for (int e = 0; e < n; ++e) dst[e] = g[e];
            } else {
              pf_store_row<T>(out + static_cast<size_t>(row) * p.ld_out + col, g, n);
            }
          }
        }
      }
    }
  }
  if (timed_out && p.status && lane == 0) atomicOr(p.status, DEV_TIMEOUT);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// [R, C] -> [C, ldo] (ldo >= R): packed down rows to the K-major B operand of GEMM 2.  64 x 64
// tiles of 16-bit elements, 16-byte global loads and stores on both sides; requires C % 8 == 0 and
// ldo % 8 == 0.  Rows >= R read as zero.  r_dev (optional): device-side row count, rows beyond its
// k-block are never reached by the contraction and are skipped.
__global__ void __launch_bounds__(256) k_pf_transpose(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int R, int C,
                                                      int ldo, const int* __restrict__ r_dev) {
  // the tile is stored transposed ([column][row], rows of 66 elements: the 8 column groups a warp
  // scatters into land in 4 different bank quarters) and read back with aligned 32-bit loads
  __shared__ __align__(16) uint16_t tile[64][66];
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  if (r_dev && r0 >= (*r_dev + PF_BK - 1) / PF_BK * PF_BK) return;
  const int t = threadIdx.x;
#pragma unroll
  for (int k = 0; k < 2; ++k) {  // 64 rows x 8 chunks of 8 elements
    const int idx = t + 256 * k, rr = idx >> 3, cc = (idx & 7) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r0 + rr < R && c0 + cc < C) v = *reinterpret_cast<const uint4*>(in + static_cast<size_t>(r0 + rr) * C + c0 + cc);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      tile[cc + 2 * e][rr] = static_cast<uint16_t>(w[e] & 0xffffu);
      tile[cc + 2 * e + 1][rr] = static_cast<uint16_t>(w[e] >> 16);
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 2; ++k) {  // 64 output rows (columns of the input tile) x 8 chunks of 8 input rows
    const int idx = t + 256 * k, cc = idx >> 3, rr = (idx & 7) * 8;
    if (c0 + cc < C && r0 + rr < ldo) {
      const uint32_t* src = reinterpret_cast<const uint32_t*>(&tile[cc][rr]);  // 132-byte rows: 4-byte aligned
      const uint4 v = make_uint4(src[0], src[1], src[2], src[3]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(c0 + cc) * ldo + r0 + rr) = v;
    }
  }
}

// ---------------------------------------------------------------------------------- host
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PFN_encodeTiled encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  }
  return fn;
}

// 2-D K-major operand [rows, kd] with row stride ld (elements); box 64 x 128, 128-byte swizzle.
static int make_map(CUtensorMap* m, const void* base, int dtype, int64_t rows, int64_t kd, int64_t ld) {
  PFN_encodeTiled enc = encode_fn();
  if (!enc) {
    set_error("prefill path: cuTensorMapEncodeTiled is not available from this driver");
    return STX_ERR_CUDA;
  }
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(kd), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {PF_BK, PF_BM};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(m, dtype == STX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("prefill path: cuTensorMapEncodeTiled failed with %d (rows=%lld k=%lld ld=%lld)", static_cast<int>(r),
              static_cast<long long>(rows), static_cast<long long>(kd), static_cast<long long>(ld));
    return STX_ERR_CUDA;
  }
  return STX_OK;
}

template <typename T, int MODE, int MH, bool DK>
static int launch_umma_dk(const CUtensorMap& a, const CUtensorMap& b, PfArgs p, cudaStream_t s) {
  constexpr uint32_t stage_bytes = (MH + 2) * PF_TILE_BYTES;
  p.stages = MH == 2 ? 3 : 4;
  const size_t smem = 1024 + static_cast<size_t>(p.stages) * stage_bytes + (2 * p.stages + 1) * sizeof(uint64_t) + 16;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    STX_CUDA(cudaFuncSetAttribute(k_umma_gemm<T, MODE, MH, DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    attr_set[dev] = true;
  }
  const int bn = MODE == 0 ? PF_BN : 2 * PF_BN, bm = MH * PF_BM;
  dim3 grid((p.N + bn - 1) / bn, (p.M + bm - 1) / bm, static_cast<unsigned>(std::max(1, p.stages_z)));
  if (MODE == 0) grid = dim3(grid.y, grid.x, grid.z);
  k_umma_gemm<T, MODE, MH, DK><<<grid, PF_THREADS, smem, s>>>(a, b, p);
  STX_LAUNCH_CHECK("k_umma_gemm");
  return STX_OK;
}

template <typename T, int MODE, int MH>
static int launch_umma_mh(const CUtensorMap& a, const CUtensorMap& b, const PfArgs& p, cudaStream_t s) {
  return (p.k_dev || p.part) ? launch_umma_dk<T, MODE, MH, true>(a, b, p, s) : launch_umma_dk<T, MODE, MH, false>(a, b, p, s);
}

template <typename T, int MODE>
static int launch_umma(const CUtensorMap& a, const CUtensorMap& b, const PfArgs& p, cudaStream_t s) {
  // one row half for small row counts, two (a 256-row CTA tile) otherwise
  return p.M > PF_BM ? launch_umma_mh<T, MODE, 2>(a, b, p, s) : launch_umma_mh<T, MODE, 1>(a, b, p, s);
}

// a[b][j] = act(sum_z gate_z[b][j]) * sum_z up_z[b][j] for j < K (zero up to the end of K's k-block),
// z ascending: the tail of a GEMM 1 whose contraction was split.
template <typename T>
__global__ void __launch_bounds__(256) k_pf_act_sum(const float* __restrict__ part, int nz, int M, int N, int ldp,
                                                    T* __restrict__ a_out, int ld_out, int act, const int* __restrict__ k_dev) {
  const int k_valid = k_dev ? min(*k_dev, N) : N;
  const int k_round = min(N, (k_valid + PF_BK - 1) / PF_BK * PF_BK);
  const int j = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (j >= k_round || b >= M) return;
  float g = 0.f, u = 0.f;
  for (int z = 0; z < nz; ++z) {
    const float* src = part + (static_cast<size_t>(z) * M + b) * (2 * static_cast<size_t>(ldp)) + j;
    g += __ldcg(src);
    u += __ldcg(src + ldp);
  }
  a_out[static_cast<size_t>(b) * ld_out + j] = DT<T>::from_f(j < k_valid ? apply_act(act, g) * u : 0.f);
}

// GEMM 1 has ceil(B/128..256) x I/128 output tiles: a shard of the intermediate dimension with few rows
// leaves most SMs without one, so its contraction (over H) is split too.
static int gemm1_splits(int64_t B, int64_t H, int64_t K) {
  const int64_t bm = B > PF_BM ? 2 * PF_BM : PF_BM;
  const int64_t tiles = ((B + bm - 1) / bm) * ((K + PF_BN - 1) / PF_BN);
  if (tiles > num_sms()) return 1;
  // round up: the tiles are counted for all K slots, but a cache is rarely full (tiles beyond the
  // device-side K exit at once), so up to 2x the SM count of CTAs still runs as about one wave
  return static_cast<int>(std::min<int64_t>({8, (num_sms() + tiles - 1) / tiles, std::max<int64_t>(1, H / (4 * PF_BK))}));
}

// GEMM 2 has only ceil(B/128..256) x H/256 output tiles; for few rows the contraction is split so
// that about one CTA per SM streams the down weight.
static int gemm2_splits(int64_t B, int64_t H) {
  const int64_t tiles = ((B + (B > PF_BM ? 2 * PF_BM : PF_BM) - 1) / (B > PF_BM ? 2 * PF_BM : PF_BM)) * ((H + 2 * PF_BN - 1) / (2 * PF_BN));
  if (tiles * 2 > num_sms()) return 1;
  return static_cast<int>(std::min<int64_t>(16, std::max<int64_t>(1, num_sms() / tiles)));
}

size_t prefill_scratch_bytes(int64_t B, int64_t H, int64_t K) {
  const int64_t K8 = (K + 7) / 8 * 8;
  const int z = gemm2_splits(B, H), z1 = gemm1_splits(B, H, K);
  return align_up(static_cast<size_t>(B) * K8 * 2, 1024) + align_up(static_cast<size_t>(H) * K8 * 2, 1024) + 1024 +
         (z > 1 ? align_up(static_cast<size_t>(z) * B * H * sizeof(float), 1024) : 0) +
         (z1 > 1 ? align_up(static_cast<size_t>(z1) * B * 2 * K8 * sizeof(float), 1024) : 0);
}

// Implemented in stx_mlp_row.cu: out[i] = sum over g < G of partial[g][i], g ascending (n % 128 == 0).
int partial_sum(const float* partial, int G, int64_t n, void* out, int dtype, cudaStream_t s);

// Row blocks of STX_GEMM_MIN_ROWS and more (16-bit, gated) run as tensor-core GEMMs.
bool prefill_wanted(int64_t B, int64_t H, int64_t K, int dtype, int has_gate) {
  return dtype != STX_F32 && has_gate && B >= STX_GEMM_MIN_ROWS && (H % 64) == 0 && K >= 64;
}

// x [B,H], concat [2K,H] (gate rows then up rows), down_packed [K,H]; scratch: prefill_scratch_bytes().
// k_dev (optional): device count of valid packed rows, <= K; the work then follows *k_dev while all
// shapes, tensor maps and grids are built for K, so the call needs no host read-back.
int prefill_forward(const void* x, int64_t B, int64_t H, const void* concat, const void* down_packed, int64_t K,
                    void* out, void* combined, int act, int dtype, void* scratch, int* status, const int* k_dev,
                    cudaStream_t s) {
  const int64_t K8 = (K + 7) / 8 * 8;
  const uintptr_t base = (reinterpret_cast<uintptr_t>(scratch) + 1023) & ~static_cast<uintptr_t>(1023);
  void* a_scr = reinterpret_cast<void*>(base);                                                   // [B, K8]
  void* dt_scr = reinterpret_cast<void*>(base + align_up(static_cast<size_t>(B) * K8 * 2, 1024));  // [H, K8]
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(concat)) & 15) {
    set_error("prefill path: x and concat_w must be 16-byte aligned");
    return STX_ERR_INVALID_ARG;
  }
  // down rows -> K-major [H, K8]
  {
    dim3 grid(static_cast<unsigned>((H + 63) / 64), static_cast<unsigned>((K + 63) / 64));
    k_pf_transpose<<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(down_packed), static_cast<uint16_t*>(dt_scr),
                                                 static_cast<int>(K), static_cast<int>(H), static_cast<int>(K8), k_dev);
    STX_LAUNCH_CHECK("k_pf_transpose");
  }
  // the activations are GEMM 2's A operand: read them straight from combined_buf[:, :K] when its
  // row stride is TMA-compatible (a multiple of 16 bytes), else from the scratch copy
  const bool a_in_combined = combined != nullptr && (K % 4) == 0 && (reinterpret_cast<uintptr_t>(combined) & 15) == 0;
  CUtensorMap mx, mw, ma, md;
  int rc = make_map(&mx, x, dtype, B, H, H);
  if (rc == STX_OK) rc = make_map(&mw, concat, dtype, 2 * K, H, H);
  if (rc == STX_OK) rc = a_in_combined ? make_map(&ma, combined, dtype, B, K, 2 * K) : make_map(&ma, a_scr, dtype, B, K, K8);
  if (rc == STX_OK) rc = make_map(&md, dt_scr, dtype, H, K, K8);
  if (rc != STX_OK) return rc;
  PfArgs g1{};
  g1.M = static_cast<int>(B);
  g1.N = static_cast<int>(K);
  g1.Kd = static_cast<int>(H);
  g1.up_off = static_cast<int>(K);
  g1.stages = 4;
  g1.a_out = a_in_combined ? nullptr : a_scr;
  g1.ld_out = static_cast<int>(K8);
  g1.combined = combined;
  g1.act = act;
  g1.status = status;
  g1.k_dev = k_dev;
  PfArgs g2{};
  g2.M = static_cast<int>(B);
  g2.N = static_cast<int>(H);
  g2.Kd = static_cast<int>(K);
  g2.stages = 6;
  g2.a_out = out;
  g2.ld_out = static_cast<int>(H);
  g2.act = act;
  g2.status = status;
  g2.k_dev = k_dev;
  const int z_sized = gemm2_splits(B, H);  // what prefill_scratch_bytes reserved
  const int z = (B * H) % 128 == 0 ? z_sized : 1;
  float* part = nullptr;
  const uintptr_t part_base = base + align_up(static_cast<size_t>(B) * K8 * 2, 1024) + align_up(static_cast<size_t>(H) * K8 * 2, 1024);
  if (z > 1) {
    part = reinterpret_cast<float*>(part_base);
    g2.part = part;
    g2.stages_z = z;
  }
  // GEMM 1 split (only without combined_buf: the activation moves to k_pf_act_sum, which writes a alone)
  const int z1 = combined == nullptr ? gemm1_splits(B, H, K) : 1;
  float* part1 = nullptr;
  if (z1 > 1) {
    part1 = reinterpret_cast<float*>(part_base + (z_sized > 1 ? align_up(static_cast<size_t>(z_sized) * B * H * sizeof(float), 1024) : 0));
    g1.part = part1;
    g1.ld_part = static_cast<int>(K8);
    g1.stages_z = z1;
  }
  const dim3 agrid(static_cast<unsigned>((K + 255) / 256), static_cast<unsigned>(B));
  if (dtype == STX_F16) {
    rc = launch_umma<__half, 0>(mx, mw, g1, s);
    if (rc == STX_OK && part1) {
      k_pf_act_sum<__half><<<agrid, 256, 0, s>>>(part1, z1, static_cast<int>(B), static_cast<int>(K), static_cast<int>(K8),
                                                 static_cast<__half*>(a_scr), static_cast<int>(K8), act, k_dev);
      STX_LAUNCH_CHECK("k_pf_act_sum");
    }
    if (rc == STX_OK) rc = launch_umma<__half, 1>(ma, md, g2, s);
  } else {
    rc = launch_umma<__nv_bfloat16, 0>(mx, mw, g1, s);
    if (rc == STX_OK && part1) {
      k_pf_act_sum<__nv_bfloat16><<<agrid, 256, 0, s>>>(part1, z1, static_cast<int>(B), static_cast<int>(K), static_cast<int>(K8),
                                                        static_cast<__nv_bfloat16*>(a_scr), static_cast<int>(K8), act, k_dev);
      STX_LAUNCH_CHECK("k_pf_act_sum");
    }
    if (rc == STX_OK) rc = launch_umma<__nv_bfloat16, 1>(ma, md, g2, s);
  }
  if (rc == STX_OK && part) rc = partial_sum(part, z, B * H, out, dtype, s);
  return rc;
}

}  // namespace stx
