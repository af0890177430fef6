// Device-side pieces shared by the persistent single-row stack kernels (stx_stack_b1.cu: layer by layer;
// stx_stack_flow.cu: all predictors first, then one uninterrupted row stream).
#pragma once

#include "stx_common.cuh"

namespace stx {

constexpr int SB1_THREADS = 512;
constexpr int SB1_WARPS = SB1_THREADS / 32;
constexpr int SB1_MAX_SLOTS = 16;
constexpr int SB1_MY_CAP = 128;    // neurons of one CTA per layer: ceil(K / G) <= 128
constexpr int SB1_MAX_PASS = 2;    // 16-byte column chunks per thread: H / V <= 2 * 512
constexpr int SB1_OFF_AS = 256;    // a_s [2 buffers][4] floats
constexpr int SB1_OFF_PD = 320;    // quarter sums [2 buffers][4 neurons][4 quarters] float2
constexpr int SB1_OFF_T = 832;     // t of the layer in the score layout, <= 512 bytes
constexpr int SB1_OFF_MY = 1344;   // the CTA's neurons of the layer [SB1_MY_CAP]
constexpr int SB1_HEADER = 1920;   // x follows, then the slots
constexpr uint32_t SB1_GRID_WAIT_LIMIT = 1u << 21;

// sync words (uint32): [0] generation, then one counter per barrier, 128 bytes apart
constexpr int SB1_SYNC_GEN = 0, SB1_SYNC_A = 32, SB1_SYNC_B = 64, SB1_SYNC_C = 96, SB1_SYNC_M = 128;
// the three barriers of the flow kernel (once per launch each)
constexpr int SB1_SYNC_FT = 160, SB1_SYNC_FM = 192, SB1_SYNC_FP = 224;

// Poll limit of a grid barrier.  Sharded, a CTA of this GPU may itself be waiting for a peer rank (that wait has
// its own, shorter limit): the barrier outlasts it.
__device__ __forceinline__ uint32_t grid_wait_limit(int world) { return world > 1 ? SB1_GRID_WAIT_LIMIT * 8u : SB1_GRID_WAIT_LIMIT; }

__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until the counter has reached `target` (wrap-safe).  False when the limit expired.
__device__ __forceinline__ bool grid_wait(const uint32_t* ctr, uint32_t target, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (static_cast<int32_t>(ld_acquire_u32(ctr) - target) >= 0) return true;
  }
  return false;
}

// floor(n / d) for 0 <= n < 2^24, d > 0, rd = 1.0f / d: one multiplication and a correction by one either way
__device__ __forceinline__ int div_small(int n, int d, float rd) {
  int q = __float2int_rz(__int2float_rz(n) * rd);
  if (q * d > n) --q;
  if ((q + 1) * d <= n) ++q;
  return q;
}

// acc + sum over the 8 (fp32: 4) elements of a 16-byte chunk of w[e] * x[e], in element order with one
// rounding per step.  16-bit types use the mixed-precision fma (both factors 16-bit, fp32 addend and
// result): the product of two 16-bit floats is exact in fp32, so the result equals convert + fmaf while
// no conversion instruction is issued.
template <typename T> struct MixDot;
template <> struct MixDot<float> {
  static __device__ __forceinline__ float run(const uint4& w, const uint4& x, float acc) {
    acc = fmaf(__uint_as_float(w.x), __uint_as_float(x.x), acc);
    acc = fmaf(__uint_as_float(w.y), __uint_as_float(x.y), acc);
    acc = fmaf(__uint_as_float(w.z), __uint_as_float(x.z), acc);
    acc = fmaf(__uint_as_float(w.w), __uint_as_float(x.w), acc);
    return acc;
  }
};
#define STX_MIXDOT_PAIR(SUFFIX)                                                                               \
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\tmov.b32 {wl, wh}, %1;\n\tmov.b32 {xl, xh}, %2;\n\t"                  \
      "fma.rn.f32." SUFFIX " %0, wl, xl, %0;\n\tfma.rn.f32." SUFFIX " %0, wh, xh, %0;\n\t}"                   \
      : "+f"(acc)                                                                                             \
      : "r"(ww), "r"(xx))
template <> struct MixDot<__half> {
  static __device__ __forceinline__ float run(const uint4& w, const uint4& x, float acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t ww = wv[i], xx = xv[i];
      STX_MIXDOT_PAIR("f16");
    }
    return acc;
  }
};
template <> struct MixDot<__nv_bfloat16> {
  static __device__ __forceinline__ float run(const uint4& w, const uint4& x, float acc) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w}, xv[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t ww = wv[i], xx = xv[i];
      STX_MIXDOT_PAIR("bf16");
    }
    return acc;
  }
};
#undef STX_MIXDOT_PAIR

}  // namespace stx
