// Shared device/host helpers for the sm_100a sparse-MLP kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "stx.h"

namespace stx {

// ---------------------------------------------------------------- error plumbing (host)
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns STX_ERR_CUDA

#define STX_CUDA(call)                                         \
  do {                                                         \
    cudaError_t e__ = (call);                                  \
    if (e__ != cudaSuccess) return ::stx::cuda_fail(e__, #call); \
  } while (0)

#define STX_CHECK_ARG(cond, ...)        \
  do {                                  \
    if (!(cond)) {                      \
      ::stx::set_error(__VA_ARGS__);    \
      return STX_ERR_INVALID_ARG;       \
    }                                   \
  } while (0)

#define STX_LAUNCH_CHECK(name)                                            \
  do {                                                                    \
    cudaError_t e__ = cudaGetLastError();                                 \
    if (e__ != cudaSuccess) return ::stx::cuda_fail(e__, "launch " name); \
  } while (0)

int num_sms();  // SM count of the current device (cached per device)

inline size_t dtype_size(int dt) { return dt == STX_F32 ? 4 : 2; }
// Row blocks of at least this many rows (16-bit, gated) run as tensor-core GEMMs over packed weights;
// fewer rows run the streaming kernels (1 row: k_mlp_b1, 2..8: k_mlp_bn).
constexpr int64_t STX_GEMM_MIN_ROWS = 9;
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ---------------------------------------------------------------- dtype traits
// V = elements per 16-byte vector.  All row lengths that take the vector path are
// multiples of V, and all row starts are 16-byte aligned.
template <typename T> struct DT;
template <> struct DT<float> {
  static constexpr int V = 4;
  static constexpr int id = STX_F32;
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
  static __device__ __forceinline__ float round_f(float v) { return v; }
};
template <> struct DT<__half> {
  static constexpr int V = 8;
  static constexpr int id = STX_F16;
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
  static __device__ __forceinline__ float round_f(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct DT<__nv_bfloat16> {
  static constexpr int V = 8;
  static constexpr int id = STX_BF16;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round_f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

// 16-byte streaming load (read-only data that no thread of this kernel writes).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// 16-byte load through L1 (small operands re-read by many threads, e.g. x).
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
  return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// fp32 vector reduction into global memory (4 consecutive floats, 16-byte aligned).
__device__ __forceinline__ void red_add_f32x4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <typename T> struct Unpack;
template <> struct Unpack<float> {
  static __device__ __forceinline__ void run(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
};
template <> struct Unpack<__half> {
  static __device__ __forceinline__ void run(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <> struct Unpack<__nv_bfloat16> {
  static __device__ __forceinline__ void run(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // bf16 -> fp32 is a 16-bit shift
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ float warp_sum_xor(float v) {
  // Butterfly: every lane ends with the same bits because a+b == b+a exactly.
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// Activations in fp32 (accurate libm variants; they run once per active neuron).
__device__ __forceinline__ float apply_act(int act, float x) {
  switch (act) {
    case STX_ACT_RELU: return fmaxf(x, 0.f);
    case STX_ACT_SILU: return x / (1.f + expf(-x));
    case STX_ACT_GELU_TANH: {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
    }
    case STX_ACT_SIGMOID: return 1.f / (1.f + expf(-x));
    case STX_ACT_GELU: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    default: return x;
  }
}

// Programmatic dependent launch: a kernel launched with launch_pdl() may start while its
// predecessor on the stream is still running; it must call pdl_wait() before it touches
// anything the predecessor wrote (or still reads), and may do set-up work before that.
// pdl_wait() returns at once in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Device status word bits (stx_cache state[STATUS]).
enum : int {
  DEV_OK = 0,
  DEV_NO_ACTIVE = 1,  // an update produced K == 0
  DEV_BAD_INDEX = 2,  // a bounds check skipped an access
  DEV_TIMEOUT = 4     // a bounded wait expired
};

}  // namespace stx
