// Error reporting, device queries and small C-ABI helpers.
#include "stx_common.cuh"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace stx {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
  return STX_ERR_CUDA;
}

int num_sms() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace stx

extern "C" {

const char* stx_last_error(void) { return stx::g_err; }

int stx_version(void) { return STX_VERSION; }

const char* stx_status_string(int status) {
  switch (status) {
    case STX_OK: return "ok";
    case STX_ERR_INVALID_ARG: return "invalid argument";
    case STX_ERR_UNSUPPORTED: return "unsupported shape or dtype";
    case STX_ERR_CUDA: return "CUDA runtime error";
    case STX_ERR_NO_ACTIVE: return "No active weights";
    case STX_ERR_CACHE_INVALID: return "Cache is not valid";
    case STX_ERR_ALLOC: return "device allocation failed";
    case STX_ERR_TIMEOUT: return "device-side wait timed out";
    case STX_ERR_TOO_LARGE: return "size exceeds a fixed limit";
    default: return "unknown status";
  }
}

int stx_act_from_name(const char* name) {
  if (!name) return -1;
  if (!strcmp(name, "relu")) return STX_ACT_RELU;
  if (!strcmp(name, "silu") || !strcmp(name, "swish")) return STX_ACT_SILU;
  if (!strcmp(name, "gelu_pytorch_tanh") || !strcmp(name, "gelu_new") || !strcmp(name, "gelu_tanh")) return STX_ACT_GELU_TANH;
  if (!strcmp(name, "sigmoid")) return STX_ACT_SIGMOID;
  if (!strcmp(name, "gelu")) return STX_ACT_GELU;
  return -1;
}

}  // extern "C"
