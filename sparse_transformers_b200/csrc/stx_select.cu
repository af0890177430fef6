// Per-row selection rules that need a whole score row, and the approximate top-k threshold.
#include "stx_common.cuh"

namespace stx {

int mask_from_scores(const void* scores, int64_t B, int64_t I, int dtype, int method, float param,
                     uint32_t* bits_out, void* scratch, cudaStream_t s) {
  (void)scores; (void)B; (void)I; (void)dtype; (void)param; (void)bits_out; (void)scratch; (void)s;
  set_error("mask rule %d is not built yet", method);
  return STX_ERR_UNSUPPORTED;
}

}  // namespace stx

using namespace stx;

extern "C" {

int stx_approx_topk_scratch_bytes(int64_t B, int64_t I, size_t* bytes_out) {
  STX_CHECK_ARG(bytes_out && B > 0 && I > 0, "stx_approx_topk_scratch_bytes: bad argument");
  *bytes_out = 256;
  return STX_OK;
}

int stx_approx_topk_threshold(const void* scores, int64_t B, int64_t I, int64_t k, int dtype, void* threshold_out,
                              void* scratch, void* stream) {
  (void)scores; (void)B; (void)I; (void)k; (void)dtype; (void)threshold_out; (void)scratch; (void)stream;
  set_error("stx_approx_topk_threshold is not built yet");
  return STX_ERR_UNSUPPORTED;
}

}  // extern "C"
