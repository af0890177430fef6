// Sparse gated MLP for decode batches: host dispatch between the streaming kernels.
//
//   a[j,b]   = act(x[b]·gate[j]) * (x[b]·up[j])      (K active neurons)
//   out[b,:] = sum_j a[j,b] * down[j,:]
//
//   stx_mlp_batch.cu   k_gateup_tma / k_gateup_mma + k_down_rows: two kernels over packed rows or a mask-listed
//                      gather; any dtype, gated or not
//   stx_mlp_row.cu     k_mlp_b1 + k_partial_reduce: one row, predictor scores of the CTA's own neurons, mask bytes,
//                      row gather and the whole MLP in one kernel; k_mlp_bn + k_partial_reduce4: 2..8 rows of
//                      16-bit gated weights, same structure with both projections on the tensor pipe
#include "stx_mlp_stream.cuh"

namespace stx {

// Returns STX_ERR_UNSUPPORTED (without setting an error text) when the shape does not fit
// these kernels; the caller then uses the plain-load kernel.
// scratch: fp32 a[K][B] at offset 256.  parts: bit 0 = gate/up kernel, bit 1 = down kernel.
int mlp_forward_tma(const void* x, int64_t B, int64_t H, const void* gate, const void* up, const void* down,
                    const int32_t* K_dev, int64_t K_host, const GatherSpec* gs, void* out, void* combined, int act,
                    int has_gate, int dtype, void* scratch, float* partial, int* status, unsigned parts,
                    cudaStream_t s) {
  const size_t es = dtype_size(dtype);
  const int V = static_cast<int>(16 / es);
  const int nchunk = static_cast<int>(H / V);
  if (nchunk < 32) return STX_ERR_UNSUPPORTED;
  const uintptr_t al = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(down);
  if (al & 15) return STX_ERR_UNSUPPORTED;
  const int nb = B >= 8 ? 8 : (B >= 4 ? 4 : (B >= 2 ? 2 : 1));
  const int nmat = has_gate ? 2 : 1;
  const size_t row_bytes = static_cast<size_t>(H) * es;
  const size_t x_bytes = (es * nb * H + 127) / 128 * 128;
  if (256 + x_bytes + 2 * nmat * row_bytes > TMA_SMEM_BUDGET) return STX_ERR_UNSUPPORTED;
  const int nwarps = static_cast<int>(std::min<size_t>(16, (TMA_SMEM_BUDGET - 256 - x_bytes) / (nmat * row_bytes)));
  GateUpArgs a;
  a.x = x;
  a.gate = gate;
  a.up = up;
  a.combined = combined;
  a.a_out = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256);
  a.status = status;
  a.K_dev = K_dev;
  a.mask_bits = gs ? gs->mask_bits : nullptr;
  a.idx_out = gs ? gs->idx : nullptr;
  a.count_out = gs ? gs->count : nullptr;
  a.I = gs ? gs->I : 0;
  a.K_host = static_cast<int>(K_host);
  a.B = static_cast<int>(B);
  a.H = static_cast<int>(H);
  a.act = act;
  a.has_gate = has_gate;
  a.nwarps = nwarps;
  const size_t smem = 256 + x_bytes + static_cast<size_t>(nwarps) * nmat * row_bytes;
  // gather mode runs next to the cache maintenance of the same layer (side stream): leave one
  // SM free for its single-block index plan instead of making a persistent CTA wait for it
  int grid = gs ? std::max(1, num_sms() - 1) : num_sms();
  if (!K_dev && !gs) grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(grid, K_host)));
  if (gs) {
    // the in-kernel listing of the mask handles 8 words per thread and 512 rows per CTA
    const size_t mma_stride = row_bytes + 64;
    const size_t mma_fixed = 256 + static_cast<size_t>(std::min<int64_t>(B, 8)) * mma_stride;
    int min_warps = nwarps;
    if (es == 2 && mma_fixed + 2 * MMA_TILE_ROWS * mma_stride <= TMA_SMEM_BUDGET)
      min_warps = std::min<int>(min_warps, static_cast<int>((TMA_SMEM_BUDGET - mma_fixed) / (MMA_TILE_ROWS * mma_stride)));
    if ((gs->I + 31) / 32 > 8 * 32 * min_warps || (gs->I + grid - 1) / grid + 4 > GATHER_MY_CAP) return STX_ERR_UNSUPPORTED;
  }
  DownArgs d;
  d.a = a.a_out;
  d.down = down;
  d.out = out;
  d.K_dev = gs ? gs->count : K_dev;
  d.row_idx = gs ? gs->idx : nullptr;
  d.K_host = static_cast<int>(K_host);
  d.B = static_cast<int>(B);
  d.H = static_cast<int>(H);
  // batch 1 with room for three rows per warp and H within the register accumulators: fused kernel
  const bool b1 = B == 1 && partial != nullptr && mlp_row_slots(static_cast<int>(H), has_gate, dtype, 0) > 0;
  if (b1) return mlp_row_launch(a, down, partial, out, grid, parts, dtype, s);
  return mlp_batch_launch(a, nb, grid, smem, d, parts, dtype, s);
}


}  // namespace stx
