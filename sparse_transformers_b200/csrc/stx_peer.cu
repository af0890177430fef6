// Peer-memory exchange object and the stand-alone all-reduce kernel (C ABI: stx_peer_*).
#include "stx_peer.cuh"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <new>

namespace stx {

bool peer_args(const stx_peer* p, PeerArgs* out) {
  if (!p || !p->connected) return false;
  out->mine = static_cast<uint2*>(p->local);
  for (int q = 0; q < PEER_MAX_WORLD; ++q) out->peer[q] = static_cast<uint2*>(q < p->world ? p->peers[q] : nullptr);
  out->ctl = p->ctl;
  out->max_elems = p->max_elems;
  out->rank = p->rank;
  out->world = p->world;
  out->wait_limit = p->wait_limit;
  return true;
}

// data[i] <- sum over ranks of data[i], in place.  Every thread first pushes all its elements,
// then collects them, so the waits for different elements overlap.
template <typename T>
__global__ void __launch_bounds__(256) k_peer_allreduce(const __grid_constant__ PeerArgs a, T* __restrict__ data, long long n) {
  pdl_wait();
  pdl_launch_dependents();
  const int epoch = peer_epoch_begin(a);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long i0 = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (long long i = i0; i < n; i += stride) peer_push(a, epoch, i, DT<T>::to_f(data[i]));
  bool timed_out = false;
  for (long long i = i0; i < n; i += stride) {
    const float s = peer_collect(a, epoch, i, DT<T>::to_f(data[i]), &timed_out);
    data[i] = DT<T>::from_f(s);
  }
  if (timed_out) atomicOr(a.ctl + 2, DEV_TIMEOUT);
  peer_epoch_end(a, epoch);
}

int peer_allreduce(const stx_peer* p, void* data, int64_t n, int dtype, cudaStream_t s) {
  PeerArgs a;
  if (!peer_args(p, &a)) {
    set_error("stx_peer_allreduce: the peer object is not connected");
    return STX_ERR_INVALID_ARG;
  }
  STX_CHECK_ARG(n >= 0 && n <= p->max_elems, "stx_peer_allreduce: n=%lld exceeds max_elems=%lld", static_cast<long long>(n),
                static_cast<long long>(p->max_elems));
  if (n == 0 || p->world == 1) return STX_OK;
  const unsigned grid = static_cast<unsigned>(std::min<int64_t>((n + 255) / 256, 8 * static_cast<int64_t>(num_sms())));
  const long long nn = n;
  switch (dtype) {
    case STX_F32: STX_CUDA(launch_pdl(k_peer_allreduce<float>, dim3(grid), dim3(256), 0, s, a, static_cast<float*>(data), nn)); break;
    case STX_F16: STX_CUDA(launch_pdl(k_peer_allreduce<__half>, dim3(grid), dim3(256), 0, s, a, static_cast<__half*>(data), nn)); break;
    default:
      STX_CUDA(launch_pdl(k_peer_allreduce<__nv_bfloat16>, dim3(grid), dim3(256), 0, s, a, static_cast<__nv_bfloat16*>(data), nn));
      break;
  }
  return STX_OK;
}

}  // namespace stx

using namespace stx;

extern "C" {

int stx_peer_create(stx_peer_t** out, int rank, int world, int64_t max_elems) {
  STX_CHECK_ARG(out, "stx_peer_create: out is null");
  *out = nullptr;
  STX_CHECK_ARG(world >= 1 && world <= PEER_MAX_WORLD && rank >= 0 && rank < world,
                "stx_peer_create: rank %d / world %d outside 1..%d", rank, world, PEER_MAX_WORLD);
  STX_CHECK_ARG(max_elems > 0, "stx_peer_create: max_elems must be positive");
  stx_peer* p = new (std::nothrow) stx_peer();
  if (!p) {
    set_error("stx_peer_create: out of host memory");
    return STX_ERR_ALLOC;
  }
  p->rank = rank;
  p->world = world;
  p->max_elems = max_elems;
  if (const char* e = getenv("STX_PEER_WAIT_ITERS")) {
    const long v = atol(e);
    if (v > 0) p->wait_limit = static_cast<unsigned>(std::min<long>(v, 1L << 30));
  }
  const size_t bytes = sizeof(uint2) * 2 * static_cast<size_t>(world) * static_cast<size_t>(max_elems);
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaMalloc(&p->local, bytes);
  if (e == cudaSuccess) e = cudaMemset(p->local, 0, bytes);
  if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->ctl), 256);
  if (e == cudaSuccess) e = cudaMemset(p->ctl, 0, 256);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    set_error("stx_peer_create: device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    cudaFree(p->local);
    cudaFree(p->ctl);
    delete p;
    return STX_ERR_ALLOC;
  }
  p->peers[rank] = p->local;
  p->connected = world == 1;
  *out = p;
  return STX_OK;
}

int stx_peer_destroy(stx_peer_t* p) {
  if (!p) return STX_OK;
  for (int q = 0; q < p->world; ++q)
    if (p->ipc_opened[q] && p->peers[q]) cudaIpcCloseMemHandle(p->peers[q]);
  cudaFree(p->local);
  cudaFree(p->ctl);
  delete p;
  return STX_OK;
}

int stx_peer_ipc_handle(stx_peer_t* p, void* handle_out) {
  STX_CHECK_ARG(p && handle_out, "stx_peer_ipc_handle: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == STX_PEER_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  STX_CUDA(cudaIpcGetMemHandle(&h, p->local));
  memcpy(handle_out, &h, sizeof(h));
  return STX_OK;
}

int stx_peer_connect_ipc(stx_peer_t* p, const void* handles) {
  STX_CHECK_ARG(p && handles, "stx_peer_connect_ipc: null pointer");
  STX_CHECK_ARG(!p->connected || p->world == 1, "stx_peer_connect_ipc: already connected");
  for (int q = 0; q < p->world; ++q) {
    if (q == p->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const char*>(handles) + static_cast<size_t>(q) * STX_PEER_HANDLE_BYTES, sizeof(h));
    void* ptr = nullptr;
    STX_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    p->peers[q] = ptr;
    p->ipc_opened[q] = true;
  }
  p->connected = true;
  return STX_OK;
}

int stx_peer_connect_ptrs(stx_peer_t* p, void* const* buffers) {
  STX_CHECK_ARG(p && buffers, "stx_peer_connect_ptrs: null pointer");
  for (int q = 0; q < p->world; ++q) {
    if (q == p->rank) continue;
    STX_CHECK_ARG(buffers[q], "stx_peer_connect_ptrs: buffer of rank %d is null", q);
    p->peers[q] = buffers[q];
  }
  p->connected = true;
  return STX_OK;
}

int stx_peer_local_buffer(stx_peer_t* p, void** buffer_out) {
  STX_CHECK_ARG(p && buffer_out, "stx_peer_local_buffer: null pointer");
  *buffer_out = p->local;
  return STX_OK;
}

int stx_peer_allreduce(stx_peer_t* p, void* data, int64_t n, int dtype, void* stream) {
  STX_CHECK_ARG(p && data, "stx_peer_allreduce: null pointer");
  STX_CHECK_ARG(dtype == STX_F32 || dtype == STX_F16 || dtype == STX_BF16, "stx_peer_allreduce: bad dtype %d", dtype);
  return peer_allreduce(p, data, n, dtype, static_cast<cudaStream_t>(stream));
}

int stx_peer_status(stx_peer_t* p, int* status_out, void* stream) {
  STX_CHECK_ARG(p && status_out, "stx_peer_status: null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  STX_CUDA(cudaMemcpyAsync(&v, p->ctl + 2, sizeof(int), cudaMemcpyDeviceToHost, s));
  STX_CUDA(cudaStreamSynchronize(s));
  *status_out = (v & DEV_TIMEOUT) ? STX_ERR_TIMEOUT : STX_OK;
  return STX_OK;
}

}  // extern "C"
