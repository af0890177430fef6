// One-shot all-reduce over peer memory (NVLink / NVSwitch), usable inside other kernels.
//
// Every rank owns an exchange buffer of 8-byte words {fp32 bits, epoch}:
//     word(parity, src, i) = buf[(parity * world + src) * max_elems + i]
// A rank pushes its value for element i into word(epoch & 1, rank, i) of every peer with one
// 8-byte store, then polls its own words of the other ranks until their epoch matches and adds
// the values in ascending rank order, so every rank gets bit-identical sums.  The epoch travels
// with the data, hence no flag, no fence and a single NVLink traversal on the critical path.
// Two parities suffice: a rank can run at most one call ahead of a peer, because finishing call
// e needs that peer's data of call e, which the peer sends only after it has finished e - 1.
// The epoch of a call lives in device memory (ctl[0]) so that a replayed CUDA graph advances it.
#pragma once

#include "stx_common.cuh"

namespace stx {

constexpr int PEER_MAX_WORLD = 8;

struct PeerArgs {
  uint2* mine;                   // this rank's exchange buffer
  uint2* peer[PEER_MAX_WORLD];   // every rank's buffer as seen from this GPU (peer[rank] == mine)
  int* ctl;                      // [0] epoch of the last finished call, [1] block ticket, [2] status bits
  long long max_elems;
  int rank, world;
  unsigned wait_limit;           // poll iterations before a wait gives up
};

// All blocks of a launch call this once after pdl_wait(): the epoch of this call.
__device__ __forceinline__ int peer_epoch_begin(const PeerArgs& a) {
  return static_cast<int>(static_cast<unsigned>(*reinterpret_cast<volatile int*>(a.ctl)) + 1u);
}

// All threads of every block call this at the end; the last block to arrive advances the epoch.
__device__ __forceinline__ void peer_epoch_end(const PeerArgs& a, int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned nblocks = gridDim.x * gridDim.y * gridDim.z;
    if (atomicAdd(reinterpret_cast<unsigned*>(a.ctl + 1), 1u) == nblocks - 1) {
      a.ctl[1] = 0;
      *reinterpret_cast<volatile int*>(a.ctl) = epoch;
    }
  }
}

__device__ __forceinline__ void peer_push(const PeerArgs& a, int epoch, long long i, float v) {
  const long long off = (static_cast<long long>(epoch & 1) * a.world + a.rank) * a.max_elems + i;
  for (int d = 1; d < a.world; ++d) {  // start with the next rank: spreads the first stores over the links
    const int p = (a.rank + d) % a.world;
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1,%2};" ::"l"(a.peer[p] + off), "r"(__float_as_uint(v)), "r"(epoch)
                 : "memory");
  }
}

// Sum over ranks in ascending order; `v` is this rank's own value.  Sets *timed_out when a peer's
// word did not arrive within the limit (the sum then lacks that term).
__device__ __forceinline__ float peer_collect(const PeerArgs& a, int epoch, long long i, float v, bool* timed_out) {
  float acc = 0.f;
  for (int q = 0; q < a.world; ++q) {
    if (q == a.rank) {
      acc += v;
      continue;
    }
    const uint2* src = a.mine + (static_cast<long long>(epoch & 1) * a.world + q) * a.max_elems + i;
    unsigned bits = 0, ep = 0;
    bool got = false;
    for (unsigned it = 0; it < a.wait_limit; ++it) {
      asm volatile("ld.relaxed.sys.global.v2.b32 {%0,%1}, [%2];" : "=r"(bits), "=r"(ep) : "l"(src) : "memory");
      if (ep == static_cast<unsigned>(epoch)) {
        got = true;
        break;
      }
      if (it > 16) __nanosleep(it > 4096 ? 1000 : 100);
    }
    if (got)
      acc += __uint_as_float(bits);
    else
      *timed_out = true;
  }
  return acc;
}

}  // namespace stx

// Host-side object behind stx_peer_t.
struct stx_peer {
  int rank = 0, world = 1;
  int64_t max_elems = 0;
  int device = 0;
  void* local = nullptr;
  void* peers[stx::PEER_MAX_WORLD] = {};
  bool ipc_opened[stx::PEER_MAX_WORLD] = {};
  bool connected = false;
  int* ctl = nullptr;
  unsigned wait_limit = 1u << 22;
};

namespace stx {
// Kernel arguments of a connected peer object; false when it is not connected.
bool peer_args(const stx_peer* p, PeerArgs* out);
}  // namespace stx
