// Arguments of the persistent single-row stack kernel (stx_stack_b1.cu).
#pragma once

#include "stx_common.cuh"
#include "stx_peer.cuh"

namespace stx {

constexpr int STACK_B1_MAX_LAYERS = 36;  // layers per launch: the descriptors travel as kernel parameters

struct UpkeepArgs;  // stx_cache_plan.cuh

struct StackLayerDesc {
  const void* cat;   // per-neuron records [I][gate row | up row | down row] ([I][up | down] without a gate)
  const void* A;     // [r,H]
  const void* Bm;    // [I,r]
  uint32_t* bits;    // the layer's mask words (written bytewise)
  void* out;         // [H] in the model dtype
  int* status;       // device status word of the layer's cache
  float tau;
  int act;
};

struct StackB1Args {
  StackLayerDesc layer[STACK_B1_MAX_LAYERS];
  const void* x;     // [H]
  float* t_buf;      // [L][r]
  float* partial;    // [max(L, 2)][G][H] per-CTA partial outputs (layer-by-layer kernel: two of them, by layer parity)
  uint32_t* sync;    // counters (see the kernel)
  int L, H, I, r, has_gate, nslot, strict;
  PeerArgs peer;     // world > 1: the output sum of a layer ends with the all-reduce over the shards
  const UpkeepArgs* upkeep;  // flow kernel only: device array [L]; the launch itself keeps the layers' weight caches up
                             // to date (index plan of layer l by CTA l, then the row copies by all CTAs).  Null: the
                             // caller launches the plan and copy kernels.
};

constexpr int FLOW_MAX_PASSES = 2;  // the flow kernel scores a CTA's mask bytes eight at a time, in up to two passes
// flow: the flow kernel will run (not the layer-by-layer one, whose CTAs score eight mask bytes in a single pass)
bool stack_b1_supported(int64_t H, int64_t I, int64_t r, int has_gate, int dtype, bool flow = false);
size_t stack_b1_scratch_bytes(int64_t L, int64_t H, int64_t r);
// One launch for layers [0, a.L), a.L <= STACK_B1_MAX_LAYERS.  scratch: stack_b1_scratch_bytes(a.L, ..)
// bytes, zeroed once at allocation and then owned by the launches of this group of layers.
int stack_b1_forward(StackB1Args& a, void* scratch, int dtype, cudaStream_t s);
// The flow kernel on the same arguments and scratch (stx_stack_flow.cu); stack_b1_forward picks it for layers
// that do not feed one another.  smem: dynamic shared memory of the launch, smem_limit: the opt-in maximum.
// True when stack_b1_forward will run the flow kernel for these arguments AND its CTAs have the shared memory
// for the caches' index plans, i.e. a.upkeep may be set.
bool stack_flow_upkeep_inside(const StackB1Args& a, int dtype);
int stack_flow_launch(const StackB1Args& a, int dtype, size_t smem, size_t smem_limit, cudaStream_t s);

}  // namespace stx
