// Internal declarations of the device-resident differential weight cache.
#pragma once

#include "stx_common.cuh"

// Slots of the cache's device state array (int32).
enum : int {
  ST_K = 0,        // number of active neurons
  ST_NJOBS = 1,    // packed rows the last plan marked for rewriting
  ST_ADDED = 2,    // neurons added by the last update
  ST_REMOVED = 3,  // neurons removed by the last update
  ST_STATUS = 4,   // stx::DEV_* bits (sticky)
  ST_VALID = 5,    // 1 once an update has rebuilt the views (reference: cache_valid)
  ST_EPOCH = 6,    // incremented by every update that changed something
  ST_COUNT = 8
};

struct stx_cache {
  int64_t I = 0, H = 0;
  int dtype = 0;
  int has_gate = 1;
  unsigned flags = 0;
  int device = 0;
  size_t row_bytes = 0;

  // full pools, one H-row per neuron ([I,H]); down is stored transposed
  const void* pool_gate = nullptr;
  const void* pool_up = nullptr;
  void* pool_down = nullptr;
  void* own_gate = nullptr;  // non-null when the cache owns copies of gate/up
  void* own_up = nullptr;
  // optional second copy of the pools, one record per neuron: [I][gate row | up row | down row]
  // ([I][up row | down row] without a gate), so that a neuron's weights are ONE contiguous read.
  // Built on demand (cache_ensure_cat) for the persistent single-row stack kernel.
  void* pool_cat = nullptr;

  // packed pools ([I,H] capacity; rows 0..K-1 valid): row j belongs to neuron active[j]
  void* pk_gate = nullptr;
  void* pk_up = nullptr;
  void* pk_down = nullptr;

  // lazily allocated [2I,H] (or [I,H]) buffer behind stx_cache_concat_weight
  void* concat = nullptr;
  int64_t concat_epoch = -1;

  int32_t* active = nullptr;   // [I] neuron id at packed position j
  int32_t* pos_of = nullptr;   // [I] packed position of neuron n, -1 when inactive
  int32_t* lists = nullptr;    // [2I] scratch: added ids | removed ids (ascending)
  int32_t* jobs = nullptr;     // [I] packed positions to rewrite from the pool
  uint32_t* cur_bits = nullptr;  // [W] current mask
  uint32_t* tmp_bits = nullptr;  // [W] staging for byte masks
  uint32_t* stale = nullptr;     // [W] packed slots whose rows lag behind the index plan (lazy mode)
  bool lazy_used = false;        // host flag: some plan was enqueued (or captured) in lazy mode
  int32_t* state = nullptr;      // [ST_COUNT]
  int32_t* host_state = nullptr; // pinned mirror for read-backs
};

namespace stx {
// Enqueue plan + row copies for a bit-packed mask already on the device.
int cache_update_bits(stx_cache* c, const uint32_t* bits, cudaStream_t s);
// Plan only (index arrays, job list, state); the caller moves the rows.
// lazy: remember the rewritten slots in `stale` instead of queueing them for cache_copy_rows
int cache_plan(stx_cache* c, const uint32_t* bits, cudaStream_t s, bool lazy = false);
int cache_copy_rows(stx_cache* c, cudaStream_t s);
int cache_flush(stx_cache* c, cudaStream_t s);  // rows of all stale slots (no-op when none are pending)
int cache_read_state(stx_cache* c, cudaStream_t s);  // syncs; fills host_state
int cache_ensure_cat(stx_cache* c, cudaStream_t s);  // allocates and fills pool_cat once (asynchronous fill)
}  // namespace stx
