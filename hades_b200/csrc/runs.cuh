// The grouping of a batch of ids into runs of equal ids (hb_runs_t): what the sort of a
// step leaves behind, shared by the forward fetch (each distinct id is looked up and read
// once), the LRU ageing, the list of cache misses and the backward aggregation.
#pragma once

#include "common.cuh"

namespace hb {

// carve of the workspace behind hb_runs_build
struct RunsPlan {
  int64_t *k0, *k1;     // sort keys (uint32 view when the ids fit 32 bits)
  uint32_t *p0, *p1;    // positions
  void* sort_temp;
  size_t sort_temp_bytes;
  int64_t* run_start;   // [m + 1]
  uint8_t* head;        // [m + 1]
  int64_t* n_valid;     // [1]
  int64_t* num_runs;    // [1]
  int64_t* class_counts;  // [4]
  int8_t* dclass;       // [m + 1]
  int32_t* dpos;        // [m + 1]
  int64_t* uniq;        // [m + 1]
  int32_t* base8;       // [m / 8 + 2]
  void* compact_ws;
  size_t compact_ws_bytes;
  size_t total;
};

RunsPlan make_runs_plan(void* ws, int64_t n);

#ifdef __CUDACC__
__device__ __forceinline__ int64_t runs_valid_entries(const hb_runs_t& r) {
  if (!r.n_dev) return r.n;
  const int64_t d = *r.n_dev;
  return d < r.n ? (d > 0 ? d : 0) : r.n;
}
#endif

}  // namespace hb
