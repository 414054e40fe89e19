// An embedding table sharded by owner (row of id on rank id % world, local row id / world):
// the handle behind hb_peer_table_* and the device-side view the fetch kernels use.
#pragma once

#include "common.cuh"

struct hb_peer_table {
  int rank, world;
  int64_t num_rows;    // rows of the whole table
  int64_t rows_local;  // rows of this rank's shard
  int64_t row_bytes;
  char* local;
  char* peer[64];
  bool opened[64];
};

namespace hb {

struct ShardView {
  const char* p[64];
  int world;
  int64_t num_rows;  // ids at and beyond it have no row
};

#ifdef __CUDACC__
__device__ __forceinline__ const char* shard_row(const ShardView& s, int64_t id, int64_t row_bytes) {
  if (s.world == 1) return s.p[0] + id * row_bytes;
  const int64_t owner = mod_nonneg(id, s.world);
  return s.p[owner] + ((id - owner) / s.world) * row_bytes;
}
#endif

// Fills `out` from a connected table; HB_ERR_INVALID when a shard is not mapped yet.
int make_shard_view(const hb_peer_table* t, ShardView* out);

}  // namespace hb
