// Device-resident cache index: state layout and the lookup device functions
// shared by the stand-alone lookup kernels and the fused lookup+fetch kernels.
//
// State of record (what add/reset/touch_lru mutate), structure-of-arrays form of
// the reference's 96-byte cache_line (src/cache/cache_line.h:7-11):
//   line_ids[lines*8]  int64   -1 = empty        one 64-byte line per set
//   lru     [lines*8]  int32   access counters
// Derived, read-only "sorted view" for HB_LOOKUP_SORTED:
//   pairs[]            (id, slot) sorted by id, padded to 8 with (INT64_MAX,-1)
//   level[1..top][]    level[1] = id of every 8th pair, level[k+1] = every 16th
//                      id of level[k]; each padded with INT64_MAX so that a
//                      16-key block read never leaves the array.  The top level
//                      (<= kTopMax ids) is staged in shared memory by each CTA.
#pragma once

#include "common.cuh"

namespace hb {

constexpr int kWays = HB_WAYS;
constexpr int kMaxLevels = 8;     // enough for 2^40 ids
constexpr int kTopMax = 2048;     // ids of the top level held in shared memory
constexpr int kLeafFan = 8;       // pairs per leaf block (128 bytes)
constexpr int kNodeFan = 16;      // ids per inner block (128 bytes)

struct IndexView {
  const int64_t* line_ids;
  int64_t lines;
  // sorted view
  const longlong2* pairs;
  const int64_t* level[kMaxLevels];  // level[0] unused
  int32_t level_len[kMaxLevels];     // valid ids per level (level[0]: pairs)
  int32_t top;                       // index of the top level (>= 1), 0 if empty
};

}  // namespace hb

struct hb_index {
  int device;
  int64_t cache_size;  // capacity = lines * 8 (reference: _init_cache, cache.h:47)
  int64_t lines;
  int64_t* line_ids;   // [lines*8]
  int32_t* lru;        // [lines*8]
  // sorted view
  bool sorted_stale;
  longlong2* pairs;            // [round_up(capacity, 8) + 8]
  int64_t* level_store;        // one allocation, levels carved from it
  int64_t level_off[hb::kMaxLevels];
  int64_t level_cap[hb::kMaxLevels];
  int64_t* scratch_count;      // device int64[4] for small reductions
  // run-based LRU ageing: which run of the current batch hit a slot (valid when
  // slot_epoch[slot] == the batch counter kept at slot_epoch[capacity]); allocated
  // on first use.  The counter is 32 bits: 2^31 batches per index.
  int32_t* slot_run;
  int32_t* slot_epoch;
  hb::IndexView view;
  // An index over another process's lines (hb_index_open): the sorted view is this process's
  // own and is rebuilt before every use, because the owner may have changed the lines since.
  // (The owner itself rebuilds after its own changes; after a change by the other process it
  // calls hb_index_build_sorted.)
  bool shared;
  bool opened;  // line_ids / lru are mappings of another process's memory
};

#ifdef __CUDACC__
namespace hb {

// ---- set-associative probe ---------------------------------------------------
// The warp resolves 32 queries (lane l owns id_l).  Groups of 8 lanes read one
// 64-byte line per step; 4 queries per step, 8 steps.  Returns the slot of this
// lane's own id (or -1).
__device__ __forceinline__ int64_t warp_lookup_setassoc(const IndexView& v, int64_t id) {
  const int lane = lane_id();
  const int sub = lane & 7;
  const int grp = lane >> 3;
  const bool valid = id >= 0;
  const int64_t line = valid ? mod_nonneg(id, v.lines) : -1;
  int64_t keys[8];
  int64_t qid[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int q = r * 4 + grp;
    const int64_t lq = __shfl_sync(0xffffffffu, line, q);
    qid[r] = __shfl_sync(0xffffffffu, id, q);
    keys[r] = lq >= 0 ? __ldg(v.line_ids + lq * kWays + sub) : (int64_t)-1;
  }
  int64_t slot = -1;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const unsigned b = __ballot_sync(0xffffffffu, qid[r] >= 0 && keys[r] == qid[r]);
    if ((lane >> 2) == r) {
      const unsigned mine = (b >> ((lane & 3) * 8)) & 0xffu;
      // the reference's find() returns the FIRST matching way (cache_line.h:49-55)
      if (mine) slot = line * kWays + (__ffs(mine) - 1);
    }
  }
  return slot;
}

// ---- sorted-view search --------------------------------------------------------
// top level must already be in shared memory (stage_top_level).
__device__ __forceinline__ void stage_top_level(const IndexView& v, int64_t* smem_top) {
  if (v.top == 0) return;
  const int n = v.level_len[v.top];
  for (int i = threadIdx.x; i < n; i += blockDim.x) smem_top[i] = __ldg(v.level[v.top] + i);
}

__device__ __forceinline__ int64_t warp_lookup_sorted(const IndexView& v, const int64_t* smem_top,
                                                      int64_t id) {
  const int lane = lane_id();
  const int sub = lane & 7;
  const int grp = lane >> 3;
  if (v.top == 0) return -1;
  // per-lane upper_bound over the shared-memory top level
  int64_t t = -1;
  if (id >= 0) {
    int lo = 0, hi = v.level_len[v.top];
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (smem_top[mid] <= id) lo = mid + 1; else hi = mid;
    }
    t = lo - 1;
  }
  // inner levels: 16 ids per block, two per lane of an 8-lane group
  for (int l = v.top - 1; l >= 1; --l) {
    const longlong2* lv = reinterpret_cast<const longlong2*>(v.level[l]);
    longlong2 k[8];
    int64_t qid[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int q = r * 4 + grp;
      const int64_t tq = __shfl_sync(0xffffffffu, t, q);
      qid[r] = __shfl_sync(0xffffffffu, id, q);
      k[r] = tq >= 0 ? __ldg(lv + tq * (kNodeFan / 2) + sub) : make_longlong2(INT64_MAX, INT64_MAX);
    }
    int64_t nt = t;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const unsigned b0 = __ballot_sync(0xffffffffu, k[r].x <= qid[r]);
      const unsigned b1 = __ballot_sync(0xffffffffu, k[r].y <= qid[r]);
      if ((lane >> 2) == r && t >= 0) {
        const int sh = (lane & 3) * 8;
        const int c = __popc((b0 >> sh) & 0xffu) + __popc((b1 >> sh) & 0xffu);
        nt = t * kNodeFan + c - 1;  // c >= 1: the block's first id is the parent id
      }
    }
    t = nt;
  }
  // leaf: 8 (id, slot) pairs per block, one per lane of the group
  longlong2 p[8];
  int64_t qid[8];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int q = r * 4 + grp;
    const int64_t tq = __shfl_sync(0xffffffffu, t, q);
    qid[r] = __shfl_sync(0xffffffffu, id, q);
    p[r] = tq >= 0 ? __ldg(v.pairs + tq * kLeafFan + sub) : make_longlong2(INT64_MAX, -1);
  }
  int64_t slot = -1;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const unsigned b = __ballot_sync(0xffffffffu, p[r].x == qid[r] && qid[r] >= 0);
    // owner lane of query (r, g) is lane r*4+g; it takes the slot from the
    // matching lane of group g
    const int g_owner = lane & 3;
    const unsigned mine = (b >> (g_owner * 8)) & 0xffu;
    const int src = mine ? g_owner * 8 + (__ffs(mine) - 1) : 0;
    const int64_t s = __shfl_sync(0xffffffffu, p[r].y, src);
    if ((lane >> 2) == r && mine) slot = s;
  }
  return slot;
}

template <int MODE>
__device__ __forceinline__ int64_t warp_lookup(const IndexView& v, const int64_t* smem_top,
                                               int64_t id) {
  if (MODE == HB_LOOKUP_SORTED) return warp_lookup_sorted(v, smem_top, id);
  return warp_lookup_setassoc(v, id);
}

}  // namespace hb
#endif  // __CUDACC__
