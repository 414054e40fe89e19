// Ordered compaction in two launches (no waiting between blocks).
//
// Items 0..n-1 each get a class in [0, 4) or -1 (dropped).  Launch 1 counts the
// classes of every tile of 2048 items.  Launch 2: every block adds up the counts
// of the tiles before its own (a tile list of a few thousand entries costs a few
// kilobytes per block), scans its own items and hands every kept item the number
// of earlier kept items OF EACH CLASS, so that a policy can number the items per
// class, over all classes, or both.  Every thread owns 8 consecutive items, so
// positions follow the input order.  The block of the last tile passes the class
// totals to the policy.
//
// Used where a three-launch partition over n items (histogram, one-block scan,
// scatter) was spending most of its time in launch gaps: run heads of a sorted
// batch, their per-class numbering, the list of cache misses of a batch.
#pragma once

#include "launch.cuh"

namespace hb {

constexpr int kCompBlock = 256;
constexpr int kCompItems = 8;
constexpr int kCompTile = kCompBlock * kCompItems;
constexpr int kCompClasses = 4;
// beyond this many tiles every block would re-read too long a list; a one-block
// scan between the two launches turns the list into prefixes instead
constexpr int64_t kCompInlinePrefixTiles = 8192;

struct CompactPlan {
  int64_t n;
  int64_t num_tiles;
  int4* tile_counts;  // [num_tiles] per-class counts, or exclusive prefixes when `prefixed`
  int prefixed;
};

static inline int64_t compact_tiles(int64_t n) { return n > 0 ? ceil_div(n, (int64_t)kCompTile) : 1; }
static inline size_t compact_workspace_bytes(int64_t n) {
  return align_up((size_t)(compact_tiles(n) + 1) * sizeof(int4), 256) + 256;
}

#ifdef __CUDACC__

// sum of four counters over the block; result valid in every thread
__device__ __forceinline__ int4 block_sum4(int4 v, int4* s_warp /* [kCompBlock/32] */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
    v.z += __shfl_xor_sync(0xffffffffu, v.z, o);
    v.w += __shfl_xor_sync(0xffffffffu, v.w, o);
  }
  if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
  __syncthreads();
  int4 t = make_int4(0, 0, 0, 0);
#pragma unroll
  for (int w = 0; w < kCompBlock / 32; ++w) {
    const int4 x = s_warp[w];
    t.x += x.x; t.y += x.y; t.z += x.z; t.w += x.w;
  }
  __syncthreads();
  return t;
}

__device__ __forceinline__ void bump4(int4& c, int cls) {
  c.x += cls == 0;
  c.y += cls == 1;
  c.z += cls == 2;
  c.w += cls == 3;
}

// The classes of a thread's 8 consecutive items.  A policy may bring its own
// classify8(base, n, cls) (e.g. vector loads of the 8 keys); otherwise classify(i) is asked
// item by item.
template <typename Policy>
__device__ __forceinline__ auto classify_items(const Policy& pol, int64_t base, int64_t n, int* cls, int)
    -> decltype(pol.classify8(base, n, cls), void()) {
  pol.classify8(base, n, cls);
}
template <typename Policy>
__device__ __forceinline__ void classify_items(const Policy& pol, int64_t base, int64_t n, int* cls, long) {
#pragma unroll
  for (int k = 0; k < kCompItems; ++k) cls[k] = base + k < n ? pol.classify(base + k) : -1;
}

// A policy may ask for the number of kept items ahead of every thread's 8 items
// (thread_begin(base, before)), e.g. to leave a coarse index of the compaction behind.
template <typename Policy>
__device__ __forceinline__ auto thread_begin_hook(const Policy& pol, int64_t base, const int4& before, int)
    -> decltype(pol.thread_begin(base, before), void()) {
  pol.thread_begin(base, before);
}
template <typename Policy>
__device__ __forceinline__ void thread_begin_hook(const Policy&, int64_t, const int4&, long) {}

template <typename Policy>
__global__ void __launch_bounds__(kCompBlock) compact_count_kernel(Policy pol, CompactPlan p) {
  __shared__ int4 s_warp[kCompBlock / 32];
  const int64_t base = (int64_t)blockIdx.x * kCompTile + (int64_t)threadIdx.x * kCompItems;
  int4 c = make_int4(0, 0, 0, 0);
  int cls[kCompItems];
  classify_items(pol, base, p.n, cls, 0);
#pragma unroll
  for (int k = 0; k < kCompItems; ++k) bump4(c, cls[k]);
  const int4 t = block_sum4(c, s_warp);
  if (threadIdx.x == 0) p.tile_counts[blockIdx.x] = t;
}

// only for very long inputs: tile counts -> exclusive prefixes, one block
static __global__ void __launch_bounds__(1024) compact_prefix_kernel(CompactPlan p) {
  __shared__ long long s_part[1024][4];
  const int64_t per = (p.num_tiles + 1023) / 1024;
  const int64_t t0 = (int64_t)threadIdx.x * per;
  const int64_t t1 = (t0 + per < p.num_tiles) ? t0 + per : p.num_tiles;
  long long a[4] = {0, 0, 0, 0};
  for (int64_t t = t0; t < t1; ++t) {
    const int4 v = p.tile_counts[t];
    a[0] += v.x; a[1] += v.y; a[2] += v.z; a[3] += v.w;
  }
  for (int k = 0; k < 4; ++k) s_part[threadIdx.x][k] = a[k];
  __syncthreads();
  if (threadIdx.x == 0) {
    long long run[4] = {0, 0, 0, 0};
    for (int x = 0; x < 1024; ++x)
      for (int k = 0; k < 4; ++k) {
        const long long v = s_part[x][k];
        s_part[x][k] = run[k];
        run[k] += v;
      }
  }
  __syncthreads();
  int run[4];
  for (int k = 0; k < 4; ++k) run[k] = (int)s_part[threadIdx.x][k];
  for (int64_t t = t0; t < t1; ++t) {
    const int4 v = p.tile_counts[t];
    p.tile_counts[t] = make_int4(run[0], run[1], run[2], run[3]);
    run[0] += v.x; run[1] += v.y; run[2] += v.z; run[3] += v.w;
  }
  if (t1 == p.num_tiles && t0 < t1)  // the thread that owns the last tile leaves the totals
    p.tile_counts[p.num_tiles] = make_int4(run[0], run[1], run[2], run[3]);
}

// Policy::emit(i, cls, before) with before.{x,y,z,w} = kept items of class 0..3 ahead
// of item i; Policy::finish(totals) once, by one thread, after all emits of the last tile
// have been issued (totals: kept items per class over the whole input).
template <typename Policy>
__global__ void __launch_bounds__(kCompBlock) compact_scatter_kernel(Policy pol, CompactPlan p) {
  __shared__ int4 s_warp[kCompBlock / 32];
  __shared__ int4 s_scan[kCompBlock / 32];
  const int64_t tile = blockIdx.x;
  // kept items in the tiles before this one
  int4 before_tile;
  if (p.prefixed) {
    before_tile = p.tile_counts[tile];
  } else {
    int4 acc = make_int4(0, 0, 0, 0);
    for (int64_t t = threadIdx.x; t < tile; t += kCompBlock) {
      const int4 v = p.tile_counts[t];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    before_tile = block_sum4(acc, s_warp);
  }
  const int64_t base = tile * kCompTile + (int64_t)threadIdx.x * kCompItems;
  int cls[kCompItems];
  int4 mine = make_int4(0, 0, 0, 0);
  classify_items(pol, base, p.n, cls, 0);
#pragma unroll
  for (int k = 0; k < kCompItems; ++k) bump4(mine, cls[k]);
  // exclusive scan of the per-thread counts over the block
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int4 inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int x = __shfl_up_sync(0xffffffffu, inc.x, o);
    const int y = __shfl_up_sync(0xffffffffu, inc.y, o);
    const int z = __shfl_up_sync(0xffffffffu, inc.z, o);
    const int w = __shfl_up_sync(0xffffffffu, inc.w, o);
    if (lane >= o) { inc.x += x; inc.y += y; inc.z += z; inc.w += w; }
  }
  if (lane == 31) s_scan[warp] = inc;
  __syncthreads();
  int4 run = before_tile;
  for (int w = 0; w < warp; ++w) {
    const int4 x = s_scan[w];
    run.x += x.x; run.y += x.y; run.z += x.z; run.w += x.w;
  }
  run.x += inc.x - mine.x; run.y += inc.y - mine.y; run.z += inc.z - mine.z; run.w += inc.w - mine.w;
  if (base < p.n) thread_begin_hook(pol, base, run, 0);
#pragma unroll
  for (int k = 0; k < kCompItems; ++k) {
    if (cls[k] >= 0) {
      pol.emit(base + k, cls[k], run);
      bump4(run, cls[k]);
    }
  }
  if (tile == p.num_tiles - 1 && threadIdx.x == kCompBlock - 1) pol.finish(run);
}

// Runs the launches.  Workspace: compact_workspace_bytes(n).
template <typename Policy>
int run_compact(const Policy& pol, int64_t n, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!ws || ws_bytes < compact_workspace_bytes(n)) {
    set_error("compact: workspace of %zu bytes needed, %zu given", compact_workspace_bytes(n), ws_bytes);
    return HB_ERR_WORKSPACE;
  }
  CompactPlan p;
  p.n = n > 0 ? n : 0;
  p.num_tiles = compact_tiles(n);
  p.tile_counts = reinterpret_cast<int4*>(align_up((size_t)ws, 256));
  p.prefixed = p.num_tiles > kCompInlinePrefixTiles;
  HB_LAUNCH(compact_count_kernel<Policy>, (int)p.num_tiles, kCompBlock, 0, st, pol, p);
  if (p.prefixed) HB_LAUNCH(compact_prefix_kernel, 1, 1024, 0, st, p);
  HB_LAUNCH(compact_scatter_kernel<Policy>, (int)p.num_tiles, kCompBlock, 0, st, pol, p);
  return HB_OK;
}

#endif  // __CUDACC__

}  // namespace hb
