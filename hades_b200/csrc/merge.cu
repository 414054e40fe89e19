// Owner-side merge of what the ranks pushed, for the case the push guarantees: every source's
// slab holds strictly ascending ids (each rank sends the sorted unique ids of its own local
// aggregation, and the bucketing by owner is stable).  unique_grads on the owner
// (python/EmbCache/sparse_optim.py:142-157) is then a merge of `num_seg` sorted lists, which
// needs no sort: every entry finds its place in the merged order with one binary search per
// other slab, a stream compaction numbers the distinct ids, and one pass adds the (at most
// num_seg) rows of each id in slab order.  Same results as hb_unique_segsum_f32 on the same
// slabs (which sorts), in four launches instead of sixteen.
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include "launch.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;

struct MergePlan {
  uint8_t* flag;        // [N]   1 = first entry of its id in merged order
  int32_t* src;         // [N]   entry (slab * cap + index) at each merged position
  int32_t* run_start;   // [N]   merged position of the first entry of each distinct id
  void* select_temp;
  size_t select_temp_bytes;
  size_t total;
};

MergePlan make_plan(void* ws, int64_t n) {
  MergePlan p;
  Carver c(ws);
  p.flag = c.take<uint8_t>((size_t)n);
  p.src = c.take<int32_t>((size_t)n);
  p.run_start = c.take<int32_t>((size_t)n);
  p.select_temp_bytes = 0;
  cub::DeviceSelect::Flagged(nullptr, p.select_temp_bytes, thrust::counting_iterator<int32_t>(0),
                             (const uint8_t*)nullptr, (int32_t*)nullptr, (int64_t*)nullptr, (int)n);
  p.select_temp = c.take<char>(p.select_temp_bytes);
  p.total = c.used();
  return p;
}

__device__ __forceinline__ int64_t seg_len(const int64_t* seg_counts, int s, int64_t cap) {
  const int64_t c = seg_counts[s];
  return c < 0 ? 0 : (c < cap ? c : cap);
}

__device__ __forceinline__ int64_t lower_bound_dev(const int64_t* a, int64_t n, int64_t x) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (__ldg(a + mid) < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// merged position of every entry (ascending id, equal ids in slab order) and whether it is
// the first of its id
__global__ void __launch_bounds__(kBlock) merge_rank_kernel(
    const int64_t* __restrict__ ids, const int64_t* __restrict__ seg_counts, int num_seg,
    int64_t cap, uint8_t* __restrict__ flag, int32_t* __restrict__ src) {
  const int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (e >= (int64_t)num_seg * cap) return;
  const int s = (int)(e / cap);
  const int64_t j = e - (int64_t)s * cap;
  if (j >= seg_len(seg_counts, s, cap)) return;
  const int64_t x = __ldg(ids + e);
  int64_t p = j;
  bool first = true;
  for (int t = 0; t < num_seg; ++t) {
    if (t == s) continue;
    const int64_t len = seg_len(seg_counts, t, cap);
    const int64_t* a = ids + (int64_t)t * cap;
    const int64_t lb = lower_bound_dev(a, len, x);
    const bool earlier_has_it = t < s && lb < len && __ldg(a + lb) == x;
    p += lb + (earlier_has_it ? 1 : 0);
    if (earlier_has_it) first = false;
  }
  flag[p] = first ? 1 : 0;
  src[p] = (int32_t)e;
}

// A warp takes 32 distinct ids per round.  Lane l reads the extent of run l, adds its counts and
// writes id and count; then the warp walks the 32 runs, G lanes per row and kRuns runs in flight,
// adding each run's rows in slab order.  (A warp per run would spend its time waiting: nearly all
// runs hold one or two rows.)
constexpr int kRuns = 4;

template <typename V>
__device__ __forceinline__ void vadd(V& a, const V& b);
template <>
__device__ __forceinline__ void vadd<float4>(float4& a, const float4& b) {
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}
template <>
__device__ __forceinline__ void vadd<float>(float& a, const float& b) { a += b; }
__device__ __forceinline__ void vdiv(float4& a, float d) { a.x /= d; a.y /= d; a.z /= d; a.w /= d; }
__device__ __forceinline__ void vdiv(float& a, float d) { a /= d; }

template <typename V>
__global__ void __launch_bounds__(kBlock) merge_sum_kernel(
    const int64_t* __restrict__ ids, const float* __restrict__ rows, const int64_t* __restrict__ cnt,
    const int64_t* __restrict__ seg_counts, int num_seg, int64_t cap, int64_t dim, int mean,
    const int32_t* __restrict__ src, const int32_t* __restrict__ run_start,
    const int64_t* __restrict__ num_unique, int64_t* __restrict__ uniq_ids,
    float* __restrict__ out_rows, int64_t* __restrict__ out_counts, int glog2) {
  int64_t total = 0;
  for (int s = 0; s < num_seg; ++s) total += seg_len(seg_counts, s, cap);
  const int64_t u = *num_unique;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int G = 1 << glog2, rpp = 32 >> glog2;
  const int sub = lane & (G - 1), which = lane >> glog2;
  const int64_t vpr = dim * 4 / (int64_t)sizeof(V);  // vectors per row
  const V* vrows = reinterpret_cast<const V*>(rows);
  V* vout = reinterpret_cast<V*>(out_rows);
  for (int64_t r0 = warp * 32; r0 < u; r0 += nwarps * 32) {
    const int64_t r = r0 + lane;
    int p0 = 0, len = 0, first = 0;
    float denom = 1.0f;
    if (r < u) {
      p0 = run_start[r];
      len = (int)((r + 1 < u ? (int64_t)run_start[r + 1] : total) - p0);
      first = src[p0];  // handed to the row loop by shuffle: its loads then wait for nothing
      int64_t csum = 0;
      for (int j = 0; j < len; ++j) csum += cnt ? __ldg(cnt + src[p0 + j]) : 1;
      denom = (float)(cnt ? csum + 1 : csum);  // counts start from ones when cnt is given
      uniq_ids[r] = __ldg(ids + first);
      if (out_counts) out_counts[r] = csum + ((cnt && mean) ? 1 : 0);
    }
    for (int pass = 0; pass < G; pass += kRuns) {
      int P0[kRuns], L[kRuns], F[kRuns];
      float D[kRuns];
      int64_t R[kRuns];
#pragma unroll
      for (int t = 0; t < kRuns; ++t) {
        const int q = ((pass + t) * rpp + which) & 31;
        P0[t] = __shfl_sync(0xffffffffu, p0, q);
        F[t] = __shfl_sync(0xffffffffu, first, q);
        L[t] = __shfl_sync(0xffffffffu, len, q);
        D[t] = __shfl_sync(0xffffffffu, denom, q);
        if (pass + t >= G) L[t] = 0;
        R[t] = r0 + q;
      }
      for (int64_t k = sub; k < vpr; k += G) {
        V acc[kRuns];
#pragma unroll
        for (int t = 0; t < kRuns; ++t)
          if (L[t] > 0) acc[t] = __ldg(vrows + (int64_t)F[t] * vpr + k);
#pragma unroll
        for (int t = 0; t < kRuns; ++t)
          for (int j = 1; j < L[t]; ++j) vadd(acc[t], __ldg(vrows + (int64_t)src[P0[t] + j] * vpr + k));
#pragma unroll
        for (int t = 0; t < kRuns; ++t)
          if (L[t] > 0) {
            if (mean) vdiv(acc[t], D[t]);
            vout[R[t] * vpr + k] = acc[t];
          }
      }
    }
  }
}

int group_log2_for(int64_t units) {
  int g = 0;
  while ((1 << g) < units && g < 5) ++g;
  return g;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

size_t hb_merge_sorted_slabs_workspace_bytes(int64_t num_seg, int64_t seg_cap) {
  const int64_t n = num_seg * seg_cap;
  if (n <= 0 || n >= ((int64_t)1 << 31)) return 0;
  return make_plan(nullptr, n).total;
}

int hb_merge_sorted_slabs_f32(const int64_t* ids, const float* rows, const int64_t* cnt,
                              const int64_t* seg_counts, int64_t num_seg, int64_t seg_cap, int64_t dim,
                              int mean, int64_t* uniq_ids, float* out_rows, int64_t* out_counts,
                              int64_t* num_unique, void* workspace, size_t workspace_bytes,
                              hb_stream_t stream) {
  HB_CHECK_ARG(num_seg >= 1 && num_seg <= 64 && seg_cap > 0 && dim > 0, "hb_merge_sorted_slabs_f32: bad sizes");
  const int64_t n = num_seg * seg_cap;
  HB_CHECK_ARG(n < ((int64_t)1 << 31), "hb_merge_sorted_slabs_f32: too many entries");
  HB_CHECK_ARG(ids && rows && seg_counts && uniq_ids && out_rows && num_unique,
               "hb_merge_sorted_slabs_f32: null argument");
  MergePlan p = make_plan(workspace, n);
  if (!workspace || workspace_bytes < p.total) {
    set_error("hb_merge_sorted_slabs_f32: workspace of %zu bytes needed, %zu given", p.total, workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  HB_CUDA(cudaMemsetAsync(p.flag, 0, (size_t)n, st));
  HB_LAUNCH(merge_rank_kernel, (int)ceil_div(n, kBlock), kBlock, 0, st, ids, seg_counts, (int)num_seg, seg_cap,
            p.flag, p.src);
  HB_CUDA(cub::DeviceSelect::Flagged(p.select_temp, p.select_temp_bytes, thrust::counting_iterator<int32_t>(0),
                                     p.flag, p.run_start, num_unique, (int)n, st));
  count_library_launches(2);
  int64_t blocks = ceil_div(n, kBlock);
  const int64_t cap_blocks = (int64_t)sm_count() * 8;
  if (blocks > cap_blocks) blocks = cap_blocks;
  const bool vec4 = dim % 4 == 0 && ((((uintptr_t)rows | (uintptr_t)out_rows)) & 15) == 0;
  const int glog2 = group_log2_for(vec4 ? dim / 4 : dim);
  if (vec4)
    HB_LAUNCH(merge_sum_kernel<float4>, (int)blocks, kBlock, 0, st, ids, rows, cnt, seg_counts, (int)num_seg,
              seg_cap, dim, mean, p.src, p.run_start, num_unique, uniq_ids, out_rows, out_counts, glog2);
  else
    HB_LAUNCH(merge_sum_kernel<float>, (int)blocks, kBlock, 0, st, ids, rows, cnt, seg_counts, (int)num_seg,
              seg_cap, dim, mean, p.src, p.run_start, num_unique, uniq_ids, out_rows, out_counts, glog2);
  return HB_OK;
}

}  // extern "C"
