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

// one warp per distinct id: add its rows in slab order, divide, write id / row / count
template <bool VEC4>
__global__ void __launch_bounds__(kBlock) merge_sum_kernel(
    const int64_t* __restrict__ ids, const float* __restrict__ rows, const int64_t* __restrict__ cnt,
    const int64_t* __restrict__ seg_counts, int num_seg, int64_t cap, int64_t dim, int mean,
    const int32_t* __restrict__ src, const int32_t* __restrict__ run_start,
    const int64_t* __restrict__ num_unique, int64_t* __restrict__ uniq_ids,
    float* __restrict__ out_rows, int64_t* __restrict__ out_counts) {
  int64_t total = 0;
  for (int s = 0; s < num_seg; ++s) total += seg_len(seg_counts, s, cap);
  const int64_t u = *num_unique;
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < u; r += nwarps) {
    const int64_t p0 = run_start[r];
    const int64_t p1 = r + 1 < u ? (int64_t)run_start[r + 1] : total;
    // at most num_seg (<= 64) entries: lane l holds entry p0 + l
    int64_t e = -1, c = 0;
    if (p0 + lane < p1) {
      e = src[p0 + lane];
      c = cnt ? __ldg(cnt + e) : 1;
    }
    int64_t csum = c;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) csum += __shfl_xor_sync(0xffffffffu, csum, o);
    int64_t e2 = -1;  // entries 32..63 of a run (more than 32 sources)
    if (p1 - p0 > 32) {
      int64_t c2 = 0;
      if (p0 + 32 + lane < p1) {
        e2 = src[p0 + 32 + lane];
        c2 = cnt ? __ldg(cnt + e2) : 1;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) c2 += __shfl_xor_sync(0xffffffffu, c2, o);
      csum += c2;
    }
    const float denom = (float)(cnt ? csum + 1 : csum);  // counts start from ones when cnt is given
    const int len = (int)(p1 - p0);
    // the k loops are uniform across the warp (k0), so that every lane takes part in the shuffles
    if (VEC4) {
      const int64_t vpr = dim >> 2;
      for (int64_t k0 = 0; k0 < vpr; k0 += 32) {
        const int64_t k = k0 + lane;
        const bool on = k < vpr;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int q = 0; q < len; ++q) {
          const int64_t eq = __shfl_sync(0xffffffffu, q < 32 ? e : e2, q & 31);
          if (on) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(rows + eq * dim) + k);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
        }
        if (mean) { acc.x /= denom; acc.y /= denom; acc.z /= denom; acc.w /= denom; }
        if (on) reinterpret_cast<float4*>(out_rows + r * dim)[k] = acc;
      }
    } else {
      for (int64_t k0 = 0; k0 < dim; k0 += 32) {
        const int64_t k = k0 + lane;
        const bool on = k < dim;
        float acc = 0.f;
        for (int q = 0; q < len; ++q) {
          const int64_t eq = __shfl_sync(0xffffffffu, q < 32 ? e : e2, q & 31);
          if (on) acc += __ldg(rows + eq * dim + k);
        }
        if (mean) acc /= denom;
        if (on) out_rows[r * dim + k] = acc;
      }
    }
    if (lane == 0) {
      uniq_ids[r] = __ldg(ids + e);
      if (out_counts) out_counts[r] = csum + ((cnt && mean) ? 1 : 0);
    }
  }
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
  int64_t blocks = ceil_div(n * 32, kBlock);
  const int64_t cap_blocks = (int64_t)sm_count() * 8;
  if (blocks > cap_blocks) blocks = cap_blocks;
  const bool vec4 = dim % 4 == 0 && ((((uintptr_t)rows | (uintptr_t)out_rows)) & 15) == 0;
  if (vec4)
    HB_LAUNCH(merge_sum_kernel<true>, (int)blocks, kBlock, 0, st, ids, rows, cnt, seg_counts, (int)num_seg, seg_cap,
              dim, mean, p.src, p.run_start, num_unique, uniq_ids, out_rows, out_counts);
  else
    HB_LAUNCH(merge_sum_kernel<false>, (int)blocks, kBlock, 0, st, ids, rows, cnt, seg_counts, (int)num_seg, seg_cap,
              dim, mean, p.src, p.run_start, num_unique, uniq_ids, out_rows, out_counts);
  return HB_OK;
}

}  // extern "C"
