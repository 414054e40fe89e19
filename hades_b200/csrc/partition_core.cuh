// Stable multi-way partition: the building block behind split+compact, owner
// bucketing ("pack"), the 3-way gradient split and the staging-table flush.
//
// Items 0..n-1 each get a class in [0, K) (or -1 = dropped).  Output position of
// an item = start of its class + number of earlier items of the same class, so
// the order inside a class is the input order (what torch.nonzero / a stable
// sort would give).  Three launches, no inter-block waiting:
//   1. per-block class histogram
//   2. one CTA turns the histograms into per-block class offsets, class totals
//      and class starts
//   3. every block recomputes the classes, ranks its items with warp match +
//      a per-warp count table in shared memory, and lets the policy emit them.
#pragma once

#include "launch.cuh"

namespace hb {

constexpr int kPartBlock = 256;
constexpr int kPartItemsMax = 8;  // items per thread: 8 for id-only partitions, fewer when
                                  // every item drags a payload row along (more CTAs in flight)
constexpr int kPartMaxClasses = 1024;

struct PartitionPlan {
  int64_t n;
  int num_classes;
  int items;              // items per thread (1..kPartItemsMax)
  int64_t num_blocks;
  int32_t* block_hist;    // [num_blocks][K] -> exclusive offsets inside the class
  int64_t* class_total;   // [K]
  int64_t* class_start;   // [K+1]
};

static inline size_t partition_workspace_bytes(int64_t n, int num_classes, int items = 1) {
  const int64_t nb = n > 0 ? ceil_div(n, (int64_t)kPartBlock * items) : 1;
  return align_up((size_t)nb * num_classes * sizeof(int32_t), 256) +
         2 * align_up((size_t)(num_classes + 1) * sizeof(int64_t), 256) + 256;
}

static inline PartitionPlan partition_plan(void* ws, int64_t n, int num_classes, int items) {
  PartitionPlan p;
  p.n = n;
  p.num_classes = num_classes;
  p.items = items;
  p.num_blocks = n > 0 ? ceil_div(n, (int64_t)kPartBlock * items) : 1;
  Carver cv(ws);
  p.block_hist = cv.take<int32_t>((size_t)p.num_blocks * num_classes);
  p.class_total = cv.take<int64_t>(num_classes + 1);
  p.class_start = cv.take<int64_t>(num_classes + 1);
  return p;
}

#ifdef __CUDACC__

template <typename Policy>
__global__ void __launch_bounds__(kPartBlock) partition_hist_kernel(Policy pol, PartitionPlan p) {
  extern __shared__ int s_hist[];
  for (int k = threadIdx.x; k < p.num_classes; k += kPartBlock) s_hist[k] = 0;
  __syncthreads();
  const int64_t base = (int64_t)blockIdx.x * kPartBlock * p.items;
  for (int s = 0; s < p.items; ++s) {
    const int64_t i = base + s * kPartBlock + threadIdx.x;
    if (i < p.n) {
      const int c = pol.classify(i);
      if (c >= 0) atomicAdd(&s_hist[c], 1);  // integer counts: order cannot change the result
    }
  }
  __syncthreads();
  for (int k = threadIdx.x; k < p.num_classes; k += kPartBlock)
    p.block_hist[(int64_t)blockIdx.x * p.num_classes + k] = s_hist[k];
}

// One CTA of kScanThreads turns the per-block histograms into exclusive offsets.
// Few classes: the whole CTA scans one class at a time (each thread owns a
// contiguous range of blocks: local sum, CTA-wide exclusive scan of the sums,
// local write-back).  Many classes: one warp per class does the same with its
// 32 lanes.
constexpr int kScanThreads = 1024;

__device__ __forceinline__ int64_t warp_exclusive_scan(int64_t v, int64_t& total) {
  const int lane = threadIdx.x & 31;
  int64_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int64_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  total = __shfl_sync(0xffffffffu, inc, 31);
  return inc - v;
}

static __global__ void __launch_bounds__(kScanThreads) partition_scan_kernel(
    PartitionPlan p, int64_t* __restrict__ counts_out) {
  __shared__ int64_t s_warp[32];
  const int K = p.num_classes;
  const int64_t nb = p.num_blocks;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  if (K <= 8) {
    const int64_t per = (nb + kScanThreads - 1) / kScanThreads;
    const int64_t b0 = (int64_t)threadIdx.x * per;
    const int64_t b1 = (b0 + per < nb) ? b0 + per : nb;
    for (int k = 0; k < K; ++k) {
      int64_t local = 0;
      for (int64_t b = b0; b < b1; ++b) local += p.block_hist[b * K + k];
      int64_t wtotal;
      const int64_t wex = warp_exclusive_scan(local, wtotal);
      if (lane == 31) s_warp[warp] = wtotal;
      __syncthreads();
      int64_t base = 0, total = 0;
      for (int w = 0; w < kScanThreads / 32; ++w) {
        if (w < warp) base += s_warp[w];
        total += s_warp[w];
      }
      int64_t run = base + wex;
      for (int64_t b = b0; b < b1; ++b) {
        int32_t* cell = p.block_hist + b * K + k;
        const int32_t c = *cell;
        *cell = (int32_t)run;
        run += c;
      }
      if (threadIdx.x == 0) {
        p.class_total[k] = total;
        if (counts_out) counts_out[k] = total;
      }
      __syncthreads();
    }
  } else {
    const int64_t per = (nb + 31) / 32;
    const int64_t b0 = (int64_t)lane * per;
    const int64_t b1 = (b0 + per < nb) ? b0 + per : nb;
    for (int k = warp; k < K; k += kScanThreads / 32) {
      int64_t local = 0;
      for (int64_t b = b0; b < b1; ++b) local += p.block_hist[b * K + k];
      int64_t total;
      int64_t run = warp_exclusive_scan(local, total);
      for (int64_t b = b0; b < b1; ++b) {
        int32_t* cell = p.block_hist + b * K + k;
        const int32_t c = *cell;
        *cell = (int32_t)run;
        run += c;
      }
      if (lane == 0) {
        p.class_total[k] = total;
        if (counts_out) counts_out[k] = total;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int k = 0; k < K; ++k) {
      p.class_start[k] = run;
      run += p.class_total[k];
    }
    p.class_start[K] = run;
  }
}

// Policy::emit(i, cls, pos_in_class, class_start, active) is called by all 32
// lanes of a warp together (inactive lanes pass active = false), so that it can
// move payload rows cooperatively.
template <typename Policy>
__global__ void __launch_bounds__(kPartBlock) partition_scatter_kernel(Policy pol, PartitionPlan p) {
  extern __shared__ __align__(16) int s_mem[];
  const int K = p.num_classes;
  int* warp_cnt = s_mem;                               // [8][K]
  int64_t* running = reinterpret_cast<int64_t*>(s_mem + (kPartBlock / 32) * K);  // [K]; 8*K ints keep it 8-byte aligned
  int64_t* cstart = running + K;                       // [K]
  for (int k = threadIdx.x; k < K; k += kPartBlock) {
    running[k] = p.block_hist[(int64_t)blockIdx.x * K + k];
    cstart[k] = p.class_start[k];
    for (int w = 0; w < kPartBlock / 32; ++w) warp_cnt[w * K + k] = 0;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const unsigned lt = (1u << lane) - 1u;
  const int64_t base = (int64_t)blockIdx.x * kPartBlock * p.items;
  for (int s = 0; s < p.items; ++s) {
    const int64_t i = base + s * kPartBlock + threadIdx.x;
    const int c = i < p.n ? pol.classify(i) : -1;
    const unsigned same = __match_any_sync(0xffffffffu, c);
    const int rank = __popc(same & lt);
    if (c >= 0 && rank == 0) warp_cnt[warp * K + c] = __popc(same);
    __syncthreads();
    int64_t pos = 0;
    if (c >= 0) {
      pos = running[c] + rank;
      for (int w = 0; w < warp; ++w) pos += warp_cnt[w * K + c];
    }
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += kPartBlock) {
      int sum = 0;
      for (int w = 0; w < kPartBlock / 32; ++w) {
        sum += warp_cnt[w * K + k];
        warp_cnt[w * K + k] = 0;
      }
      running[k] += sum;
    }
    __syncthreads();
    pol.emit(i, c, pos, c >= 0 ? cstart[c] : 0, c >= 0);
  }
}

static inline size_t partition_scatter_smem(int K) {
  return (size_t)((kPartBlock / 32) * K) * sizeof(int) + 2 * (size_t)K * sizeof(int64_t);
}

// Runs the three launches.  counts_out (nullable): device int64[K].  items: items
// per thread (a workspace sized for items = 1 fits every choice).
template <typename Policy>
int run_partition(const Policy& pol, int64_t n, int num_classes, void* ws, size_t ws_bytes,
                  int64_t* counts_out, cudaStream_t st, int items = kPartItemsMax,
                  PartitionPlan* plan_out = nullptr) {
  if (items < 1) items = 1;
  if (items > kPartItemsMax) items = kPartItemsMax;
  if (num_classes < 1 || num_classes > kPartMaxClasses) {
    set_error("partition: number of classes %d outside [1, %d]", num_classes, kPartMaxClasses);
    return HB_ERR_INVALID;
  }
  if (!ws || ws_bytes < partition_workspace_bytes(n, num_classes, items)) {
    set_error("partition: workspace of %zu bytes needed, %zu given",
              partition_workspace_bytes(n, num_classes, items), ws_bytes);
    return HB_ERR_WORKSPACE;
  }
  PartitionPlan p = partition_plan(ws, n, num_classes, items);
  if (plan_out) *plan_out = p;
  if (n <= 0) {
    HB_CUDA(cudaMemsetAsync(p.block_hist, 0, (size_t)num_classes * sizeof(int32_t), st));
    HB_LAUNCH(partition_scan_kernel, 1, kScanThreads, 0, st, p, counts_out);
    return HB_OK;
  }
  HB_LAUNCH(partition_hist_kernel<Policy>, (int)p.num_blocks, kPartBlock,
            (size_t)num_classes * sizeof(int), st, pol, p);
  HB_LAUNCH(partition_scan_kernel, 1, kScanThreads, 0, st, p, counts_out);
  HB_LAUNCH(partition_scatter_kernel<Policy>, (int)p.num_blocks, kPartBlock,
            partition_scatter_smem(num_classes), st, pol, p);
  return HB_OK;
}

// Cooperative payload-row mover for Policy::emit: every lane passes its own
// (src row, dst row, active); the warp copies the active rows, 4 at a time.
__device__ __forceinline__ void warp_move_rows(const char* src_row, char* dst_row, bool active,
                                               int64_t row_bytes, int vb) {
  const int lane = threadIdx.x & 31;
  const unsigned act = __ballot_sync(0xffffffffu, active);
  if (act == 0u) return;
  const unsigned long long sb = (unsigned long long)src_row;
  const unsigned long long db = (unsigned long long)dst_row;
  if (vb == 16 && row_bytes <= 256) {
    // narrow rows: G = 2..16 lanes per row, 32/G rows per pass, 4 passes in flight
    const int vpr = (int)(row_bytes >> 4);
    int G = 16;
    while ((G >> 1) >= vpr && G > 1) G >>= 1;
    const int rpp = 32 / G;
    const int sub = lane & (G - 1);
    const int which = lane / G;
    for (int q0 = 0; q0 < 32; q0 += 4 * rpp) {
      const uint4* s[4];
      uint4* d[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u * rpp + which;
        const unsigned long long a = __shfl_sync(0xffffffffu, sb, q & 31);
        const unsigned long long b = __shfl_sync(0xffffffffu, db, q & 31);
        const bool on = q < 32 && ((act >> q) & 1u) && sub < vpr;
        s[u] = on ? reinterpret_cast<const uint4*>(a) : nullptr;
        d[u] = reinterpret_cast<uint4*>(b);
      }
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s[u]) v[u] = __ldg(s[u] + sub);
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s[u]) d[u][sub] = v[u];
    }
  } else if (vb == 16) {
    const int64_t vpr = row_bytes >> 4;
    for (int q0 = 0; q0 < 32; q0 += 4) {
      if (((act >> q0) & 0xfu) == 0u) continue;
      const uint4* s[4];
      uint4* d[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const unsigned long long a = __shfl_sync(0xffffffffu, sb, q0 + u);
        const unsigned long long b = __shfl_sync(0xffffffffu, db, q0 + u);
        const bool on = (act >> (q0 + u)) & 1u;
        s[u] = on ? reinterpret_cast<const uint4*>(a) : nullptr;
        d[u] = reinterpret_cast<uint4*>(b);
      }
      for (int64_t k = lane; k < vpr; k += 32) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s[u]) v[u] = __ldg(s[u] + k);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s[u]) d[u][k] = v[u];
      }
    }
  } else {
    for (int q = 0; q < 32; ++q) {
      const unsigned long long a = __shfl_sync(0xffffffffu, sb, q);
      const unsigned long long b = __shfl_sync(0xffffffffu, db, q);
      if (!((act >> q) & 1u)) continue;
      const char* s = reinterpret_cast<const char*>(a);
      char* d = reinterpret_cast<char*>(b);
      if (vb == 4) {
        for (int64_t k = lane; k < (row_bytes >> 2); k += 32)
          reinterpret_cast<uint32_t*>(d)[k] = __ldg(reinterpret_cast<const uint32_t*>(s) + k);
      } else {
        for (int64_t k = lane; k < row_bytes; k += 32) d[k] = s[k];
      }
    }
  }
}

static inline int payload_vec_bytes(int64_t row_bytes, const void* a, const void* b) {
  const uintptr_t bits = (uintptr_t)row_bytes | (uintptr_t)a | (uintptr_t)b;
  if ((bits & 15) == 0) return 16;
  if ((bits & 3) == 0) return 4;
  return 1;
}

#endif  // __CUDACC__

}  // namespace hb
