// Hot/cold split (+ compaction), owner search, owner bucketing ("pack") and the
// 3-way gradient split.
#include "partition_core.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;

// ---- hot/cold split masks: src/cuda/split.cu:34-44 -------------------------------
__global__ void split_masks_kernel(const int64_t* __restrict__ ids, int64_t n,
                                   const int8_t* __restrict__ table, uint8_t* __restrict__ local,
                                   uint8_t* __restrict__ hot, uint8_t* __restrict__ cold) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int8_t v = __ldg(table + __ldg(ids + i));
  local[i] = v == 0;
  hot[i] = v == 1;
  cold[i] = v == 2;
}

// split + the nonzero() calls that follow it in python/EmbCache/dist_emb.py:174-191
struct SplitCompactPolicy {
  const int64_t* ids;
  const int8_t* table;
  uint8_t* local;
  uint8_t* hot;
  uint8_t* cold;
  int64_t* index_out;
  int64_t n;
  __device__ __forceinline__ int classify(int64_t i) const {
    const int8_t v = __ldg(table + __ldg(ids + i));
    return (v >= 0 && v <= 2) ? (int)v : -1;
  }
  __device__ __forceinline__ void emit(int64_t i, int c, int64_t pos, int64_t start,
                                       bool active) const {
    if (active) index_out[start + pos] = i;
    if (local && i < n) {  // any other table value leaves all three masks false
      local[i] = c == 0;
      hot[i] = c == 1;
      cold[i] = c == 2;
    }
  }
};

// ---- owner search: src/cuda/binary_search.cu ---------------------------------------
template <typename T>
__device__ __forceinline__ int64_t upper_bound_dev(const T* a, int64_t n, T v) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (a[mid] <= v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

template <typename T>
__global__ void owner_mod_kernel(const T* __restrict__ in, int64_t n, int64_t g,
                                 T* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = (T)(in[i] % (T)g);
}

template <typename T>
__global__ void owner_range_kernel(const T* __restrict__ in, int64_t n,
                                   const T* __restrict__ range, int64_t parts, int64_t g,
                                   T* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const T v = in[i];
  out[i] = (T)((upper_bound_dev(range, parts, v) - 1) * g + v % (T)g);
}

template <typename T>
__global__ void upper_bound_kernel(const T* __restrict__ in, int64_t n,
                                   const T* __restrict__ sorted, int64_t m, T* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) out[i] = (T)upper_bound_dev(sorted, m, in[i]);
}

// ---- owner bucketing: python/EmbCache/sparse_optim.py:36-55 --------------------------
struct OwnerFn {
  const int64_t* range;  // nullable: owner = id % g
  int64_t parts;
  int64_t g;
  __device__ __forceinline__ int operator()(int64_t id) const {
    if (!range) return (int)mod_nonneg(id, g);
    return (int)((upper_bound_dev(range, parts, id) - 1) * g + mod_nonneg(id, g));
  }
};

struct BucketPackPolicy {
  OwnerFn owner;
  int num_buckets;
  const int64_t* n_dev;  // nullable device count that caps n
  const int64_t* ids;
  const char* rows;
  const int64_t* cnt;
  int64_t row_bytes;
  int vb;
  int64_t* out_ids;
  char* out_rows;
  int64_t* out_cnt;
  __device__ __forceinline__ int classify(int64_t i) const {
    if (n_dev && i >= *n_dev) return -1;
    const int64_t id = __ldg(ids + i);
    if (id < 0) return -1;
    const int o = owner(id);
    return (o >= 0 && o < num_buckets) ? o : -1;
  }
  __device__ __forceinline__ void emit(int64_t i, int, int64_t pos, int64_t start,
                                       bool active) const {
    const int64_t d = start + pos;
    if (active) {
      out_ids[d] = ids[i];
      if (cnt) out_cnt[d] = cnt[i];
    }
    if (rows)
      warp_move_rows(rows + i * row_bytes, out_rows + d * row_bytes, active, row_bytes, vb);
  }
};

// ---- 3-way gradient split: python/EmbCache/sparse_optim.py:243-259 --------------------
// class 0 = hot, 1 = cold local (~hot & local), 2 = cold remote (~hot & ~local)
struct GradSplitPolicy {
  const int64_t* ids;
  const char* rows;
  const uint8_t* hot;
  const uint8_t* local;
  int64_t row_bytes;
  int vb;
  int64_t* out_ids;
  char* out_rows;
  __device__ __forceinline__ int classify(int64_t i) const {
    if (hot[i]) return 0;
    return local[i] ? 1 : 2;
  }
  __device__ __forceinline__ void emit(int64_t i, int, int64_t pos, int64_t start,
                                       bool active) const {
    const int64_t d = start + pos;
    if (active) out_ids[d] = ids[i];
    warp_move_rows(rows + i * row_bytes, out_rows + d * row_bytes, active, row_bytes, vb);
  }
};

// ---- 3-way split of (ids, rows, cnt) by a per-node class table ---------------------------
// class = table[id] in {0, 1, 2}; the split of src/cuda/split.cu applied to rows that
// travel with their ids (gradient rows after local aggregation).
struct TableSplitPolicy {
  const int64_t* ids;
  const char* rows;
  const int64_t* cnt;
  const int64_t* n_dev;
  const int8_t* table;
  int64_t row_bytes;
  int vb;
  int64_t* out_ids[3];   // per class, each compacted from 0; null = count only
  char* out_rows[3];
  int64_t* out_cnt[3];
  __device__ __forceinline__ int classify(int64_t i) const {
    if (n_dev && i >= *n_dev) return -1;
    const int64_t id = __ldg(ids + i);
    if (id < 0) return -1;
    const int8_t v = __ldg(table + id);
    return (v >= 0 && v <= 2) ? (int)v : -1;
  }
  __device__ __forceinline__ void emit(int64_t i, int c, int64_t pos, int64_t, bool active) const {
    const bool write = active && out_ids[c] != nullptr;
    if (write) {
      out_ids[c][pos] = ids[i];
      if (cnt && out_cnt[c]) out_cnt[c][pos] = cnt[i];
    }
    const bool move = write && out_rows[c] != nullptr;
    warp_move_rows(rows + i * row_bytes, move ? out_rows[c] + pos * row_bytes : nullptr, move,
                   row_bytes, vb);
  }
};

int grid_for(int64_t n) { return (int)(n > 0 ? ceil_div(n, kBlock) : 1); }

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

size_t hb_partition_workspace_bytes(int64_t n, int num_classes) {
  return partition_workspace_bytes(n, num_classes);
}

int hb_split_masks(const int64_t* ids, int64_t n, const int8_t* mask_table, uint8_t* local_mask,
                   uint8_t* hot_mask, uint8_t* cold_mask, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0, "hb_split_masks: negative n");
  HB_CHECK_ARG(n == 0 || (ids && mask_table && local_mask && hot_mask && cold_mask),
               "hb_split_masks: null argument");
  if (n == 0) return HB_OK;
  HB_LAUNCH(split_masks_kernel, grid_for(n), kBlock, 0, (cudaStream_t)stream, ids, n, mask_table,
            local_mask, hot_mask, cold_mask);
  return HB_OK;
}

int hb_split_compact(const int64_t* ids, int64_t n, const int8_t* mask_table, uint8_t* local_mask,
                     uint8_t* hot_mask, uint8_t* cold_mask, int64_t* index_out, int64_t* counts,
                     void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31), "hb_split_compact: n out of range");
  HB_CHECK_ARG(counts != nullptr, "hb_split_compact: counts is null");
  HB_CHECK_ARG(n == 0 || (ids && mask_table && index_out), "hb_split_compact: null argument");
  const bool masks = local_mask || hot_mask || cold_mask;
  HB_CHECK_ARG(!masks || (local_mask && hot_mask && cold_mask),
               "hb_split_compact: give all three masks or none");
  SplitCompactPolicy pol{ids, mask_table, local_mask, hot_mask, cold_mask, index_out, n};
  return run_partition(pol, n, 3, workspace, workspace_bytes, counts, (cudaStream_t)stream);
}

#define HB_INT_SWITCH(idx_bytes, T, ...) \
  if ((idx_bytes) == 8) {                \
    typedef int64_t T;                   \
    __VA_ARGS__                          \
  } else {                               \
    typedef int32_t T;                   \
    __VA_ARGS__                          \
  }

int hb_owner_mod(const void* in, int64_t n, int idx_bytes, int64_t g, void* out,
                 hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && g > 0, "hb_owner_mod: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_owner_mod: ids must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (in && out), "hb_owner_mod: null argument");
  if (n == 0) return HB_OK;
  HB_INT_SWITCH(idx_bytes, T, {
    HB_LAUNCH(owner_mod_kernel<T>, grid_for(n), kBlock, 0, (cudaStream_t)stream, (const T*)in, n, g,
              (T*)out);
  })
  return HB_OK;
}

int hb_owner_range(const void* in, int64_t n, int idx_bytes, const void* range_partition,
                   int64_t num_part, int64_t g, void* out, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && g > 0 && num_part > 0, "hb_owner_range: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_owner_range: ids must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (in && out && range_partition), "hb_owner_range: null argument");
  if (n == 0) return HB_OK;
  HB_INT_SWITCH(idx_bytes, T, {
    HB_LAUNCH(owner_range_kernel<T>, grid_for(n), kBlock, 0, (cudaStream_t)stream, (const T*)in, n,
              (const T*)range_partition, num_part, g, (T*)out);
  })
  return HB_OK;
}

int hb_upper_bound(const void* in, int64_t n, int idx_bytes, const void* sorted, int64_t m,
                   void* out, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && m >= 0, "hb_upper_bound: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_upper_bound: values must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (in && out && (m == 0 || sorted)), "hb_upper_bound: null argument");
  if (n == 0) return HB_OK;
  HB_INT_SWITCH(idx_bytes, T, {
    HB_LAUNCH(upper_bound_kernel<T>, grid_for(n), kBlock, 0, (cudaStream_t)stream, (const T*)in, n,
              (const T*)sorted, m, (T*)out);
  })
  return HB_OK;
}

int hb_bucket_pack(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                   const int64_t* n_dev, int64_t row_bytes, int num_buckets,
                   const int64_t* range_partition,
                   int64_t num_part, int64_t g, int64_t* out_ids, void* out_rows, int64_t* out_cnt,
                   int64_t* counts, void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31), "hb_bucket_pack: n out of range");
  HB_CHECK_ARG(g > 0 && num_buckets > 0, "hb_bucket_pack: bad bucket parameters");
  HB_CHECK_ARG(counts != nullptr, "hb_bucket_pack: counts is null");
  HB_CHECK_ARG(n == 0 || (ids && out_ids), "hb_bucket_pack: null ids");
  HB_CHECK_ARG(!rows || (out_rows && row_bytes > 0), "hb_bucket_pack: rows without output");
  HB_CHECK_ARG(!cnt || out_cnt, "hb_bucket_pack: cnt without output");
  HB_CHECK_ARG(!range_partition || num_part > 0, "hb_bucket_pack: empty range partition");
  BucketPackPolicy pol{{range_partition, num_part, g}, num_buckets, n_dev, ids, (const char*)rows, cnt,
                       row_bytes, rows ? payload_vec_bytes(row_bytes, rows, out_rows) : 1,
                       out_ids, (char*)out_rows, out_cnt};
  return run_partition(pol, n, num_buckets, workspace, workspace_bytes, counts,
                       (cudaStream_t)stream, rows ? 1 : kPartItemsMax);
}

int hb_table_split3(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                    const int64_t* n_dev, int64_t row_bytes, const int8_t* table,
                    int64_t* const* out_ids, void* const* out_rows, int64_t* const* out_cnt,
                    int64_t* counts, void* workspace, size_t workspace_bytes,
                    hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31) && row_bytes > 0, "hb_table_split3: bad sizes");
  HB_CHECK_ARG(counts != nullptr && table != nullptr, "hb_table_split3: null counts or table");
  HB_CHECK_ARG(out_ids && out_rows, "hb_table_split3: null output tables");
  HB_CHECK_ARG(n == 0 || (ids && rows), "hb_table_split3: null argument");
  TableSplitPolicy pol;
  pol.ids = ids;
  pol.rows = (const char*)rows;
  pol.cnt = cnt;
  pol.n_dev = n_dev;
  pol.table = table;
  pol.row_bytes = row_bytes;
  uintptr_t bits = (uintptr_t)row_bytes | (uintptr_t)rows;
  for (int c = 0; c < 3; ++c) {
    pol.out_ids[c] = out_ids[c];
    pol.out_rows[c] = (char*)out_rows[c];
    pol.out_cnt[c] = out_cnt ? out_cnt[c] : nullptr;
    bits |= (uintptr_t)out_rows[c];
  }
  pol.vb = (bits & 15) == 0 ? 16 : ((bits & 3) == 0 ? 4 : 1);
  return run_partition(pol, n, 3, workspace, workspace_bytes, counts, (cudaStream_t)stream, 1);
}

int hb_grad_split3(const int64_t* ids, const void* rows, const uint8_t* hot_mask,
                   const uint8_t* local_mask, int64_t n, int64_t row_bytes, int64_t* out_ids,
                   void* out_rows, int64_t* counts, void* workspace, size_t workspace_bytes,
                   hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31) && row_bytes > 0, "hb_grad_split3: bad sizes");
  HB_CHECK_ARG(counts != nullptr, "hb_grad_split3: counts is null");
  HB_CHECK_ARG(n == 0 || (ids && rows && hot_mask && local_mask && out_ids && out_rows),
               "hb_grad_split3: null argument");
  GradSplitPolicy pol{ids, (const char*)rows, hot_mask, local_mask, row_bytes,
                      payload_vec_bytes(row_bytes, rows, out_rows), out_ids, (char*)out_rows};
  return run_partition(pol, n, 3, workspace, workspace_bytes, counts, (cudaStream_t)stream, 1);
}

// ---- owner bucketing for callers that must not allocate ---------------------------------
// Some hosts of this library cannot hand it a workspace: code that runs inside a
// region where device allocation is forbidden or unpredictable (a serving loop
// with a frozen memory plan, a foreign runtime that owns the allocator and offers
// no scratch hook, an interrupt-style callback that must not block in the driver).
// For them the block histograms and offsets of the partition live in a fixed
// array that is part of the loaded module, so the call itself creates nothing.
//
// The array below is DEVICE memory.  In host code its name only stands for the
// symbol; the usable address is asked from the runtime once per device
// (cudaGetSymbolAddress) and that address is what the kernels receive.
constexpr int64_t kNoAllocMaxItems = (int64_t)1 << 20;  // 1,048,576 ids per call
constexpr int kNoAllocMaxBuckets = 64;
// partition_workspace_bytes(kNoAllocMaxItems, kNoAllocMaxBuckets, 8 items per thread) = 132,864 bytes
constexpr size_t kNoAllocScratchBytes = 135168;  // 132 KiB, held by every GPU that loads the library

static __device__ __align__(256) unsigned char g_noalloc_pack_scratch[kNoAllocScratchBytes];

namespace {

// Device address of the scratch array on the current device; looked up on the
// first call per device and remembered.
int noalloc_scratch_address(void** out) {
  static void* addr[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    hb::set_error("hb_bucket_pack_noalloc: cannot identify the current device (%s)",
                  cudaGetErrorString(e));
    return HB_ERR_CUDA;
  }
  if (addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_pack_scratch);
    if (e != cudaSuccess || p == nullptr) {
      hb::set_error("hb_bucket_pack_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return HB_ERR_CUDA;
    }
    addr[dev] = p;
  }
  *out = addr[dev];
  return HB_OK;
}

}  // namespace

int64_t hb_bucket_pack_noalloc_max_items(void) { return kNoAllocMaxItems; }
int hb_bucket_pack_noalloc_max_buckets(void) { return kNoAllocMaxBuckets; }

int hb_bucket_pack_noalloc(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                           const int64_t* n_dev, int64_t row_bytes, int num_buckets,
                           const int64_t* range_partition, int64_t num_part, int64_t g,
                           int64_t* out_ids, void* out_rows, int64_t* out_cnt, int64_t* counts,
                           hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0, "hb_bucket_pack_noalloc: negative n");
  if (n > kNoAllocMaxItems || num_buckets > kNoAllocMaxBuckets) {
    hb::set_error("hb_bucket_pack_noalloc: %lld ids / %d buckets exceed the built-in scratch "
                  "(at most %lld ids and %d buckets per call); use hb_bucket_pack with a workspace",
                  (long long)n, num_buckets, (long long)kNoAllocMaxItems, kNoAllocMaxBuckets);
    return HB_ERR_CAPACITY;
  }
  HB_CHECK_ARG(g > 0 && num_buckets > 0, "hb_bucket_pack_noalloc: bad bucket parameters");
  HB_CHECK_ARG(counts != nullptr, "hb_bucket_pack_noalloc: counts is null");
  HB_CHECK_ARG(n == 0 || (ids && out_ids), "hb_bucket_pack_noalloc: null ids");
  HB_CHECK_ARG(!rows || (out_rows && row_bytes > 0), "hb_bucket_pack_noalloc: rows without output");
  HB_CHECK_ARG(!cnt || out_cnt, "hb_bucket_pack_noalloc: cnt without output");
  HB_CHECK_ARG(!range_partition || num_part > 0, "hb_bucket_pack_noalloc: empty range partition");
  if (partition_workspace_bytes(n, num_buckets, kPartItemsMax) > kNoAllocScratchBytes) {
    hb::set_error("hb_bucket_pack_noalloc: internal scratch too small for this request");
    return HB_ERR_CAPACITY;
  }
  void* scratch = nullptr;
  int rc = noalloc_scratch_address(&scratch);
  if (rc != HB_OK) return rc;
  // Nothing in the scratch has to start at zero: the histogram kernel writes
  // every cell it later reads and the scan kernel writes the totals and starts,
  // so whatever the previous call left behind is overwritten before use.
  BucketPackPolicy pol{{range_partition, num_part, g}, num_buckets, n_dev, ids, (const char*)rows, cnt,
                       row_bytes, rows ? payload_vec_bytes(row_bytes, rows, out_rows) : 1,
                       out_ids, (char*)out_rows, out_cnt};
  return run_partition(pol, n, num_buckets, scratch, kNoAllocScratchBytes, counts,
                       (cudaStream_t)stream, kPartItemsMax);
}


}  // extern "C"
