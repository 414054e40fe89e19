// Row movers: gather, scatter (set / combine), cached gather / scatter through a
// dense index map, accumulate, and the fused cache lookup + fetch.
//
// Two data paths:
//  * LSU: a group of 1..32 lanes owns a row and moves it with the widest vector
//    (16/8/4/2/1 bytes) that the row size and the base addresses allow; each
//    group keeps kRows rows in flight so that a warp has several independent
//    128-bit loads outstanding.
//  * BULK: rows go through shared memory with cp.async.bulk.  For a gather the
//    lanes of a warp each fetch one row into a per-warp stage and a single bulk
//    store writes the stage to the (contiguous) output; for a scatter one bulk
//    load brings a contiguous stage in and the lanes store one row each.
#include "bulk.cuh"
#include "index.cuh"
#include <initializer_list>

#include "launch.cuh"

namespace hb {
int* device_error_word();  // runtime.cu

namespace {

constexpr int kBlock = 256;
constexpr int kRows = 4;            // rows in flight per lane group (LSU path)
constexpr int kStageBytes = 16384;  // per-warp shared-memory stage (BULK path)
constexpr int kBulkWarps = 8;

template <int VB> struct Vec;
template <> struct Vec<16> { using T = uint4; };
template <> struct Vec<8> { using T = uint2; };
template <> struct Vec<4> { using T = uint32_t; };
template <> struct Vec<2> { using T = uint16_t; };
template <> struct Vec<1> { using T = uint8_t; };

// ---- address resolvers ---------------------------------------------------------
// resolve(i, leader, src, dst): row i's source and destination; false = skip.
template <typename IdxT, bool HAS_DST_INDEX>
struct GatherRes {
  const char* src; const IdxT* si; char* dst; const IdxT* di; int64_t rb;
  __device__ __forceinline__ bool resolve(int64_t i, bool, const char*& s, char*& d) const {
    s = src + (int64_t)__ldg(si + i) * rb;
    d = dst + (HAS_DST_INDEX ? (int64_t)__ldg(di + i) : i) * rb;
    return true;
  }
};

template <typename IdxT>
struct ScatterRes {
  const char* src; char* dst; const IdxT* di; int64_t rb;
  __device__ __forceinline__ bool resolve(int64_t i, bool, const char*& s, char*& d) const {
    s = src + i * rb;
    d = dst + (int64_t)__ldg(di + i) * rb;
    return true;
  }
};

template <typename IdxT>
struct CachedGatherRes {
  const char* backing; const char* cached; const IdxT* index; const IdxT* map; char* dst;
  uint8_t* found; int64_t rb;
  __device__ __forceinline__ bool resolve(int64_t i, bool leader, const char*& s, char*& d) const {
    const int64_t idx = (int64_t)__ldg(index + i);
    const int64_t g = (int64_t)__ldg(map + idx);
    s = g != -1 ? cached + g * rb : backing + idx * rb;
    d = dst + i * rb;
    if (leader && found) found[i] = g != -1;
    return true;
  }
};

template <typename IdxT>
struct CachedScatterRes {
  const char* src; char* backing; char* cached; const IdxT* index; const IdxT* map; int64_t rb;
  __device__ __forceinline__ bool resolve(int64_t i, bool, const char*& s, char*& d) const {
    const int64_t idx = (int64_t)__ldg(index + i);
    const int64_t g = (int64_t)__ldg(map + idx);
    s = src + i * rb;
    d = g != -1 ? cached + g * rb : backing + idx * rb;
    return true;
  }
};

// ---- LSU mover -------------------------------------------------------------------
template <int VB, typename R>
__global__ void __launch_bounds__(kBlock) move_rows_kernel(R rs, int64_t n, int64_t row_bytes,
                                                            int glog2) {
  using V = typename Vec<VB>::T;
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t group = tid >> glog2;
  const int sub = (int)(tid & ((1 << glog2) - 1));
  const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) >> glog2;
  const int64_t vpr = row_bytes / VB;
  const int G = 1 << glog2;
  for (int64_t i0 = group; i0 < n; i0 += ngroups * kRows) {
    const V* s[kRows];
    V* d[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int64_t i = i0 + r * ngroups;
      s[r] = nullptr;
      d[r] = nullptr;
      if (i < n) {
        const char* sp;
        char* dp;
        if (rs.resolve(i, sub == 0, sp, dp)) {
          s[r] = reinterpret_cast<const V*>(sp);
          d[r] = reinterpret_cast<V*>(dp);
        }
      }
    }
    for (int64_t k = sub; k < vpr; k += G) {
      V v[kRows];
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (s[r]) v[r] = __ldg(s[r] + k);
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (s[r]) __stcs(d[r] + k, v[r]);
    }
  }
}

// ---- cached gather, rows of up to 512 bytes in 16-byte vectors -----------------------------
// A warp takes 32 consecutive outputs: lane l reads index[i] and index_map[index[i]] for its own
// output (32 independent chains, coalesced index reads), then the warp moves the 32 rows eight
// at a time, 16 bytes per lane.  With one lane group per row (move_rows_kernel) the two
// dependent index reads of a row are made by every lane of the group and only four rows are in
// flight per warp.
template <typename IdxT>
__global__ void __launch_bounds__(kBlock, 3) cached_gather_warp_kernel(
    const char* __restrict__ backing, const char* __restrict__ cached, const IdxT* __restrict__ index,
    const IdxT* __restrict__ map, char* __restrict__ dst, uint8_t* __restrict__ found, int64_t n,
    int64_t row_bytes) {
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int vpr = (int)(row_bytes >> 4);
  const bool on = lane < vpr;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const char* src = nullptr;
    if (i < n) {
      const int64_t idx = (int64_t)__ldg(index + i);
      const int64_t g = (int64_t)__ldg(map + idx);
      src = g != -1 ? cached + g * row_bytes : backing + idx * row_bytes;
      if (found) found[i] = g != -1;
    }
    const unsigned have = __ballot_sync(0xffffffffu, src != nullptr);
    const unsigned long long src_bits = (unsigned long long)src;
    for (int q0 = 0; q0 < 32; q0 += 8) {
      if (((have >> q0) & 0xffu) == 0u) continue;
      uint4 val[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q0 + u);
        if (((have >> (q0 + u)) & 1u) && on) val[u] = __ldg(reinterpret_cast<const uint4*>(sb) + lane);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (((have >> (q0 + u)) & 1u) && on)
          __stcs(reinterpret_cast<uint4*>(dst + (base + q0 + u) * row_bytes) + lane, val[u]);
    }
  }
}

// ---- accumulate: dst[idx[i],:] += src[i,:], cnt[idx[i]] += 1 (unique indices) ------
template <typename IdxT>
__global__ void __launch_bounds__(kBlock) accumulate_rows_kernel(
    const float* __restrict__ src, float* __restrict__ dst, const IdxT* __restrict__ di,
    int32_t* __restrict__ cnt, int64_t n, int64_t dim, int glog2, bool vec4) {
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t group = tid >> glog2;
  const int sub = (int)(tid & ((1 << glog2) - 1));
  const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) >> glog2;
  const int G = 1 << glog2;
  for (int64_t i0 = group; i0 < n; i0 += ngroups * kRows) {
    int64_t row[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int64_t i = i0 + r * ngroups;
      row[r] = i < n ? (int64_t)__ldg(di + i) : -1;
      if (row[r] >= 0 && sub == 0 && cnt) cnt[row[r]] += 1;
    }
    if (vec4) {
      const int64_t vpr = dim >> 2;
      for (int64_t k = sub; k < vpr; k += G) {
        float4 a[kRows], b[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          if (row[r] >= 0) {
            a[r] = __ldg(reinterpret_cast<const float4*>(src + (i0 + r * ngroups) * dim) + k);
            b[r] = *(reinterpret_cast<const float4*>(dst + row[r] * dim) + k);
          }
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          if (row[r] >= 0) {
            b[r].x += a[r].x; b[r].y += a[r].y; b[r].z += a[r].z; b[r].w += a[r].w;
            *(reinterpret_cast<float4*>(dst + row[r] * dim) + k) = b[r];
          }
      }
    } else {
      for (int64_t k = sub; k < dim; k += G) {
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          if (row[r] >= 0) dst[row[r] * dim + k] += __ldg(src + (i0 + r * ngroups) * dim + k);
      }
    }
  }
}

// ---- fused lookup + fetch, LSU ---------------------------------------------------
template <int MODE, int VB>
__global__ void __launch_bounds__(kBlock) lookup_fetch_kernel(
    IndexView v, const int64_t* __restrict__ ids, int64_t n, const char* __restrict__ cache_rows,
    const char* __restrict__ backing, int64_t row_bytes, char* __restrict__ out,
    int64_t* __restrict__ locs, uint8_t* __restrict__ found, int glog2) {
  using V = typename Vec<VB>::T;
  __shared__ int64_t s_top[MODE == HB_LOOKUP_SORTED ? kTopMax : 1];
  if (MODE == HB_LOOKUP_SORTED) {
    stage_top_level(v, s_top);
    __syncthreads();
  }
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int G = 1 << glog2;
  const int sub = lane & (G - 1);
  const int which = lane >> glog2;
  const int rows_per_pass = 32 >> glog2;
  const int64_t vpr = row_bytes / VB;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    if (i < n) {
      if (locs) locs[i] = slot;
      if (found) found[i] = slot >= 0;
    }
    const char* src = nullptr;
    if (slot >= 0) src = cache_rows + slot * row_bytes;
    else if (backing && id >= 0) src = backing + id * row_bytes;
    const unsigned long long src_bits = (unsigned long long)src;
    // G lanes per row, 32/G rows per pass, kRows passes in flight
    for (int p = 0; p < G; p += kRows) {
      const V* s[kRows];
      V* d[kRows];
#pragma unroll
      for (int u = 0; u < kRows; ++u) {
        const int q = ((p + u) * rows_per_pass + which) & 31;
        const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q);
        const bool ok = (p + u) < G && sb != 0ull;
        s[u] = ok ? reinterpret_cast<const V*>(sb) : nullptr;
        d[u] = reinterpret_cast<V*>(out + (base + q) * row_bytes);
      }
      for (int64_t k = sub; k < vpr; k += G) {
        V val[kRows];
#pragma unroll
        for (int u = 0; u < kRows; ++u)
          if (s[u]) val[u] = __ldg(s[u] + k);
#pragma unroll
        for (int u = 0; u < kRows; ++u)
          if (s[u]) __stcs(d[u] + k, val[u]);
      }
    }
  }
}

// ---- fused lookup + fetch, 512-byte rows (dim 128 fp32) ---------------------------------
// One lane moves 16 bytes of a row, so a warp moves a whole row per instruction.
// The 32 rows of a warp's chunk go in 8 batches of 4; with DEPTH = 2 the loads of
// batch b+1 are issued before the stores of batch b, which doubles the bytes a warp
// keeps in flight without waiting.
template <int MODE, int MINB, int DEPTH>
__global__ void __launch_bounds__(kBlock, MINB) lookup_fetch512_kernel(
    IndexView v, const int64_t* __restrict__ ids, int64_t n, const char* __restrict__ cache_rows,
    const char* __restrict__ backing, char* __restrict__ out, int64_t* __restrict__ locs,
    uint8_t* __restrict__ found) {
  __shared__ int64_t s_top[MODE == HB_LOOKUP_SORTED ? kTopMax : 1];
  if (MODE == HB_LOOKUP_SORTED) {
    stage_top_level(v, s_top);
    __syncthreads();
  }
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    if (i < n) {
      if (locs) locs[i] = slot;
      if (found) found[i] = slot >= 0;
    }
    const char* src = nullptr;
    if (slot >= 0) src = cache_rows + slot * 512;
    else if (backing && id >= 0) src = backing + id * 512;
    const unsigned long long src_bits = (unsigned long long)src;
    const unsigned have = __ballot_sync(0xffffffffu, src != nullptr);  // rows to move
    uint4* dst = reinterpret_cast<uint4*>(out + base * 512) + lane;
    uint4 buf[DEPTH][4];
    auto load = [&](int b, uint4* into) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = b * 4 + u;
        const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q);
        if ((have >> q) & 1u) into[u] = __ldg(reinterpret_cast<const uint4*>(sb) + lane);
      }
    };
    auto store = [&](int b, const uint4* from) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = b * 4 + u;
        if ((have >> q) & 1u) __stcs(dst + q * 32, from[u]);
      }
    };
    if (DEPTH == 1) {
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        load(b, buf[0]);
        store(b, buf[0]);
      }
    } else {
      load(0, buf[0]);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        if (b + 1 < 8) load(b + 1, buf[(b + 1) & (DEPTH - 1)]);
        store(b, buf[b & (DEPTH - 1)]);
      }
    }
  }
}

// ---- BULK path ----------------------------------------------------------------------
// Shared memory per CTA: kBulkWarps stages of kStageBytes, then one mbarrier per
// warp, then (sorted lookup only) the staged top level.
struct BulkSmem {
  char* stage;
  uint64_t* bar;
};

__device__ __forceinline__ BulkSmem bulk_smem_setup(char* smem) {
  BulkSmem b;
  const int w = threadIdx.x >> 5;
  b.stage = smem + (size_t)w * kStageBytes;
  b.bar = reinterpret_cast<uint64_t*>(smem + (size_t)kBulkWarps * kStageBytes) + w;
  if (lane_id() == 0) mbar_init(b.bar, 1);
  mbar_init_fence();
  __syncthreads();
  return b;
}

// One stage: lanes [0, rows) each fetch `row_bytes` from their own src (nullptr =
// keep out of the copy), then the stage is written out.  When every row of the
// stage is present the output is one contiguous bulk store; otherwise present
// rows are stored one by one.  Returns false when the bounded wait gave up.
__device__ __forceinline__ bool bulk_stage_gather(const BulkSmem& b, uint32_t& parity,
                                                  const char* src, char* dst_first, int rows,
                                                  uint32_t row_bytes) {
  const int lane = lane_id();
  const bool have = lane < rows && src != nullptr;
  const unsigned present = __ballot_sync(0xffffffffu, have);
  if (present == 0u) return true;
  // the previous store out of this stage must have finished reading it
  bulk_wait_read_all();
  __syncwarp();
  if (lane == 0) mbar_arrive_expect_tx(b.bar, (uint32_t)__popc(present) * row_bytes);
  __syncwarp();
  if (have) bulk_g2s(b.stage + (size_t)lane * row_bytes, src, row_bytes, b.bar);
  const bool ok = mbar_wait_bounded(b.bar, parity);
  parity ^= 1u;
  if (!__all_sync(0xffffffffu, ok)) return false;
  const unsigned full = rows >= 32 ? 0xffffffffu : ((1u << rows) - 1u);
  if (present == full) {
    if (lane == 0) {
      bulk_s2g(dst_first, b.stage, (uint32_t)rows * row_bytes);
      bulk_commit();
    }
  } else if (have) {
    bulk_s2g(dst_first + (size_t)lane * row_bytes, b.stage + (size_t)lane * row_bytes, row_bytes);
    bulk_commit();
  }
  return true;
}

template <typename IdxT>
__global__ void __launch_bounds__(kBulkWarps * 32) bulk_gather_kernel(
    const char* __restrict__ src, const IdxT* __restrict__ si, char* __restrict__ dst, int64_t n,
    uint32_t row_bytes, int rows_per_stage, int* __restrict__ err) {
  extern __shared__ __align__(128) char smem[];
  BulkSmem b = bulk_smem_setup(smem);
  uint32_t parity = 0;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * rows_per_stage; base < n; base += nwarps * rows_per_stage) {
    const int64_t left = n - base;
    const int rows = left < rows_per_stage ? (int)left : rows_per_stage;
    const char* s = lane < rows ? src + (int64_t)__ldg(si + base + lane) * row_bytes : nullptr;
    if (!bulk_stage_gather(b, parity, s, dst + base * row_bytes, rows, row_bytes)) {
      if (lane == 0) atomicExch(err, HB_ERR_TIMEOUT);
      break;
    }
  }
  bulk_wait_all();
}

template <typename IdxT>
__global__ void __launch_bounds__(kBulkWarps * 32) bulk_scatter_kernel(
    const char* __restrict__ src, char* __restrict__ dst, const IdxT* __restrict__ di, int64_t n,
    uint32_t row_bytes, int rows_per_stage, int* __restrict__ err) {
  extern __shared__ __align__(128) char smem[];
  BulkSmem b = bulk_smem_setup(smem);
  uint32_t parity = 0;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * rows_per_stage; base < n; base += nwarps * rows_per_stage) {
    const int64_t left = n - base;
    const int rows = left < rows_per_stage ? (int)left : rows_per_stage;
    char* d = lane < rows ? dst + (int64_t)__ldg(di + base + lane) * row_bytes : nullptr;
    bulk_wait_read_all();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive_expect_tx(b.bar, (uint32_t)rows * row_bytes);
      bulk_g2s(b.stage, src + base * row_bytes, (uint32_t)rows * row_bytes, b.bar);
    }
    const bool ok = mbar_wait_bounded(b.bar, parity);
    parity ^= 1u;
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0) atomicExch(err, HB_ERR_TIMEOUT);
      break;
    }
    if (d) {
      bulk_s2g(d, b.stage + (size_t)lane * row_bytes, row_bytes);
      bulk_commit();
    }
  }
  bulk_wait_all();
}

template <int MODE>
__global__ void __launch_bounds__(kBulkWarps * 32) bulk_lookup_fetch_kernel(
    IndexView v, const int64_t* __restrict__ ids, int64_t n, const char* __restrict__ cache_rows,
    const char* __restrict__ backing, uint32_t row_bytes, char* __restrict__ out,
    int64_t* __restrict__ locs, uint8_t* __restrict__ found, int rows_per_stage,
    int* __restrict__ err) {
  extern __shared__ __align__(128) char smem[];
  int64_t* s_top = reinterpret_cast<int64_t*>(smem + (size_t)kBulkWarps * kStageBytes + 128);
  if (MODE == HB_LOOKUP_SORTED) stage_top_level(v, s_top);
  BulkSmem b = bulk_smem_setup(smem);  // ends with __syncthreads()
  uint32_t parity = 0;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  bool alive = true;
  for (int64_t base = warp * 32; base < n && alive; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    if (i < n) {
      if (locs) locs[i] = slot;
      if (found) found[i] = slot >= 0;
    }
    const char* src = nullptr;
    if (slot >= 0) src = cache_rows + slot * (int64_t)row_bytes;
    else if (backing && id >= 0) src = backing + id * (int64_t)row_bytes;
    const unsigned long long src_bits = (unsigned long long)src;
    const int chunk = (n - base) < 32 ? (int)(n - base) : 32;
    for (int r0 = 0; r0 < chunk; r0 += rows_per_stage) {
      const int rows = (chunk - r0) < rows_per_stage ? (chunk - r0) : rows_per_stage;
      const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, (r0 + lane) & 31);
      const char* s = lane < rows ? reinterpret_cast<const char*>(sb) : nullptr;
      if (!bulk_stage_gather(b, parity, s, out + (base + r0) * (int64_t)row_bytes, rows,
                             row_bytes)) {
        if (lane == 0) atomicExch(err, HB_ERR_TIMEOUT);
        alive = false;
        break;
      }
    }
  }
  bulk_wait_all();
}

// ---- host-side dispatch helpers ---------------------------------------------------------
int group_log2_for(int64_t vecs_per_row) {
  int g = 0;
  while ((1 << g) < vecs_per_row && g < 5) ++g;
  return g;
}

int vec_bytes_for(int64_t row_bytes, std::initializer_list<const void*> ptrs) {
  uintptr_t bits = (uintptr_t)row_bytes;
  for (const void* p : ptrs) bits |= (uintptr_t)p;
  if ((bits & 15) == 0) return 16;
  if ((bits & 7) == 0) return 8;
  if ((bits & 3) == 0) return 4;
  if ((bits & 1) == 0) return 2;
  return 1;
}

int grid_for_groups(int64_t n, int glog2) {
  const int64_t groups = ceil_div(n, kRows);
  int64_t blocks = ceil_div(groups << glog2, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename R>
int launch_move(R rs, int64_t n, int64_t row_bytes, int vb, cudaStream_t st) {
  const int glog2 = group_log2_for(row_bytes / vb);
  const int grid = grid_for_groups(n, glog2);
  switch (vb) {
    case 16: HB_LAUNCH((move_rows_kernel<16, R>), grid, kBlock, 0, st, rs, n, row_bytes, glog2); break;
    case 8: HB_LAUNCH((move_rows_kernel<8, R>), grid, kBlock, 0, st, rs, n, row_bytes, glog2); break;
    case 4: HB_LAUNCH((move_rows_kernel<4, R>), grid, kBlock, 0, st, rs, n, row_bytes, glog2); break;
    case 2: HB_LAUNCH((move_rows_kernel<2, R>), grid, kBlock, 0, st, rs, n, row_bytes, glog2); break;
    default: HB_LAUNCH((move_rows_kernel<1, R>), grid, kBlock, 0, st, rs, n, row_bytes, glog2); break;
  }
  return HB_OK;
}

bool bulk_eligible(int64_t row_bytes, std::initializer_list<const void*> ptrs) {
  if (row_bytes < 16 || row_bytes > kStageBytes || (row_bytes & 15)) return false;
  for (const void* p : ptrs)
    if ((uintptr_t)p & 15) return false;
  return true;
}

int rows_per_stage_for(int64_t row_bytes) {
  int64_t r = kStageBytes / row_bytes;
  if (r > 32) r = 32;
  return (int)r;
}

size_t bulk_smem_bytes(bool with_top) {
  return (size_t)kBulkWarps * kStageBytes + 128 + (with_top ? kTopMax * sizeof(int64_t) : 0);
}

int bulk_grid(int64_t n, int rows_per_stage) {
  const int64_t stages = ceil_div(n, rows_per_stage);
  int64_t blocks = ceil_div(stages, kBulkWarps);
  const int64_t cap = sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename K>
int allow_big_smem(K kernel, size_t bytes) {
  HB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return HB_OK;
}

#define HB_IDX_SWITCH(idx_bytes, IdxT, ...)              \
  if ((idx_bytes) == 8) {                                \
    typedef int64_t IdxT;                                \
    __VA_ARGS__                                          \
  } else {                                               \
    typedef int32_t IdxT;                                \
    __VA_ARGS__                                          \
  }

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_rows_gather(const void* src, const void* src_index, void* dst, const void* dst_index,
                   int64_t n, int64_t row_bytes, int idx_bytes, int mover, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_rows_gather: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_rows_gather: index must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (src && src_index && dst), "hb_rows_gather: null argument");
  HB_CHECK_ARG(mover >= HB_MOVER_AUTO && mover <= HB_MOVER_BULK, "hb_rows_gather: unknown mover");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const bool can_bulk = dst_index == nullptr && bulk_eligible(row_bytes, {src, dst});
  if (mover == HB_MOVER_BULK && !can_bulk) {
    set_error("hb_rows_gather: bulk mover needs a contiguous output, 16-byte aligned buffers and "
              "a row size that is a multiple of 16 and at most %d bytes", kStageBytes);
    return HB_ERR_UNSUPPORTED;
  }
  if (mover == HB_MOVER_BULK) {
    const int rps = rows_per_stage_for(row_bytes);
    const size_t smem = bulk_smem_bytes(false);
    int* err = device_error_word();
    HB_IDX_SWITCH(idx_bytes, IdxT, {
      int rc = allow_big_smem(bulk_gather_kernel<IdxT>, smem);
      if (rc) return rc;
      HB_LAUNCH(bulk_gather_kernel<IdxT>, bulk_grid(n, rps), kBulkWarps * 32, smem, st,
                (const char*)src, (const IdxT*)src_index, (char*)dst, n, (uint32_t)row_bytes, rps,
                err);
    })
    return HB_OK;
  }
  const int vb = vec_bytes_for(row_bytes, {src, dst});
  HB_IDX_SWITCH(idx_bytes, IdxT, {
    if (dst_index) {
      GatherRes<IdxT, true> rs{(const char*)src, (const IdxT*)src_index, (char*)dst,
                               (const IdxT*)dst_index, row_bytes};
      return launch_move(rs, n, row_bytes, vb, st);
    } else {
      GatherRes<IdxT, false> rs{(const char*)src, (const IdxT*)src_index, (char*)dst, nullptr,
                                row_bytes};
      return launch_move(rs, n, row_bytes, vb, st);
    }
  })
}

int hb_rows_scatter(const void* src, void* dst, const void* dst_index, int64_t n,
                    int64_t row_bytes, int idx_bytes, int mover, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_rows_scatter: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_rows_scatter: index must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (src && dst && dst_index), "hb_rows_scatter: null argument");
  HB_CHECK_ARG(mover >= HB_MOVER_AUTO && mover <= HB_MOVER_BULK, "hb_rows_scatter: unknown mover");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (mover == HB_MOVER_BULK) {
    if (!bulk_eligible(row_bytes, {src, dst})) {
      set_error("hb_rows_scatter: bulk mover needs 16-byte aligned buffers and a row size that is "
                "a multiple of 16 and at most %d bytes", kStageBytes);
      return HB_ERR_UNSUPPORTED;
    }
    const int rps = rows_per_stage_for(row_bytes);
    const size_t smem = bulk_smem_bytes(false);
    int* err = device_error_word();
    HB_IDX_SWITCH(idx_bytes, IdxT, {
      int rc = allow_big_smem(bulk_scatter_kernel<IdxT>, smem);
      if (rc) return rc;
      HB_LAUNCH(bulk_scatter_kernel<IdxT>, bulk_grid(n, rps), kBulkWarps * 32, smem, st,
                (const char*)src, (char*)dst, (const IdxT*)dst_index, n, (uint32_t)row_bytes, rps,
                err);
    })
    return HB_OK;
  }
  const int vb = vec_bytes_for(row_bytes, {src, dst});
  HB_IDX_SWITCH(idx_bytes, IdxT, {
    ScatterRes<IdxT> rs{(const char*)src, (char*)dst, (const IdxT*)dst_index, row_bytes};
    return launch_move(rs, n, row_bytes, vb, st);
  })
}

int hb_rows_gather_cached(const void* backing_src, const void* cached_src, const void* index,
                          const void* index_map, void* dst, uint8_t* found, int64_t n,
                          int64_t row_bytes, int idx_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_rows_gather_cached: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_rows_gather_cached: index must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (backing_src && cached_src && index && index_map && dst),
               "hb_rows_gather_cached: null argument");
  if (n == 0) return HB_OK;
  const int vb = vec_bytes_for(row_bytes, {backing_src, cached_src, dst});
  if (vb == 16 && row_bytes <= 512) {
    int64_t blocks = ceil_div(ceil_div(n, 32) * 32, kBlock);
    if (blocks > (int64_t)sm_count() * 24) blocks = (int64_t)sm_count() * 24;
    HB_IDX_SWITCH(idx_bytes, IdxT, {
      HB_LAUNCH(cached_gather_warp_kernel<IdxT>, (int)blocks, kBlock, 0, (cudaStream_t)stream,
                (const char*)backing_src, (const char*)cached_src, (const IdxT*)index, (const IdxT*)index_map,
                (char*)dst, found, n, row_bytes);
      return HB_OK;
    })
  }
  HB_IDX_SWITCH(idx_bytes, IdxT, {
    CachedGatherRes<IdxT> rs{(const char*)backing_src, (const char*)cached_src, (const IdxT*)index,
                             (const IdxT*)index_map, (char*)dst, found, row_bytes};
    return launch_move(rs, n, row_bytes, vb, (cudaStream_t)stream);
  })
}

int hb_rows_scatter_cached(const void* src, void* backing_dst, void* cached_dst, const void* index,
                           const void* index_map, int64_t n, int64_t row_bytes, int idx_bytes,
                           hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_rows_scatter_cached: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_rows_scatter_cached: index must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (src && backing_dst && cached_dst && index && index_map),
               "hb_rows_scatter_cached: null argument");
  if (n == 0) return HB_OK;
  const int vb = vec_bytes_for(row_bytes, {src, backing_dst, cached_dst});
  HB_IDX_SWITCH(idx_bytes, IdxT, {
    CachedScatterRes<IdxT> rs{(const char*)src, (char*)backing_dst, (char*)cached_dst,
                              (const IdxT*)index, (const IdxT*)index_map, row_bytes};
    return launch_move(rs, n, row_bytes, vb, (cudaStream_t)stream);
  })
}

int hb_rows_accumulate_f32(const float* src, float* dst, const void* dst_index, int32_t* cnt,
                           int64_t n, int64_t dim, int idx_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && dim > 0, "hb_rows_accumulate_f32: bad sizes");
  HB_CHECK_ARG(idx_bytes == 4 || idx_bytes == 8, "hb_rows_accumulate_f32: index must be int32 or int64");
  HB_CHECK_ARG(n == 0 || (src && dst && dst_index), "hb_rows_accumulate_f32: null argument");
  if (n == 0) return HB_OK;
  const bool vec4 = (dim % 4 == 0) && (((uintptr_t)src | (uintptr_t)dst) & 15) == 0;
  const int glog2 = group_log2_for(vec4 ? dim / 4 : dim);
  const int grid = grid_for_groups(n, glog2);
  HB_IDX_SWITCH(idx_bytes, IdxT, {
    HB_LAUNCH(accumulate_rows_kernel<IdxT>, grid, kBlock, 0, (cudaStream_t)stream, src, dst,
              (const IdxT*)dst_index, cnt, n, dim, glog2, vec4);
  })
  return HB_OK;
}

int hb_lookup_fetch(hb_index_t* h, const int64_t* ids, int64_t n, const void* cache_rows,
                    const void* backing_rows, int64_t row_bytes, void* out_rows, int64_t* locs,
                    uint8_t* found, int mode, int mover, hb_stream_t stream) {
  HB_CHECK_ARG(h && n >= 0 && row_bytes > 0, "hb_lookup_fetch: bad argument");
  HB_CHECK_ARG(n == 0 || (ids && cache_rows && out_rows), "hb_lookup_fetch: null argument");
  HB_CHECK_ARG(mode == HB_LOOKUP_SETASSOC || mode == HB_LOOKUP_SORTED,
               "hb_lookup_fetch: unknown mode %d", mode);
  HB_CHECK_ARG(mover >= HB_MOVER_AUTO && mover <= HB_MOVER_BULK, "hb_lookup_fetch: unknown mover");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == HB_LOOKUP_SORTED && h->sorted_stale) {
    int rc = hb_index_build_sorted(h, stream);
    if (rc != HB_OK) return rc;
  }
  const bool can_bulk = bulk_eligible(row_bytes, {cache_rows, backing_rows, out_rows});
  if (mover == HB_MOVER_BULK && !can_bulk) {
    set_error("hb_lookup_fetch: bulk mover needs 16-byte aligned buffers and a row size that is a "
              "multiple of 16 and at most %d bytes", kStageBytes);
    return HB_ERR_UNSUPPORTED;
  }
  if (mover == HB_MOVER_BULK) {
    const int rps = rows_per_stage_for(row_bytes);
    const bool sorted = mode == HB_LOOKUP_SORTED;
    const size_t smem = bulk_smem_bytes(sorted);
    int64_t blocks = ceil_div(ceil_div(n, 32), kBulkWarps);
    if (blocks > sm_count()) blocks = sm_count();
    int* err = device_error_word();
    if (sorted) {
      int rc = allow_big_smem(bulk_lookup_fetch_kernel<HB_LOOKUP_SORTED>, smem);
      if (rc) return rc;
      HB_LAUNCH(bulk_lookup_fetch_kernel<HB_LOOKUP_SORTED>, (int)blocks, kBulkWarps * 32, smem, st,
                h->view, ids, n, (const char*)cache_rows, (const char*)backing_rows,
                (uint32_t)row_bytes, (char*)out_rows, locs, found, rps, err);
    } else {
      int rc = allow_big_smem(bulk_lookup_fetch_kernel<HB_LOOKUP_SETASSOC>, smem);
      if (rc) return rc;
      HB_LAUNCH(bulk_lookup_fetch_kernel<HB_LOOKUP_SETASSOC>, (int)blocks, kBulkWarps * 32, smem,
                st, h->view, ids, n, (const char*)cache_rows, (const char*)backing_rows,
                (uint32_t)row_bytes, (char*)out_rows, locs, found, rps, err);
    }
    return HB_OK;
  }
  const int vb = vec_bytes_for(row_bytes, {cache_rows, backing_rows, out_rows});
  const int glog2 = group_log2_for(row_bytes / vb);
  int64_t blocks = ceil_div(ceil_div(n, 32) * 32, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (vb == 16 && row_bytes == 512) {
    // dim 128 fp32: the specialised kernel (measured 2-4 % faster than the generic mover;
    // deeper prefetch or 4 CTAs/SM measured no better: the kernel sits at the random-row
    // bandwidth of the memory system)
    if (mode == HB_LOOKUP_SORTED)
      HB_LAUNCH((lookup_fetch512_kernel<HB_LOOKUP_SORTED, 3, 1>), (int)blocks, kBlock, 0, st, h->view,
                ids, n, (const char*)cache_rows, (const char*)backing_rows, (char*)out_rows, locs, found);
    else
      HB_LAUNCH((lookup_fetch512_kernel<HB_LOOKUP_SETASSOC, 3, 1>), (int)blocks, kBlock, 0, st, h->view,
                ids, n, (const char*)cache_rows, (const char*)backing_rows, (char*)out_rows, locs, found);
    return HB_OK;
  }
#define HB_LF(MODE, VB)                                                                         \
  HB_LAUNCH((lookup_fetch_kernel<MODE, VB>), (int)blocks, kBlock, 0, st, h->view, ids, n,       \
            (const char*)cache_rows, (const char*)backing_rows, row_bytes, (char*)out_rows, locs, \
            found, glog2)
#define HB_LF_VB(MODE)                 \
  switch (vb) {                        \
    case 16: HB_LF(MODE, 16); break;   \
    case 8: HB_LF(MODE, 8); break;     \
    case 4: HB_LF(MODE, 4); break;     \
    case 2: HB_LF(MODE, 2); break;     \
    default: HB_LF(MODE, 1); break;    \
  }
  if (mode == HB_LOOKUP_SORTED) {
    HB_LF_VB(HB_LOOKUP_SORTED)
  } else {
    HB_LF_VB(HB_LOOKUP_SETASSOC)
  }
#undef HB_LF_VB
#undef HB_LF
  return HB_OK;
}

}  // extern "C"
