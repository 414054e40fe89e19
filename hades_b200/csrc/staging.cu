// Cold-gradient staging table in HBM: accumulate, flush and insert.  Replaces the
// arithmetic of the reference's cache-server process (python/EmbCache/server.py:
// _accumulate_gradients_cold_remote/_local :546-574, _send_staled_gradients
// :346-497, _update_cache :499-544), which does it with torch CPU indexing on
// shared-memory tensors behind sockets.
#include "index.cuh"
#include <type_traits>

#include "partition_core.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ int64_t effective_n(int64_t n, const int64_t* n_dev) {
  if (!n_dev) return n;
  const int64_t d = *n_dev;
  return d < n ? d : n;
}

// rows[q] of the warp's 32 items: dst_row += src_row (fp32), 4 rows in flight
template <int VEC>
__device__ __forceinline__ void warp_add_rows(const float* src_row, float* dst_row, bool active,
                                              int64_t dim) {
  const int lane = threadIdx.x & 31;
  const unsigned act = __ballot_sync(0xffffffffu, active);
  if (act == 0u) return;
  const unsigned long long sb = (unsigned long long)src_row;
  const unsigned long long db = (unsigned long long)dst_row;
  for (int q0 = 0; q0 < 32; q0 += 4) {
    if (((act >> q0) & 0xfu) == 0u) continue;
    const float* s[4];
    float* d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned long long a = __shfl_sync(0xffffffffu, sb, q0 + u);
      const unsigned long long b = __shfl_sync(0xffffffffu, db, q0 + u);
      const bool on = (act >> (q0 + u)) & 1u;
      s[u] = on ? reinterpret_cast<const float*>(a) : nullptr;
      d[u] = reinterpret_cast<float*>(b);
    }
    if (VEC == 4) {
      const int64_t vpr = dim >> 2;
      for (int64_t k = lane; k < vpr; k += 32) {
        float4 x[4], y[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s[u]) {
            x[u] = __ldg(reinterpret_cast<const float4*>(s[u]) + k);
            y[u] = reinterpret_cast<float4*>(d[u])[k];
          }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s[u]) {
            y[u].x += x[u].x; y[u].y += x[u].y; y[u].z += x[u].z; y[u].w += x[u].w;
            reinterpret_cast<float4*>(d[u])[k] = y[u];
          }
      }
    } else {
      for (int64_t k = lane; k < dim; k += 32) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (s[u]) d[u][k] += __ldg(s[u] + k);
      }
    }
  }
}

// ---- accumulate through the cache index (cold remote, server.py:546-562) --------------
template <int MODE, int VEC>
__global__ void __launch_bounds__(kBlock) staging_accumulate_cached_kernel(
    IndexView v, hb_staging_t s, const int64_t* __restrict__ ids, const float* __restrict__ grads,
    int64_t n, const int64_t* __restrict__ n_dev, const int32_t* __restrict__ thr_table,
    int32_t default_thr, unsigned long long* __restrict__ dropped, int64_t* __restrict__ locs_out) {
  __shared__ int64_t s_top[MODE == HB_LOOKUP_SORTED ? kTopMax : 1];
  if (MODE == HB_LOOKUP_SORTED) {
    stage_top_level(v, s_top);
    __syncthreads();
  }
  n = effective_n(n, n_dev);
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    const bool hit = slot >= 0;
    if (locs_out && i < n) locs_out[i] = slot;
    if (hit) {
      s.idx[slot] = id;
      s.iter_threshold[slot] = thr_table ? __ldg(thr_table + id) : default_thr;
      s.cnt[slot] += 1;
    }
    if (dropped) {
      const unsigned miss = __ballot_sync(0xffffffffu, i < n && id >= 0 && !hit);
      if (lane == 0 && miss) atomicAdd(dropped, (unsigned long long)__popc(miss));
    }
    warp_add_rows<VEC>(grads + i * s.dim, s.grad + (hit ? slot : 0) * s.dim, hit, s.dim);
  }
}

// ---- accumulate by direct address (cold local, server.py:564-574) -----------------------
template <int VEC>
__global__ void __launch_bounds__(kBlock) staging_accumulate_direct_kernel(
    hb_staging_t s, const int64_t* __restrict__ ids, const float* __restrict__ grads, int64_t n,
    const int64_t* __restrict__ n_dev, int64_t id_offset, int64_t id_stride) {
  n = effective_n(n, n_dev);
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    int64_t slot = -1;
    if (id >= id_offset) {
      slot = (id - id_offset) / id_stride;
      if (slot >= s.slots) slot = -1;
    }
    const bool ok = slot >= 0;
    if (ok) {
      s.idx[slot] = id;
      s.cnt[slot] += 1;
    }
    warp_add_rows<VEC>(grads + i * s.dim, s.grad + (ok ? slot : 0) * s.dim, ok, s.dim);
  }
}

// ---- flush (server.py:346-425 remote / :427-497 local) ---------------------------------------
// Item = staging slot.  A slot is stale when cnt > 0 and (iter_count >=
// iter_threshold or cnt >= cnt_threshold); stale rows leave in slot order,
// bucketed by id % num_clients, and the slot is cleared; live slots with cnt > 0
// age by one iteration.
//
// Two passes.  The partition selects: it writes the id of every stale slot to its place in
// the output (slot order within a bucket), leaves the slot number where the count will go,
// resets the cache entry and ages the live slots; no row moves there, because with a few
// per cent of the slots stale a warp of the partition would move one or two rows at a time.
// The second pass runs over the stale entries only: count out and cleared, row out and zeroed.
struct FlushPolicy {
  hb_staging_t s;
  int32_t cnt_threshold;
  int num_clients;
  int64_t out_cap;    // rows the output can take (only with one client); the rest stays staged
  int64_t* line_ids;  // nullable: the cache index entries of flushed ids are reset
  int32_t* lru;
  int64_t* out_ids;
  int64_t* out_cnt;   // holds the slot number until the second pass
  __device__ __forceinline__ int classify(int64_t i) const {
    const int32_t c = s.cnt[i];
    if (c <= 0) return -1;
    if (!(s.iter_count[i] >= s.iter_threshold[i] || c >= cnt_threshold)) return -1;
    const int64_t id = s.idx[i];
    return id >= 0 ? (int)mod_nonneg(id, num_clients) : -1;
  }
  __device__ __forceinline__ void emit(int64_t i, int, int64_t pos, int64_t start,
                                       bool active) const {
    const int64_t d = start + pos;
    if (active && d < out_cap) {
      const int64_t id = s.idx[i];
      out_ids[d] = id;
      out_cnt[d] = i;
      if (line_ids && line_ids[i] == id) {  // _idx_cache.reset(ids), server.py:413
        line_ids[i] = -1;
        lru[i] = 0;
      }
    } else if (i < s.slots && s.cnt[i] > 0) {
      s.iter_count[i] += 1;  // server.py:418 (a stale row the output had no room for waits for the next flush)
    }
  }
};

// Second pass of the flush: entry d < sum(counts) left slot out_cnt[d]; its count goes out
// and starts again (server.py:419), its row goes out and is zeroed.  VB: bytes per vector.
template <int VB>
__global__ void __launch_bounds__(kBlock) staging_flush_move_kernel(
    hb_staging_t s, const int64_t* __restrict__ counts, int num_clients, int64_t out_cap,
    int64_t* __restrict__ out_cnt, float* __restrict__ out_rows) {
  using V = typename std::conditional<VB == 16, uint4, uint32_t>::type;
  int64_t total = 0;
  for (int c = 0; c < num_clients; ++c) total += counts[c];
  if (total > out_cap) total = out_cap;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t vpr = (int64_t)s.dim * 4 / VB;
  V zero;
  memset(&zero, 0, sizeof(zero));
  for (int64_t base = warp * 32; base < total; base += nwarps * 32) {
    const int64_t d = base + lane;
    int64_t slot = -1;
    if (d < total) {
      slot = out_cnt[d];
      out_cnt[d] = (int64_t)s.cnt[slot];
      s.cnt[slot] = 0;
      s.iter_count[slot] = 0;
    }
    const int rows_here = (int)((total - base) < 32 ? (total - base) : 32);
    for (int q0 = 0; q0 < rows_here; q0 += 4) {
      V* src[4];
      V* dst[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t sl = __shfl_sync(0xffffffffu, slot, (q0 + u) & 31);
        const bool on = q0 + u < rows_here;
        src[u] = on ? reinterpret_cast<V*>(s.grad + sl * s.dim) : nullptr;
        dst[u] = reinterpret_cast<V*>(out_rows + (base + q0 + u) * s.dim);
      }
      for (int64_t k = lane; k < vpr; k += 32) {
        V v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (src[u]) v[u] = src[u][k];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (src[u]) {
            __stcs(dst[u] + k, v[u]);
            src[u][k] = zero;
          }
      }
    }
  }
}

// ---- insert (server.py:499-544): rows into the cache buffer at the slots add() gave ----------
template <int VEC_BYTES>
__global__ void __launch_bounds__(kBlock) staging_insert_kernel(
    hb_staging_t s, const int64_t* __restrict__ locs, const uint8_t* __restrict__ last_writer,
    const char* __restrict__ emb_rows, const int64_t* __restrict__ row_index,
    char* __restrict__ cache_rows, int64_t row_bytes, int64_t n) {
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    // of several ids that received the same slot, the last of the batch writes it
    const int64_t slot = (i < n && last_writer[i]) ? __ldg(locs + i) : -1;
    const bool ok = slot >= 0;
    if (ok && s.cnt) {
      s.cnt[slot] = 0;   // server.py:539-541
      s.idx[slot] = -1;
    }
    const int64_t from = (ok && row_index) ? __ldg(row_index + i) : i;  // row of entry i in emb_rows
    warp_move_rows(emb_rows + from * row_bytes, cache_rows + (ok ? slot : 0) * row_bytes, ok, row_bytes,
                   VEC_BYTES);
    if (s.grad) {
      const unsigned act = __ballot_sync(0xffffffffu, ok);
      for (int q = 0; q < 32; ++q) {
        if (!((act >> q) & 1u)) continue;
        const int64_t sq = __shfl_sync(0xffffffffu, slot, q);
        float* row = s.grad + sq * s.dim;
        for (int64_t k = lane; k < s.dim; k += 32) row[k] = 0.f;
      }
    }
  }
}

int warp_grid(int64_t n) {
  int64_t blocks = ceil_div(ceil_div(n, 32) * 32, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int check_staging(const hb_staging_t* s, const char* who) {
  if (!s || !s->grad || !s->cnt || !s->idx || !s->iter_count || !s->iter_threshold ||
      s->slots <= 0 || s->dim <= 0) {
    set_error("%s: incomplete staging table description", who);
    return HB_ERR_INVALID;
  }
  return HB_OK;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_staging_accumulate_cached(hb_index_t* h, const hb_staging_t* s, const int64_t* ids,
                                 const float* grads, int64_t n, const int64_t* n_dev,
                                 const int32_t* threshold_table, int32_t default_threshold,
                                 int mode, int64_t* dropped, int64_t* locs_out,
                                 hb_stream_t stream) {
  HB_CHECK_ARG(h != nullptr, "hb_staging_accumulate_cached: null index");
  int rc = check_staging(s, "hb_staging_accumulate_cached");
  if (rc) return rc;
  HB_CHECK_ARG(n >= 0 && (n == 0 || (ids && grads)), "hb_staging_accumulate_cached: null argument");
  HB_CHECK_ARG(s->slots == h->cache_size,
               "hb_staging_accumulate_cached: the staging table must have one slot per cache slot");
  HB_CHECK_ARG(mode == HB_LOOKUP_SETASSOC || mode == HB_LOOKUP_SORTED,
               "hb_staging_accumulate_cached: unknown mode");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == HB_LOOKUP_SORTED && h->sorted_stale) {
    rc = hb_index_build_sorted(h, stream);
    if (rc) return rc;
  }
  const bool vec4 = (s->dim % 4 == 0) && (((uintptr_t)grads | (uintptr_t)s->grad) & 15) == 0;
  const int grid = warp_grid(n);
#define HB_ACC(MODE, VEC)                                                                     \
  HB_LAUNCH((staging_accumulate_cached_kernel<MODE, VEC>), grid, kBlock, 0, st, h->view, *s,  \
            ids, grads, n, n_dev, threshold_table, default_threshold,                         \
            (unsigned long long*)dropped, locs_out)
  if (mode == HB_LOOKUP_SORTED) {
    if (vec4) HB_ACC(HB_LOOKUP_SORTED, 4); else HB_ACC(HB_LOOKUP_SORTED, 1);
  } else {
    if (vec4) HB_ACC(HB_LOOKUP_SETASSOC, 4); else HB_ACC(HB_LOOKUP_SETASSOC, 1);
  }
#undef HB_ACC
  return HB_OK;
}

int hb_staging_accumulate_direct(const hb_staging_t* s, const int64_t* ids, const float* grads,
                                 int64_t n, const int64_t* n_dev, int64_t id_offset,
                                 int64_t id_stride, hb_stream_t stream) {
  int rc = check_staging(s, "hb_staging_accumulate_direct");
  if (rc) return rc;
  HB_CHECK_ARG(n >= 0 && (n == 0 || (ids && grads)), "hb_staging_accumulate_direct: null argument");
  HB_CHECK_ARG(id_stride > 0, "hb_staging_accumulate_direct: id_stride must be positive");
  if (n == 0) return HB_OK;
  const bool vec4 = (s->dim % 4 == 0) && (((uintptr_t)grads | (uintptr_t)s->grad) & 15) == 0;
  if (vec4)
    HB_LAUNCH(staging_accumulate_direct_kernel<4>, warp_grid(n), kBlock, 0, (cudaStream_t)stream,
              *s, ids, grads, n, n_dev, id_offset, id_stride);
  else
    HB_LAUNCH(staging_accumulate_direct_kernel<1>, warp_grid(n), kBlock, 0, (cudaStream_t)stream,
              *s, ids, grads, n, n_dev, id_offset, id_stride);
  return HB_OK;
}

size_t hb_staging_flush_workspace_bytes(int64_t slots, int num_clients) {
  return partition_workspace_bytes(slots, num_clients);
}

int hb_staging_flush(hb_index_t* h, const hb_staging_t* s, int32_t cnt_threshold, int num_clients,
                     int64_t out_cap, int64_t* out_ids, float* out_rows, int64_t* out_cnt,
                     int64_t* counts, void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  int rc = check_staging(s, "hb_staging_flush");
  if (rc) return rc;
  if (out_cap <= 0 || out_cap > s->slots) out_cap = s->slots;
  HB_CHECK_ARG(out_cap == s->slots || num_clients == 1,
               "hb_staging_flush: an output smaller than the table needs num_clients == 1");
  HB_CHECK_ARG(out_ids && out_rows && out_cnt && counts, "hb_staging_flush: null output");
  HB_CHECK_ARG(num_clients >= 1, "hb_staging_flush: num_clients must be positive");
  HB_CHECK_ARG(s->slots < ((int64_t)1 << 31), "hb_staging_flush: too many slots");
  HB_CHECK_ARG(!h || h->cache_size == s->slots,
               "hb_staging_flush: the staging table must have one slot per cache slot");
  FlushPolicy pol{*s, cnt_threshold, num_clients, out_cap, h ? h->line_ids : nullptr,
                  h ? h->lru : nullptr, out_ids, out_cnt};
  rc = run_partition(pol, s->slots, num_clients, workspace, workspace_bytes, counts,
                     (cudaStream_t)stream, 8);
  if (rc != HB_OK) return rc;
  if (h) h->sorted_stale = true;
  // the number of stale rows is only known on the device: size the grid for a full output
  const int grid = warp_grid(out_cap);
  if (payload_vec_bytes(s->dim * (int64_t)sizeof(float), s->grad, out_rows) == 16)
    HB_LAUNCH(staging_flush_move_kernel<16>, grid, kBlock, 0, (cudaStream_t)stream, *s, counts, num_clients,
              out_cap, out_cnt, out_rows);
  else
    HB_LAUNCH(staging_flush_move_kernel<4>, grid, kBlock, 0, (cudaStream_t)stream, *s, counts, num_clients,
              out_cap, out_cnt, out_rows);
  return HB_OK;
}

size_t hb_staging_insert_workspace_bytes(int64_t n) {
  return hb_index_add_workspace_bytes(n) + align_up((size_t)(n > 0 ? n : 1), 256);
}

int hb_staging_insert(hb_index_t* h, const hb_staging_t* s, const int64_t* ids,
                      const void* emb_rows, int64_t n, void* cache_rows, int64_t row_bytes,
                      int64_t* locs_out, void* workspace, size_t workspace_bytes,
                      hb_stream_t stream) {
  return hb_staging_insert_gather(h, s, ids, emb_rows, nullptr, n, cache_rows, row_bytes, locs_out,
                                  workspace, workspace_bytes, stream);
}

int hb_staging_insert_gather(hb_index_t* h, const hb_staging_t* s, const int64_t* ids,
                             const void* emb_rows, const int64_t* row_index, int64_t n,
                             void* cache_rows, int64_t row_bytes, int64_t* locs_out, void* workspace,
                             size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(h != nullptr, "hb_staging_insert: null index");
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_staging_insert: bad sizes");
  HB_CHECK_ARG(n == 0 || (ids && emb_rows && cache_rows && locs_out), "hb_staging_insert: null argument");
  HB_CHECK_ARG(!s || s->slots == h->cache_size,
               "hb_staging_insert: the staging table must have one slot per cache slot");
  if (n == 0) return HB_OK;
  const size_t flag_bytes = align_up((size_t)n, 256);
  if (!workspace || workspace_bytes < hb_staging_insert_workspace_bytes(n)) {
    set_error("hb_staging_insert: workspace of %zu bytes needed, %zu given",
              hb_staging_insert_workspace_bytes(n), workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  uint8_t* last_writer = static_cast<uint8_t*>(workspace);
  int rc = hb_index_add(h, ids, n, locs_out, last_writer, static_cast<char*>(workspace) + flag_bytes,
                        workspace_bytes - flag_bytes, stream);
  if (rc) return rc;
  return hb_staging_insert_rows(s, emb_rows, row_index, n, cache_rows, row_bytes, locs_out, last_writer, stream);
}

int hb_staging_insert_rows(const hb_staging_t* s, const void* emb_rows, const int64_t* row_index, int64_t n,
                           void* cache_rows, int64_t row_bytes, const int64_t* locs, const uint8_t* last_writer,
                           hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && row_bytes > 0, "hb_staging_insert_rows: bad sizes");
  HB_CHECK_ARG(n == 0 || (emb_rows && cache_rows && locs && last_writer), "hb_staging_insert_rows: null argument");
  if (n == 0) return HB_OK;
  hb_staging_t none;
  memset(&none, 0, sizeof(none));
  const hb_staging_t st_desc = s ? *s : none;
  const int vb = payload_vec_bytes(row_bytes, emb_rows, cache_rows);
  cudaStream_t st = (cudaStream_t)stream;
  if (vb == 16)
    HB_LAUNCH(staging_insert_kernel<16>, warp_grid(n), kBlock, 0, st, st_desc, locs, last_writer,
              (const char*)emb_rows, row_index, (char*)cache_rows, row_bytes, n);
  else if (vb == 4)
    HB_LAUNCH(staging_insert_kernel<4>, warp_grid(n), kBlock, 0, st, st_desc, locs, last_writer,
              (const char*)emb_rows, row_index, (char*)cache_rows, row_bytes, n);
  else
    HB_LAUNCH(staging_insert_kernel<1>, warp_grid(n), kBlock, 0, st, st_desc, locs, last_writer,
              (const char*)emb_rows, row_index, (char*)cache_rows, row_bytes, n);
  return HB_OK;
}

}  // extern "C"
