// An embedding table sharded over the GPUs of one box by owner (row of id lives on rank
// id % world at local row id / world), every shard mapped into every process with CUDA IPC, so
// that a kernel on any GPU reads the authoritative row of any id with plain loads over NVLink.
// This is the forward direction of the owner partitioning: the reference pulls such rows from
// DGL's DistTensor through the host (python/EmbCache/dist_emb.py:241-243) and reads pinned host
// memory from its kernels by unified addressing (src/cuda/uva_fetch.cu:72-106); here the remote
// memory is a peer GPU's HBM.
//
// Loads from a shard are plain ld.global (no multicast, no bulk copies).  Ordering against the
// owners' writes is the caller's: a fence of all ranks between an optimiser update and the next
// read (hb_a2a_fence or any collective on the stream).
#include <cstring>

#include "index.cuh"
#include "launch.cuh"
#include "shard.cuh"

namespace hb {
int* device_error_word();  // runtime.cu

int make_shard_view(const hb_peer_table* t, ShardView* out) {
  memset(out, 0, sizeof(*out));
  out->world = t->world;
  out->num_rows = t->num_rows;
  for (int r = 0; r < t->world; ++r) {
    if (!t->peer[r]) {
      set_error("hb_peer_table: shard of rank %d is not mapped (connect or set_peer first)", r);
      return HB_ERR_INVALID;
    }
    out->p[r] = t->peer[r];
  }
  return HB_OK;
}

namespace {

constexpr int kBlock = 256;

// Copy the rows whose sources the 32 lanes hold (nullptr = none) to out rows base .. base+31,
// 16 bytes per lane and instruction, four rows in flight.
__device__ __forceinline__ void warp_copy_rows16(const char* src, char* out_first, int64_t row_bytes) {
  const int lane = lane_id();
  const unsigned long long src_bits = (unsigned long long)src;
  const unsigned have = __ballot_sync(0xffffffffu, src != nullptr);
  const int64_t vpr = row_bytes >> 4;
  for (int q0 = 0; q0 < 32; q0 += 4) {
    if (((have >> q0) & 0xfu) == 0u) continue;
    const uint4* s[4];
    uint4* d[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q0 + u);
      s[u] = ((have >> (q0 + u)) & 1u) ? reinterpret_cast<const uint4*>(sb) : nullptr;
      d[u] = reinterpret_cast<uint4*>(out_first + (int64_t)(q0 + u) * row_bytes);
    }
    for (int64_t k = lane; k < vpr; k += 32) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s[u]) v[u] = s[u][k];  // plain load: the source may be a peer GPU's memory
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (s[u]) __stcs(d[u] + k, v[u]);
    }
  }
}

// out[i] = cache row of ids[i] when the index holds it, else the authoritative row from the
// owner's shard; slots and found mask as hb_lookup_fetch.
template <int MODE>
__global__ void __launch_bounds__(kBlock, MODE == HB_LOOKUP_SORTED ? 2 : 3) sharded_lookup_fetch_kernel(
    IndexView v, ShardView sh, const int64_t* __restrict__ ids, int64_t n,
    const char* __restrict__ cache_rows, int64_t row_bytes, char* __restrict__ out,
    int64_t* __restrict__ locs, uint8_t* __restrict__ found, int* __restrict__ err) {
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
    if (slot >= 0) src = cache_rows + slot * row_bytes;
    else if (id >= 0 && id < sh.num_rows) src = shard_row(sh, id, row_bytes);
    else if (id >= sh.num_rows) atomicExch(err, HB_ERR_INVALID);  // no such row: the output row stays as it was
    warp_copy_rows16(src, out + base * row_bytes, row_bytes);
  }
}

// out[i] = authoritative row of ids[i] for i < min(n, *n_dev)
__global__ void __launch_bounds__(kBlock) sharded_gather_kernel(
    ShardView sh, const int64_t* __restrict__ ids, int64_t n, const int64_t* __restrict__ n_dev,
    int64_t row_bytes, char* __restrict__ out, int* __restrict__ err) {
  if (n_dev && *n_dev < n) n = *n_dev;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane;
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    if (id >= sh.num_rows) atomicExch(err, HB_ERR_INVALID);  // no such row: the output row stays as it was
    warp_copy_rows16((id >= 0 && id < sh.num_rows) ? shard_row(sh, id, row_bytes) : nullptr,
                     out + base * row_bytes, row_bytes);
  }
}

// The owner's half of a forward fetch in which the owners deliver: requests (id, row of the
// requester's stage) lie in per-requester segments of seg_cap entries (the receive view of an
// hb_a2a exchange: counts[s] valid in segment s); every requested row of this rank's shard is
// stored into the stage of its requester, which this rank has mapped.  Peer STORES run at the
// links' bandwidth where scattered peer LOADS of the same rows do not.  One warp per request and
// step, 4 requests in flight per warp; the warps take the requesters in rotated order.
__global__ void __launch_bounds__(kBlock, 4) fetch_serve_kernel(
    const char* __restrict__ shard, int64_t rows_local, int rank, int world, ShardView stages,
    int64_t stage_rows, const int64_t* __restrict__ req_ids, const int64_t* __restrict__ req_rows,
    const int64_t* __restrict__ counts, int64_t seg_cap, int64_t row_bytes, int* __restrict__ err) {
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  constexpr int kFly = 4;
  const int64_t vpr = row_bytes >> 4;
  for (int j = 0; j < world; ++j) {
    // every warp starts with another requester (and every rank with another one again): all
    // links carry rows all the time, instead of every owner storing into the same GPU first
    const int s = (int)((warp + rank + 1 + j) % world);
    int64_t cnt = counts[s];
    if (cnt > seg_cap) cnt = seg_cap;
    char* stage = const_cast<char*>(stages.p[s]);
    for (int64_t k0 = warp * kFly; k0 < cnt; k0 += nwarps * kFly) {
      const uint4* from[kFly];
      uint4* to[kFly];
#pragma unroll
      for (int x = 0; x < kFly; ++x) {
        from[x] = nullptr;
        to[x] = nullptr;
        if (k0 + x < cnt) {
          const int64_t id = __ldg(req_ids + s * seg_cap + k0 + x);
          const int64_t row = __ldg(req_rows + s * seg_cap + k0 + x);
          const int64_t local = (id - rank) / world;
          const bool ok = id >= 0 && mod_nonneg(id, world) == rank && local < rows_local && row >= 0 &&
                          row < stage_rows;
          if (ok) {
            from[x] = reinterpret_cast<const uint4*>(shard + local * row_bytes);
            to[x] = reinterpret_cast<uint4*>(stage + row * row_bytes);
          } else if (lane == 0) {
            atomicExch(err, HB_ERR_INVALID);  // not this rank's row, or no such row of the stage: skipped
          }
        }
      }
      for (int64_t k = lane; k < vpr; k += 32) {
        uint4 val[kFly];
#pragma unroll
        for (int x = 0; x < kFly; ++x)
          if (from[x]) val[x] = from[x][k];
#pragma unroll
        for (int x = 0; x < kFly; ++x)
          if (from[x]) to[x][k] = val[x];
      }
    }
  }
}

int64_t grid_for(int64_t n) {
  int64_t blocks = ceil_div(ceil_div(n, 32) * 32, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  return blocks > cap ? cap : blocks;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_peer_table_create(int rank, int world, int64_t num_rows, int64_t row_bytes, hb_peer_table_t** out) {
  HB_CHECK_ARG(out && world >= 1 && world <= 64 && rank >= 0 && rank < world, "hb_peer_table_create: bad rank/world");
  HB_CHECK_ARG(num_rows > 0 && row_bytes > 0 && row_bytes % 16 == 0,
               "hb_peer_table_create: rows must be a positive multiple of 16 bytes");
  hb_peer_table_t* t = new hb_peer_table_t();
  memset(t, 0, sizeof(*t));
  t->rank = rank;
  t->world = world;
  t->num_rows = num_rows;
  t->rows_local = (num_rows - rank + world - 1) / world;
  t->row_bytes = row_bytes;
  const size_t bytes = (size_t)(t->rows_local > 0 ? t->rows_local : 1) * row_bytes;
  cudaError_t e = cudaMalloc(&t->local, bytes);
  if (e != cudaSuccess) {
    set_error("hb_peer_table_create: cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    delete t;
    return HB_ERR_CUDA;
  }
  t->peer[rank] = t->local;
  *out = t;
  return HB_OK;
}

size_t hb_peer_table_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int hb_peer_table_export_handle(hb_peer_table_t* t, void* handle_out) {
  HB_CHECK_ARG(t && handle_out, "hb_peer_table_export_handle: null argument");
  cudaIpcMemHandle_t h;
  HB_CUDA(cudaIpcGetMemHandle(&h, t->local));
  memcpy(handle_out, &h, sizeof(h));
  return HB_OK;
}

int hb_peer_table_connect(hb_peer_table_t* t, const void* handles) {
  HB_CHECK_ARG(t && (t->world == 1 || handles), "hb_peer_table_connect: null argument");
  const char* hp = static_cast<const char*>(handles);
  for (int r = 0; r < t->world; ++r) {
    if (r == t->rank || t->peer[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, hp + (size_t)r * sizeof(h), sizeof(h));
    void* ptr = nullptr;
    HB_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    t->peer[r] = static_cast<char*>(ptr);
    t->opened[r] = true;
  }
  return HB_OK;
}

int hb_peer_table_set_peer(hb_peer_table_t* t, int rank, const void* shard_rows) {
  HB_CHECK_ARG(t && rank >= 0 && rank < t->world && rank != t->rank && shard_rows,
               "hb_peer_table_set_peer: bad argument");
  HB_CHECK_ARG(!t->opened[rank], "hb_peer_table_set_peer: rank %d is already mapped", rank);
  t->peer[rank] = static_cast<char*>(const_cast<void*>(shard_rows));
  return HB_OK;
}

int hb_peer_table_local(hb_peer_table_t* t, void** rows, int64_t* rows_local) {
  HB_CHECK_ARG(t != nullptr, "hb_peer_table_local: null table");
  if (rows) *rows = t->local;
  if (rows_local) *rows_local = t->rows_local;
  return HB_OK;
}

// Close this process's mappings of the peers' shards; see hb_a2a_disconnect for the order of
// a tear-down (all ranks disconnect, barrier, all ranks destroy).
int hb_peer_table_disconnect(hb_peer_table_t* t) {
  if (!t) return HB_OK;
  for (int r = 0; r < t->world; ++r) {
    if (!t->opened[r]) continue;
    cudaIpcCloseMemHandle(t->peer[r]);
    t->peer[r] = nullptr;
    t->opened[r] = false;
  }
  return HB_OK;
}

int hb_peer_table_destroy(hb_peer_table_t* t) {
  if (!t) return HB_OK;
  for (int r = 0; r < t->world; ++r)
    if (t->opened[r]) cudaIpcCloseMemHandle(t->peer[r]);
  cudaFree(t->local);
  delete t;
  return HB_OK;
}

int hb_peer_table_gather(hb_peer_table_t* t, const int64_t* ids, int64_t n, const int64_t* n_dev,
                         void* dst, hb_stream_t stream) {
  HB_CHECK_ARG(t && n >= 0, "hb_peer_table_gather: bad argument");
  HB_CHECK_ARG(n == 0 || (ids && dst), "hb_peer_table_gather: null argument");
  HB_CHECK_ARG(((uintptr_t)dst & 15) == 0, "hb_peer_table_gather: dst must be 16-byte aligned");
  if (n == 0) return HB_OK;
  ShardView sv;
  int rc = make_shard_view(t, &sv);
  if (rc != HB_OK) return rc;
  HB_LAUNCH(sharded_gather_kernel, (int)grid_for(n), kBlock, 0, (cudaStream_t)stream, sv, ids, n, n_dev,
            t->row_bytes, (char*)dst, device_error_word());
  return HB_OK;
}

int hb_fetch_serve(hb_peer_table_t* table, hb_peer_table_t* stages, const int64_t* req_ids,
                   const int64_t* req_rows, const int64_t* req_counts, int64_t seg_cap, hb_stream_t stream) {
  HB_CHECK_ARG(table && stages && req_ids && req_rows && req_counts && seg_cap > 0, "hb_fetch_serve: null argument");
  HB_CHECK_ARG(table->world == stages->world && table->rank == stages->rank,
               "hb_fetch_serve: table and stages belong to different groups");
  HB_CHECK_ARG(table->row_bytes == stages->row_bytes, "hb_fetch_serve: row sizes differ");
  ShardView sv;
  int rc = make_shard_view(stages, &sv);
  if (rc != HB_OK) return rc;
  // every rank's stage has the rows of the shortest one
  const int64_t stage_rows = stages->num_rows / stages->world;
  HB_LAUNCH(fetch_serve_kernel, sm_count() * 4, kBlock, 0, (cudaStream_t)stream, (const char*)table->local,
            table->rows_local, table->rank, table->world, sv, stage_rows, req_ids, req_rows, req_counts, seg_cap,
            table->row_bytes, device_error_word());
  return HB_OK;
}

int hb_lookup_fetch_sharded(hb_index_t* h, const int64_t* ids, int64_t n, const void* cache_rows,
                            hb_peer_table_t* table, void* out_rows, int64_t* locs, uint8_t* found,
                            int mode, hb_stream_t stream) {
  HB_CHECK_ARG(h && table && n >= 0, "hb_lookup_fetch_sharded: bad argument");
  HB_CHECK_ARG(n == 0 || (ids && cache_rows && out_rows), "hb_lookup_fetch_sharded: null argument");
  HB_CHECK_ARG(mode == HB_LOOKUP_SETASSOC || mode == HB_LOOKUP_SORTED,
               "hb_lookup_fetch_sharded: unknown mode %d", mode);
  HB_CHECK_ARG((((uintptr_t)cache_rows | (uintptr_t)out_rows) & 15) == 0,
               "hb_lookup_fetch_sharded: buffers must be 16-byte aligned");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == HB_LOOKUP_SORTED && h->sorted_stale) {
    int rc = hb_index_build_sorted(h, stream);
    if (rc != HB_OK) return rc;
  }
  ShardView sv;
  int rc = make_shard_view(table, &sv);
  if (rc != HB_OK) return rc;
  if (mode == HB_LOOKUP_SORTED)
    HB_LAUNCH(sharded_lookup_fetch_kernel<HB_LOOKUP_SORTED>, (int)grid_for(n), kBlock, 0, st, h->view, sv,
              ids, n, (const char*)cache_rows, table->row_bytes, (char*)out_rows, locs, found, device_error_word());
  else
    HB_LAUNCH(sharded_lookup_fetch_kernel<HB_LOOKUP_SETASSOC>, (int)grid_for(n), kBlock, 0, st, h->view, sv,
              ids, n, (const char*)cache_rows, table->row_bytes, (char*)out_rows, locs, found, device_error_word());
  return HB_OK;
}

}  // extern "C"
