// Cache index in HBM: create/destroy, add, lookup, LRU touch, reset, getall,
// sorted-view build, raw export/import.  Semantics follow the reference's
// SACacheIndex (src/cache/cache.h) and cache_line (src/cache/cache_line.h);
// the data structures and kernels are new.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>
#include <cub/iterator/counting_input_iterator.cuh>

#include "index.cuh"
#include "launch.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;

__global__ void fill_i64_kernel(int64_t* p, int64_t n, int64_t v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

__global__ void fill_i32_kernel(int32_t* p, int64_t n, int32_t v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// ---- add ---------------------------------------------------------------------
// key = set of the id (or `lines` for an unusable id), value = position in batch.
__global__ void add_keys_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t lines,
                                uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t id = ids[i];
  keys[i] = id >= 0 ? (uint32_t)mod_nonneg(id, lines) : (uint32_t)lines;
  vals[i] = (uint32_t)i;
}

// One thread per set that appears in the batch: it owns the line, applies the
// batch's ids for that set in input order (keys were stably sorted, so vals are
// ascending inside a set).  Placement policy: src/cache/cache.h:51-88 with
// find_or_empty_entry (cache_line.h:67-78) and find_lru (cache_line.h:92-103).
__global__ void add_walk_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t lines,
                                const uint32_t* __restrict__ keys,
                                const uint32_t* __restrict__ vals, int64_t* __restrict__ line_ids,
                                int32_t* __restrict__ lru, int64_t* __restrict__ locs,
                                uint8_t* __restrict__ last_writer) {
  const int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (j >= n) return;
  const uint32_t line = keys[j];
  if ((int64_t)line >= lines) {              // unusable ids (negative: padding) sort last
    locs[vals[j]] = -1;                      // every thread answers for its own entry
    if (last_writer) last_writer[vals[j]] = 0;
    return;
  }
  if (j > 0 && keys[j - 1] == line) return;  // not the head of its segment
  int64_t last_k[kWays];  // sorted position of the last id of the batch placed in each way
#pragma unroll
  for (int w = 0; w < kWays; ++w) last_k[w] = -1;
  int64_t lid[kWays];
  int32_t cnt[kWays];
#pragma unroll
  for (int w = 0; w < kWays; ++w) {
    lid[w] = line_ids[(int64_t)line * kWays + w];
    cnt[w] = lru[(int64_t)line * kWays + w];
  }
  for (int64_t k = j; k < n && keys[k] == line; ++k) {
    const uint32_t pos = vals[k];
    const int64_t id = ids[pos];
    int way = -1;
    bool exists = false;
#pragma unroll
    for (int w = 0; w < kWays; ++w) {
      if (!exists) {
        if (lid[w] == id) { way = w; exists = true; }
        else if (lid[w] == -1) way = w;  // keeps the LAST empty way
      }
    }
    if (way < 0) {
      // no empty way: least recently used = largest non-zero counter, first on ties
      int best = 0;
      int32_t tmp = cnt[0];
#pragma unroll
      for (int w = 0; w < kWays; ++w) {
        if (cnt[w] > tmp && cnt[w] != 0) { best = w; tmp = cnt[w]; }
      }
      way = tmp == 0 ? -1 : best;
    }
    if (way >= 0) {
      if (!exists) {
#pragma unroll
        for (int w = 0; w < kWays; ++w) {
          if (w == way) { lid[w] = id; cnt[w] = 0; }  // set_id zeroes the counter
        }
      }
      locs[pos] = (int64_t)line * kWays + way;
#pragma unroll
      for (int w = 0; w < kWays; ++w)
        if (w == way) last_k[w] = k;
    } else {
      locs[pos] = -1;
    }
  }
#pragma unroll
  for (int w = 0; w < kWays; ++w) {
    line_ids[(int64_t)line * kWays + w] = lid[w];
    lru[(int64_t)line * kWays + w] = cnt[w];
  }
  if (last_writer) {
    for (int64_t k = j; k < n && keys[k] == line; ++k) {
      const uint32_t pos = vals[k];
      const int64_t loc = locs[pos];
      bool last = false;
      if (loc >= 0) {
        const int way = (int)(loc & (kWays - 1));
#pragma unroll
        for (int w = 0; w < kWays; ++w)
          if (w == way) last = last_k[w] == k;
      }
      last_writer[pos] = last;
    }
  }
}

// ---- lookup ------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(kBlock) lookup_kernel(IndexView v, const int64_t* __restrict__ ids,
                                                         int64_t n, int64_t* __restrict__ locs,
                                                         uint8_t* __restrict__ found) {
  __shared__ int64_t s_top[MODE == HB_LOOKUP_SORTED ? kTopMax : 1];
  if (MODE == HB_LOOKUP_SORTED) {
    stage_top_level(v, s_top);
    __syncthreads();
  }
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = warp * 32; base < n; base += nwarps * 32) {
    const int64_t i = base + lane_id();
    const int64_t id = i < n ? __ldg(ids + i) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    if (i < n) {
      if (locs) locs[i] = slot;
      if (found) found[i] = slot >= 0;
    }
  }
}

// ---- LRU touch ---------------------------------------------------------------
__global__ void touch_keys_kernel(const int64_t* __restrict__ locs, int64_t n, int64_t capacity,
                                  uint32_t* __restrict__ keys, uint32_t* __restrict__ vals) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t s = locs[i];
  keys[i] = (s >= 0 && s < capacity) ? (uint32_t)s : (uint32_t)capacity;
  vals[i] = (uint32_t)i;
}

__device__ __forceinline__ int64_t lower_bound_u32(const uint32_t* a, int64_t lo, int64_t hi,
                                                   uint32_t key) {
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (a[mid] < key) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// keys = hit slots sorted ascending (stable, so batch positions ascend inside a
// slot).  The thread at the head of each line's segment computes the counters
// that the sequential rule "all counters of the line += 1, hit way = 0"
// (cache_line.h:80-86) leaves after the whole batch:
//   way hit in the batch   -> number of hits on the line after its last hit
//   way not hit            -> old counter + hits on the line
__global__ void touch_apply_kernel(const uint32_t* __restrict__ keys,
                                   const uint32_t* __restrict__ vals, int64_t n, int64_t capacity,
                                   int32_t* __restrict__ lru) {
  const int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (j >= n) return;
  const uint32_t key = keys[j];
  if ((int64_t)key >= capacity) return;  // misses sort last
  const uint32_t line = key >> 3;
  if (j > 0 && (keys[j - 1] >> 3) == line) return;
  // run boundaries of the 8 ways inside this line's segment
  int64_t rb[kWays + 1];
  rb[0] = j;
  // first position whose key belongs to a later line (or a miss)
  int64_t seg_hi = n;
  {
    // gallop to bound the binary search by the segment length, not by n
    int64_t step = 8;
    int64_t hi = j + 1;
    const uint32_t next = (line + 1) << 3;
    while (hi < n && keys[hi] < next) { hi = (hi + step < n) ? hi + step : n; step <<= 1; }
    seg_hi = lower_bound_u32(keys, j, hi, next);
  }
#pragma unroll
  for (int w = 1; w < kWays; ++w) rb[w] = lower_bound_u32(keys, rb[w - 1], seg_hi, (line << 3) + w);
  rb[kWays] = seg_hi;
  const int32_t total = (int32_t)(seg_hi - j);
#pragma unroll
  for (int w = 0; w < kWays; ++w) {
    int32_t* c = lru + (int64_t)line * kWays + w;
    if (rb[w + 1] == rb[w]) {
      *c += total;
    } else {
      const uint32_t last = vals[rb[w + 1] - 1];
      int32_t after = 0;
#pragma unroll
      for (int x = 0; x < kWays; ++x) {
        if (x == w || rb[x + 1] == rb[x]) continue;
        // positions in run x greater than `last`
        int64_t lo = rb[x], hi = rb[x + 1];
        while (lo < hi) {
          const int64_t mid = (lo + hi) >> 1;
          if (vals[mid] <= last) lo = mid + 1; else hi = mid;
        }
        after += (int32_t)(rb[x + 1] - lo);
      }
      *c = after;
    }
  }
}

// ---- LRU touch from runs -------------------------------------------------------
// The batch is given as runs of equal ids (each run = the sorted batch positions
// of one id, ascending), so no sort is needed: a first kernel notes which run hit
// each slot, a second computes per hit slot the same closed form as above, with
// "hits on the line after my last hit" counted by binary search in the position
// lists of the other hit ways of the line.
struct RunsView {
  const int64_t* locs;       // slot of every batch position (or of every sorted entry, see below)
  const uint32_t* perm;      // nullable: position list of the runs (identity when null)
  const int64_t* run_start;  // nullable: run u = [run_start[u], run_start[u+1]) (run u = {u} when null)
  const int64_t* num_runs;   // nullable device count
  const int64_t* n_dev;      // nullable device count of positions
  int64_t max_runs;
  int64_t n;
  int locs_kind;             // locs holds a slot per batch position (0), per sorted entry (1), per run (2)
  __device__ __forceinline__ int64_t slot_of_run(int64_t u) const {
    if (locs_kind == 2) return locs[u];
    const int64_t j = start(u);
    return locs[locs_kind == 1 ? j : pos(j)];
  }
  __device__ __forceinline__ int64_t positions() const {
    if (!n_dev) return n;
    const int64_t d = *n_dev;
    return d < n ? (d > 0 ? d : 0) : n;
  }
  __device__ __forceinline__ int64_t runs() const {
    int64_t r = max_runs;
    if (num_runs && *num_runs < r) r = *num_runs;
    if (!run_start) { const int64_t p = positions(); if (p < r) r = p; }
    return r;
  }
  __device__ __forceinline__ int64_t start(int64_t u) const { return run_start ? run_start[u] : u; }
  __device__ __forceinline__ int64_t end(int64_t u, int64_t nruns, int64_t npos) const {
    return (u + 1 < nruns) ? start(u + 1) : npos;
  }
  __device__ __forceinline__ int64_t pos(int64_t j) const { return perm ? (int64_t)perm[j] : j; }
};

// The batch number lives on the device and is advanced by a kernel, so that a
// captured CUDA graph that contains the ageing can be replayed.
__global__ void touch_runs_next_epoch_kernel(int32_t* epoch) { *epoch += 1; }

__global__ void touch_runs_mark_kernel(RunsView v, int64_t capacity, const int32_t* epoch_dev,
                                       int32_t* __restrict__ slot_run,
                                       int32_t* __restrict__ slot_epoch) {
  const int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (u >= v.runs()) return;
  const int32_t epoch = *epoch_dev;
  const int64_t slot = v.slot_of_run(u);
  if (slot < 0 || slot >= capacity) return;
  slot_run[slot] = (int32_t)u;
  slot_epoch[slot] = epoch;
}

__global__ void touch_runs_apply_kernel(RunsView v, int64_t capacity, const int32_t* epoch_dev,
                                        const int32_t* __restrict__ slot_run,
                                        const int32_t* __restrict__ slot_epoch,
                                        int32_t* __restrict__ lru) {
  const int64_t u = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t nruns = v.runs();
  if (u >= nruns) return;
  const int32_t epoch = *epoch_dev;
  const int64_t npos = v.positions();
  const int64_t slot = v.slot_of_run(u);
  if (slot < 0 || slot >= capacity) return;
  const int64_t line = slot >> 3;
  const int way = (int)(slot & 7);
  const int64_t last = v.pos(v.end(u, nruns, npos) - 1);
  int32_t total = 0, after = 0;
  bool leader = true;
  bool hit[kWays];
#pragma unroll
  for (int w = 0; w < kWays; ++w) {
    hit[w] = slot_epoch[line * kWays + w] == epoch;
    if (!hit[w]) continue;
    const int64_t u2 = slot_run[line * kWays + w];
    const int64_t s2 = v.start(u2), e2 = v.end(u2, nruns, npos);
    total += (int32_t)(e2 - s2);
    if (w < way) leader = false;
    if (w != way) {
      int64_t lo = s2, hi = e2;  // first position of the run greater than `last`
      while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        if (v.pos(mid) <= last) lo = mid + 1; else hi = mid;
      }
      after += (int32_t)(e2 - lo);
    }
  }
  lru[slot] = after;
  if (leader) {
#pragma unroll
    for (int w = 0; w < kWays; ++w)
      if (!hit[w]) lru[line * kWays + w] += total;
  }
}

// ---- reset -------------------------------------------------------------------
__global__ void reset_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t lines,
                             int64_t* __restrict__ line_ids, int32_t* __restrict__ lru) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t id = ids[i];
  if (id < 0) return;
  const int64_t line = mod_nonneg(id, lines);
#pragma unroll
  for (int w = 0; w < kWays; ++w) {
    if (line_ids[line * kWays + w] == id) {
      line_ids[line * kWays + w] = -1;  // set_id(way, -1) also zeroes the counter
      lru[line * kWays + w] = 0;
      break;
    }
  }
}

// ---- enumerate / sorted view -------------------------------------------------
struct SlotValid {
  const int64_t* line_ids;
  __device__ bool operator()(int64_t slot) const { return line_ids[slot] != -1; }
};

__global__ void gather_ids_kernel(const int64_t* __restrict__ line_ids,
                                  const int64_t* __restrict__ slots, int64_t n,
                                  int64_t* __restrict__ ids_out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i < n) ids_out[i] = line_ids[slots[i]];
}

__global__ void write_pairs_kernel(const int64_t* __restrict__ ids, const int64_t* __restrict__ slots,
                                   int64_t n, int64_t n_pad, longlong2* __restrict__ pairs) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n_pad) return;
  pairs[i] = i < n ? make_longlong2(ids[i], slots[i]) : make_longlong2(INT64_MAX, -1);
}

// level 1 samples the pairs with stride 8, higher levels sample the level below
// with stride 16
__global__ void build_level1_kernel(const longlong2* __restrict__ pairs, int64_t len,
                                    int64_t len_pad, int64_t* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= len_pad) return;
  out[i] = i < len ? pairs[i * kLeafFan].x : INT64_MAX;
}

__global__ void build_level_kernel(const int64_t* __restrict__ below, int64_t len, int64_t len_pad,
                                   int64_t* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= len_pad) return;
  out[i] = i < len ? below[i * kNodeFan] : INT64_MAX;
}

__global__ void count_valid_kernel(const int64_t* __restrict__ line_ids, int64_t n,
                                   unsigned long long* __restrict__ out) {
  unsigned long long c = 0;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    c += line_ids[i] != -1;
  for (int o = 16; o > 0; o >>= 1) c += __shfl_down_sync(0xffffffffu, c, o);
  if (lane_id() == 0 && c) atomicAdd(out, c);
}

int grid_for(int64_t n, int block = kBlock) {
  int64_t g = ceil_div(n, block);
  if (g < 1) g = 1;
  return (int)g;
}

int grid_capped(int64_t n, int block = kBlock) {
  int64_t g = ceil_div(n, block);
  const int64_t cap = (int64_t)sm_count() * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

int sort_bits(int64_t max_key_exclusive) {
  int b = 1;
  while (b < 32 && ((int64_t)1 << b) < max_key_exclusive) ++b;
  return b;
}

size_t pair_sort_temp_bytes(int64_t n) {
  size_t bytes = 0;
  cub::DoubleBuffer<uint32_t> k(nullptr, nullptr), v(nullptr, nullptr);
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, k, v, (int)n, 0, 32, (cudaStream_t)0);
  return bytes;
}

}  // namespace

// workspace layout shared by add and touch_lru: 2x keys, 2x vals, cub temp
static size_t keyval_workspace_bytes(int64_t n) {
  if (n <= 0) return 256;
  size_t per = align_up((size_t)n * sizeof(uint32_t), 256);
  return 4 * per + align_up(pair_sort_temp_bytes(n), 256) + 256;
}

}  // namespace hb

using namespace hb;

extern "C" {

namespace {
// everything of an index except its lines: the sorted view's storage and the scratch word
int alloc_derived(hb_index_t* h) {
  const int64_t cap = h->cache_size;
  HB_CUDA(cudaMalloc(&h->pairs, (cap + kLeafFan) * sizeof(longlong2)));
  HB_CUDA(cudaMalloc(&h->scratch_count, 4 * sizeof(int64_t)));
  // level capacities for a full index
  int64_t len = h->lines;  // level 1: one id per leaf block
  int64_t total = 0;
  for (int l = 1; l < kMaxLevels; ++l) {
    h->level_off[l] = total;
    h->level_cap[l] = len + kNodeFan;
    total += align_up(h->level_cap[l], 32);
    len = ceil_div(len, kNodeFan);
  }
  HB_CUDA(cudaMalloc(&h->level_store, total * sizeof(int64_t)));
  h->sorted_stale = true;
  h->view.line_ids = h->line_ids;
  h->view.lines = h->lines;
  h->view.pairs = h->pairs;
  h->view.top = 0;
  return HB_OK;
}

struct IndexIpcHandle {
  int64_t cache_size;
  int64_t lines;
  cudaIpcMemHandle_t line_ids;
  cudaIpcMemHandle_t lru;
};
}  // namespace

int hb_index_create(int64_t cache_size, hb_index_t** out) {
  HB_CHECK_ARG(out != nullptr, "hb_index_create: out is null");
  HB_CHECK_ARG(cache_size > 0, "hb_index_create: cache_size must be positive");
  const int64_t lines = ceil_div(cache_size, kWays);
  HB_CHECK_ARG(lines <= ((int64_t)1 << 28), "hb_index_create: at most 2^31 slots are supported");
  hb_index_t* h = new hb_index_t();
  memset(h, 0, sizeof(*h));
  HB_CUDA(cudaGetDevice(&h->device));
  h->lines = lines;
  h->cache_size = lines * kWays;
  const int64_t cap = h->cache_size;
  HB_CUDA(cudaMalloc(&h->line_ids, cap * sizeof(int64_t)));
  HB_CUDA(cudaMalloc(&h->lru, cap * sizeof(int32_t)));
  int rc = alloc_derived(h);
  if (rc != HB_OK) return rc;
  HB_LAUNCH(fill_i64_kernel, grid_capped(cap), kBlock, 0, 0, h->line_ids, cap, (int64_t)-1);
  HB_LAUNCH(fill_i32_kernel, grid_capped(cap), kBlock, 0, 0, h->lru, cap, 0);
  HB_CUDA(cudaStreamSynchronize(0));
  *out = h;
  return HB_OK;
}

// An index shared between the processes of one box, as the reference shares its index through
// a named POSIX segment (SACacheIndex(name, create, ...), src/cache/cache.h:145-167): the
// creating process exports a handle, another process opens it and works on the SAME lines
// (ids and LRU counters) in the creator's HBM.  As in the reference nothing orders the two
// processes' calls: callers do (its test does with barriers, test/test_cache.py:20-55).
size_t hb_index_handle_bytes(void) { return sizeof(IndexIpcHandle); }

int hb_index_export_handle(hb_index_t* h, void* handle_out) {
  HB_CHECK_ARG(h && handle_out, "hb_index_export_handle: null argument");
  HB_CHECK_ARG(!h->opened, "hb_index_export_handle: only the creating process exports");
  IndexIpcHandle x;
  memset(&x, 0, sizeof(x));
  x.cache_size = h->cache_size;
  x.lines = h->lines;
  HB_CUDA(cudaIpcGetMemHandle(&x.line_ids, h->line_ids));
  HB_CUDA(cudaIpcGetMemHandle(&x.lru, h->lru));
  memcpy(handle_out, &x, sizeof(x));
  return HB_OK;
}

int hb_index_open(const void* handle, hb_index_t** out) {
  HB_CHECK_ARG(handle && out, "hb_index_open: null argument");
  IndexIpcHandle x;
  memcpy(&x, handle, sizeof(x));
  HB_CHECK_ARG(x.lines > 0 && x.cache_size == x.lines * kWays, "hb_index_open: not an index handle");
  hb_index_t* h = new hb_index_t();
  memset(h, 0, sizeof(*h));
  HB_CUDA(cudaGetDevice(&h->device));
  h->lines = x.lines;
  h->cache_size = x.cache_size;
  h->shared = true;
  h->opened = true;
  void* p = nullptr;
  HB_CUDA(cudaIpcOpenMemHandle(&p, x.line_ids, cudaIpcMemLazyEnablePeerAccess));
  h->line_ids = static_cast<int64_t*>(p);
  HB_CUDA(cudaIpcOpenMemHandle(&p, x.lru, cudaIpcMemLazyEnablePeerAccess));
  h->lru = static_cast<int32_t*>(p);
  int rc = alloc_derived(h);
  if (rc != HB_OK) return rc;
  *out = h;
  return HB_OK;
}

int hb_index_destroy(hb_index_t* h) {
  if (!h) return HB_OK;
  if (h->opened) {
    cudaIpcCloseMemHandle(h->line_ids);
    cudaIpcCloseMemHandle(h->lru);
  } else {
    cudaFree(h->line_ids);
    cudaFree(h->lru);
  }
  cudaFree(h->pairs);
  cudaFree(h->level_store);
  cudaFree(h->scratch_count);
  cudaFree(h->slot_run);
  cudaFree(h->slot_epoch);
  delete h;
  return HB_OK;
}

int64_t hb_index_size(const hb_index_t* h) { return h ? h->cache_size : -1; }
int64_t hb_index_capacity(const hb_index_t* h) { return h ? h->lines * kWays : -1; }
// bytes of one reference cache line: 8 int64 ids + 8 int32 counters
int64_t hb_index_space(const hb_index_t* h) { return h ? h->lines * 96 : -1; }
int64_t hb_index_lines(const hb_index_t* h) { return h ? h->lines : -1; }

int hb_index_valid_entries(hb_index_t* h, int64_t* out_host, hb_stream_t stream) {
  HB_CHECK_ARG(h && out_host, "hb_index_valid_entries: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  HB_CUDA(cudaMemsetAsync(h->scratch_count, 0, sizeof(int64_t), st));
  HB_LAUNCH(count_valid_kernel, grid_capped(h->cache_size), kBlock, 0, st, h->line_ids,
            h->cache_size, (unsigned long long*)h->scratch_count);
  HB_CUDA(cudaMemcpyAsync(out_host, h->scratch_count, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
  HB_CUDA(cudaStreamSynchronize(st));
  return HB_OK;
}

size_t hb_index_add_workspace_bytes(int64_t n) { return keyval_workspace_bytes(n); }
size_t hb_index_touch_lru_workspace_bytes(int64_t n) { return keyval_workspace_bytes(n); }

int hb_index_add(hb_index_t* h, const int64_t* ids, int64_t n, int64_t* locs,
                 uint8_t* last_writer, void* workspace, size_t workspace_bytes,
                 hb_stream_t stream) {
  HB_CHECK_ARG(h && (n == 0 || (ids && locs)), "hb_index_add: null argument");
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31), "hb_index_add: n out of range");
  if (n == 0) return HB_OK;
  if (workspace_bytes < keyval_workspace_bytes(n) || !workspace) {
    set_error("hb_index_add: workspace of %zu bytes needed, %zu given", keyval_workspace_bytes(n),
              workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  Carver cv(workspace);
  uint32_t* k0 = cv.take<uint32_t>(n);
  uint32_t* k1 = cv.take<uint32_t>(n);
  uint32_t* v0 = cv.take<uint32_t>(n);
  uint32_t* v1 = cv.take<uint32_t>(n);
  size_t temp_bytes = pair_sort_temp_bytes(n);
  void* temp = cv.take<char>(temp_bytes);
  HB_LAUNCH(add_keys_kernel, grid_for(n), kBlock, 0, st, ids, n, h->lines, k0, v0);
  cub::DoubleBuffer<uint32_t> keys(k0, k1), vals(v0, v1);
  HB_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys, vals, (int)n, 0,
                                          sort_bits(h->lines + 1), st));
  count_library_launches(3);
  HB_LAUNCH(add_walk_kernel, grid_for(n), kBlock, 0, st, ids, n, h->lines, keys.Current(),
            vals.Current(), h->line_ids, h->lru, locs, last_writer);
  h->sorted_stale = true;
  return HB_OK;
}

int hb_index_touch_lru(hb_index_t* h, const int64_t* locs, int64_t n, void* workspace,
                       size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(h && (n == 0 || locs), "hb_index_touch_lru: null argument");
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31), "hb_index_touch_lru: n out of range");
  if (n == 0) return HB_OK;
  if (workspace_bytes < keyval_workspace_bytes(n) || !workspace) {
    set_error("hb_index_touch_lru: workspace of %zu bytes needed, %zu given",
              keyval_workspace_bytes(n), workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  Carver cv(workspace);
  uint32_t* k0 = cv.take<uint32_t>(n);
  uint32_t* k1 = cv.take<uint32_t>(n);
  uint32_t* v0 = cv.take<uint32_t>(n);
  uint32_t* v1 = cv.take<uint32_t>(n);
  size_t temp_bytes = pair_sort_temp_bytes(n);
  void* temp = cv.take<char>(temp_bytes);
  HB_LAUNCH(touch_keys_kernel, grid_for(n), kBlock, 0, st, locs, n, h->cache_size, k0, v0);
  cub::DoubleBuffer<uint32_t> keys(k0, k1), vals(v0, v1);
  HB_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, keys, vals, (int)n, 0,
                                          sort_bits(h->cache_size + 1), st));
  count_library_launches(3);
  HB_LAUNCH(touch_apply_kernel, grid_for(n), kBlock, 0, st, keys.Current(), vals.Current(), n,
            h->cache_size, h->lru);
  return HB_OK;
}

int hb_index_touch_lru_runs(hb_index_t* h, const int64_t* locs, const uint32_t* perm,
                            const int64_t* run_start, int64_t max_runs, const int64_t* num_runs,
                            int64_t n, const int64_t* n_dev, int locs_kind, hb_stream_t stream) {
  HB_CHECK_ARG(h && (n == 0 || locs), "hb_index_touch_lru_runs: null argument");
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31) && max_runs >= 0 && max_runs <= n,
               "hb_index_touch_lru_runs: sizes out of range");
  HB_CHECK_ARG(!(perm && !run_start), "hb_index_touch_lru_runs: a position list needs run starts");
  HB_CHECK_ARG(locs_kind >= 0 && locs_kind <= 2, "hb_index_touch_lru_runs: locs_kind is 0, 1 or 2");
  if (n == 0 || max_runs == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t cap = h->cache_size;
  if (!h->slot_run) {
    // first use (do it outside any stream capture): marks start at batch 0, the counter at 0
    HB_CUDA(cudaMalloc(&h->slot_run, cap * sizeof(int32_t)));
    HB_CUDA(cudaMalloc(&h->slot_epoch, (cap + 1) * sizeof(int32_t)));
    HB_CUDA(cudaMemsetAsync(h->slot_epoch, 0, (cap + 1) * sizeof(int32_t), st));
  }
  int32_t* epoch_dev = h->slot_epoch + cap;  // the batch counter sits after the marks
  RunsView v{locs, perm, run_start, num_runs, n_dev, max_runs, n, locs_kind};
  HB_LAUNCH(touch_runs_next_epoch_kernel, 1, 1, 0, st, epoch_dev);
  HB_LAUNCH(touch_runs_mark_kernel, grid_for(max_runs), kBlock, 0, st, v, cap, epoch_dev, h->slot_run,
            h->slot_epoch);
  HB_LAUNCH(touch_runs_apply_kernel, grid_for(max_runs), kBlock, 0, st, v, cap, epoch_dev,
            h->slot_run, h->slot_epoch, h->lru);
  return HB_OK;
}

int hb_index_lookup(hb_index_t* h, const int64_t* ids, int64_t n, int64_t* locs, uint8_t* found,
                    int mode, hb_stream_t stream) {
  HB_CHECK_ARG(h && (n == 0 || ids), "hb_index_lookup: null argument");
  HB_CHECK_ARG(mode == HB_LOOKUP_SETASSOC || mode == HB_LOOKUP_SORTED,
               "hb_index_lookup: unknown mode %d", mode);
  HB_CHECK_ARG(n >= 0, "hb_index_lookup: negative n");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_capped(n);
  if (mode == HB_LOOKUP_SORTED) {
    if (h->sorted_stale) {
      int rc = hb_index_build_sorted(h, stream);
      if (rc != HB_OK) return rc;
    }
    HB_LAUNCH(lookup_kernel<HB_LOOKUP_SORTED>, grid, kBlock, 0, st, h->view, ids, n, locs, found);
  } else {
    HB_LAUNCH(lookup_kernel<HB_LOOKUP_SETASSOC>, grid, kBlock, 0, st, h->view, ids, n, locs, found);
  }
  return HB_OK;
}

int hb_index_reset(hb_index_t* h, const int64_t* ids, int64_t n, hb_stream_t stream) {
  HB_CHECK_ARG(h && (n == 0 || ids), "hb_index_reset: null argument");
  if (n <= 0) return HB_OK;
  HB_LAUNCH(reset_kernel, grid_for(n), kBlock, 0, (cudaStream_t)stream, ids, n, h->lines,
            h->line_ids, h->lru);
  h->sorted_stale = true;
  return HB_OK;
}

// Select the valid slots (ascending) into a fresh device buffer; returns their
// count on the host.  Setup path: allocates and synchronises.
static int select_valid_slots(hb_index_t* h, cudaStream_t st, int64_t** slots_out,
                              int64_t* count_host) {
  const int64_t cap = h->cache_size;
  int64_t* slots = nullptr;
  HB_CUDA(cudaMalloc(&slots, cap * sizeof(int64_t)));
  cub::CountingInputIterator<int64_t> it(0);
  SlotValid pred{h->line_ids};
  size_t temp_bytes = 0;
  cub::DeviceSelect::If(nullptr, temp_bytes, it, slots, h->scratch_count, cap, pred, st);
  void* temp = nullptr;
  HB_CUDA(cudaMalloc(&temp, temp_bytes ? temp_bytes : 1));
  cudaError_t e = cub::DeviceSelect::If(temp, temp_bytes, it, slots, h->scratch_count, cap, pred, st);
  count_library_launches(2);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(count_host, h->scratch_count, sizeof(int64_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(temp);
  if (e != cudaSuccess) {
    cudaFree(slots);
    set_error("select_valid_slots: %s", cudaGetErrorString(e));
    return HB_ERR_CUDA;
  }
  *slots_out = slots;
  return HB_OK;
}

int hb_index_getall(hb_index_t* h, int64_t* ids_out, int64_t* locs_out, int64_t len,
                    int64_t* n_written_host, hb_stream_t stream) {
  HB_CHECK_ARG(h && len >= 0, "hb_index_getall: bad argument");
  HB_CHECK_ARG(len == 0 || (ids_out && locs_out), "hb_index_getall: null output");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t* slots = nullptr;
  int64_t valid = 0;
  int rc = select_valid_slots(h, st, &slots, &valid);
  if (rc != HB_OK) return rc;
  const int64_t m = valid < len ? valid : len;
  cudaError_t e = cudaSuccess;
  if (m > 0) {
    e = cudaMemcpyAsync(locs_out, slots, m * sizeof(int64_t), cudaMemcpyDeviceToDevice, st);
    if (e == cudaSuccess) {
      gather_ids_kernel<<<grid_for(m), kBlock, 0, st>>>(h->line_ids, slots, m, ids_out);
      count_launch();
      e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  }
  cudaFree(slots);
  if (e != cudaSuccess) {
    set_error("hb_index_getall: %s", cudaGetErrorString(e));
    return HB_ERR_CUDA;
  }
  if (n_written_host) *n_written_host = m;
  return HB_OK;
}

int hb_index_build_sorted(hb_index_t* h, hb_stream_t stream) {
  HB_CHECK_ARG(h, "hb_index_build_sorted: null index");
  cudaStream_t st = (cudaStream_t)stream;
  int64_t* slots = nullptr;
  int64_t valid = 0;
  int rc = select_valid_slots(h, st, &slots, &valid);
  if (rc != HB_OK) return rc;
  IndexView& v = h->view;
  v.line_ids = h->line_ids;
  v.lines = h->lines;
  v.pairs = h->pairs;
  for (int l = 0; l < kMaxLevels; ++l) { v.level[l] = nullptr; v.level_len[l] = 0; }
  v.top = 0;
  cudaError_t e = cudaSuccess;
  int64_t *ids = nullptr, *ids_sorted = nullptr, *slots_sorted = nullptr;
  void* temp = nullptr;
  if (valid > 0) {
    do {
      if ((e = cudaMalloc(&ids, valid * sizeof(int64_t))) != cudaSuccess) break;
      if ((e = cudaMalloc(&ids_sorted, valid * sizeof(int64_t))) != cudaSuccess) break;
      if ((e = cudaMalloc(&slots_sorted, valid * sizeof(int64_t))) != cudaSuccess) break;
      gather_ids_kernel<<<grid_for(valid), kBlock, 0, st>>>(h->line_ids, slots, valid, ids);
      count_launch();
      size_t temp_bytes = 0;
      cub::DeviceRadixSort::SortPairs(nullptr, temp_bytes, ids, ids_sorted, slots, slots_sorted,
                                      (int)valid, 0, 64, st);
      if ((e = cudaMalloc(&temp, temp_bytes ? temp_bytes : 1)) != cudaSuccess) break;
      if ((e = cub::DeviceRadixSort::SortPairs(temp, temp_bytes, ids, ids_sorted, slots,
                                               slots_sorted, (int)valid, 0, 64, st)) != cudaSuccess)
        break;
      count_library_launches(9);
      const int64_t n_pad = align_up(valid, kLeafFan);
      write_pairs_kernel<<<grid_for(n_pad), kBlock, 0, st>>>(ids_sorted, slots_sorted, valid, n_pad,
                                                             h->pairs);
      count_launch();
      v.level_len[0] = (int32_t)valid;
      int64_t len = n_pad / kLeafFan;
      for (int l = 1; l < kMaxLevels; ++l) {
        int64_t* out = h->level_store + h->level_off[l];
        const int64_t len_pad = align_up(len, kNodeFan);
        if (l == 1)
          build_level1_kernel<<<grid_for(len_pad), kBlock, 0, st>>>(h->pairs, len, len_pad, out);
        else
          build_level_kernel<<<grid_for(len_pad), kBlock, 0, st>>>(
              h->level_store + h->level_off[l - 1], len, len_pad, out);
        count_launch();
        v.level[l] = out;
        v.level_len[l] = (int32_t)len;
        if (len <= kTopMax) { v.top = l; break; }
        len = ceil_div(len, kNodeFan);
      }
      if ((e = cudaGetLastError()) != cudaSuccess) break;
      e = cudaStreamSynchronize(st);
    } while (0);
  }
  cudaFree(slots);
  cudaFree(ids);
  cudaFree(ids_sorted);
  cudaFree(slots_sorted);
  cudaFree(temp);
  if (e != cudaSuccess) {
    set_error("hb_index_build_sorted: %s", cudaGetErrorString(e));
    return HB_ERR_CUDA;
  }
  h->sorted_stale = h->shared;  // a shared index may change under this process
  return HB_OK;
}

int hb_index_export(hb_index_t* h, int64_t* line_ids, int32_t* lru, hb_stream_t stream) {
  HB_CHECK_ARG(h, "hb_index_export: null index");
  cudaStream_t st = (cudaStream_t)stream;
  if (line_ids)
    HB_CUDA(cudaMemcpyAsync(line_ids, h->line_ids, h->cache_size * sizeof(int64_t),
                            cudaMemcpyDefault, st));
  if (lru)
    HB_CUDA(cudaMemcpyAsync(lru, h->lru, h->cache_size * sizeof(int32_t), cudaMemcpyDefault, st));
  HB_CUDA(cudaStreamSynchronize(st));
  return HB_OK;
}

int hb_index_import(hb_index_t* h, const int64_t* line_ids, const int32_t* lru,
                    hb_stream_t stream) {
  HB_CHECK_ARG(h, "hb_index_import: null index");
  cudaStream_t st = (cudaStream_t)stream;
  if (line_ids)
    HB_CUDA(cudaMemcpyAsync(h->line_ids, line_ids, h->cache_size * sizeof(int64_t),
                            cudaMemcpyDefault, st));
  if (lru)
    HB_CUDA(cudaMemcpyAsync(h->lru, lru, h->cache_size * sizeof(int32_t), cudaMemcpyDefault, st));
  HB_CUDA(cudaStreamSynchronize(st));
  h->sorted_stale = true;
  return HB_OK;
}

}  // extern "C"
