// Sort-once step: the batch of ids is sorted ONCE (radix sort of (id, position)), its runs
// of equal ids are numbered, and everything that the reference does per occurrence is then
// done per distinct id:
//   * hb_runs_build         sort + run heads + class and per-class position of every
//                           distinct id (torch.unique of python/EmbCache/sparse_optim.py:133
//                           and the class lookups of dist_emb.py:174-191, sparse_optim.py:243-259)
//   * hb_lookup_fetch_runs  cache lookup + cached fetch over the sorted batch: consecutive
//                           copies of an id reuse the row already in registers, so a row is read
//                           once per warp that meets it (dist_emb.py:184-243; a DGL sampler hands
//                           the reference unique ids, a raw id stream does not)
//   * hb_runs_miss_list     ids of one class that the cache did not hold, ascending, with
//                           the batch position whose output row holds their embedding
//                           (the uncached cold ids sent to the server, dist_emb.py:218-259)
// The backward aggregation (segsum.cu) and the LRU ageing (index.cu) take the same runs.
#include <cub/device/device_radix_sort.cuh>

#include "a2a.cuh"
#include "compact.cuh"
#include "index.cuh"
#include "runs.cuh"
#include "shard.cuh"

namespace hb {
int* device_error_word();  // runtime.cu

namespace {

constexpr int kBlock = 256;

size_t sort_temp_bytes(int64_t n) {
  size_t b64 = 0, b32 = 0;
  cub::DoubleBuffer<int64_t> k(nullptr, nullptr);
  cub::DoubleBuffer<uint32_t> k32(nullptr, nullptr);
  cub::DoubleBuffer<uint32_t> v(nullptr, nullptr);
  cub::DeviceRadixSort::SortPairs(nullptr, b64, k, v, (int)n, 0, 64, (cudaStream_t)0);
  cub::DeviceRadixSort::SortPairs(nullptr, b32, k32, v, (int)n, 0, 32, (cudaStream_t)0);
  return b64 > b32 ? b64 : b32;
}

// number of valid entries of a segmented input = sum of the segment counts
__global__ void sum_counts_kernel(const int64_t* __restrict__ seg_counts, int64_t num_segs,
                                  int64_t seg_cap, int64_t* __restrict__ out) {
  if (threadIdx.x || blockIdx.x) return;
  int64_t t = 0;
  for (int64_t k = 0; k < num_segs; ++k) {
    const int64_t c = seg_counts[k];
    t += c < 0 ? 0 : (c > seg_cap ? seg_cap : c);
  }
  *out = t;
}

// keys = ids (entries at and beyond the device count, or beyond their segment's count, get
// the largest key of id_bits bits, so they sort last), perm = 0..n-1.  A valid id that does
// not fit below that key raises HB_ERR_INVALID in the device status word: it would collide
// with another id or with the padding.
template <typename KeyT>
__global__ void prepare_keys_kernel(const int64_t* __restrict__ ids, int64_t n,
                                    const int64_t* __restrict__ n_dev,
                                    const int64_t* __restrict__ seg_counts, int64_t seg_cap,
                                    int64_t sentinel, KeyT* __restrict__ keys,
                                    uint32_t* __restrict__ perm, int* __restrict__ err) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const bool keep = seg_counts ? (i % seg_cap) < seg_counts[i / seg_cap] : (!n_dev || i < *n_dev);
  int64_t id = keep ? ids[i] : sentinel;
  if (keep && (id < 0 || id >= sentinel)) {
    atomicExch(err, HB_ERR_INVALID);
    id = sentinel;
  }
  keys[i] = (KeyT)id;
  perm[i] = (uint32_t)i;
}

// run heads of the sorted keys, numbered over all runs and inside their class
template <typename KeyT>
struct HeadPolicy {
  const KeyT* keys;
  const int64_t* n_dev;
  int64_t n;
  const int8_t* table;   // nullable: no classes
  int64_t table_len;
  uint8_t* head;
  int64_t* uniq;
  int64_t* uniq2;        // nullable second copy (the caller's buffer)
  int64_t* run_start;
  int8_t* dclass;
  int32_t* dpos;
  int64_t* out_ids[3];
  int64_t* num_runs;
  int64_t* num_runs2;    // nullable second copy
  int64_t* class_counts;
  int64_t* class_counts2;
  int32_t* base8;        // [ceil(n / 8)] runs that start before entry 8k
  __device__ __forceinline__ void thread_begin(int64_t base, const int4& before) const {
    base8[base >> 3] = before.x + before.y + before.z + before.w;
  }
  __device__ __forceinline__ int64_t valid_entries() const {
    if (!n_dev) return n;
    const int64_t d = *n_dev;
    return d < n ? (d > 0 ? d : 0) : n;
  }
  __device__ __forceinline__ int classify(int64_t i) const {
    const bool is_head = i < valid_entries() && (i == 0 || __ldg(keys + i - 1) != __ldg(keys + i));
    head[i] = is_head;
    if (!is_head) return -1;
    if (!table) return 0;
    const int64_t id = (int64_t)__ldg(keys + i);
    if (id >= table_len) return 3;
    const int8_t v = __ldg(table + id);
    return (v >= 0 && v <= 2) ? (int)v : 3;
  }
  // the 8 items of a thread at once: their keys come in two 16-byte loads (32-bit keys) and
  // the head flags leave in one 8-byte store
  __device__ __forceinline__ void classify8(int64_t base, int64_t n_items, int* cls) const {
    const int64_t ne = valid_entries();
    if (base + 8 > n_items || sizeof(KeyT) != 4) {
#pragma unroll
      for (int k = 0; k < 8; ++k) cls[k] = base + k < n_items ? classify(base + k) : -1;
      return;
    }
    uint32_t key[9];
    key[0] = base > 0 ? (uint32_t)__ldg(keys + base - 1) : 0u;
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(keys + base));
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(keys + base) + 1);
    key[1] = a.x; key[2] = a.y; key[3] = a.z; key[4] = a.w;
    key[5] = b.x; key[6] = b.y; key[7] = b.z; key[8] = b.w;
    unsigned long long flags = 0ull;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int64_t i = base + k;
      const bool is_head = i < ne && (i == 0 || key[k] != key[k + 1]);
      flags |= (unsigned long long)is_head << (8 * k);
      int c = -1;
      if (is_head) {
        c = 0;
        if (table) {
          const int64_t id = (int64_t)key[k + 1];
          c = 3;
          if (id < table_len) {
            const int8_t v = __ldg(table + id);
            if (v >= 0 && v <= 2) c = (int)v;
          }
        }
      }
      cls[k] = c;
    }
    *reinterpret_cast<unsigned long long*>(head + base) = flags;
  }
  __device__ __forceinline__ void emit(int64_t i, int cls, const int4& before) const {
    const int64_t u = (int64_t)before.x + before.y + before.z + before.w;
    const int64_t id = (int64_t)keys[i];
    uniq[u] = id;
    if (uniq2) uniq2[u] = id;
    run_start[u] = i;
    if (table) {
      const int pos = cls == 0 ? before.x : (cls == 1 ? before.y : (cls == 2 ? before.z : before.w));
      dclass[u] = cls < 3 ? (int8_t)cls : (int8_t)-1;
      dpos[u] = pos;
      if (cls < 3 && out_ids[cls]) out_ids[cls][pos] = id;
    }
  }
  __device__ __forceinline__ void finish(const int4& tot) const {
    const int64_t u = (int64_t)tot.x + tot.y + tot.z + tot.w;
    *num_runs = u;
    if (num_runs2) *num_runs2 = u;
    run_start[u] = valid_entries();
    class_counts[0] = tot.x; class_counts[1] = tot.y; class_counts[2] = tot.z; class_counts[3] = tot.w;
    if (class_counts2) { class_counts2[0] = tot.x; class_counts2[1] = tot.y; class_counts2[2] = tot.z; }
  }
};

// ---- forward: lookup + fetch over the sorted batch -----------------------------------------
// RESOLVE works per distinct id (one lane per run): the index probe, the slot of the run, and
// where the row of the run is to be read from -- the cache row, the row of the table on this
// GPU, or, for a row that lives on ANOTHER GPU, its place in a staging buffer on this GPU; such
// runs go on a list.  STAGE (sharded tables only) copies the listed rows from their owners, so
// that every remote row crosses NVLink once per step however often its id occurs in the batch
// (a row read again by every warp that meets the id, from seven GPUs at once, serialises on one
// L2 slice of its owner).  EXPAND works per entry of the sorted batch: the row goes to the
// entry's batch position; entries of one run inside a warp take the registers of the first.
struct RowSource {
  const char* backing;  // one table on this GPU, or null
  int64_t backing_rows;
  ShardView shards;     // used when PEER
  int rank;             // whose shard is local (PEER)
  char* stage;          // [stage_cap][row_bytes] copies of remote rows, by run (PEER)
  int64_t stage_cap;
  int32_t* remote_runs;            // runs whose row STAGE has to copy, in any order (PEER)
  unsigned long long* remote_count;  // [1], zero before RESOLVE
  // when the OWNERS deliver the remote rows (hb_runs_resolve_requests): a remote run becomes the
  // request (id, run) -- the run is also the row of this GPU's stage that the owner fills --
  // stored straight into this rank's slab of the owner's receive area
  const hb_a2a::Dest* req_dest;
  unsigned long long* req_counts;  // [world] requests so far per owner, zero before RESOLVE
  int64_t req_cap;                 // requests one owner's slab takes from this rank
};

template <bool PEER>
__device__ __forceinline__ uint4 load_row16(const uint4* p) {
  if (PEER) return *p;  // may be a peer GPU's memory that its owner rewrites between steps
  return __ldg(p);
}

// run_src[u]: address of the run's row (16-byte aligned, 0 = none) | 1 when it is a cache row
template <int MODE, bool PEER>
__global__ void __launch_bounds__(kBlock) runs_resolve_kernel(
    IndexView v, hb_runs_t r, RowSource rs, const char* __restrict__ cache_rows, int64_t row_bytes,
    int vb, unsigned long long* __restrict__ run_src, int64_t* __restrict__ run_slots,
    int* __restrict__ err) {
  __shared__ int64_t s_top[MODE == HB_LOOKUP_SORTED ? kTopMax : 1];
  if (MODE == HB_LOOKUP_SORTED) {
    stage_top_level(v, s_top);
    __syncthreads();
  }
  const int64_t U = *r.num_runs;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t limit = PEER ? rs.shards.num_rows : rs.backing_rows;
  for (int64_t u0 = warp * 32; u0 < U; u0 += nwarps * 32) {
    const int64_t u = u0 + lane;
    const bool valid = u < U;
    const int64_t id = valid ? __ldg(r.uniq_ids + u) : -1;
    const int64_t slot = warp_lookup<MODE>(v, s_top, id);
    const char* src = nullptr;
    const char* remote = nullptr;  // to be copied to the stage
    if (slot >= 0) {
      src = cache_rows + slot * row_bytes;
    } else if (valid && id < limit) {
      if (PEER) {
        const char* row = shard_row(rs.shards, id, row_bytes);
        const bool mine = rs.shards.world == 1 || mod_nonneg(id, rs.shards.world) == rs.rank;
        if (mine || u >= rs.stage_cap) {
          src = row;  // local shard, or no room in the stage: EXPAND reads the owner's memory itself
        } else {
          remote = row;
          src = rs.stage + u * row_bytes;
        }
      } else {
        src = rs.backing ? rs.backing + id * row_bytes : nullptr;
      }
    } else if (valid && (PEER || rs.backing)) {
      atomicExch(err, HB_ERR_INVALID);  // no such row: the output rows of the run stay as they were
    }
    if (valid) {
      run_src[u] = (unsigned long long)src | (slot >= 0 ? 1ull : 0ull);
      if (run_slots) run_slots[u] = slot;
    }
    if (PEER) {
      // remote runs go on a list; STAGE copies their rows with every row in flight at once (the
      // copy is bound by round trips over NVLink, which a kernel that also probes the index
      // cannot keep enough of in flight)
      const unsigned todo = __ballot_sync(0xffffffffu, remote != nullptr);
      if (todo && rs.req_dest) {
        if (remote) {
          // one counter per owner: the lanes that ask the same owner take consecutive places
          const int owner = (int)mod_nonneg(id, rs.shards.world);
          const unsigned same = __match_any_sync(todo, owner);
          const int leader = __ffs(same) - 1;
          unsigned long long at = 0;
          if (lane == leader) at = atomicAdd(rs.req_counts + owner, (unsigned long long)__popc(same));
          at = __shfl_sync(same, at, leader);
          const int64_t k = (int64_t)at + __popc(same & ((1u << lane) - 1u));
          if (k < rs.req_cap) {
            const int64_t slot = (int64_t)rs.rank * rs.req_cap + k;  // my slab in the owner's area
            rs.req_dest->ids[owner][slot] = id;
            rs.req_dest->cnt[owner][slot] = u;
          } else {
            atomicExch(err, HB_ERR_CAPACITY);  // the row is not delivered: the stage keeps what it held
          }
        }
      } else if (todo) {
        unsigned long long at = 0;
        if (lane == 0) at = atomicAdd(rs.remote_count, (unsigned long long)__popc(todo));
        at = __shfl_sync(0xffffffffu, at, 0);
        if (remote) rs.remote_runs[at + __popc(todo & ((1u << lane) - 1u))] = (int32_t)u;
      }
    }
  }
}

// STAGE: the rows of the listed runs, from their owners' shards into this GPU's stage.  One
// warp per row and step, 4 rows in flight per warp, 32 warps per SM: some 19,000 rows are on
// their way at once, several times what the links need to run at their bandwidth.
__global__ void __launch_bounds__(kBlock, 4) runs_stage_kernel(hb_runs_t r, RowSource rs, int64_t row_bytes, int vb) {
  const int64_t cnt = (int64_t)*rs.remote_count;
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  constexpr int kFly = 4;
  for (int64_t i0 = warp * kFly; i0 < cnt; i0 += nwarps * kFly) {
    const char* from[kFly];
    char* to[kFly];
#pragma unroll
    for (int x = 0; x < kFly; ++x) {
      from[x] = nullptr;
      to[x] = nullptr;
      if (i0 + x < cnt) {
        // every rank starts at another place of its list: the lists of the ranks hold much the same
        // popular ids in much the same order, and readers that walk an owner's rows in step with
        // each other queue on the same lines
        int64_t at = i0 + x + (cnt / rs.shards.world) * rs.rank;
        if (at >= cnt) at -= cnt;
        const int64_t u = rs.remote_runs[at];
        from[x] = shard_row(rs.shards, __ldg(r.uniq_ids + u), row_bytes);
        to[x] = rs.stage + u * row_bytes;
      }
    }
    if (vb == 16) {
      for (int64_t k = lane; k < (row_bytes >> 4); k += 32) {
        uint4 val[kFly];
#pragma unroll
        for (int x = 0; x < kFly; ++x)
          if (from[x]) val[x] = *(reinterpret_cast<const uint4*>(from[x]) + k);
#pragma unroll
        for (int x = 0; x < kFly; ++x)
          if (from[x]) *(reinterpret_cast<uint4*>(to[x]) + k) = val[x];
      }
    } else {
      for (int x = 0; x < kFly; ++x) {
        if (!from[x]) continue;
        for (int64_t k = lane; k < row_bytes; k += 32) to[x][k] = from[x][k];
      }
    }
  }
}

// the run an entry of the sorted batch belongs to: runs that start before its group of 8
// entries (base8) + the heads inside the group up to the entry
__device__ __forceinline__ int64_t run_of_entry(const hb_runs_t& r, int64_t j) {
  const unsigned long long flags = *reinterpret_cast<const unsigned long long*>(r.head + (j & ~(int64_t)7));
  const int k = (int)(j & 7);
  const unsigned long long mask = k == 7 ? ~0ull : ((1ull << (8 * (k + 1))) - 1ull);
  return (int64_t)__ldg(r.base8 + (j >> 3)) + __popcll(flags & mask) - 1;
}

// RB: 512 = rows of exactly 512 bytes (128 fp32: the address arithmetic folds, no lane is idle);
// 16 = any multiple of 16 bytes; 0 = words or bytes.  PEER: a source may be another GPU's memory
// (runs that found no room in the stage), so rows are read with plain loads.
template <bool PEER, int RB>
__global__ void __launch_bounds__(kBlock, RB == 512 ? 4 : 3) runs_expand_kernel(
    hb_runs_t r, const unsigned long long* __restrict__ run_src, const int64_t* __restrict__ run_slots,
    int64_t row_bytes_arg, int vb, char* __restrict__ out, int64_t* __restrict__ locs,
    uint8_t* __restrict__ found) {
  constexpr bool V16 = RB != 0;
  const int64_t row_bytes = RB == 512 ? (int64_t)512 : row_bytes_arg;
  const int64_t n = runs_valid_entries(r);
  const int lane = lane_id();
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t stride = (((int64_t)gridDim.x * blockDim.x) >> 5) * 32;
  int64_t base = warp * 32;
  uint32_t pos_next = 0;
  int64_t run_next = -1;
  if (base + lane < n) {
    pos_next = __ldg(r.perm + base + lane);
    run_next = run_of_entry(r, base + lane);
  }
  for (; base < n; base += stride) {
    const bool valid = base + lane < n;
    const uint32_t pos = pos_next;
    const int64_t u = valid ? run_next : -1;
    if (base + stride + lane < n) {
      pos_next = __ldg(r.perm + base + stride + lane);
      run_next = run_of_entry(r, base + stride + lane);
    }
    const int64_t prev = __shfl_up_sync(0xffffffffu, u, 1);
    const unsigned fresh = __ballot_sync(0xffffffffu, lane == 0 || u != prev);
    const unsigned long long word = valid ? run_src[u] : 0ull;
    const unsigned long long src_bits = word & ~1ull;
    if (valid) {
      if (found) found[pos] = (uint8_t)(word & 1ull);
      if (locs) locs[pos] = run_slots[u];  // 8 bytes scattered over the batch: costly
    }
    const unsigned have = __ballot_sync(0xffffffffu, src_bits != 0ull);
    if (V16) {
      const int64_t vpr = row_bytes >> 4;
      if (RB == 512 || vpr <= 32) {
        const bool on = RB == 512 || lane < vpr;
        uint4 last = make_uint4(0, 0, 0, 0);
        constexpr int kFly = RB == 512 ? 8 : 4;  // rows whose loads are in flight together
        for (int q0 = 0; q0 < 32; q0 += kFly) {
          if (((have >> q0) & ((1u << kFly) - 1u)) == 0u) continue;
          uint4 val[kFly];
          uint32_t pq[kFly];
#pragma unroll
          for (int x = 0; x < kFly; ++x) {
            const int q = q0 + x;
            const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q);
            pq[x] = __shfl_sync(0xffffffffu, pos, q);
            if (((have & fresh) >> q) & 1u)
              if (on) val[x] = load_row16<PEER>(reinterpret_cast<const uint4*>(sb) + lane);
          }
#pragma unroll
          for (int x = 0; x < kFly; ++x) {
            const int q = q0 + x;
            if (!((have >> q) & 1u)) continue;
            if (!((fresh >> q) & 1u)) val[x] = last;
            last = val[x];
            if (on) __stcs(reinterpret_cast<uint4*>(out + (int64_t)pq[x] * row_bytes) + lane, val[x]);
          }
        }
      } else {
        for (int q0 = 0; q0 < 32; q0 += 4) {
          if (((have >> q0) & 0xfu) == 0u) continue;
          const uint4* sp[4];
          uint4* dp[4];
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const int q = q0 + x;
            const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q);
            const uint32_t pq = __shfl_sync(0xffffffffu, pos, q);
            sp[x] = ((have >> q) & 1u) ? reinterpret_cast<const uint4*>(sb) : nullptr;
            dp[x] = reinterpret_cast<uint4*>(out + (int64_t)pq * row_bytes);
          }
          for (int64_t k = lane; k < vpr; k += 32) {
            uint4 val[4];
#pragma unroll
            for (int x = 0; x < 4; ++x)
              if (sp[x]) val[x] = load_row16<PEER>(sp[x] + k);
#pragma unroll
            for (int x = 0; x < 4; ++x)
              if (sp[x]) __stcs(dp[x] + k, val[x]);
          }
        }
      }
    } else {
      // rows that are not a multiple of 16 bytes (or unaligned buffers): words or bytes
      for (int q = 0; q < 32; ++q) {
        const unsigned long long sb = __shfl_sync(0xffffffffu, src_bits, q);
        const uint32_t pq = __shfl_sync(0xffffffffu, pos, q);
        if (!((have >> q) & 1u)) continue;
        char* d = out + (int64_t)pq * row_bytes;
        if (vb == 4) {
          const uint32_t* s4 = reinterpret_cast<const uint32_t*>(sb);
          for (int64_t k = lane; k < (row_bytes >> 2); k += 32) reinterpret_cast<uint32_t*>(d)[k] = s4[k];
        } else {
          const char* s1 = reinterpret_cast<const char*>(sb);
          for (int64_t k = lane; k < row_bytes; k += 32) d[k] = s1[k];
        }
      }
    }
  }
}

// ---- ids of one class that missed the cache -----------------------------------------------
struct MissPolicy {
  hb_runs_t r;
  const int64_t* locs;   // slot per batch position (kind 0), per sorted entry (1) or per run (2)
  int locs_kind;
  int want_class;        // < 0: every class
  int64_t cap;
  int64_t* miss_ids;     // [cap], filled from entry 0
  int64_t* miss_src;     // [cap] batch position whose output row holds the embedding
  int64_t* miss_count;
  __device__ __forceinline__ int classify(int64_t u) const {
    if (u >= *r.num_runs) return -1;
    if (want_class >= 0 && (!r.dclass || r.dclass[u] != want_class)) return -1;
    const int64_t j = r.run_start[u];
    const int64_t at = locs_kind == 2 ? u : (locs_kind == 1 ? j : (int64_t)r.perm[j]);
    return locs[at] < 0 ? 0 : -1;
  }
  __device__ __forceinline__ void emit(int64_t u, int, const int4& before) const {
    if (before.x >= cap) return;
    miss_ids[before.x] = r.uniq_ids[u];
    miss_src[before.x] = (int64_t)r.perm[r.run_start[u]];
  }
  __device__ __forceinline__ void finish(const int4& tot) const {
    *miss_count = tot.x < cap ? tot.x : cap;
  }
};

__global__ void fill_i64_kernel(int64_t* p, int64_t n, int64_t v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

}  // namespace

RunsPlan make_runs_plan(void* ws, int64_t n) {
  RunsPlan s;
  Carver cv(ws ? ws : (void*)256);  // a null workspace still yields the sizes
  const int64_t m = n > 0 ? n : 1;
  s.k0 = cv.take<int64_t>(m);
  s.k1 = cv.take<int64_t>(m);
  s.p0 = cv.take<uint32_t>(m);
  s.p1 = cv.take<uint32_t>(m);
  s.sort_temp_bytes = sort_temp_bytes(m);
  s.sort_temp = cv.take<char>(s.sort_temp_bytes);
  s.run_start = cv.take<int64_t>(m + 1);
  s.head = cv.take<uint8_t>(m + 1);
  s.n_valid = cv.take<int64_t>(1);
  s.num_runs = cv.take<int64_t>(1);
  s.class_counts = cv.take<int64_t>(4);
  s.dclass = cv.take<int8_t>(m + 1);
  s.dpos = cv.take<int32_t>(m + 1);
  s.uniq = cv.take<int64_t>(m + 1);
  s.base8 = cv.take<int32_t>(m / 8 + 2);
  s.compact_ws_bytes = compact_workspace_bytes(m);
  s.compact_ws = cv.take<char>(s.compact_ws_bytes);
  s.total = cv.used() + 256;
  return s;
}

}  // namespace hb

using namespace hb;

extern "C" {

size_t hb_runs_workspace_bytes(int64_t n) { return make_runs_plan(nullptr, n).total; }

int hb_runs_build(const int64_t* ids, int64_t n, const int64_t* n_dev, const int64_t* seg_counts,
                  int64_t seg_cap, int id_bits, const int8_t* class_table, int64_t table_len,
                  int64_t* const* class_ids_out, int64_t* class_counts_out, int64_t* uniq_ids_out,
                  int64_t* num_unique_out, void* workspace, size_t workspace_bytes,
                  hb_runs_t* runs_out, hb_stream_t stream) {
  HB_CHECK_ARG(runs_out != nullptr, "hb_runs_build: runs_out is null");
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31), "hb_runs_build: n out of range");
  HB_CHECK_ARG(n == 0 || ids, "hb_runs_build: null ids");
  HB_CHECK_ARG(id_bits >= 1 && id_bits <= 64, "hb_runs_build: id_bits must be in [1, 64]");
  HB_CHECK_ARG(!seg_counts || (seg_cap > 0 && n % seg_cap == 0),
               "hb_runs_build: a segmented input holds whole segments of seg_cap entries");
  HB_CHECK_ARG(!class_table || table_len > 0, "hb_runs_build: a class table needs its length");
  RunsPlan s = make_runs_plan(workspace, n);
  if (!workspace || workspace_bytes < s.total) {
    set_error("hb_runs_build: workspace of %zu bytes needed, %zu given", s.total, workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  cudaStream_t st = (cudaStream_t)stream;
  memset(runs_out, 0, sizeof(*runs_out));
  runs_out->n = n;
  runs_out->num_runs = s.num_runs;
  runs_out->class_counts = s.class_counts;
  runs_out->run_start = s.run_start;
  runs_out->head = s.head;
  runs_out->uniq_ids = s.uniq;
  runs_out->base8 = s.base8;
  runs_out->dclass = class_table ? s.dclass : nullptr;
  runs_out->dpos = class_table ? s.dpos : nullptr;
  if (n == 0) {
    HB_CUDA(cudaMemsetAsync(s.num_runs, 0, sizeof(int64_t), st));
    HB_CUDA(cudaMemsetAsync(s.class_counts, 0, 4 * sizeof(int64_t), st));
    HB_CUDA(cudaMemsetAsync(s.run_start, 0, sizeof(int64_t), st));
    if (num_unique_out) HB_CUDA(cudaMemsetAsync(num_unique_out, 0, sizeof(int64_t), st));
    if (class_counts_out) HB_CUDA(cudaMemsetAsync(class_counts_out, 0, 3 * sizeof(int64_t), st));
    return HB_OK;
  }
  if (seg_counts) {
    // valid entries are scattered over the segments; their number becomes the device count
    HB_LAUNCH(sum_counts_kernel, 1, 32, 0, st, seg_counts, n / seg_cap, seg_cap, s.n_valid);
    n_dev = s.n_valid;
  }
  runs_out->n_dev = n_dev;
  const int64_t sentinel = id_bits >= 63 ? INT64_MAX : (((int64_t)1 << id_bits) - 1);
  cub::DoubleBuffer<uint32_t> perm(s.p0, s.p1);
  int rc;
  int64_t* cls_out[3] = {class_ids_out ? class_ids_out[0] : nullptr, class_ids_out ? class_ids_out[1] : nullptr,
                         class_ids_out ? class_ids_out[2] : nullptr};
  if (id_bits <= 32) {
    uint32_t* k0 = reinterpret_cast<uint32_t*>(s.k0);
    uint32_t* k1 = reinterpret_cast<uint32_t*>(s.k1);
    HB_LAUNCH(prepare_keys_kernel<uint32_t>, (int)ceil_div(n, kBlock), kBlock, 0, st, ids, n, n_dev,
              seg_counts, seg_cap, sentinel, k0, s.p0, device_error_word());
    cub::DoubleBuffer<uint32_t> keys(k0, k1);
    HB_CUDA(cub::DeviceRadixSort::SortPairs(s.sort_temp, s.sort_temp_bytes, keys, perm, (int)n, 0,
                                            id_bits, st));
    HeadPolicy<uint32_t> pol{keys.Current(), n_dev, n, class_table, table_len, s.head, s.uniq, uniq_ids_out,
                             s.run_start, s.dclass, s.dpos, {cls_out[0], cls_out[1], cls_out[2]},
                             s.num_runs, num_unique_out, s.class_counts, class_counts_out, s.base8};
    rc = run_compact(pol, n, s.compact_ws, s.compact_ws_bytes, st);
    runs_out->keys = keys.Current();
    runs_out->key_bytes = 4;
  } else {
    HB_LAUNCH(prepare_keys_kernel<int64_t>, (int)ceil_div(n, kBlock), kBlock, 0, st, ids, n, n_dev,
              seg_counts, seg_cap, sentinel, s.k0, s.p0, device_error_word());
    cub::DoubleBuffer<int64_t> keys(s.k0, s.k1);
    HB_CUDA(cub::DeviceRadixSort::SortPairs(s.sort_temp, s.sort_temp_bytes, keys, perm, (int)n, 0,
                                            id_bits, st));
    HeadPolicy<int64_t> pol{keys.Current(), n_dev, n, class_table, table_len, s.head, s.uniq, uniq_ids_out,
                            s.run_start, s.dclass, s.dpos, {cls_out[0], cls_out[1], cls_out[2]},
                            s.num_runs, num_unique_out, s.class_counts, class_counts_out, s.base8};
    rc = run_compact(pol, n, s.compact_ws, s.compact_ws_bytes, st);
    runs_out->keys = keys.Current();
    runs_out->key_bytes = 8;
  }
  count_library_launches(1 + (id_bits + 7) / 8);
  runs_out->perm = perm.Current();
  return rc;
}

namespace {
// scratch of hb_lookup_fetch_runs: where every run's row is read from, the slot of every run
// when the caller does not ask for it, and (sharded table) the copies of the remote rows
struct FetchPlan {
  unsigned long long* run_src;
  int64_t* run_slots;
  char* stage;
  int64_t stage_cap;
  int32_t* remote_runs;
  unsigned long long* remote_count;
  unsigned long long* req_counts;  // [64]
  size_t total;
};
constexpr int64_t kStageMaxBytes = (int64_t)1 << 30;  // at most 1 GiB of staged remote rows

FetchPlan make_fetch_plan(void* ws, int64_t n, int64_t row_bytes, bool sharded) {
  FetchPlan f;
  Carver cv(ws ? ws : (void*)256);
  const int64_t m = n > 0 ? n : 1;
  f.run_src = cv.take<unsigned long long>(m);
  f.run_slots = cv.take<int64_t>(m);
  f.req_counts = cv.take<unsigned long long>(64);
  f.stage_cap = 0;
  f.stage = nullptr;
  f.remote_runs = nullptr;
  f.remote_count = nullptr;
  if (sharded) {
    f.stage_cap = kStageMaxBytes / row_bytes < m ? kStageMaxBytes / row_bytes : m;
    f.stage = cv.take<char>((size_t)f.stage_cap * row_bytes);
    f.remote_runs = cv.take<int32_t>(m);
    f.remote_count = cv.take<unsigned long long>(2);
  }
  f.total = cv.used() + 256;
  return f;
}
// Who brings the remote rows: nobody (one table on this GPU), this GPU (STAGE reads the owners'
// shards), or the owners (`dv`: RESOLVE lists (id, run) requests, the owners store the rows into
// dv->stage, which they have mapped, before EXPAND runs).
struct Delivery {
  char* stage;
  int64_t stage_cap;
  hb_a2a* requests;  // the exchange that carries the requests (null: expansion only)
  int* parity_out;   // which of its receive areas this call filled
  bool peer_sources; // expansion only: a run's row may lie in another GPU's memory (plain loads)
};

int fetch_runs_impl(hb_index_t* h, const hb_runs_t* runs, const void* cache_rows, const void* backing_rows,
                    int64_t backing_num_rows, hb_peer_table_t* table, int64_t row_bytes, void* out_rows,
                    int64_t* locs, uint8_t* found, int64_t* run_slots, int mode, void* workspace,
                    size_t workspace_bytes, hb_stream_t stream, const Delivery* dv, bool resolve, bool expand) {
  HB_CHECK_ARG((h || !resolve) && runs, "hb_lookup_fetch_runs: null argument");
  HB_CHECK_ARG(row_bytes > 0, "hb_lookup_fetch_runs: bad row size");
  HB_CHECK_ARG(runs->n == 0 || ((cache_rows || !resolve) && runs->perm && runs->head && runs->base8 &&
                                runs->uniq_ids),
               "hb_lookup_fetch_runs: null argument");
  HB_CHECK_ARG(mode == HB_LOOKUP_SETASSOC || mode == HB_LOOKUP_SORTED,
               "hb_lookup_fetch_runs: unknown mode %d", mode);
  HB_CHECK_ARG(!(table && backing_rows), "hb_lookup_fetch_runs: give a backing table or a sharded one");
  HB_CHECK_ARG(!table || table->row_bytes == row_bytes, "hb_lookup_fetch_runs: row size differs from the table's");
  HB_CHECK_ARG(!backing_rows || backing_num_rows > 0, "hb_lookup_fetch_runs: a backing table needs its row count");
  cudaStream_t st = (cudaStream_t)stream;
  FetchPlan f0 = make_fetch_plan(workspace, runs->n, row_bytes, false);
  if (resolve && dv && dv->requests) {
    // also with an empty batch: the owners read this rank's counts after the fence
    if (!workspace || workspace_bytes < f0.total) {
      set_error("hb_runs_resolve_requests: workspace of %zu bytes needed, %zu given", f0.total, workspace_bytes);
      return HB_ERR_WORKSPACE;
    }
    HB_CUDA(cudaMemsetAsync(f0.req_counts, 0, 64 * sizeof(unsigned long long), st));
  }
  if (runs->n == 0) {
    if (resolve && dv && dv->requests) {
      const hb_a2a::Dest* dest;
      int rc = a2a_direct_begin(dv->requests, &dest, dv->parity_out);
      if (rc != HB_OK) return rc;
      return a2a_direct_publish(dv->requests, *dv->parity_out, f0.req_counts, st);
    }
    return HB_OK;
  }
  const bool sharded = !dv && table != nullptr && table->world > 1;  // this GPU copies the remote rows
  FetchPlan f = make_fetch_plan(workspace, runs->n, row_bytes, sharded);
  if (!workspace || workspace_bytes < f.total) {
    set_error("hb_lookup_fetch_runs: workspace of %zu bytes needed, %zu given", f.total, workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  if (resolve && mode == HB_LOOKUP_SORTED && h->sorted_stale) {
    int rc = hb_index_build_sorted(h, stream);
    if (rc != HB_OK) return rc;
  }
  RowSource rs;
  memset(&rs, 0, sizeof(rs));
  rs.backing = (const char*)backing_rows;
  rs.backing_rows = backing_rows ? backing_num_rows : 0;
  rs.stage = f.stage;
  rs.stage_cap = f.stage_cap;
  rs.remote_runs = f.remote_runs;
  rs.remote_count = f.remote_count;
  if (dv) {
    rs.stage = dv->stage;
    rs.stage_cap = dv->stage_cap;
    if (resolve && dv->requests) {
      HB_CHECK_ARG(dv->requests->world == table->world && dv->requests->rank == table->rank,
                   "hb_runs_resolve_requests: the exchange and the table belong to different groups");
      int rc = a2a_direct_begin(dv->requests, &rs.req_dest, dv->parity_out);
      if (rc != HB_OK) return rc;
      rs.req_counts = f.req_counts;
      rs.req_cap = dv->requests->cap;
    }
  }
  if (table) {
    int rc = make_shard_view(table, &rs.shards);
    if (rc != HB_OK) return rc;
    rs.rank = table->rank;
  }
  uintptr_t bits = (uintptr_t)row_bytes | (uintptr_t)cache_rows | (uintptr_t)out_rows | (uintptr_t)backing_rows |
                   (uintptr_t)(dv ? dv->stage : nullptr);
  HB_CHECK_ARG((bits & 1) == 0, "hb_lookup_fetch_runs: rows must start at even addresses");
  const bool v16 = (bits & 15) == 0;  // shards come from cudaMalloc and hold whole rows
  const int vb = v16 ? 16 : ((bits & 3) == 0 ? 4 : 1);
  int* err = device_error_word();
  int64_t* slots = run_slots ? run_slots : f.run_slots;
  if (resolve && sharded) HB_CUDA(cudaMemsetAsync(rs.remote_count, 0, sizeof(unsigned long long), st));
  if (resolve) {
    int64_t blocks = ceil_div(ceil_div(runs->n, 32) * 32, kBlock);  // one lane per run, at most n runs
    if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
    const int grid = (int)(blocks < 1 ? 1 : blocks);
#define HB_RES(MODE, PEER)                                                                              \
  HB_LAUNCH((runs_resolve_kernel<MODE, PEER>), grid, kBlock, 0, st, h->view, *runs, rs,                \
            (const char*)cache_rows, row_bytes, vb, f.run_src, slots, err)
    if (mode == HB_LOOKUP_SORTED) {
      if (table) HB_RES(HB_LOOKUP_SORTED, true); else HB_RES(HB_LOOKUP_SORTED, false);
    } else {
      if (table) HB_RES(HB_LOOKUP_SETASSOC, true); else HB_RES(HB_LOOKUP_SETASSOC, false);
    }
#undef HB_RES
  }
  if (resolve && sharded)
    HB_LAUNCH(runs_stage_kernel, sm_count() * 4, kBlock, 0, st, *runs, rs, row_bytes, vb);
  if (resolve && dv && dv->requests) {
    int rc = a2a_direct_publish(dv->requests, *dv->parity_out, f.req_counts, st);
    if (rc != HB_OK) return rc;
  }
  if (!expand) return HB_OK;  // per distinct id only: slots in run_slots, remote rows staged or asked for
  int64_t blocks = ceil_div(ceil_div(runs->n, 32) * 32, kBlock);
  if (blocks > (int64_t)sm_count() * 32) blocks = (int64_t)sm_count() * 32;
  const int grid = (int)(blocks < 1 ? 1 : blocks);
#define HB_EXP(PEER, RB)                                                                         \
  HB_LAUNCH((runs_expand_kernel<PEER, RB>), grid, kBlock, 0, st, *runs, f.run_src, slots, row_bytes, \
            vb, (char*)out_rows, locs, found)
#define HB_EXP_V(PEER)                                \
  do {                                                \
    if (v16 && row_bytes == 512) HB_EXP(PEER, 512);   \
    else if (v16) HB_EXP(PEER, 16);                   \
    else HB_EXP(PEER, 0);                             \
  } while (0)
  if (sharded || (dv && dv->peer_sources)) HB_EXP_V(true); else HB_EXP_V(false);
#undef HB_EXP_V
#undef HB_EXP
  return HB_OK;
}
}  // namespace

size_t hb_lookup_fetch_runs_workspace_bytes(int64_t n, int64_t row_bytes, int sharded) {
  return make_fetch_plan(nullptr, n, row_bytes > 0 ? row_bytes : 1, sharded != 0).total;
}

int hb_lookup_fetch_runs(hb_index_t* h, const hb_runs_t* runs, const void* cache_rows,
                         const void* backing_rows, int64_t backing_num_rows, hb_peer_table_t* table,
                         int64_t row_bytes, void* out_rows, int64_t* locs, uint8_t* found,
                         int64_t* run_slots, int mode, void* workspace, size_t workspace_bytes,
                         hb_stream_t stream) {
  return fetch_runs_impl(h, runs, cache_rows, backing_rows, backing_num_rows, table, row_bytes, out_rows, locs,
                         found, run_slots, mode, workspace, workspace_bytes, stream, nullptr, true,
                         out_rows != nullptr);
}

int hb_runs_resolve_requests(hb_index_t* h, const hb_runs_t* runs, const void* cache_rows,
                             hb_peer_table_t* table, int64_t row_bytes, void* stage_rows, int64_t stage_cap,
                             int64_t* run_slots, hb_a2a_t* requests, int* parity_out, int mode, void* workspace,
                             size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(table && stage_rows && stage_cap > 0 && requests && parity_out,
               "hb_runs_resolve_requests: null argument");
  HB_CHECK_ARG(((uintptr_t)stage_rows & 15) == 0, "hb_runs_resolve_requests: the stage is 16-byte aligned");
  Delivery dv{(char*)stage_rows, stage_cap, requests, parity_out, true};
  return fetch_runs_impl(h, runs, cache_rows, nullptr, 0, table, row_bytes, nullptr, nullptr, nullptr, run_slots,
                         mode, workspace, workspace_bytes, stream, &dv, true, false);
}

int hb_runs_expand(const hb_runs_t* runs, const void* cache_rows, const void* other_rows, int64_t row_bytes,
                   int peer_sources, void* out_rows, int64_t* locs, uint8_t* found, const int64_t* run_slots,
                   void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(out_rows != nullptr && cache_rows != nullptr, "hb_runs_expand: null argument");
  Delivery dv{(char*)other_rows, 0, nullptr, nullptr, peer_sources != 0};
  return fetch_runs_impl(nullptr, runs, cache_rows, nullptr, 0, nullptr, row_bytes, out_rows, locs, found,
                         const_cast<int64_t*>(run_slots), HB_LOOKUP_SETASSOC, workspace, workspace_bytes, stream,
                         &dv, false, true);
}

size_t hb_runs_miss_list_workspace_bytes(int64_t n) { return compact_workspace_bytes(n); }

int hb_runs_miss_list(const hb_runs_t* runs, const int64_t* locs, int locs_kind, int want_class,
                      int64_t cap, int64_t* miss_ids, int64_t* miss_src, int64_t* miss_count,
                      void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(runs && locs && miss_ids && miss_src && miss_count && cap > 0,
               "hb_runs_miss_list: null argument");
  HB_CHECK_ARG(locs_kind >= 0 && locs_kind <= 2, "hb_runs_miss_list: locs_kind is 0, 1 or 2");
  HB_CHECK_ARG(want_class < 0 || runs->dclass || runs->n == 0,
               "hb_runs_miss_list: the runs were built without a class table");
  cudaStream_t st = (cudaStream_t)stream;
  // entries beyond the count hold -1, which the index's add() ignores
  int64_t blocks = ceil_div(cap, kBlock);
  if (blocks > (int64_t)sm_count() * 8) blocks = (int64_t)sm_count() * 8;
  HB_LAUNCH(fill_i64_kernel, (int)blocks, kBlock, 0, st, miss_ids, cap, (int64_t)-1);
  if (runs->n == 0) {
    HB_CUDA(cudaMemsetAsync(miss_count, 0, sizeof(int64_t), st));
    return HB_OK;
  }
  MissPolicy pol{*runs, locs, locs_kind, want_class, cap, miss_ids, miss_src, miss_count};
  return run_compact(pol, runs->n, workspace, workspace_bytes, st);
}

}  // extern "C"
