/*
 * libhades_b200 -- C ABI of the B200 (sm_100a) embedding-cache / sparse-gradient
 * hot path.  Plain pointers and sizes only; no torch types.  Every entry point
 * returns an hb_status (0 = success) and never exits the process;
 * hb_last_error() gives the message of the last failure on the calling thread.
 *
 * Unless stated otherwise every pointer is a DEVICE pointer (pinned host memory
 * mapped into the device address space also works for the row movers, as it
 * does for the reference's UVA kernels), every call is asynchronous on the
 * given stream (a cudaStream_t passed as void*), and the caller owns all
 * buffers.  Kernels that need scratch memory are given it by the caller as a
 * workspace: hb_xxx_workspace_bytes() tells how much.
 *
 * Each declaration cites the reference interface (HADES, path inside the
 * reference project) that it replaces.
 */
#ifndef HADES_B200_H_
#define HADES_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hb_status {
  HB_OK = 0,
  HB_ERR_INVALID = 1,     /* bad argument (shape, dtype size, null pointer, alignment) */
  HB_ERR_CUDA = 2,        /* a CUDA runtime call failed */
  HB_ERR_WORKSPACE = 3,   /* caller workspace too small */
  HB_ERR_UNSUPPORTED = 4, /* valid request that this build does not implement */
  HB_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out */
  HB_ERR_CAPACITY = 6     /* a fixed-capacity buffer would overflow */
} hb_status;

typedef void* hb_stream_t; /* cudaStream_t */

const char* hb_last_error(void);
int hb_version(void);
/* Number of kernels this library has launched in this process (all threads). */
int64_t hb_launch_count(void);
/* Kernels that wait on hardware barriers do so with an iteration limit; one that
 * gives up records an hb_status in a per-device word instead of trapping.  This
 * call synchronises the stream, returns that word (0 = none) and clears it. */
int hb_device_status(int* status_host, hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Cache index: 8-way set-associative ID -> slot map, state resident in HBM.   */
/* Replaces SACacheIndex / IndexCache (src/cache/cache.h:11-257,               */
/* src/cache/cache_line.h:7-103, bound in src/pybind.cc:17-33).                */
/* slot = (id % lines) * 8 + way; -1 = absent.  ids must be >= 0.              */
/* ------------------------------------------------------------------------- */
typedef struct hb_index hb_index_t;
typedef struct hb_peer_table hb_peer_table_t; /* a table sharded over the GPUs of a box, see the end of this file */
typedef struct hb_a2a hb_a2a_t;               /* a peer-memory exchange, see hb_a2a_create */

#define HB_WAYS 8

/* Lookup algorithm.  Both give identical outputs. */
#define HB_LOOKUP_SETASSOC 0 /* probe the 64-byte line id % lines              */
#define HB_LOOKUP_SORTED 1   /* warp-cooperative search of the sorted view     */

/* IndexCache(cache_size, ...) ctor, src/cache/cache.h:138-167: lines =
 * ceil(cache_size/8); capacity rounds up to a multiple of 8.  Allocates the
 * state on the current device. */
int hb_index_create(int64_t cache_size, hb_index_t** out);
int hb_index_destroy(hb_index_t* h);

/* One index for several processes of a box, as IndexCache(name, create=False) opens the
 * creator's POSIX segment in the reference (src/cache/cache.h:145-167, exercised by
 * test/test_cache.py:6-61): the creator exports a handle of hb_index_handle_bytes() bytes,
 * passes it through any host channel, and hb_index_open gives another process an index over
 * the SAME lines (ids and LRU counters stay in the creator's HBM; the creator destroys last).
 * Nothing orders the processes' calls against each other: the callers do, as in the
 * reference.  HB_LOOKUP_SORTED on an opened index rebuilds its sorted view before every
 * lookup; the creator calls hb_index_build_sorted after the other process changed the
 * index.  At most 2^31 slots per index (hb_index_create refuses more). */
size_t hb_index_handle_bytes(void);
int hb_index_export_handle(hb_index_t* h, void* handle_out /* host */);
int hb_index_open(const void* handle /* host */, hb_index_t** out);
/* get_size / get_capacity / get_space, src/cache/cache.h:176-194 */
int64_t hb_index_size(const hb_index_t* h);
int64_t hb_index_capacity(const hb_index_t* h);
int64_t hb_index_space(const hb_index_t* h);
int64_t hb_index_lines(const hb_index_t* h);
/* get_valid_entries_num, src/cache/cache.h:178-183.  Synchronises the stream. */
int hb_index_valid_entries(hb_index_t* h, int64_t* out_host, hb_stream_t stream);

/* add(ids) -> locs, src/cache/cache.h:51-88,196-206: existing id -> its slot;
 * else the LAST empty way; else the least-recently-used way (largest counter,
 * first on ties) unless all counters are 0, then -1.  Ids are applied in input
 * order per set (the reference result at OMP_NUM_THREADS=1).  Two ids of one
 * batch can receive the same slot (a later id evicts an earlier one, or the same
 * id repeats); last_writer (nullable, n bytes) marks for each id whether it is
 * the last of the batch to hold its slot, i.e. whose row a sequential
 * "rows[locs] = batch rows" leaves there. */
size_t hb_index_add_workspace_bytes(int64_t n);
int hb_index_add(hb_index_t* h, const int64_t* ids, int64_t n, int64_t* locs,
                 uint8_t* last_writer, void* workspace, size_t workspace_bytes,
                 hb_stream_t stream);

/* lookup(ids) -> locs (and optional found mask = locs >= 0),
 * src/cache/cache.h:90-104,213-222 and cudalookup, src/cache/lookup.cu:13-85.
 * Does not touch the LRU counters; see hb_index_touch_lru. */
int hb_index_lookup(hb_index_t* h, const int64_t* ids, int64_t n, int64_t* locs,
                    uint8_t* found /* nullable */, int mode, hb_stream_t stream);

/* The side effect of the reference's CPU lookup, cache_line::access_loc,
 * src/cache/cache_line.h:80-86 via src/cache/cache.h:101: for each hit in batch
 * order, every counter of the hit line += 1 and the hit way's counter = 0. */
size_t hb_index_touch_lru_workspace_bytes(int64_t n);
int hb_index_touch_lru(hb_index_t* h, const int64_t* locs, int64_t n,
                       void* workspace, size_t workspace_bytes, hb_stream_t stream);

/* The same LRU effect for a batch that is already grouped: run u holds the batch
 * positions perm[run_start[u] .. run_start[u+1]) (ascending) of ONE id, so all of
 * them carry the same slot locs[position], and different runs carry different
 * slots.  This is what the sort inside hb_unique_segsum_f32 leaves behind
 * (hb_runs_t), so a step that aggregates the gradients of the ids it looked up
 * needs no second sort for the ageing.  perm NULL = identity; run_start NULL =
 * every position is its own run (a batch of unique ids); num_runs / n_dev:
 * nullable device counts capping max_runs / n.  locs_kind: locs holds a slot per batch
 * position (0), per sorted entry (1) or per run (2: the run_slots of hb_lookup_fetch_runs).  The first call allocates two int32 arrays of `capacity`
 * entries inside the index. */
int hb_index_touch_lru_runs(hb_index_t* h, const int64_t* locs, const uint32_t* perm,
                            const int64_t* run_start, int64_t max_runs,
                            const int64_t* num_runs, int64_t n, const int64_t* n_dev,
                            int locs_kind, hb_stream_t stream);

/* reset(ids), src/cache/cache.h:106-118,208-211: a hit way becomes empty. */
int hb_index_reset(hb_index_t* h, const int64_t* ids, int64_t n, hb_stream_t stream);

/* getall(len) -> (ids, locs) in slot order, src/cache/cache.h:120-135,243-257.
 * Writes min(len, valid) pairs; *n_written_host receives that count.
 * Synchronises the stream. */
int hb_index_getall(hb_index_t* h, int64_t* ids_out, int64_t* locs_out, int64_t len,
                    int64_t* n_written_host, hb_stream_t stream);

/* Rebuild the sorted (id, slot) view and its pivot levels used by
 * HB_LOOKUP_SORTED after add/reset/import changed the index.  hb_index_lookup
 * and hb_lookup_fetch call it themselves when the view is stale. */
int hb_index_build_sorted(hb_index_t* h, hb_stream_t stream);

/* Raw state in/out (device or host pointers): line_ids[capacity] int64,
 * lru[capacity] int32.  For tests, checkpoints and a host mirror. */
int hb_index_export(hb_index_t* h, int64_t* line_ids, int32_t* lru, hb_stream_t stream);
int hb_index_import(hb_index_t* h, const int64_t* line_ids, const int32_t* lru,
                    hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Row movers.  Rows are opaque byte strings of row_bytes (= dim * elem size); */
/* index arrays are int32 (idx_bytes 4) or int64 (idx_bytes 8).  Out-of-range   */
/* indices are undefined behaviour, as in the reference.                        */
/* ------------------------------------------------------------------------- */
#define HB_MOVER_AUTO 0 /* pick by row size and alignment                      */
#define HB_MOVER_LSU 1  /* vectorised ld.global / st.global                    */
#define HB_MOVER_BULK 2 /* cp.async.bulk through shared memory (TMA engine)    */

/* dst[dst_index[i], :] = src[src_index[i], :]; dst_index NULL means i.
 * Replaces CUDAFetch (src/cuda/uva_fetch.cu:28-45) and CUDAFetch2 (:72-106). */
int hb_rows_gather(const void* src, const void* src_index, void* dst,
                   const void* dst_index /* nullable */, int64_t n, int64_t row_bytes,
                   int idx_bytes, int mover, hb_stream_t stream);

/* dst[dst_index[i], :] = src[i, :] (overwrite; with duplicate indices one of
 * the writers wins).  Replaces CUDASet (src/cuda/uva_set.cu:35-69) and
 * CUDACombine (src/cuda/uva_fetch.cu:212-228), which compute the same thing. */
int hb_rows_scatter(const void* src, void* dst, const void* dst_index, int64_t n,
                    int64_t row_bytes, int idx_bytes, int mover, hb_stream_t stream);

/* g = index_map[index[i]]; dst[i,:] = g != -1 ? cached_src[g,:] : backing_src[index[i],:].
 * found (nullable) receives g != -1.  Replaces CUDAFetchWithCache2
 * (src/cuda/uva_fetch.cu:149-192). */
int hb_rows_gather_cached(const void* backing_src, const void* cached_src,
                          const void* index, const void* index_map, void* dst,
                          uint8_t* found /* nullable */, int64_t n, int64_t row_bytes,
                          int idx_bytes, hb_stream_t stream);

/* g = index_map[index[i]]; (g != -1 ? cached_dst[g,:] : backing_dst[index[i],:]) = src[i,:].
 * Replaces CUDASetWithCache (src/cuda/uva_set.cu:112-154). */
int hb_rows_scatter_cached(const void* src, void* backing_dst, void* cached_dst,
                           const void* index, const void* index_map, int64_t n,
                           int64_t row_bytes, int idx_bytes, hb_stream_t stream);

/* dst[dst_index[i], :] += src[i, :] in fp32 and, when cnt is given,
 * cnt[dst_index[i]] += 1.  Indices must be unique (the reference's assumption,
 * python/EmbCache/server.py:547,565); duplicates go through
 * hb_unique_segsum_f32 first.  Replaces the torch CPU indexing of
 * _accumulate_gradients_cold_local, python/EmbCache/server.py:564-574. */
int hb_rows_accumulate_f32(const float* src, float* dst, const void* dst_index,
                           int32_t* cnt /* nullable */, int64_t n, int64_t dim,
                           int idx_bytes, hb_stream_t stream);

/* Fused cache lookup + cached fetch: slot = lookup(ids[i]);
 * out_rows[i,:] = slot >= 0 ? cache_rows[slot,:] : backing_rows[ids[i],:]
 * (a miss leaves the output row untouched when backing_rows is NULL);
 * locs[i] = slot (nullable), found[i] = slot >= 0 (nullable).
 * One pass for IndexCache.lookup + cudaFetch + the backing-table fetch of
 * python/EmbCache/dist_emb.py:184-243. */
int hb_lookup_fetch(hb_index_t* h, const int64_t* ids, int64_t n, const void* cache_rows,
                    const void* backing_rows /* nullable */, int64_t row_bytes,
                    void* out_rows, int64_t* locs /* nullable */,
                    uint8_t* found /* nullable */, int mode, int mover,
                    hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Hot/cold split, owner search, owner bucketing.                              */
/* ------------------------------------------------------------------------- */
/* Workspace of the stable multi-way partition that split_compact, bucket_pack,
 * grad_split3 and the staging flush share. */
size_t hb_partition_workspace_bytes(int64_t n, int num_classes);

/* v = mask_table[ids[i]]: local = (v==0), hot = (v==1), cold = (v==2), one byte
 * each.  Replaces splitCUDA / cudaSplit (src/cuda/split.cu:12-56). */
int hb_split_masks(const int64_t* ids, int64_t n, const int8_t* mask_table,
                   uint8_t* local_mask, uint8_t* hot_mask, uint8_t* cold_mask,
                   hb_stream_t stream);

/* hb_split_masks fused with the nonzero() calls that follow it in
 * python/EmbCache/dist_emb.py:174-191: index_out holds the positions of the
 * local ids, then of the hot ids, then of the cold ids, each ascending;
 * counts (device int64[3]) their numbers.  Masks are optional (all or none). */
int hb_split_compact(const int64_t* ids, int64_t n, const int8_t* mask_table,
                     uint8_t* local_mask, uint8_t* hot_mask, uint8_t* cold_mask,
                     int64_t* index_out, int64_t* counts, void* workspace,
                     size_t workspace_bytes, hb_stream_t stream);

/* out = in % g.  Replaces Reminder / cudaReminder (src/cuda/binary_search.cu:76-89). */
int hb_owner_mod(const void* in, int64_t n, int idx_bytes, int64_t g, void* out,
                 hb_stream_t stream);
/* out = (upper_bound(range_partition, in) - 1) * g + in % g.  Replaces
 * CUDABinarySearch / cudaBinarySearch (src/cuda/binary_search.cu:45-59). */
int hb_owner_range(const void* in, int64_t n, int idx_bytes, const void* range_partition,
                   int64_t num_part, int64_t g, void* out, hb_stream_t stream);
/* out = upper_bound(sorted, in).  Replaces CUDABinarySearch2 / cudaBinarySearch2
 * (src/cuda/binary_search.cu:61-74). */
int hb_upper_bound(const void* in, int64_t n, int idx_bytes, const void* sorted, int64_t m,
                   void* out, hb_stream_t stream);

/* Bucket (ids, rows, cnt) by owner, stable inside a bucket: the owner search,
 * torch.sort, three gathers and cudaBinarySearch2 of swap_gradients
 * (python/EmbCache/sparse_optim.py:36-55) in one pass with the counts left on
 * the device.  owner = id % g when range_partition is NULL, else the
 * hb_owner_range rule.  rows and cnt are optional.  counts: device
 * int64[num_buckets]; bucket b starts at the sum of the counts before it. */
int hb_bucket_pack(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                   const int64_t* n_dev /* nullable device count capping n */,
                   int64_t row_bytes, int num_buckets, const int64_t* range_partition,
                   int64_t num_part, int64_t g, int64_t* out_ids, void* out_rows,
                   int64_t* out_cnt, int64_t* counts, void* workspace,
                   size_t workspace_bytes, hb_stream_t stream);

/* hb_bucket_pack for hosts that cannot give the library scratch memory or let it
 * allocate: a runtime that owns the device allocator and exposes no workspace
 * hook, a serving loop whose memory plan is frozen, a callback that must not
 * enter the driver's allocator.  No counterpart in the reference (it allocates
 * freely through torch).  The partition's histograms and offsets live in a
 * fixed 132 KiB device array inside the library (every GPU that loads the
 * library holds it until the process exits), which limits one call to
 * hb_bucket_pack_noalloc_max_items() = 1,048,576 ids and
 * hb_bucket_pack_noalloc_max_buckets() = 64 buckets; larger requests return
 * HB_ERR_CAPACITY.  Inputs, outputs and counts are still the caller's.  The
 * call performs no cudaMalloc / cudaFree and calls no allocating routine.  Its
 * FIRST call on each device also asks the runtime for the array's device
 * address (cudaGetSymbolAddress); make that first call outside any stream
 * capture.  All calls on a device share the one array, which keeps whatever the
 * last call wrote: every cell is rewritten before it is read, so nothing needs
 * clearing, but two calls that overlap on the GPU (different streams, or
 * different threads without ordering) race on it -- order them. */
int64_t hb_bucket_pack_noalloc_max_items(void);
int hb_bucket_pack_noalloc_max_buckets(void);
int hb_bucket_pack_noalloc(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                           const int64_t* n_dev, int64_t row_bytes, int num_buckets,
                           const int64_t* range_partition, int64_t num_part, int64_t g,
                           int64_t* out_ids, void* out_rows, int64_t* out_cnt,
                           int64_t* counts, hb_stream_t stream);

/* (ids, rows, cnt) split three ways by a per-node class table, class =
 * table[id] in {0,1,2} (the classes of src/cuda/split.cu:34-44).  out_ids,
 * out_rows, out_cnt are HOST arrays of three device pointers: class c is
 * compacted, in input order, into its own buffers starting at entry 0; a NULL
 * out_ids[c] counts the class without writing it.  counts: device int64[3].
 * cnt / out_cnt are optional; n_dev (nullable device int64) caps n. */
int hb_table_split3(const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                    const int64_t* n_dev, int64_t row_bytes, const int8_t* table,
                    int64_t* const* out_ids, void* const* out_rows, int64_t* const* out_cnt,
                    int64_t* counts, void* workspace, size_t workspace_bytes,
                    hb_stream_t stream);

/* The hot / cold-local / cold-remote selects of DistembSparseGradOptimizer.step
 * (python/EmbCache/sparse_optim.py:243-259) in one pass: out holds the hot rows
 * (hot_mask), then ~hot & local, then ~hot & ~local; counts: device int64[3]. */
int hb_grad_split3(const int64_t* ids, const void* rows, const uint8_t* hot_mask,
                   const uint8_t* local_mask, int64_t n, int64_t row_bytes,
                   int64_t* out_ids, void* out_rows, int64_t* counts, void* workspace,
                   size_t workspace_bytes, hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Hot-node local aggregation.                                                 */
/* ------------------------------------------------------------------------- */
/* Sorted unique ids with the per-id fp32 sum (mean = 0) or mean (mean = 1) of
 * their gradient rows, deterministic.  Replaces only_unique_grads and
 * unique_grads (python/EmbCache/sparse_optim.py:132-157).  counts (nullable):
 * occurrences per id; when mean = 1 and cnt_in is given, 1 + sum of cnt_in,
 * which is also the divisor (the reference starts its counts from ones,
 * sparse_optim.py:145-148).  uniq_ids / sums / counts must hold n entries;
 * num_unique is a device int64.  id_bits: ids are < 2^id_bits - 1 (sort passes).
 * n_dev (nullable device int64) caps n: entries at and beyond it are ignored.
 * seg_counts (nullable, device int64[n / seg_cap]): the input is a sequence of
 * segments of seg_cap entries and only the first seg_counts[s] entries of segment
 * s are valid -- the receive slabs of hb_a2a_push, consumed in place. */
/* The grouping of a batch into runs of equal ids: the input positions sorted by id
 * (stable, so positions ascend inside a run) and the start of every run, with the
 * distinct ids and, when a class table was given, the class of every distinct id and
 * its position among the ids of its class.  What torch.unique(return_inverse,
 * return_counts) computes at python/EmbCache/sparse_optim.py:133, kept so that the
 * forward fetch, the LRU ageing, the miss list and the backward aggregation of one
 * step share one sort.  All pointers are device pointers into the workspace given to
 * hb_runs_build (valid until that workspace is written again). */
typedef struct hb_runs {
  const uint32_t* perm;       /* [n] input position of each sorted element */
  const int64_t* run_start;   /* [num_runs + 1]; run_start[num_runs] = valid entries */
  const int64_t* num_runs;    /* device int64 (= number of distinct ids) */
  int64_t n;
  const void* keys;           /* [n] sorted ids: uint32 (key_bytes 4) or int64 (key_bytes 8) */
  int key_bytes;
  const uint8_t* head;        /* [n] 1 where a run starts */
  const int64_t* uniq_ids;    /* [num_runs] ascending */
  const int8_t* dclass;       /* [num_runs] class of the id, -1 = none; NULL without a table */
  const int32_t* dpos;        /* [num_runs] position among the ids of its class */
  const int64_t* class_counts;/* device int64[4]: distinct ids of class 0, 1, 2, other */
  const int64_t* n_dev;       /* nullable device count of valid input entries */
  const int32_t* base8;       /* [ceil(n / 8)] runs that start before sorted entry 8k: with the
                                 head flags it gives the run of any entry in two small loads */
} hb_runs_t;

/* Optional split of the aggregated rows by a per-node class table (class =
 * table[id] in {0,1,2}, the classes of src/cuda/split.cu:34-44): the row, id and
 * count of every unique id go straight to the buffers of its class, compacted
 * from entry 0 in id order, instead of to uniq_ids / sums / counts -- the hot /
 * cold selects of python/EmbCache/sparse_optim.py:243-259 without a second pass
 * over the rows.  A NULL out_rows[c] / out_ids[c] / out_cnt[c] drops that part of
 * class c.  class_counts: device int64[3]. */
typedef struct hb_class_split {
  const int8_t* table;
  int64_t table_len;          /* entries of table; ids at and beyond it have no class */
  int64_t* out_ids[3];
  float* out_rows[3];
  int64_t* out_cnt[3];
  int64_t* class_counts;
} hb_class_split_t;

size_t hb_unique_segsum_workspace_bytes(int64_t n, int64_t dim);
int hb_unique_segsum_f32(const int64_t* ids, const float* grads, const int64_t* cnt_in,
                         int64_t n, const int64_t* n_dev, const int64_t* seg_counts,
                         int64_t seg_cap, int64_t dim, int id_bits, int mean,
                         int64_t* uniq_ids,
                         float* sums, int64_t* counts /* nullable */, int64_t* num_unique,
                         hb_runs_t* runs_out /* nullable, host */,
                         const hb_class_split_t* split /* nullable, host; then uniq_ids, sums,
                         counts may be NULL */, void* workspace, size_t workspace_bytes,
                         hb_stream_t stream);

/* Sort a batch once: runs of equal ids (hb_runs_t above).  class_table (nullable, int8
 * per node, table_len entries): class and per-class position of every distinct id; with
 * class_ids_out (nullable host array of 3 device buffers, each nullable) the distinct
 * ids of class c are also written to class_ids_out[c] from entry 0, ascending -- the id
 * half of the hot / cold selects of python/EmbCache/sparse_optim.py:243-259 --
 * and class_counts_out (nullable device int64[3]) receives their numbers.
 * uniq_ids_out / num_unique_out: nullable second copies in caller memory.  n_dev,
 * seg_counts, seg_cap, id_bits as for hb_unique_segsum_f32.  An id that is negative or
 * not below 2^id_bits - 1 raises HB_ERR_INVALID in the device status word. */
size_t hb_runs_workspace_bytes(int64_t n);
int hb_runs_build(const int64_t* ids, int64_t n, const int64_t* n_dev /* nullable */,
                  const int64_t* seg_counts /* nullable */, int64_t seg_cap, int id_bits,
                  const int8_t* class_table /* nullable */, int64_t table_len,
                  int64_t* const* class_ids_out /* nullable, host */,
                  int64_t* class_counts_out /* nullable */, int64_t* uniq_ids_out /* nullable */,
                  int64_t* num_unique_out /* nullable */, void* workspace, size_t workspace_bytes,
                  hb_runs_t* runs_out /* host */, hb_stream_t stream);

/* The aggregation half of hb_unique_segsum_f32 over runs that already exist (the ids of
 * `grads` are the ids the runs were built from, same order): per-id sums or means into
 * `sums` [num_runs][dim] (+ counts), or with `split` straight into the class buffers
 * out_rows / out_cnt (table, out_ids and class_counts of `split` are not used here: the
 * runs carry the classes).  python/EmbCache/sparse_optim.py:134-139 (index_add_). */
size_t hb_segsum_runs_workspace_bytes(int64_t n, int64_t dim);
int hb_segsum_runs_f32(const hb_runs_t* runs /* host */, const float* grads,
                       const int64_t* cnt_in /* nullable */, int64_t dim, int mean, float* sums,
                       int64_t* counts /* nullable */, const hb_class_split_t* split /* nullable */,
                       void* workspace, size_t workspace_bytes, hb_stream_t stream);

/* hb_lookup_fetch (or hb_lookup_fetch_sharded when `table` is given) over a batch that
 * hb_runs_build has sorted: same outputs at the same batch positions (locs, found,
 * out_rows), in two launches (three with a sharded table).  The first works per DISTINCT id:
 * index probe, the slot of every run (run_slots[u], nullable output, n entries) and the place
 * its row is read from; rows that live in another GPU's shard are then copied once, by a
 * launch of their own, into a staging buffer on this GPU (up to 1 GiB of them; the rest is
 * read from the owner directly), so every remote row crosses NVLink once per step however
 * often its id occurs.  The last launch writes the row of every entry to its batch position;
 * entries of one run inside a warp share one read.
 * locs (nullable): the per-position slots, 8-byte writes scattered over the batch (about
 * 15 % of the time at 512-byte rows): hb_index_touch_lru_runs and hb_runs_miss_list take
 * run_slots instead.  out_rows == NULL leaves the last launch out (the lookup of the distinct
 * ids; remote rows staged).  A miss whose id is not below the table's row count leaves its
 * output rows untouched and raises HB_ERR_INVALID in the device status word.
 * python/EmbCache/dist_emb.py:184-243. */
size_t hb_lookup_fetch_runs_workspace_bytes(int64_t n, int64_t row_bytes, int sharded);
int hb_lookup_fetch_runs(hb_index_t* h, const hb_runs_t* runs /* host */, const void* cache_rows,
                         const void* backing_rows /* nullable */, int64_t backing_num_rows,
                         hb_peer_table_t* table /* nullable */, int64_t row_bytes, void* out_rows,
                         int64_t* locs /* nullable */, uint8_t* found /* nullable */,
                         int64_t* run_slots /* nullable */, int mode, void* workspace,
                         size_t workspace_bytes, hb_stream_t stream);

/* The same forward fetch with the OWNERS delivering the remote rows (several GPUs; on this pool
 * scattered peer loads of rows collapse to a few tens of GB/s once more than one peer is read,
 * while peer stores run at the links' bandwidth).  Three calls around two fences:
 *   hb_runs_resolve_requests  the first launch of hb_lookup_fetch_runs; a run whose row lives on
 *       another GPU is not copied but asked for: the request (id, run u) is stored straight into
 *       this rank's slab of the owner's receive area of `requests` (an hb_a2a exchange of
 *       cap_rows >= the distinct ids one owner can be asked for; its row payload is not used),
 *       id in the ids array and u in the cnt array; u is also the row of stage_rows the owner is
 *       to fill.  *parity_out: the receive area filled, as from hb_a2a_push.  A slab that is full
 *       raises HB_ERR_CAPACITY in the device status word.  Runs at and beyond stage_cap are read
 *       from the owner directly by the last launch.  stage_rows: this GPU's stage,
 *       [stage_cap][row_bytes], that the peers have mapped (the local shard of an hb_peer_table
 *       created for the purpose).
 *   hb_a2a_fence(requests); every rank, as an owner: hb_fetch_serve on the receive view of that
 *       area; hb_a2a_fence(requests)
 *   hb_runs_expand            the last launch: rows to their batch positions, with locs / found.
 * workspace: hb_lookup_fetch_runs_workspace_bytes(n, row_bytes, 0), the same for both calls and
 * untouched in between.
 * hb_runs_expand also finishes a hb_lookup_fetch_runs call that was given out_rows == NULL (same
 * workspace), so that a caller can put work between the two launches: the index maintenance of
 * the batch (LRU ageing, insertion of the misses) needs the first only.  cache_rows / other_rows:
 * what the first call was given as cache rows and as backing table or stage (their alignment
 * decides the width of the copies); peer_sources: non-zero when the first call had a table
 * sharded over several GPUs (rows may then be read from a peer's memory, with plain loads). */
int hb_runs_resolve_requests(hb_index_t* h, const hb_runs_t* runs /* host */, const void* cache_rows,
                             hb_peer_table_t* table, int64_t row_bytes, void* stage_rows, int64_t stage_cap,
                             int64_t* run_slots /* nullable */, hb_a2a_t* requests, int* parity_out /* host */,
                             int mode, void* workspace, size_t workspace_bytes, hb_stream_t stream);
int hb_runs_expand(const hb_runs_t* runs /* host */, const void* cache_rows, const void* other_rows /* nullable */,
                   int64_t row_bytes, int peer_sources, void* out_rows, int64_t* locs /* nullable */,
                   uint8_t* found /* nullable */, const int64_t* run_slots /* nullable: the workspace's */,
                   void* workspace, size_t workspace_bytes, hb_stream_t stream);

/* The distinct ids of class want_class (< 0: any) that the lookup missed (locs[position]
 * < 0; locs_kind: locs holds a slot per batch position (0), per sorted entry (1) or per
 * run (2, the run_slots of hb_lookup_fetch_runs)), ascending, at
 * most cap of them: miss_ids[cap] (entries past the count are -1, which
 * hb_index_add ignores), miss_src[cap] = a batch position of the id (its row in the fetch
 * output), *miss_count.  The uncached cold ids that DistEmbeddingTensor.__call__ sends to
 * the cache server, python/EmbCache/dist_emb.py:218-259. */
size_t hb_runs_miss_list_workspace_bytes(int64_t n);
int hb_runs_miss_list(const hb_runs_t* runs /* host */, const int64_t* locs, int locs_kind,
                      int want_class, int64_t cap, int64_t* miss_ids, int64_t* miss_src,
                      int64_t* miss_count, void* workspace, size_t workspace_bytes,
                      hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Cold-gradient staging table (the reference's cache-server buffers).         */
/* ------------------------------------------------------------------------- */
/* Caller-owned device buffers, python/EmbCache/server.py:76-160:
 * _grad_cache_buff, _grad_cnt_cache_buff, _grad_idx_cache_buff,
 * _grad_iter_count, _grad_iter_threshold (and their _local_ twins). */
typedef struct hb_staging {
  float* grad;             /* [slots][dim], zero when idle */
  int32_t* cnt;            /* [slots] messages accumulated since the last flush */
  int64_t* idx;            /* [slots] id staged in the slot, -1 = none */
  int32_t* iter_count;     /* [slots] iterations since the last flush */
  int32_t* iter_threshold; /* [slots] flush after this many iterations */
  int64_t slots;
  int64_t dim;
} hb_staging_t;

/* Cold remote gradients, _accumulate_gradients_cold_remote, server.py:546-562:
 * slot = lookup(id); found: idx[slot] = id, iter_threshold[slot] =
 * threshold_table[id] (default_threshold when the table is NULL), grad[slot] +=
 * grads[i], cnt[slot] += 1; a miss is dropped (counted in *dropped, a device
 * int64, when given).  ids must be unique.  n_dev (nullable device int64) caps n,
 * so that the count left on the device by hb_unique_segsum_f32 can be used
 * without a host read.  locs_out (nullable, n entries) receives the slots, for
 * hb_index_touch_lru: the server's lookup is the CPU one, which ages the LRU
 * counters.  The staging table has one slot per cache slot. */
int hb_staging_accumulate_cached(hb_index_t* h, const hb_staging_t* s, const int64_t* ids,
                                 const float* grads, int64_t n, const int64_t* n_dev,
                                 const int32_t* threshold_table, int32_t default_threshold,
                                 int mode, int64_t* dropped, int64_t* locs_out,
                                 hb_stream_t stream);

/* Cold local gradients, _accumulate_gradients_cold_local, server.py:564-574:
 * slot = (id - id_offset) / id_stride; grad[slot] += grads[i]; cnt[slot] += 1;
 * idx[slot] = id.  ids must be unique. */
int hb_staging_accumulate_direct(const hb_staging_t* s, const int64_t* ids, const float* grads,
                                 int64_t n, const int64_t* n_dev, int64_t id_offset,
                                 int64_t id_stride, hb_stream_t stream);

/* _send_staled_gradients, server.py:346-497: slots with cnt > 0 and (iter_count
 * >= iter_threshold or cnt >= cnt_threshold) leave in slot order, bucketed by
 * id % num_clients (counts: device int64[num_clients]); their rows are read AND
 * zeroed, cnt and iter_count return to 0 and, when an index is given, their ids
 * are reset in it; other slots with cnt > 0 age by one iteration.  (The
 * reference zeroes a temporary copy of the rows, server.py:414, so its buffers
 * are never cleared; this library implements the intended read-and-zero.)
 * out_cap: entries the outputs hold; 0 = `slots`.  A smaller output needs num_clients
 * == 1 (no bucketing): the first out_cap stale slots in slot order leave, the others
 * stay staged and age like live ones until the next flush; counts[0] then still reports
 * ALL stale slots, so a consumer takes min(counts[0], out_cap) rows. */
size_t hb_staging_flush_workspace_bytes(int64_t slots, int num_clients);
int hb_staging_flush(hb_index_t* h /* nullable */, const hb_staging_t* s, int32_t cnt_threshold,
                     int num_clients, int64_t out_cap, int64_t* out_ids, float* out_rows,
                     int64_t* out_cnt, int64_t* counts, void* workspace, size_t workspace_bytes,
                     hb_stream_t stream);

/* _update_cache, server.py:499-544: locs = add(ids); cache_rows[locs[i]] =
 * emb_rows[i] where locs[i] >= 0; the staging state of those slots is cleared
 * (s may be NULL). */
size_t hb_staging_insert_workspace_bytes(int64_t n);
int hb_staging_insert(hb_index_t* h, const hb_staging_t* s /* nullable */, const int64_t* ids,
                      const void* emb_rows, int64_t n, void* cache_rows, int64_t row_bytes,
                      int64_t* locs_out, void* workspace, size_t workspace_bytes,
                      hb_stream_t stream);
/* The same with the embedding of ids[i] at emb_rows[row_index[i]] (row_index NULL: at
 * emb_rows[i]): a step inserts the cold ids its lookup missed from the rows its fetch
 * has just written (hb_runs_miss_list gives ids and row_index), as the reference's
 * trainer ships them to the server (python/EmbCache/dist_emb.py:218-259).  Negative
 * ids (padding) are ignored and get locs_out = -1. */
/* The second half of hb_staging_insert_gather for callers that run hb_index_add themselves (and
 * put other work between the two): rows emb_rows[row_index[i]] (row_index nullable: i) into the
 * cache rows at locs[i] where last_writer[i] is set (both from hb_index_add), staging slots of
 * the inserted entries reset. */
int hb_staging_insert_rows(const hb_staging_t* s /* nullable */, const void* emb_rows, const int64_t* row_index,
                           int64_t n, void* cache_rows, int64_t row_bytes, const int64_t* locs,
                           const uint8_t* last_writer, hb_stream_t stream);
int hb_staging_insert_gather(hb_index_t* h, const hb_staging_t* s /* nullable */,
                             const int64_t* ids, const void* emb_rows,
                             const int64_t* row_index /* nullable */, int64_t n, void* cache_rows,
                             int64_t row_bytes, int64_t* locs_out, void* workspace,
                             size_t workspace_bytes, hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Sparse optimiser update on the owning shard.                                */
/* ------------------------------------------------------------------------- */
/* Local row of an id: (id - id_offset) / id_stride, ids outside [0, rows) are
 * skipped; ids must be unique.  grads are divided by cnt when cnt is given
 * (the is_unique path, sparse_optim.py:608-611).  emb is fp32 (emb_elem_bytes
 * 4) or fp16 (2); state is fp32.
 *
 * SparseAdam.update, python/EmbCache/sparse_optim.py:590-685: step += 1;
 * mem = b1*mem + (1-b1)*g; power = b2*power + (1-b2)*g*g;
 * emb -= lr * (mem/(1-b1^step)) / (sqrt(power/(1-b2^step)) + eps). */
int hb_sparse_adam(const int64_t* ids, const float* grads, const int64_t* cnt, int64_t n,
                   const int64_t* n_dev, int64_t dim, int64_t id_offset, int64_t id_stride,
                   int64_t rows, float* step, float* mem, float* power, void* emb,
                   int emb_elem_bytes, double lr, double beta1, double beta2, double eps,
                   hb_stream_t stream);
/* Sparse Adagrad: sum += g*g; emb -= lr * g / (sqrt(sum) + eps).  The reference
 * ships no Adagrad (only SparseAdam); this rule has no reference counterpart to
 * compare against. */
int hb_sparse_adagrad(const int64_t* ids, const float* grads, const int64_t* cnt, int64_t n,
                      const int64_t* n_dev, int64_t dim, int64_t id_offset, int64_t id_stride,
                      int64_t rows, float* state_sum, void* emb, int emb_elem_bytes, double lr,
                      double eps, hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Owner-partitioned exchange over peer memory (one box, NVLink / NVSwitch).   */
/* ------------------------------------------------------------------------- */
/* Replaces the owner search + torch.sort + gathers + four all_to_all_single
 * calls + two host reads of swap_gradients (python/EmbCache/sparse_optim.py:
 * 36-118): hb_a2a_push buckets (id, cnt, row) by owner = id % world and stores
 * every bucket straight into the owner GPU's receive slab (CUDA IPC mapping,
 * plain stores, no multicast).  Every rank owns two receive areas that
 * alternate from push to push; between a push and the use of what was received
 * the caller runs ONE barrier among the ranks on the same stream (e.g. a
 * one-element NCCL all-reduce).  A slab holds cap_rows rows per source rank;
 * rows beyond it are dropped and HB_ERR_CAPACITY is recorded for
 * hb_device_status.  Set-up: create on every rank, exchange the handles
 * (hb_a2a_handle_bytes() bytes each) by any host channel, connect. */
int hb_a2a_create(int rank, int world, int64_t cap_rows, int64_t row_bytes, hb_a2a_t** out);
size_t hb_a2a_handle_bytes(void);
int hb_a2a_export_handle(hb_a2a_t* a, void* handle_out /* host */);
int hb_a2a_connect(hb_a2a_t* a, const void* handles /* host, world entries in rank order */);
int hb_a2a_disconnect(hb_a2a_t* a); /* first step of a tear-down, see hb_peer_table_disconnect */
int hb_a2a_destroy(hb_a2a_t* a);
size_t hb_a2a_push_workspace_bytes(int64_t n, int world);
/* sent_counts (nullable): device int64[world], rows sent to each owner.
 * *parity_out: which receive area this push used on every rank. */
int hb_a2a_push(hb_a2a_t* a, const int64_t* ids, const void* rows, const int64_t* cnt /* nullable: 1 */,
                int64_t n, const int64_t* n_dev, int64_t* sent_counts, int* parity_out,
                void* workspace, size_t workspace_bytes, hb_stream_t stream);
/* The barrier between a push and the use of what was received, without a
 * collective library: every rank stores its exchange number into every peer's
 * flag array and polls its own until all peers have done so.  The wait has an
 * iteration limit (about a second); a rank that gives up records HB_ERR_TIMEOUT
 * for hb_device_status and returns.  Every rank must call it once per push, and
 * the ranks must be on different GPUs.  The exchange number lives on the device,
 * so a captured graph holding push + fence can be replayed. */
int hb_a2a_fence(hb_a2a_t* a, hb_stream_t stream);
/* Back to the state after hb_a2a_connect (exchange number 0, flags and counts cleared,
 * next push into area 0).  After a fence gave up on a missing peer the ranks' exchange
 * numbers differ; when the host side has agreed that every rank is back, ALL ranks call
 * this between two host barriers (before: nobody still pushes or polls; after: nobody
 * pushes into an area that is being cleared) and the exchange works again.  Graphs
 * captured over the exchange stay valid (they hold no exchange number), but their
 * alternation restarts with the graph of area 0. */
int hb_a2a_reset(hb_a2a_t* a, hb_stream_t stream);
/* The bounded wait that hb_a2a_fence uses, on its own: a one-thread kernel polls
 * the device word *flag until it is >= value, for at most about a second; if it
 * gives up it records HB_ERR_TIMEOUT for hb_device_status and returns, and the
 * context stays usable.  (Failure detection is built on this: a peer that never
 * arrives shows up as a status code, never as a hung or trapped GPU.) */
int hb_wait_flag(const uint64_t* flag, uint64_t value, hb_stream_t stream);
/* This rank's receive area of a parity: ids/cnt [world][cap_rows], rows
 * [world][cap_rows][row_bytes], counts[world] (device int64: rows from each
 * source).  Feed hb_unique_segsum_f32 with seg_counts = counts, seg_cap = cap_rows. */
int hb_a2a_recv_view(hb_a2a_t* a, int parity, int64_t** ids, void** rows, int64_t** cnt,
                     int64_t** counts, int64_t* cap_rows);

/* unique_grads (python/EmbCache/sparse_optim.py:142-157) on the owner for slabs whose
 * ids are strictly ascending within each segment, which is what hb_a2a_push delivers
 * when every rank sends the sorted unique ids of its own aggregation: a merge of
 * num_seg sorted lists instead of a sort.  Layout and results as hb_unique_segsum_f32
 * with seg_counts (ids/cnt [num_seg][seg_cap], rows [num_seg][seg_cap][dim]; unique ids
 * ascending, rows added in segment order, mean != 0 divides by the count, which starts
 * from one when cnt is given; out_counts nullable).  Segments that are not ascending
 * give undefined results. */
size_t hb_merge_sorted_slabs_workspace_bytes(int64_t num_seg, int64_t seg_cap);
int hb_merge_sorted_slabs_f32(const int64_t* ids, const float* rows, const int64_t* cnt /* nullable */,
                              const int64_t* seg_counts, int64_t num_seg, int64_t seg_cap, int64_t dim,
                              int mean, int64_t* uniq_ids, float* out_rows,
                              int64_t* out_counts /* nullable */, int64_t* num_unique,
                              void* workspace, size_t workspace_bytes, hb_stream_t stream);

/* ------------------------------------------------------------------------- */
/* Table sharded over the GPUs of one box, readable from every GPU.            */
/* ------------------------------------------------------------------------- */
/* The forward direction of the owner partitioning.  The row of id lives on rank
 * id % world at local row id / world (python/EmbCache/sparse_optim.py:38,
 * cache.py:149-150); every shard is mapped into every process (CUDA IPC), and
 * the kernels below read the authoritative row of any id with plain loads over
 * NVLink.  Replaces the pull of remote rows from DGL's DistTensor through the
 * host, `self.tensor[remote_ids.cpu()]` (python/EmbCache/dist_emb.py:241-243),
 * in the manner of the reference's own unified-addressing reads of pinned host
 * memory (src/cuda/uva_fetch.cu:72-106).  Rows are multiples of 16 bytes.
 * Set-up as hb_a2a_*: create on every rank, exchange the handles, connect.  A
 * single process that drives several GPUs itself passes the shard pointers with
 * hb_peer_table_set_peer instead (peer access enabled by the caller).
 * Ordering is the caller's: all ranks pass a fence (hb_a2a_fence or a
 * collective on the stream) between an owner's update of its shard and the
 * next read by anyone. */
int hb_peer_table_create(int rank, int world, int64_t num_rows /* whole table */, int64_t row_bytes,
                         hb_peer_table_t** out);
size_t hb_peer_table_handle_bytes(void);
int hb_peer_table_export_handle(hb_peer_table_t* t, void* handle_out /* host */);
int hb_peer_table_connect(hb_peer_table_t* t, const void* handles /* host, world entries in rank order */);
int hb_peer_table_set_peer(hb_peer_table_t* t, int rank, const void* shard_rows);
/* This rank's shard: rows_local = ceil((num_rows - rank) / world) rows. */
int hb_peer_table_local(hb_peer_table_t* t, void** rows, int64_t* rows_local);
/* Tear-down of anything shared through CUDA IPC (this table, an exchange) takes two steps
 * with a barrier of all ranks before each: every rank disconnects (closes its mappings of the
 * peers' memory), then every rank destroys (frees its own).  Freeing memory that a peer still
 * has mapped is undefined behaviour of the IPC interface. */
int hb_peer_table_disconnect(hb_peer_table_t* t);
int hb_peer_table_destroy(hb_peer_table_t* t);
/* dst[i, :] = row of ids[i] from its owner's shard, i < min(n, *n_dev). */
int hb_peer_table_gather(hb_peer_table_t* t, const int64_t* ids, int64_t n,
                         const int64_t* n_dev /* nullable */, void* dst, hb_stream_t stream);
/* hb_lookup_fetch whose misses read the owner's shard: out_rows[i] = cached row
 * when the index holds ids[i], else the authoritative row.  The one pass that
 * python/EmbCache/dist_emb.py:184-243 makes of lookup, cache fetch and the
 * DistTensor pull. */
/* The owner's half of hb_runs_resolve_requests: for every requester s (segment s of seg_cap
 * entries, req_counts[s] of them valid: the receive view of the hb_a2a exchange that carried the
 * requests) the row of req_ids[k] in THIS rank's shard of `table` is stored into row req_rows[k] of
 * rank s's stage.  stages: an hb_peer_table whose local shard on every rank is that rank's stage
 * (num_rows = world x rows of one stage).  A request for a row this rank does not own, or beyond
 * the stage, is skipped and raises HB_ERR_INVALID in the device status word. */
int hb_fetch_serve(hb_peer_table_t* table, hb_peer_table_t* stages, const int64_t* req_ids,
                   const int64_t* req_rows, const int64_t* req_counts, int64_t seg_cap, hb_stream_t stream);

int hb_lookup_fetch_sharded(hb_index_t* h, const int64_t* ids, int64_t n, const void* cache_rows,
                            hb_peer_table_t* table, void* out_rows, int64_t* locs /* nullable */,
                            uint8_t* found /* nullable */, int mode, hb_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* HADES_B200_H_ */
