/*
 * TEST INFRASTRUCTURE -- not part of the product.  Plain-C, single-threaded
 * restatement of the reference's algorithms for the embedding-cache hot path,
 * used only by tests/, __graft_entry__.smoke() and bench.py's cpu_baseline leg
 * as the checker for the CUDA library.  Each function cites the reference
 * file:line (paths inside the HADES project) that it follows.
 *
 * Parity is pinned: tests/test_oracle_pins.py checks this file against the
 * reference's own compiled CPU index (oracle/_ref, built from the reference
 * sources where they lie) and against golden vectors generated from it
 * (tests/golden/).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define WAYS 8 /* CACHE_LINE_SIZE, src/cache/cache_line.h:5 */

typedef struct {
  int64_t lines;  /* index_size, src/cache/cache.h:140 */
  int64_t* ids;   /* [lines][WAYS], -1 = empty (cache_line.h:13-18) */
  int32_t* lru;   /* [lines][WAYS] access_table (cache_line.h:10) */
} oracle_index;

/* SACacheIndex ctor + _init_cache, src/cache/cache.h:40-48,138-143 */
oracle_index* oracle_index_create(int64_t cache_size) {
  oracle_index* x = (oracle_index*)malloc(sizeof(oracle_index));
  x->lines = (cache_size + WAYS - 1) / WAYS;
  x->ids = (int64_t*)malloc(sizeof(int64_t) * x->lines * WAYS);
  x->lru = (int32_t*)calloc(x->lines * WAYS, sizeof(int32_t));
  for (int64_t i = 0; i < x->lines * WAYS; ++i) x->ids[i] = -1;
  return x;
}

void oracle_index_destroy(oracle_index* x) {
  if (!x) return;
  free(x->ids);
  free(x->lru);
  free(x);
}

int64_t oracle_index_lines(const oracle_index* x) { return x->lines; }
/* get_cache_size_ / get_capacity_, src/cache/cache.h:176,185-187 */
int64_t oracle_index_capacity(const oracle_index* x) { return x->lines * WAYS; }
/* get_space_, src/cache/cache.h:189-192: sizeof(cache_line) = 8*8 + 8*4 */
int64_t oracle_index_space(const oracle_index* x) { return x->lines * 96; }

/* get_valid_entries_, src/cache/cache.h:178-183 */
int64_t oracle_index_valid(const oracle_index* x) {
  int64_t v = 0;
  for (int64_t i = 0; i < x->lines * WAYS; ++i) v += x->ids[i] != -1;
  return v;
}

/* _add, src/cache/cache.h:51-88, in input order (OMP_NUM_THREADS=1) */
void oracle_index_add(oracle_index* x, const int64_t* ids, int64_t n, int64_t* locs) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    if (id < 0) { locs[i] = -1; continue; } /* the reference indexes out of bounds here */
    const int64_t line = id % x->lines;
    int64_t* lid = x->ids + line * WAYS;
    int32_t* cnt = x->lru + line * WAYS;
    /* find_or_empty_entry, cache_line.h:67-78 */
    int idx = -1, exist = 0;
    for (int w = 0; w < WAYS; ++w) {
      if (lid[w] == id) { idx = w; exist = 1; break; }
      else if (lid[w] == -1) idx = w;
    }
    if (idx >= 0) {
      if (!exist) { lid[idx] = id; cnt[idx] = 0; } /* set_id, cache_line.h:20-24 */
      locs[i] = line * WAYS + idx;
    } else {
      /* find_lru, cache_line.h:92-103 */
      int best = 0;
      int32_t tmp = cnt[0];
      for (int w = 0; w < WAYS; ++w)
        if (cnt[w] > tmp && cnt[w] != 0) { best = w; tmp = cnt[w]; }
      if (tmp == 0) {
        locs[i] = -1;
      } else {
        lid[best] = id;
        cnt[best] = 0;
        locs[i] = line * WAYS + best;
      }
    }
  }
}

/* _lookup, src/cache/cache.h:90-104; touch != 0 applies access_loc
 * (cache_line.h:80-86) as the CPU lookup does, touch == 0 is the GPU lookup
 * (src/cache/lookup.cu:13-44), which leaves the counters alone. */
void oracle_index_lookup(oracle_index* x, const int64_t* ids, int64_t n, int64_t* locs, int touch) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    locs[i] = -1;
    if (id < 0) continue;
    const int64_t line = id % x->lines;
    const int64_t* lid = x->ids + line * WAYS;
    int32_t* cnt = x->lru + line * WAYS;
    for (int w = 0; w < WAYS; ++w) {
      if (lid[w] == id) { /* find, cache_line.h:49-55 */
        locs[i] = line * WAYS + w;
        if (touch) {
          for (int k = 0; k < WAYS; ++k) cnt[k]++;
          cnt[w] = 0;
        }
        break;
      }
    }
  }
}

/* access_loc for a list of already resolved slots, in order */
void oracle_index_touch(oracle_index* x, const int64_t* locs, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    if (locs[i] < 0) continue;
    int32_t* cnt = x->lru + (locs[i] / WAYS) * WAYS;
    for (int k = 0; k < WAYS; ++k) cnt[k]++;
    cnt[locs[i] % WAYS] = 0;
  }
}

/* _reset, src/cache/cache.h:106-118 */
void oracle_index_reset(oracle_index* x, const int64_t* ids, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = ids[i];
    if (id < 0) continue;
    const int64_t line = id % x->lines;
    for (int w = 0; w < WAYS; ++w) {
      if (x->ids[line * WAYS + w] == id) {
        x->ids[line * WAYS + w] = -1;
        x->lru[line * WAYS + w] = 0;
        break;
      }
    }
  }
}

/* _getall, src/cache/cache.h:120-135: slot order, at most len pairs */
int64_t oracle_index_getall(const oracle_index* x, int64_t* ids, int64_t* locs, int64_t len) {
  int64_t k = 0;
  for (int64_t s = 0; s < x->lines * WAYS && k < len; ++s) {
    if (x->ids[s] != -1) {
      ids[k] = x->ids[s];
      locs[k] = s;
      ++k;
    }
  }
  return k;
}

void oracle_index_export(const oracle_index* x, int64_t* ids, int32_t* lru) {
  memcpy(ids, x->ids, sizeof(int64_t) * x->lines * WAYS);
  memcpy(lru, x->lru, sizeof(int32_t) * x->lines * WAYS);
}

/* ---- row movers: the loops of src/cuda/uva_fetch.cu and src/cuda/uva_set.cu ---- */
static int64_t idx_at(const void* p, int64_t i, int idx_bytes) {
  return idx_bytes == 8 ? ((const int64_t*)p)[i] : (int64_t)((const int32_t*)p)[i];
}

/* UVAFetchKernel, uva_fetch.cu:10-26 (dst_index NULL: UVAFetchKernel2, :47-61) */
void oracle_rows_gather(const char* src, const void* si, char* dst, const void* di, int64_t n,
                        int64_t row_bytes, int idx_bytes) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t d = di ? idx_at(di, i, idx_bytes) : i;
    memcpy(dst + d * row_bytes, src + idx_at(si, i, idx_bytes) * row_bytes, row_bytes);
  }
}

/* UVASetKernel, uva_set.cu:10-24 == UVACombineKernel, uva_fetch.cu:194-210 */
void oracle_rows_scatter(const char* src, char* dst, const void* di, int64_t n, int64_t row_bytes,
                         int idx_bytes) {
  for (int64_t i = 0; i < n; ++i)
    memcpy(dst + idx_at(di, i, idx_bytes) * row_bytes, src + i * row_bytes, row_bytes);
}

/* CUDAFetchWithCacheKernel2, uva_fetch.cu:107-130 */
void oracle_rows_gather_cached(const char* backing, const char* cached, const void* index,
                               const void* map, char* dst, uint8_t* found, int64_t n,
                               int64_t row_bytes, int idx_bytes) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t idx = idx_at(index, i, idx_bytes);
    const int64_t g = idx_at(map, idx, idx_bytes);
    memcpy(dst + i * row_bytes, g != -1 ? cached + g * row_bytes : backing + idx * row_bytes,
           row_bytes);
    if (found) found[i] = g != -1;
  }
}

/* CUDASetWithCacheKernel, uva_set.cu:70-93 */
void oracle_rows_scatter_cached(const char* src, char* backing, char* cached, const void* index,
                                const void* map, int64_t n, int64_t row_bytes, int idx_bytes) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t idx = idx_at(index, i, idx_bytes);
    const int64_t g = idx_at(map, idx, idx_bytes);
    memcpy(g != -1 ? cached + g * row_bytes : backing + idx * row_bytes, src + i * row_bytes,
           row_bytes);
  }
}

/* ---- split, src/cuda/split.cu:34-44: 0 local, 1 remote hot, 2 remote cold ---- */
void oracle_split(const int64_t* ids, int64_t n, const int8_t* mask, uint8_t* local,
                  uint8_t* hot, uint8_t* cold) {
  for (int64_t i = 0; i < n; ++i) {
    const int8_t v = mask[ids[i]];
    local[i] = v == 0;
    hot[i] = v == 1;
    cold[i] = v == 2;
  }
}

/* ---- owner search, src/cuda/binary_search.cu ---- */
static int64_t upper_bound_i64(const int64_t* a, int64_t n, int64_t v) {
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) / 2;
    if (a[mid] <= v) lo = mid + 1; else hi = mid;
  }
  return lo;
}

/* ReminderKernel, binary_search.cu:35-43 */
void oracle_owner_mod(const int64_t* in, int64_t n, int64_t g, int64_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = in[i] % g;
}

/* BinarySearchKernel, binary_search.cu:10-21 */
void oracle_owner_range(const int64_t* in, int64_t n, const int64_t* range, int64_t parts,
                        int64_t g, int64_t* out) {
  for (int64_t i = 0; i < n; ++i)
    out[i] = (upper_bound_i64(range, parts, in[i]) - 1) * g + in[i] % g;
}

/* BinarySearchKernel2, binary_search.cu:23-33 */
void oracle_upper_bound(const int64_t* in, int64_t n, const int64_t* sorted, int64_t m,
                        int64_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = upper_bound_i64(sorted, m, in[i]);
}
