// TEST INFRASTRUCTURE -- not part of the product.  C-callable doorway into the
// reference's own CPU cache index: this file only #includes the reference header
// src/cache/cache.h from where the reference checkout lies and forwards to the
// public methods that its pybind module binds (src/pybind.cc:17-33).  No reference
// source is copied.  Built into oracle/_ref/ by oracle/build_oracle.py.
#include <omp.h>

#include <vector>

#include "cache/cache.h"

using RefIndex = distemb::SACacheIndex<int64_t, int64_t>;  // src/pybind.cc:13-14

namespace {
torch::Tensor wrap(const int64_t* p, int64_t n) {
  return torch::from_blob(const_cast<int64_t*>(p), {n},
                          torch::TensorOptions().dtype(torch::kInt64));
}
}  // namespace

extern "C" {

// heap-backed constructor, src/cache/cache.h:138-143 (no shared memory, no pinning)
void* ref_index_create(int64_t cache_size) { return new RefIndex((size_t)cache_size); }
void ref_index_destroy(void* h) { delete static_cast<RefIndex*>(h); }
void ref_set_threads(int n) { omp_set_num_threads(n); }
int ref_max_threads() { return omp_get_max_threads(); }

int64_t ref_index_size(void* h) { return static_cast<RefIndex*>(h)->get_cache_size_(); }
int64_t ref_index_capacity(void* h) { return (int64_t) static_cast<RefIndex*>(h)->get_capacity_(); }
int64_t ref_index_space(void* h) { return (int64_t) static_cast<RefIndex*>(h)->get_space_(); }
int64_t ref_index_valid(void* h) { return static_cast<RefIndex*>(h)->get_valid_entries_(); }

void ref_index_add(void* h, const int64_t* ids, int64_t n, int64_t* locs) {
  auto out = static_cast<RefIndex*>(h)->add_(wrap(ids, n));
  memcpy(locs, out.data_ptr<int64_t>(), n * sizeof(int64_t));
}

void ref_index_lookup(void* h, const int64_t* ids, int64_t n, int64_t* locs) {
  auto out = static_cast<RefIndex*>(h)->lookup_(wrap(ids, n));
  memcpy(locs, out.data_ptr<int64_t>(), n * sizeof(int64_t));
}

void ref_index_reset(void* h, const int64_t* ids, int64_t n) {
  static_cast<RefIndex*>(h)->reset_(wrap(ids, n));
}

void ref_index_getall(void* h, int64_t* ids, int64_t* locs, int64_t len) {
  auto out = static_cast<RefIndex*>(h)->getall_(len);
  memcpy(ids, std::get<0>(out).data_ptr<int64_t>(), len * sizeof(int64_t));
  memcpy(locs, std::get<1>(out).data_ptr<int64_t>(), len * sizeof(int64_t));
}

}  // extern "C"
