// Shared device/host helpers for libhades_b200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/hades_b200.h"

namespace hb {

// ---- error reporting -------------------------------------------------------
// Every C-ABI entry point returns an hb_status; the message of the last failure
// on the calling thread is kept for hb_last_error().  Nothing here exits the
// process (the reference's CUDA_CALL macro does, src/utils.h:12-24).
void set_error(const char* fmt, ...);

#define HB_CHECK_ARG(cond, ...)       \
  do {                                \
    if (!(cond)) {                    \
      hb::set_error(__VA_ARGS__);     \
      return HB_ERR_INVALID;          \
    }                                 \
  } while (0)

#define HB_CUDA(call)                                                      \
  do {                                                                     \
    cudaError_t e_ = (call);                                               \
    if (e_ != cudaSuccess) {                                               \
      hb::set_error("%s:%d %s failed: %s", __FILE__, __LINE__, #call,      \
                    cudaGetErrorString(e_));                               \
      return HB_ERR_CUDA;                                                  \
    }                                                                      \
  } while (0)

#define HB_LAUNCH_CHECK() HB_CUDA(cudaGetLastError())

// ---- device properties (cached per device) ---------------------------------
int sm_count();  // multiprocessors of the current device

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Carve aligned sub-buffers out of a caller-provided workspace.
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base(static_cast<char*>(p)) {}
  template <typename T>
  T* take(size_t count) {
    off = align_up(off, 256);
    T* p = reinterpret_cast<T*>(base + off);
    off += count * sizeof(T);
    return p;
  }
  size_t used() const { return align_up(off, 256); }
};

// ---- device helpers ---------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// id % m for non-negative id; 32-bit fast path when both fit.
__device__ __forceinline__ int64_t mod_nonneg(int64_t id, int64_t m) {
  if (((uint64_t)id | (uint64_t)m) >> 32) return id % m;
  return (int64_t)((uint32_t)id % (uint32_t)m);
}

template <typename IdxT>
__device__ __forceinline__ int64_t load_index(const void* p, int64_t i) {
  return (int64_t) __ldg(reinterpret_cast<const IdxT*>(p) + i);
}

#endif  // __CUDACC__

}  // namespace hb
