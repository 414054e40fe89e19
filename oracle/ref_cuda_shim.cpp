// TEST INFRASTRUCTURE -- not part of the product.  C-callable doorway into the
// reference's own CUDA operators (src/cuda/ops.h:9-41, bound in src/pybind.cc:46-70):
// this file only #includes the reference header from where the reference checkout
// lies, wraps raw device pointers in tensors (torch::from_blob) and forwards.  The
// reference's kernels are compiled from its own .cu files by oracle/build_oracle.py
// (nvcc on those files directly; its build system is not run) and linked with this
// shim into oracle/_ref/libhades_ref_cuda.so.  No reference source is copied.
//
// The reference launches on the legacy default stream without synchronising
// (e.g. src/cuda/uva_fetch.cu:39); callers order their own work accordingly.
// The reference's cudalookup (src/cache/lookup.cu) is deliberately not exposed:
// lanes of lookupkernel2 return before a warp-wide reduce, which is undefined.
#include <torch/script.h>

#include <cstring>
#include <vector>

#include "cuda/ops.h"

namespace {

torch::Tensor dev_rows(const void* p, int64_t n, int64_t dim, int elem_bytes) {
  auto opt = torch::TensorOptions().device(torch::kCUDA).dtype(elem_bytes == 8 ? torch::kDouble : torch::kFloat);
  if (dim <= 0) return torch::from_blob(const_cast<void*>(p), {n}, opt);
  return torch::from_blob(const_cast<void*>(p), {n, dim}, opt);
}

torch::Tensor dev_index(const void* p, int64_t n, int idx_bytes) {
  auto opt = torch::TensorOptions().device(torch::kCUDA).dtype(idx_bytes == 4 ? torch::kInt32 : torch::kInt64);
  return torch::from_blob(const_cast<void*>(p), {n}, opt);
}

}  // namespace

extern "C" {

// dst[dst_index[i]] = src[src_index[i]]                       src/cuda/uva_fetch.cu:28-45
void ref_cuda_fetch(const void* src, int64_t src_rows, const void* src_index, void* dst, int64_t dst_rows,
                    const void* dst_index, int64_t n, int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDAFetch(dev_rows(src, src_rows, dim, elem_bytes), dev_index(src_index, n, idx_bytes),
                           dev_rows(dst, dst_rows, dim, elem_bytes), dev_index(dst_index, n, idx_bytes));
}

// dst[i] = src[src_index[i]]  (dim <= 0: 1-D tensors)          src/cuda/uva_fetch.cu:72-106
void ref_cuda_fetch2(const void* src, int64_t src_rows, const void* src_index, void* dst, int64_t n,
                     int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDAFetch2(dev_rows(src, src_rows, dim, elem_bytes), dev_index(src_index, n, idx_bytes),
                            dev_rows(dst, n, dim, elem_bytes));
}

// cached fetch through a dense index map                      src/cuda/uva_fetch.cu:149-192
void ref_cuda_fetch_with_cache2(const void* backing, int64_t backing_rows, const void* cached,
                                int64_t cached_rows, const void* src_index, const void* index_map,
                                void* dst, int64_t n, int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDAFetchWithCache2(dev_rows(backing, backing_rows, dim, elem_bytes),
                                     dev_rows(cached, cached_rows, dim, elem_bytes),
                                     dev_index(src_index, n, idx_bytes),
                                     dev_index(index_map, backing_rows, idx_bytes),
                                     dev_rows(dst, n, dim, elem_bytes));
}

// dst[dst_index[i]] = src[i]                                   src/cuda/uva_set.cu:35-69
void ref_cuda_set(const void* src, void* dst, int64_t dst_rows, const void* dst_index, int64_t n,
                  int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDASet(dev_rows(src, n, dim, elem_bytes), dev_rows(dst, dst_rows, dim, elem_bytes),
                         dev_index(dst_index, n, idx_bytes));
}

// cached set through a dense index map                        src/cuda/uva_set.cu:112-154
void ref_cuda_set_with_cache(const void* src, void* backing, int64_t backing_rows, void* cached,
                             int64_t cached_rows, const void* dst_index, const void* index_map, int64_t n,
                             int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDASetWithCache(dev_rows(src, n, dim, elem_bytes),
                                  dev_rows(backing, backing_rows, dim, elem_bytes),
                                  dev_rows(cached, cached_rows, dim, elem_bytes),
                                  dev_index(dst_index, n, idx_bytes),
                                  dev_index(index_map, backing_rows, idx_bytes));
}

// dst[dst_index[i]] = src[i]                                   src/cuda/uva_fetch.cu:212-228
void ref_cuda_combine(const void* src, void* dst, int64_t dst_rows, const void* dst_index, int64_t n,
                      int64_t dim, int elem_bytes, int idx_bytes) {
  distemb::cuda::CUDACombine(dev_rows(src, n, dim, elem_bytes), dev_rows(dst, dst_rows, dim, elem_bytes),
                             dev_index(dst_index, n, idx_bytes));
}

// three bool masks (local, remote hot, remote cold)            src/cuda/split.cu:12-56
void ref_cuda_split(const int64_t* ids, int64_t n, const int8_t* mask, int64_t mask_len, bool* local,
                    bool* hot, bool* cold) {
  auto m = torch::from_blob(const_cast<int8_t*>(mask), {mask_len},
                            torch::TensorOptions().device(torch::kCUDA).dtype(torch::kInt8));
  auto out = distemb::cuda::splitCUDA(dev_index(ids, n, 8), m);
  cudaMemcpy(local, out[0].data_ptr<bool>(), (size_t)n, cudaMemcpyDeviceToDevice);
  cudaMemcpy(hot, out[1].data_ptr<bool>(), (size_t)n, cudaMemcpyDeviceToDevice);
  cudaMemcpy(cold, out[2].data_ptr<bool>(), (size_t)n, cudaMemcpyDeviceToDevice);
}

// in % g                                                       src/cuda/binary_search.cu:76-89
void ref_cuda_reminder(const void* in, int64_t n, int64_t g, void* out, int idx_bytes) {
  auto r = distemb::cuda::Reminder(dev_index(in, n, idx_bytes), g);
  cudaMemcpy(out, r.data_ptr(), (size_t)n * idx_bytes, cudaMemcpyDeviceToDevice);
}

// (upper_bound(range, in) - 1) * g + in % g                    src/cuda/binary_search.cu:45-59
void ref_cuda_binary_search(const void* in, int64_t n, const void* range, int64_t parts, int64_t g,
                            void* out, int idx_bytes) {
  auto r = distemb::cuda::CUDABinarySearch(dev_index(in, n, idx_bytes), dev_index(range, parts, idx_bytes), g);
  cudaMemcpy(out, r.data_ptr(), (size_t)n * idx_bytes, cudaMemcpyDeviceToDevice);
}

// upper_bound(range, in)                                       src/cuda/binary_search.cu:61-74
void ref_cuda_binary_search2(const void* in, int64_t n, const void* range, int64_t m, void* out,
                             int idx_bytes) {
  auto r = distemb::cuda::CUDABinarySearch2(dev_index(in, n, idx_bytes), dev_index(range, m, idx_bytes));
  cudaMemcpy(out, r.data_ptr(), (size_t)n * idx_bytes, cudaMemcpyDeviceToDevice);
}

}  // extern "C"
