// The translation unit a maintainer of the reference adds next to src/pybind.cc to put
// libhades_b200 behind the reference's own torch-typed operators (src/cuda/ops.h:9-41) and its
// index class (src/cache/cache.h:11-257): same function names and argument order, bodies that
// forward to the C ABI of include/hades_b200.h on torch's current stream.  Build it with the
// extension (links -lhades_b200; include/ on the include path); the m.def(...) lines of
// src/pybind.cc:16-71 stay as they are.  It is not part of libhades_b200.so; a test compiles it
// against the torch headers so that it cannot rot.
#include <ATen/cuda/CUDAContext.h>
#include <torch/script.h>

#include <vector>

#include "hades_b200.h"

namespace distemb {
namespace cuda {

static void check(int rc) { TORCH_CHECK(rc == HB_OK, hb_last_error()); }
static void* stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static int64_t row_bytes(const torch::Tensor& t) {
  return (t.dim() == 1 ? 1 : t.size(1)) * t.element_size();
}

// replaces CUDAFetch, src/cuda/uva_fetch.cu:28-45
void CUDAFetch(torch::Tensor src, torch::Tensor src_index, torch::Tensor dst, torch::Tensor dst_index) {
  TORCH_CHECK(src.size(1) == dst.size(1));
  TORCH_CHECK(dst_index.numel() == src_index.numel());
  check(hb_rows_gather(src.data_ptr(), src_index.data_ptr(), dst.data_ptr(), dst_index.data_ptr(),
                       src_index.numel(), row_bytes(src), (int)src_index.element_size(),
                       HB_MOVER_AUTO, stream()));
}

// replaces CUDAFetch2, src/cuda/uva_fetch.cu:72-106
void CUDAFetch2(torch::Tensor src, torch::Tensor src_index, torch::Tensor dst) {
  TORCH_CHECK(src.dim() == dst.dim());
  check(hb_rows_gather(src.data_ptr(), src_index.data_ptr(), dst.data_ptr(), nullptr,
                       src_index.numel(), row_bytes(src), (int)src_index.element_size(),
                       HB_MOVER_AUTO, stream()));
}

// replaces CUDAFetchWithCache2, src/cuda/uva_fetch.cu:149-192
void CUDAFetchWithCache2(torch::Tensor cpu_src, torch::Tensor gpu_src, torch::Tensor src_index,
                         torch::Tensor index_map, torch::Tensor dst) {
  check(hb_rows_gather_cached(cpu_src.data_ptr(), gpu_src.data_ptr(), src_index.data_ptr(),
                              index_map.data_ptr(), dst.data_ptr(), nullptr, src_index.numel(),
                              row_bytes(gpu_src), (int)src_index.element_size(), stream()));
}

// replaces CUDASet, src/cuda/uva_set.cu:35-69, and CUDACombine, src/cuda/uva_fetch.cu:212-228
void CUDASet(torch::Tensor src, torch::Tensor dst, torch::Tensor dst_index) {
  check(hb_rows_scatter(src.data_ptr(), dst.data_ptr(), dst_index.data_ptr(), dst_index.numel(),
                        row_bytes(src), (int)dst_index.element_size(), HB_MOVER_AUTO, stream()));
}
void CUDACombine(torch::Tensor src, torch::Tensor dst, torch::Tensor dst_index) { CUDASet(src, dst, dst_index); }

// replaces CUDASetWithCache, src/cuda/uva_set.cu:112-154
void CUDASetWithCache(torch::Tensor src, torch::Tensor cpu_dst, torch::Tensor gpu_dst,
                      torch::Tensor dst_index, torch::Tensor index_map) {
  check(hb_rows_scatter_cached(src.data_ptr(), cpu_dst.data_ptr(), gpu_dst.data_ptr(),
                               dst_index.data_ptr(), index_map.data_ptr(), dst_index.numel(),
                               row_bytes(gpu_dst), (int)dst_index.element_size(), stream()));
}

// replaces splitCUDA, src/cuda/split.cu:53-56
std::vector<torch::Tensor> splitCUDA(torch::Tensor ids, torch::Tensor mask) {
  auto opt = torch::TensorOptions().dtype(torch::kBool).device(ids.device());
  std::vector<torch::Tensor> out = {torch::zeros({ids.numel()}, opt), torch::zeros({ids.numel()}, opt),
                                    torch::zeros({ids.numel()}, opt)};
  check(hb_split_masks(ids.data_ptr<int64_t>(), ids.numel(), mask.data_ptr<int8_t>(),
                       (uint8_t*)out[0].data_ptr<bool>(), (uint8_t*)out[1].data_ptr<bool>(),
                       (uint8_t*)out[2].data_ptr<bool>(), stream()));
  return out;
}

// replace Reminder / CUDABinarySearch / CUDABinarySearch2, src/cuda/binary_search.cu:45-89
torch::Tensor Reminder(torch::Tensor in, int64_t local_num_gpus) {
  auto out = torch::empty_like(in);
  check(hb_owner_mod(in.data_ptr(), in.size(0), (int)in.element_size(), local_num_gpus, out.data_ptr(), stream()));
  return out;
}
torch::Tensor CUDABinarySearch(torch::Tensor in, torch::Tensor range_partition, int64_t local_num_gpus) {
  auto out = torch::empty_like(in);
  check(hb_owner_range(in.data_ptr(), in.size(0), (int)in.element_size(), range_partition.data_ptr(),
                       range_partition.size(0), local_num_gpus, out.data_ptr(), stream()));
  return out;
}
torch::Tensor CUDABinarySearch2(torch::Tensor in, torch::Tensor range) {
  auto out = torch::empty_like(in);
  check(hb_upper_bound(in.data_ptr(), in.size(0), (int)in.element_size(), range.data_ptr(), range.size(0),
                       out.data_ptr(), stream()));
  return out;
}

}  // namespace cuda

// Stands where SACacheIndex<int64_t, int64_t> stands in src/pybind.cc:13-33; ids and slots are
// CUDA tensors (the reference's CPU entry points copy to the device first).
struct B200Index {
  hb_index_t* h = nullptr;
  explicit B200Index(int64_t cache_size) { TORCH_CHECK(hb_index_create(cache_size, &h) == HB_OK, hb_last_error()); }
  ~B200Index() { hb_index_destroy(h); }
  B200Index(const B200Index&) = delete;
  B200Index& operator=(const B200Index&) = delete;
  int64_t get_cache_size_() { return hb_index_size(h); }
  int64_t get_capacity_() { return hb_index_capacity(h); }
  // cudalookup_, src/cache/cache.h:225-234
  torch::Tensor cudalookup_(torch::Tensor ids) {
    auto locs = torch::empty_like(ids);
    cuda::check(hb_index_lookup(h, ids.data_ptr<int64_t>(), ids.numel(), locs.data_ptr<int64_t>(), nullptr,
                                HB_LOOKUP_SETASSOC, cuda::stream()));
    return locs;
  }
  // add_, src/cache/cache.h:196-206
  torch::Tensor add_(torch::Tensor ids) {
    auto locs = torch::empty_like(ids);
    auto ws = torch::empty({(int64_t)hb_index_add_workspace_bytes(ids.numel())},
                           torch::TensorOptions().dtype(torch::kUInt8).device(ids.device()));
    cuda::check(hb_index_add(h, ids.data_ptr<int64_t>(), ids.numel(), locs.data_ptr<int64_t>(), nullptr,
                             ws.data_ptr(), (size_t)ws.numel(), cuda::stream()));
    return locs;
  }
  // reset_, src/cache/cache.h:208-211
  void reset_(torch::Tensor ids) {
    cuda::check(hb_index_reset(h, ids.data_ptr<int64_t>(), ids.numel(), cuda::stream()));
  }
};

}  // namespace distemb
