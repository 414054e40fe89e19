// Kernel-launch bookkeeping: every launch of this library goes through
// HB_LAUNCH so that hb_launch_count() reports how many kernels really ran.
#pragma once

#include "common.cuh"

namespace hb {
void count_launch();                 // one of this library's own kernels
void count_library_launches(int n);  // kernels launched for us by CUB
}  // namespace hb

// A kernel name with template commas must be wrapped in parentheses.
#define HB_LAUNCH(kernel, grid, block, smem, stream, ...)        \
  do {                                                           \
    kernel<<<(grid), (block), (smem), (stream)>>>(__VA_ARGS__);  \
    hb::count_launch();                                          \
    HB_CUDA(cudaGetLastError());                                 \
  } while (0)
