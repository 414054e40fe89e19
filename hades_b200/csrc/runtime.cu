// Process-wide pieces of the C ABI: error text, launch counter, device facts.
#include <atomic>
#include <cstdarg>
#include <cstring>

#include "launch.cuh"

namespace hb {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
void count_library_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_sms = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    cached_dev = dev;
    cached_sms = sms;
  }
  return cached_sms;
}

// One int per device, allocated on first use: kernels with bounded waits record
// an hb_status there instead of trapping.
int* device_error_word() {
  static int* words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    words[dev] = p;
  }
  return words[dev];
}

}  // namespace hb

extern "C" {

const char* hb_last_error(void) { return hb::g_error; }
int hb_version(void) { return 100; }
int64_t hb_launch_count(void) { return hb::g_launches.load(std::memory_order_relaxed); }

int hb_device_status(int* status_host, hb_stream_t stream) {
  HB_CHECK_ARG(status_host != nullptr, "hb_device_status: null argument");
  int* w = hb::device_error_word();
  if (!w) {
    hb::set_error("hb_device_status: no error word on this device");
    return HB_ERR_CUDA;
  }
  cudaStream_t st = (cudaStream_t)stream;
  HB_CUDA(cudaMemcpyAsync(status_host, w, sizeof(int), cudaMemcpyDeviceToHost, st));
  HB_CUDA(cudaStreamSynchronize(st));
  if (*status_host != 0) HB_CUDA(cudaMemsetAsync(w, 0, sizeof(int), st));
  return HB_OK;
}

}  // extern "C"
