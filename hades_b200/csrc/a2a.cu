// Owner-partitioned sparse-gradient exchange over peer memory: one fused
// "pack + push" pass buckets (id, cnt, row) by owner and stores every bucket
// straight into the owner GPU's receive slab over NVLink (plain st.global to
// memory mapped with CUDA IPC; no staging copy, no host-side sizes).  Replaces
// the sort + gathers + four all_to_all_single calls + two host reads of
// swap_gradients (python/EmbCache/sparse_optim.py:36-118).
//
// Receive area of a rank (one cudaMalloc per parity, mapped by every peer):
//   counts[world]                 rows delivered by each source
//   flags [world]                 (parity 0 only) last exchange each source has finished pushing
//   ids   [world][cap]            slab s = rows sent by rank s
//   cnt   [world][cap]
//   rows  [world][cap][row_bytes]
// Two parities alternate so that a fast rank's next push cannot overwrite what a
// slow rank is still reading; one barrier per exchange (the caller's, between
// push and consume) is then enough.  The barrier is either the caller's collective or
// hb_a2a_fence: every rank stores its exchange number into every peer's flag array
// and waits, WITH AN ITERATION LIMIT, until all peers have done the same; a rank
// that gives up records HB_ERR_TIMEOUT and returns.  (The ranks run on different
// GPUs, so the waiting kernels do run at the same time.)
#include <cstring>

#include "a2a.cuh"
#include "partition_core.cuh"

namespace hb {
int* device_error_word();  // runtime.cu
}

namespace hb {
namespace {

size_t off_counts() { return 0; }
size_t off_flags() { return 1024; }  // world <= 64: counts end at 512
size_t off_ids(int) { return 2048; }
size_t off_cnt(int world, int64_t cap) { return off_ids(world) + align_up((size_t)world * cap * 8, 256); }
size_t off_rows(int world, int64_t cap) { return off_cnt(world, cap) + align_up((size_t)world * cap * 8, 256); }
size_t area_size(int world, int64_t cap, int64_t row_bytes) {
  return off_rows(world, cap) + align_up((size_t)world * cap * row_bytes, 256);
}

struct PushPolicy {
  const int64_t* ids;
  const char* rows;
  const int64_t* cnt;
  const int64_t* n_dev;
  const hb_a2a::Dest* dest;
  int world, rank;
  int64_t cap, row_bytes;
  int vb;
  int* err;
  __device__ __forceinline__ int classify(int64_t i) const {
    if (n_dev && i >= *n_dev) return -1;
    const int64_t id = __ldg(ids + i);
    return id >= 0 ? (int)mod_nonneg(id, world) : -1;
  }
  __device__ __forceinline__ void emit(int64_t i, int c, int64_t pos, int64_t, bool active) const {
    bool ok = active && pos < cap;
    if (active && !ok) atomicExch(err, HB_ERR_CAPACITY);  // never write past a slab
    const int64_t at = (int64_t)rank * cap + pos;        // my slab in the owner's area
    if (ok) {
      dest->ids[c][at] = ids[i];
      dest->cnt[c][at] = cnt ? cnt[i] : 1;
    }
    warp_move_rows(rows + i * row_bytes, ok ? dest->rows[c] + at * row_bytes : nullptr, ok, row_bytes, vb);
  }
};

// after the scatter: tell every owner how many rows it got from this rank
__global__ void push_counts_kernel(PartitionPlan p, const hb_a2a::Dest* dest, int rank, int64_t cap,
                                   int64_t* __restrict__ sent_out) {
  const int b = threadIdx.x;
  if (b >= p.num_classes) return;
  int64_t c = p.class_total[b];
  if (c > cap) c = cap;
  dest->counts[b][rank] = c;
  if (sent_out) sent_out[b] = c;
  __threadfence_system();
}

// the same for a sender that stored its records itself (a2a_direct_publish)
__global__ void publish_counts_kernel(const unsigned long long* __restrict__ counts, const hb_a2a::Dest* dest,
                                      int rank, int world, int64_t cap) {
  const int b = threadIdx.x;
  if (b >= world) return;
  int64_t c = (int64_t)counts[b];
  if (c > cap) c = cap;
  dest->counts[b][rank] = c;
  __threadfence_system();
}

// Poll a flag until it reaches `value`, at most about a second; false = gave up.
__device__ __forceinline__ bool wait_flag_bounded(const volatile unsigned long long* flag,
                                                  unsigned long long value) {
  for (int it = 0; it < (1 << 20); ++it) {
    if (*flag >= value) return true;
    __nanosleep(it < 64 ? 100 : 1000);
  }
  return false;
}

__global__ void wait_flag_kernel(const unsigned long long* flag, unsigned long long value, int* err) {
  if (!wait_flag_bounded(flag, value)) atomicExch(err, HB_ERR_TIMEOUT);
}

// One CTA per rank.  Thread t: tell rank t that this rank has finished pushing exchange
// number e (everything before this kernel in the stream), then wait until rank t says the
// same.  Bounded: about a second of polling, then HB_ERR_TIMEOUT and return.
__global__ void a2a_fence_kernel(const hb_a2a::Dest* dest, const unsigned long long* local_flags,
                                 unsigned long long* epoch, int rank, int world, int* err) {
  __shared__ unsigned long long e;
  if (threadIdx.x == 0) e = ++(*epoch);
  __syncthreads();
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();  // my rows and counts are visible before my flag
  *reinterpret_cast<volatile unsigned long long*>(dest->flags[t] + rank) = e;
  if (!wait_flag_bounded(local_flags + t, e)) atomicExch(err, HB_ERR_TIMEOUT);
  __threadfence_system();  // reads of the slabs stay after the flag
}

}  // namespace
}  // namespace hb

namespace hb {

int a2a_direct_begin(hb_a2a* a, const hb_a2a::Dest** dest, int* parity) {
  HB_CHECK_ARG(a && dest && parity, "a2a_direct_begin: null argument");
  *parity = a->parity;
  *dest = a->dest_dev[a->parity];
  a->parity ^= 1;
  return HB_OK;
}

int a2a_direct_publish(hb_a2a* a, int parity, const unsigned long long* counts_dev, cudaStream_t st) {
  HB_CHECK_ARG(a && counts_dev && (parity == 0 || parity == 1), "a2a_direct_publish: bad argument");
  HB_LAUNCH(publish_counts_kernel, 1, 64, 0, st, counts_dev, a->dest_dev[parity], a->rank, a->world, a->cap);
  return HB_OK;
}

}  // namespace hb

using namespace hb;

extern "C" {

int hb_a2a_create(int rank, int world, int64_t cap_rows, int64_t row_bytes, hb_a2a_t** out) {
  HB_CHECK_ARG(out && world >= 1 && world <= 64 && rank >= 0 && rank < world, "hb_a2a_create: bad rank/world");
  HB_CHECK_ARG(cap_rows > 0 && row_bytes > 0, "hb_a2a_create: bad sizes");
  hb_a2a_t* a = new hb_a2a_t();
  memset(a, 0, sizeof(*a));
  a->rank = rank;
  a->world = world;
  a->cap = cap_rows;
  a->row_bytes = row_bytes;
  a->area_bytes = area_size(world, cap_rows, row_bytes);
  // a failed allocation releases what the earlier ones took
  cudaError_t e = cudaSuccess;
  for (int p = 0; p < 2 && e == cudaSuccess; ++p) {
    e = cudaMalloc(&a->local[p], a->area_bytes);
    if (e == cudaSuccess) e = cudaMemset(a->local[p], 0, a->area_bytes);
    a->peer[p][rank] = a->local[p];
    if (e == cudaSuccess) e = cudaMalloc(&a->dest_dev[p], sizeof(hb_a2a::Dest));
  }
  if (e == cudaSuccess) e = cudaMalloc(&a->epoch_dev, sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaMemset(a->epoch_dev, 0, sizeof(unsigned long long));
  if (e != cudaSuccess) {
    set_error("hb_a2a_create: allocating the receive areas (%zu bytes each) failed: %s", a->area_bytes,
              cudaGetErrorString(e));
    hb_a2a_destroy(a);
    return HB_ERR_CUDA;
  }
  *out = a;
  return HB_OK;
}

// Back to the state after hb_a2a_connect: exchange number 0, no flag set, next push into
// area 0.  After a fence gave up (HB_ERR_TIMEOUT: a peer never arrived) the ranks' exchange
// numbers differ for good; once the host side has agreed that every rank is alive again,
// all ranks call this -- with a host barrier before it (nobody is still pushing or polling)
// and after it (nobody pushes into an area that is about to be cleared) -- and go on.
int hb_a2a_reset(hb_a2a_t* a, hb_stream_t stream) {
  HB_CHECK_ARG(a != nullptr, "hb_a2a_reset: null exchange");
  cudaStream_t st = (cudaStream_t)stream;
  HB_CUDA(cudaMemsetAsync(a->epoch_dev, 0, sizeof(unsigned long long), st));
  for (int p = 0; p < 2; ++p) HB_CUDA(cudaMemsetAsync(a->local[p], 0, off_ids(a->world), st));  // counts and flags
  a->parity = 0;
  return HB_OK;
}

size_t hb_a2a_handle_bytes(void) { return 2 * sizeof(cudaIpcMemHandle_t); }

int hb_a2a_export_handle(hb_a2a_t* a, void* handle_out) {
  HB_CHECK_ARG(a && handle_out, "hb_a2a_export_handle: null argument");
  cudaIpcMemHandle_t h[2];
  for (int p = 0; p < 2; ++p) HB_CUDA(cudaIpcGetMemHandle(&h[p], a->local[p]));
  memcpy(handle_out, h, sizeof(h));
  return HB_OK;
}

// handles: world entries of hb_a2a_handle_bytes() each, entry r from rank r
int hb_a2a_connect(hb_a2a_t* a, const void* handles) {
  HB_CHECK_ARG(a && (a->world == 1 || handles), "hb_a2a_connect: null argument");
  const char* hp = static_cast<const char*>(handles);
  for (int r = 0; r < a->world; ++r) {
    if (r == a->rank) continue;
    cudaIpcMemHandle_t h[2];
    memcpy(h, hp + (size_t)r * sizeof(h), sizeof(h));
    for (int p = 0; p < 2; ++p) {
      void* ptr = nullptr;
      HB_CUDA(cudaIpcOpenMemHandle(&ptr, h[p], cudaIpcMemLazyEnablePeerAccess));
      a->peer[p][r] = static_cast<char*>(ptr);
    }
    a->opened[r] = true;
  }
  for (int p = 0; p < 2; ++p) {
    hb_a2a::Dest d;
    memset(&d, 0, sizeof(d));
    for (int r = 0; r < a->world; ++r) {
      char* base = a->peer[p][r];
      d.flags[r] = reinterpret_cast<unsigned long long*>(a->peer[0][r] + off_flags());
      d.counts[r] = reinterpret_cast<int64_t*>(base + off_counts());
      d.ids[r] = reinterpret_cast<int64_t*>(base + off_ids(a->world));
      d.cnt[r] = reinterpret_cast<int64_t*>(base + off_cnt(a->world, a->cap));
      d.rows[r] = base + off_rows(a->world, a->cap);
    }
    HB_CUDA(cudaMemcpy(a->dest_dev[p], &d, sizeof(d), cudaMemcpyHostToDevice));
  }
  return HB_OK;
}

// Close this process's mappings of the peers' areas.  Tear-down in two steps, with a
// barrier of all ranks before each: first every rank disconnects (nobody touches a peer's
// memory any more), then every rank destroys (frees its own areas).  Freeing an area that a
// peer still has mapped is undefined behaviour of the CUDA IPC interface.
int hb_a2a_disconnect(hb_a2a_t* a) {
  if (!a) return HB_OK;
  for (int r = 0; r < a->world; ++r) {
    if (!a->opened[r]) continue;
    for (int p = 0; p < 2; ++p) {
      cudaIpcCloseMemHandle(a->peer[p][r]);
      a->peer[p][r] = nullptr;
    }
    a->opened[r] = false;
  }
  return HB_OK;
}

int hb_a2a_destroy(hb_a2a_t* a) {
  if (!a) return HB_OK;
  for (int r = 0; r < a->world; ++r)
    if (a->opened[r])
      for (int p = 0; p < 2; ++p) cudaIpcCloseMemHandle(a->peer[p][r]);
  for (int p = 0; p < 2; ++p) {
    cudaFree(a->local[p]);
    cudaFree(a->dest_dev[p]);
  }
  cudaFree(a->epoch_dev);
  delete a;
  return HB_OK;
}

size_t hb_a2a_push_workspace_bytes(int64_t n, int world) { return partition_workspace_bytes(n, world, 1); }

int hb_a2a_push(hb_a2a_t* a, const int64_t* ids, const void* rows, const int64_t* cnt, int64_t n,
                const int64_t* n_dev, int64_t* sent_counts, int* parity_out, void* workspace,
                size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(a && n >= 0 && n < ((int64_t)1 << 31), "hb_a2a_push: bad argument");
  HB_CHECK_ARG(n == 0 || (ids && rows), "hb_a2a_push: null argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int p = a->parity;
  a->parity ^= 1;
  if (parity_out) *parity_out = p;
  PushPolicy pol{ids, (const char*)rows, cnt, n_dev, a->dest_dev[p], a->world, a->rank, a->cap,
                 a->row_bytes, payload_vec_bytes(a->row_bytes, rows, a->local[p] + off_rows(a->world, a->cap)),
                 device_error_word()};
  PartitionPlan plan;
  int rc = run_partition(pol, n, a->world, workspace, workspace_bytes, nullptr, st, 1, &plan);
  if (rc != HB_OK) return rc;
  HB_LAUNCH(push_counts_kernel, 1, 64, 0, st, plan, a->dest_dev[p], a->rank, a->cap, sent_counts);
  return HB_OK;
}

int hb_a2a_fence(hb_a2a_t* a, hb_stream_t stream) {
  HB_CHECK_ARG(a != nullptr, "hb_a2a_fence: null exchange");
  if (a->world == 1) return HB_OK;
  HB_LAUNCH(a2a_fence_kernel, 1, 64, 0, (cudaStream_t)stream, a->dest_dev[0],
            reinterpret_cast<const unsigned long long*>(a->local[0] + off_flags()), a->epoch_dev,
            a->rank, a->world, device_error_word());
  return HB_OK;
}

int hb_wait_flag(const uint64_t* flag, uint64_t value, hb_stream_t stream) {
  HB_CHECK_ARG(flag != nullptr, "hb_wait_flag: null flag");
  HB_LAUNCH(wait_flag_kernel, 1, 1, 0, (cudaStream_t)stream,
            reinterpret_cast<const unsigned long long*>(flag), (unsigned long long)value,
            device_error_word());
  return HB_OK;
}

int hb_a2a_recv_view(hb_a2a_t* a, int parity, int64_t** ids, void** rows, int64_t** cnt,
                     int64_t** counts, int64_t* cap_rows) {
  HB_CHECK_ARG(a && (parity == 0 || parity == 1), "hb_a2a_recv_view: bad argument");
  char* base = a->local[parity];
  if (counts) *counts = reinterpret_cast<int64_t*>(base + off_counts());
  if (ids) *ids = reinterpret_cast<int64_t*>(base + off_ids(a->world));
  if (cnt) *cnt = reinterpret_cast<int64_t*>(base + off_cnt(a->world, a->cap));
  if (rows) *rows = base + off_rows(a->world, a->cap);
  if (cap_rows) *cap_rows = a->cap;
  return HB_OK;
}

}  // extern "C"
