// Hot-node local aggregation: sorted unique ids, per-id fp32 sum (or mean) of the
// duplicate-id gradient rows, per-id counts.  Replaces only_unique_grads /
// unique_grads (python/EmbCache/sparse_optim.py:132-157: torch.unique +
// index_add_).
//
// Deterministic, no floating-point atomics:
//   1. radix sort of (id, position) pairs (CUB), stable          } hb_runs_build (runs.cu); a step
//   2. run heads numbered: unique ids, run starts, class/position } that fetched the same ids first
//                                                                   hands its runs over instead
//   3. main pass: the sorted positions are cut into fixed chunks of R rows; a
//      group of G lanes (G*4 floats wide) walks its chunk in order, reading
//      gradient rows through the permutation, broadcasting positions with warp
//      shuffles and adding in registers.  A run that lies inside the chunk is
//      written straight to its output row.  A run that crosses a chunk boundary
//      leaves a partial row (head partial: the run began earlier; tail partial:
//      it goes on) and the chunk where it begins enters it in a fix-up list.
//   4. fix-up: partials of a crossing run are added in chunk order (short runs by
//      one lane group, long runs by a whole CTA in a fixed strided+sequential
//      order).
// The order of additions depends only on the sorted order and the chunk size, so
// two runs on the same input give the same bits.  Counts are integers, so they
// use atomicAdd (order cannot change an integer sum).
#include "launch.cuh"
#include "runs.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;
constexpr int kShortSpan = 16;   // crossing runs over at most this many chunks: group fix-up
constexpr int kLongBlock = 512;

struct SegArgs {
  const uint8_t* head;        // [n] 1 where a run of equal ids starts in the sorted order
  const uint32_t* perm;       // position in the input of each sorted element [n]
  const int64_t* run_start;   // [U] first sorted position of each run
  const int64_t* num_runs;    // device scalar U
  // (run_start holds U + 1 entries: the last is the number of valid rows)
  const float* grads;         // [n][dim]
  const int64_t* cnt_in;      // nullable [n]
  const int64_t* n_dev;       // nullable device count that caps n
  int64_t n;
  int64_t dim;
  int64_t col0;               // first column of this pass
  int cols;                   // columns of this pass (<= 32*VEC*VPL)
  int chunk;                  // R
  int64_t num_chunks;
  int mean;                   // divide by the count
  float* sums;                // [U][dim] (null when the rows go to class buffers)
  // optional split of the output by a per-id class (hot / cold): run u goes to
  // row dpos[u] of class_rows[dclass[u]] (a null buffer drops the class)
  const int8_t* dclass;       // [U], null = no split
  const int32_t* dpos;        // [U]
  float* class_rows[3];
  unsigned long long* counts; // [U], zeroed before the main pass
  float* head_part;           // [num_chunks][cols]
  float* tail_part;           // [num_chunks][cols]
  int2* short_list;           // (chunk, run)
  int2* long_list;
  int* list_counts;           // [0] short, [1] long
  float* slice_part;          // [long entries][kSlices][cols]
};

template <int VEC> struct VecF;
template <> struct VecF<4> { using T = float4; };
template <> struct VecF<1> { using T = float; };

__device__ __forceinline__ void vadd(float4& a, const float4& b) {
  a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
}
__device__ __forceinline__ void vadd(float& a, const float& b) { a += b; }
__device__ __forceinline__ void vzero(float4& a) { a = make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ void vzero(float& a) { a = 0.f; }
__device__ __forceinline__ void vdiv(float4& a, float d) { a.x /= d; a.y /= d; a.z /= d; a.w /= d; }
__device__ __forceinline__ void vdiv(float& a, float d) { a /= d; }

__device__ __forceinline__ int64_t run_of(const int64_t* run_start, int64_t U, int64_t pos) {
  int64_t lo = 0, hi = U;  // upper_bound(run_start, pos) - 1
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (__ldg(run_start + mid) <= pos) lo = mid + 1; else hi = mid;
  }
  return lo - 1;
}

// where the finished row of run u goes (null = nowhere)
__device__ __forceinline__ float* out_row(const SegArgs& a, int64_t u) {
  if (!a.dclass) return a.sums + u * a.dim + a.col0;
  const int c = a.dclass[u];
  float* base = (c >= 0 && c < 3) ? a.class_rows[c] : nullptr;
  return base ? base + (int64_t)a.dpos[u] * a.dim + a.col0 : nullptr;
}

// rows of run u (no weights) or the sum of their weights: the weights are added up with
// integer atomics in the main pass, the plain count is the length of the run
__device__ __forceinline__ long long run_count(const SegArgs& a, int64_t u) {
  if (a.cnt_in) return (long long)a.counts[u];
  return (long long)(__ldg(a.run_start + u + 1) - __ldg(a.run_start + u));
}

__device__ __forceinline__ float denominator(const SegArgs& a, long long c) {
  // unique_grads starts its counts from ones when cnt is given (sparse_optim.py:145-148)
  return (float)(a.cnt_in ? c + 1 : c);
}

__device__ __forceinline__ int64_t effective_n(const SegArgs& a) {
  if (!a.n_dev) return a.n;
  const int64_t d = *a.n_dev;
  return d < a.n ? (d > 0 ? d : 0) : a.n;
}

// ---- main pass -------------------------------------------------------------------
// HAS_CNT: per-row weights are given (unique_grads with cnt); otherwise the count
// of a run is the number of its rows and needs no per-row traffic.
template <int VEC, int G, int VPL, bool HAS_CNT>
__global__ void __launch_bounds__(kBlock, 4) segsum_main_kernel(SegArgs a) {
  using V = typename VecF<VEC>::T;
  constexpr int U = (8 / VPL) < G ? (8 / VPL) : G;  // rows whose loads are in flight together
  const int lane = threadIdx.x & 31;
  const int sub = lane & (G - 1);
  const int grp_in_warp = lane / G;
  const unsigned grp_shift = grp_in_warp * G;
  const unsigned grp_mask = G == 32 ? 0xffffffffu : ((1u << G) - 1u);
  const int64_t c = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) / G;
  const int64_t n_eff = effective_n(a);  // ignored entries were given the largest key
  const bool live = c < a.num_chunks && c * a.chunk < n_eff;
  const int64_t U_runs = *a.num_runs;
  const int64_t j0 = live ? c * a.chunk : 0;
  const int64_t j1 = live ? ((j0 + a.chunk < n_eff) ? j0 + a.chunk : n_eff) : 0;
  const int vpr = a.cols / VEC;  // vectors per row in this pass

  int64_t u = live ? run_of(a.run_start, U_runs, j0) : 0;
  bool first_partial = live && __ldg(a.run_start + u) < j0;  // chunk starts inside a run
  bool have = first_partial;  // a run is open
  V acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) vzero(acc[v]);
  unsigned long long cacc = 0;

  auto flush = [&](bool tail) {
    // write the open run: complete -> output row; crossing -> partial row
    float* dst;
    bool complete = !first_partial && !tail;
    if (complete) dst = out_row(a, u);
    else if (first_partial) dst = a.head_part + c * a.cols;
    else dst = a.tail_part + c * a.cols;
    if (complete && a.mean) {
      const float d = denominator(a, (long long)cacc);
#pragma unroll
      for (int v = 0; v < VPL; ++v) vdiv(acc[v], d);
    }
    if (dst) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int k = sub + v * G;
        if (k < vpr) reinterpret_cast<V*>(dst)[k] = acc[v];
      }
    }
    if (HAS_CNT && sub == 0 && a.col0 == 0 && cacc) atomicAdd(a.counts + u, cacc);
  };

  const int steps = a.chunk / G;  // uniform trip count (chunk is a multiple of 32)
  for (int sidx = 0; sidx < steps; ++sidx) {
    const int64_t j = j0 + (int64_t)sidx * G + sub;
    const bool valid = j < j1;
    uint32_t p = 0;
    bool head = false;
    int cv = 1;
    if (valid) {
      p = __ldg(a.perm + j);
      head = __ldg(a.head + j) != 0;
      if (HAS_CNT) cv = (int)__ldg(a.cnt_in + p);
    }
    const unsigned hb_all = __ballot_sync(0xffffffffu, head);
    const unsigned vb_all = __ballot_sync(0xffffffffu, valid);
    const unsigned heads = (hb_all >> grp_shift) & grp_mask;
    const unsigned valids = (vb_all >> grp_shift) & grp_mask;
#pragma unroll 1
    for (int t0 = 0; t0 < G; t0 += U) {
      V val[U][VPL];
      int cvs[U];
#pragma unroll
      for (int x = 0; x < U; ++x) {
        const uint32_t px = __shfl_sync(0xffffffffu, p, t0 + x, G);
        cvs[x] = HAS_CNT ? __shfl_sync(0xffffffffu, cv, t0 + x, G) : 1;
        if ((valids >> (t0 + x)) & 1u) {
          const V* src = reinterpret_cast<const V*>(a.grads + (int64_t)px * a.dim + a.col0);
#pragma unroll
          for (int v = 0; v < VPL; ++v) {
            const int k = sub + v * G;
            if (k < vpr) val[x][v] = __ldg(src + k);
          }
        }
      }
#pragma unroll
      for (int x = 0; x < U; ++x) {
        if (!((valids >> (t0 + x)) & 1u)) continue;
        if ((heads >> (t0 + x)) & 1u) {
          if (have) {
            flush(false);
            ++u;
          }
          first_partial = false;
          have = true;
#pragma unroll
          for (int v = 0; v < VPL; ++v) vzero(acc[v]);
          cacc = 0;
        }
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          const int k = sub + v * G;
          if (k < vpr) vadd(acc[v], val[x][v]);
        }
        cacc += (unsigned long long)(unsigned)cvs[x];
      }
    }
  }
  if (live && have) {
    // does the open run go on after this chunk?
    const bool tail = j1 < n_eff && __ldg(a.head + j1) == 0;
    if (tail && !first_partial && sub == 0 && a.col0 == 0) {
      // this chunk holds the head of a crossing run: enter it in a fix-up list
      const int64_t run_end = __ldg(a.run_start + u + 1);
      const int64_t last_chunk = (run_end - 1) / a.chunk;
      const bool is_short = (last_chunk - c) <= kShortSpan;
      const int slot = atomicAdd(a.list_counts + (is_short ? 0 : 1), 1);
      (is_short ? a.short_list : a.long_list)[slot] = make_int2((int)c, (int)u);
    }
    flush(tail);
  }
}

// ---- after the main pass (and stage A of the long runs): one launch, three kinds of blocks ----
// Blocks [0, g_short): short crossing runs, one lane group per entry.  Blocks [g_short,
// g_short + g_long): stage B of the long crossing runs.  The rest: the counts of every run in
// the form the reference reports them, to `counts` or to the class buffers.
struct CountsOut {
  int plus_one;        // 1 + sum of cnt when cnt is given and the mean is asked (sparse_optim.py:145-148)
  int64_t* counts;     // [U], nullable
  int64_t* cls[3];     // per class, nullable
  int64_t n;
};

template <int VEC, int G, int VPL>
__global__ void __launch_bounds__(kBlock) segsum_finish_kernel(SegArgs a, CountsOut co, int g_short, int g_long) {
  using V = typename VecF<VEC>::T;
  const int64_t U_runs = *a.num_runs;
  if ((int)blockIdx.x >= g_short + g_long) {
    const int64_t i = (int64_t)(blockIdx.x - g_short - g_long) * blockDim.x + threadIdx.x;
    if (i >= co.n || i >= U_runs) return;
    const int64_t c = (int64_t)run_count(a, i) + co.plus_one;
    if (co.counts) co.counts[i] = c;
    if (a.dclass) {
      const int k = a.dclass[i];
      int64_t* out = (k >= 0 && k < 3) ? co.cls[k] : nullptr;
      if (out) out[a.dpos[i]] = c;
    }
    return;
  }
  if ((int)blockIdx.x >= g_short) {
    // stage B of a long run: tail partial + the slice sums 0..kSlices-1, in that order
    const int count = a.list_counts[1];
    const int cols = a.cols;
    for (int64_t e = blockIdx.x - g_short; e < count; e += g_long) {
      const int2 ent = a.long_list[e];
      const int64_t c = ent.x, u = ent.y;
      for (int col = threadIdx.x; col < cols; col += blockDim.x) {
        float acc = a.tail_part[c * cols + col];
        for (int sl = 0; sl < 32; ++sl) acc += a.slice_part[(e * 32 + sl) * cols + col];
        if (a.mean) acc /= denominator(a, run_count(a, u));
        float* dst = out_row(a, u);
        if (dst) dst[col] = acc;
      }
    }
    return;
  }
  const int sub = threadIdx.x & (G - 1);
  const int64_t grp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) / G;
  const int64_t ngrp = ((int64_t)g_short * blockDim.x) / G;
  const int count = a.list_counts[0];
  const int vpr = a.cols / VEC;
  for (int64_t e = grp; e < count; e += ngrp) {
    const int2 ent = a.short_list[e];
    const int64_t c = ent.x, u = ent.y;
    const int64_t run_end = __ldg(a.run_start + u + 1);
    const int64_t last_chunk = (run_end - 1) / a.chunk;
    V acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const int k = sub + v * G;
      if (k < vpr) acc[v] = reinterpret_cast<const V*>(a.tail_part + c * a.cols)[k];
    }
    for (int64_t cc = c + 1; cc <= last_chunk; ++cc) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int k = sub + v * G;
        if (k < vpr) vadd(acc[v], reinterpret_cast<const V*>(a.head_part + cc * a.cols)[k]);
      }
    }
    if (a.mean) {
      const float d = denominator(a, run_count(a, u));
#pragma unroll
      for (int v = 0; v < VPL; ++v) vdiv(acc[v], d);
    }
    float* dst = out_row(a, u);
    if (dst) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const int k = sub + v * G;
        if (k < vpr) reinterpret_cast<V*>(dst)[k] = acc[v];
      }
    }
  }
}

// ---- fix-up of long crossing runs, two launches ----------------------------------------------
// A long run leaves hundreds to thousands of partial rows (the hottest id of a
// Zipf batch).  Stage A cuts the partial list of every long run into kSlices
// contiguous slices; one CTA adds one slice (its threads form `strands` that walk
// the slice interleaved, then the strand sums are added 0,1,2,...).  Stage B adds
// the tail partial and the slice sums 0..kSlices-1 of a run and writes the row.
// Shapes depend only on the run length, so the result is reproducible.
constexpr int kSlices = 32;
constexpr int kEntriesInFlight = 8;

__global__ void __launch_bounds__(kLongBlock) segsum_fix_long_a_kernel(SegArgs a) {
  extern __shared__ float s_part[];  // [strands][cols]
  const int count = a.list_counts[1];
  const int64_t U_runs = *a.num_runs;
  const int cols = a.cols;
  const int strands = kLongBlock / cols;  // cols <= kLongBlock
  const int slice = blockIdx.x % kSlices;
  const int col = threadIdx.x % cols;
  const int strand = threadIdx.x / cols;
  for (int64_t e = blockIdx.x / kSlices; e < count; e += kEntriesInFlight) {
    const int2 ent = a.long_list[e];
    const int64_t c = ent.x, u = ent.y;
    const int64_t run_end = (u + 1 < U_runs) ? __ldg(a.run_start + u + 1) : effective_n(a);
    const int64_t last_chunk = (run_end - 1) / a.chunk;
    const int64_t parts = last_chunk - c;  // head partials c+1 .. last_chunk
    const int64_t seg = (parts + kSlices - 1) / kSlices;
    const int64_t lo = c + 1 + slice * seg;
    const int64_t hi = (lo + seg < last_chunk + 1) ? lo + seg : last_chunk + 1;
    if (strand < strands) {
      float acc = 0.f;
      int64_t cc = lo + strand;
      // four loads in flight, added in index order
      for (; cc + 3 * strands < hi; cc += 4 * strands) {
        const float x0 = a.head_part[cc * cols + col];
        const float x1 = a.head_part[(cc + strands) * cols + col];
        const float x2 = a.head_part[(cc + 2 * strands) * cols + col];
        const float x3 = a.head_part[(cc + 3 * strands) * cols + col];
        acc += x0; acc += x1; acc += x2; acc += x3;
      }
      for (; cc < hi; cc += strands) acc += a.head_part[cc * cols + col];
      s_part[strand * cols + col] = acc;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < cols; k += kLongBlock) {
      float acc = 0.f;
      for (int st = 0; st < strands; ++st) acc += s_part[st * cols + k];
      a.slice_part[(e * kSlices + slice) * cols + k] = acc;
    }
    __syncthreads();
  }
}

// ---- small helpers ----------------------------------------------------------------------------
int choose_chunk(int64_t n) {
  // at least ~16 chunks per SM, between 32 and 128 rows
  int64_t target = n / ((int64_t)sm_count() * 16);
  int r = 32;
  while (r * 2 <= target && r < 128) r *= 2;
  return r;
}

struct SegPlan {
  unsigned long long* raw_counts;
  float *head_part, *tail_part, *slice_part;
  int2 *short_list, *long_list;
  int* list_counts;
  int chunk;
  int64_t num_chunks;
  int cols_max;
  size_t total;
};

SegPlan make_plan(void* ws, int64_t n, int64_t dim) {
  SegPlan s;
  Carver cv(ws ? ws : (void*)256);  // a null workspace still yields the sizes
  const int64_t m = n > 0 ? n : 1;
  s.raw_counts = cv.take<unsigned long long>(m);
  s.chunk = choose_chunk(m);
  s.num_chunks = ceil_div(m, s.chunk);
  s.cols_max = (int)(dim < 512 ? dim : 512);
  s.head_part = cv.take<float>((size_t)s.num_chunks * s.cols_max);
  s.tail_part = cv.take<float>((size_t)s.num_chunks * s.cols_max);
  // a long run covers more than kShortSpan chunks, so there are fewer than
  // num_chunks / kShortSpan of them; 32 slices each
  s.slice_part = cv.take<float>((size_t)(s.num_chunks / kShortSpan + 1) * 32 * s.cols_max);
  s.short_list = cv.take<int2>(s.num_chunks);
  s.long_list = cv.take<int2>(s.num_chunks);
  s.list_counts = cv.take<int>(4);
  s.total = cv.used() + 256;
  return s;
}

template <int VEC, int G, int VPL>
int launch_pass(const SegArgs& a, const CountsOut& co, cudaStream_t st) {
  const int64_t threads = a.num_chunks * G;
  if (a.cnt_in)
    HB_LAUNCH((segsum_main_kernel<VEC, G, VPL, true>), (int)ceil_div(threads, kBlock), kBlock, 0, st, a);
  else
    HB_LAUNCH((segsum_main_kernel<VEC, G, VPL, false>), (int)ceil_div(threads, kBlock), kBlock, 0, st, a);
  const int strands = kLongBlock / a.cols > 0 ? kLongBlock / a.cols : 1;
  const size_t smem = (size_t)strands * a.cols * sizeof(float);
  HB_LAUNCH(segsum_fix_long_a_kernel, kSlices * kEntriesInFlight, kLongBlock, smem, st, a);
  int g_short = (int)ceil_div(a.num_chunks * G, kBlock);
  const int cap = sm_count() * 8;
  if (g_short > cap) g_short = cap;
  const int g_long = 64;
  // counts are the same for every column pass: written with the first
  const bool want_counts = a.col0 == 0 && (co.counts || co.cls[0] || co.cls[1] || co.cls[2]);
  const int g_counts = want_counts ? (int)ceil_div(co.n, kBlock) : 0;
  HB_LAUNCH((segsum_finish_kernel<VEC, G, VPL>), g_short + g_long + g_counts, kBlock, 0, st, a, co, g_short, g_long);
  return HB_OK;
}

int dispatch_pass(const SegArgs& a, const CountsOut& co, bool vec4, cudaStream_t st) {
  if (vec4) {
    const int vpr = a.cols / 4;
    if (vpr > 64) return launch_pass<4, 32, 4>(a, co, st);
    if (vpr > 32) return launch_pass<4, 32, 2>(a, co, st);
    if (vpr > 16) return launch_pass<4, 32, 1>(a, co, st);
    if (vpr > 8) return launch_pass<4, 16, 1>(a, co, st);
    if (vpr > 4) return launch_pass<4, 8, 1>(a, co, st);
    if (vpr > 2) return launch_pass<4, 4, 1>(a, co, st);
    if (vpr > 1) return launch_pass<4, 2, 1>(a, co, st);
    return launch_pass<4, 1, 1>(a, co, st);
  }
  const int vpr = a.cols;
  if (vpr > 64) return launch_pass<1, 32, 4>(a, co, st);
  if (vpr > 32) return launch_pass<1, 32, 2>(a, co, st);
  if (vpr > 16) return launch_pass<1, 32, 1>(a, co, st);
  if (vpr > 8) return launch_pass<1, 16, 1>(a, co, st);
  if (vpr > 4) return launch_pass<1, 8, 1>(a, co, st);
  if (vpr > 2) return launch_pass<1, 4, 1>(a, co, st);
  if (vpr > 1) return launch_pass<1, 2, 1>(a, co, st);
  return launch_pass<1, 1, 1>(a, co, st);
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

size_t hb_segsum_runs_workspace_bytes(int64_t n, int64_t dim) { return make_plan(nullptr, n, dim).total; }

int hb_segsum_runs_f32(const hb_runs_t* runs, const float* grads, const int64_t* cnt_in, int64_t dim,
                       int mean, float* sums, int64_t* counts, const hb_class_split_t* split,
                       void* workspace, size_t workspace_bytes, hb_stream_t stream) {
  HB_CHECK_ARG(runs != nullptr && dim > 0, "hb_segsum_runs_f32: bad argument");
  const int64_t n = runs->n;
  HB_CHECK_ARG(n == 0 || (grads && runs->perm && runs->head && runs->run_start && runs->num_runs),
               "hb_segsum_runs_f32: null argument");
  HB_CHECK_ARG(n == 0 || split || sums, "hb_segsum_runs_f32: null output");
  HB_CHECK_ARG(!split || n == 0 || (runs->dclass && runs->dpos),
               "hb_segsum_runs_f32: a split needs runs built with the class table");
  if (n == 0) return HB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  SegPlan s = make_plan(workspace, n, dim);
  if (!workspace || workspace_bytes < s.total) {
    set_error("hb_segsum_runs_f32: workspace of %zu bytes needed, %zu given", s.total, workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  if (cnt_in) HB_CUDA(cudaMemsetAsync(s.raw_counts, 0, n * sizeof(unsigned long long), st));
  uintptr_t align_bits = (uintptr_t)grads | (uintptr_t)sums;
  if (split)
    for (int c = 0; c < 3; ++c) align_bits |= (uintptr_t)split->out_rows[c];
  const bool vec4 = (dim % 4 == 0) && (align_bits & 15) == 0;
  SegArgs a;
  a.head = runs->head;
  a.perm = runs->perm;
  a.run_start = runs->run_start;
  a.num_runs = runs->num_runs;
  a.grads = grads;
  a.cnt_in = cnt_in;
  a.n_dev = runs->n_dev;
  a.n = n;
  a.dim = dim;
  a.chunk = s.chunk;
  a.num_chunks = s.num_chunks;
  a.mean = mean;
  a.sums = sums;
  a.dclass = split ? runs->dclass : nullptr;
  a.dpos = runs->dpos;
  for (int c = 0; c < 3; ++c) a.class_rows[c] = split ? split->out_rows[c] : nullptr;
  a.counts = s.raw_counts;
  a.head_part = s.head_part;
  a.tail_part = s.tail_part;
  a.short_list = s.short_list;
  a.long_list = s.long_list;
  a.list_counts = s.list_counts;
  a.slice_part = s.slice_part;
  CountsOut co;
  co.plus_one = (cnt_in && mean) ? 1 : 0;
  co.counts = counts;
  for (int c = 0; c < 3; ++c) co.cls[c] = split ? split->out_cnt[c] : nullptr;
  co.n = n;
  const int tile = vec4 ? 512 : 128;
  int rc;
  for (int64_t col0 = 0; col0 < dim; col0 += tile) {
    a.col0 = col0;
    a.cols = (int)((dim - col0) < tile ? (dim - col0) : tile);
    if (col0 == 0) HB_CUDA(cudaMemsetAsync(s.list_counts, 0, 4 * sizeof(int), st));
    rc = dispatch_pass(a, co, vec4, st);
    if (rc != HB_OK) return rc;
  }
  return HB_OK;
}

size_t hb_unique_segsum_workspace_bytes(int64_t n, int64_t dim) {
  return align_up(hb_runs_workspace_bytes(n), 256) + make_plan(nullptr, n, dim).total;
}

int hb_unique_segsum_f32(const int64_t* ids, const float* grads, const int64_t* cnt_in, int64_t n,
                         const int64_t* n_dev, const int64_t* seg_counts, int64_t seg_cap,
                         int64_t dim, int id_bits, int mean,
                         int64_t* uniq_ids, float* sums,
                         int64_t* counts, int64_t* num_unique, hb_runs_t* runs_out,
                         const hb_class_split_t* split, void* workspace, size_t workspace_bytes,
                         hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && n < ((int64_t)1 << 31) && dim > 0, "hb_unique_segsum_f32: bad sizes");
  HB_CHECK_ARG(num_unique != nullptr, "hb_unique_segsum_f32: num_unique is null");
  HB_CHECK_ARG(n == 0 || (ids && grads), "hb_unique_segsum_f32: null argument");
  HB_CHECK_ARG(n == 0 || split || (uniq_ids && sums), "hb_unique_segsum_f32: null output");
  HB_CHECK_ARG(!split || (split->table && split->class_counts && split->table_len > 0),
               "hb_unique_segsum_f32: a split needs the class table, its length and class_counts");
  const size_t runs_bytes = align_up(hb_runs_workspace_bytes(n), 256);
  if (!workspace || workspace_bytes < hb_unique_segsum_workspace_bytes(n, dim)) {
    set_error("hb_unique_segsum_f32: workspace of %zu bytes needed, %zu given",
              hb_unique_segsum_workspace_bytes(n, dim), workspace_bytes);
    return HB_ERR_WORKSPACE;
  }
  hb_runs_t runs;
  int64_t* cls_ids[3] = {split ? split->out_ids[0] : nullptr, split ? split->out_ids[1] : nullptr,
                         split ? split->out_ids[2] : nullptr};
  int rc = hb_runs_build(ids, n, n_dev, seg_counts, seg_cap, id_bits, split ? split->table : nullptr,
                         split ? split->table_len : 0, split ? cls_ids : nullptr,
                         split ? split->class_counts : nullptr, uniq_ids, num_unique, workspace,
                         runs_bytes, &runs, stream);
  if (rc != HB_OK) return rc;
  if (runs_out) *runs_out = runs;
  return hb_segsum_runs_f32(&runs, grads, cnt_in, dim, mean, sums, counts, split,
                            static_cast<char*>(workspace) + runs_bytes, workspace_bytes - runs_bytes,
                            stream);
}

}  // extern "C"
