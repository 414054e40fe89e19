// Sparse optimiser row updates on the owning shard: Adam as the reference's
// SparseAdam.update (python/EmbCache/sparse_optim.py:590-685) and Adagrad (the
// reference has no Adagrad; the rule is the usual sparse Adagrad
// sum += g*g; emb -= lr * g / (sqrt(sum) + eps)).  State, gradient and embedding
// rows are read and written once, in one kernel; the reference moves state
// through cached fetch/set kernels and the embedding through a CPU write.
#include <cuda_fp16.h>

#include "launch.cuh"

namespace hb {
namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ int64_t effective_n(int64_t n, const int64_t* n_dev) {
  if (!n_dev) return n;
  const int64_t d = *n_dev;
  return d < n ? d : n;
}

struct RowMap {
  int64_t offset, stride, rows;
  __device__ __forceinline__ int64_t operator()(int64_t id) const {
    if (id < offset) return -1;
    const int64_t r = (id - offset) / stride;
    return r < rows ? r : -1;
  }
};

template <typename E> struct EmbIO;
template <> struct EmbIO<float> {
  static __device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct EmbIO<__half> {
  static __device__ __forceinline__ float4 load4(const __half* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __half2 a = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 b = *reinterpret_cast<const __half2*>(&raw.y);
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
  }
  static __device__ __forceinline__ void store4(__half* p, float4 v) {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
  static __device__ __forceinline__ float load(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};

struct AdamParams {
  float lr, beta1, beta2, eps, one_minus_beta1, one_minus_beta2;
};

__device__ __forceinline__ float adam_elem(float g, float& m, float& v, float bias1, float bias2,
                                           const AdamParams& p) {
  // update_mem = beta1*mem + (1-beta1)*grad; update_power = beta2*power + (1-beta2)*grad^2
  m = p.beta1 * m + p.one_minus_beta1 * g;
  v = p.beta2 * v + p.one_minus_beta2 * (g * g);
  const float mc = m / bias1;
  const float vc = v / bias2;
  return p.lr * mc / (sqrtf(vc) + p.eps);  // std_values, sparse_optim.py:654-655
}

// A group of G lanes per row, kOptRows rows in flight per group (their loads are
// issued together, then the arithmetic and the stores follow).
constexpr int kOptRows = 2;

template <typename E, bool VEC4>
__global__ void __launch_bounds__(kBlock, 4) sparse_adam_kernel(
    const int64_t* __restrict__ ids, const float* __restrict__ grads,
    const int64_t* __restrict__ cnt, int64_t n, const int64_t* __restrict__ n_dev, int64_t dim,
    RowMap map, float* __restrict__ step, float* __restrict__ mem, float* __restrict__ power,
    E* __restrict__ emb, AdamParams p, int glog2) {
  n = effective_n(n, n_dev);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t group = tid >> glog2;
  const int sub = (int)(tid & ((1 << glog2) - 1));
  const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) >> glog2;
  const int G = 1 << glog2;
  const int lane = threadIdx.x & 31;
  const int leader = lane & ~(G - 1);       // first lane of this row group
  const int64_t warp_first = group - (lane >> glog2);  // the loop bound is the same for the whole warp
  for (int64_t w0 = warp_first, i0 = group; w0 < n; w0 += ngroups * kOptRows, i0 += ngroups * kOptRows) {
    int64_t row[kOptRows];
    float bias1[kOptRows], bias2[kOptRows], c[kOptRows];
#pragma unroll
    for (int r = 0; r < kOptRows; ++r) {
      const int64_t i = i0 + r * ngroups;
      row[r] = i < n ? map(__ldg(ids + i)) : -1;
      // the per-row scalars are worked out by the group's first lane and handed round
      float b1 = 1.0f, b2 = 1.0f, cc = 1.0f;
      if (row[r] >= 0 && sub == 0) {
        // state_step = state_step + 1 (per row), sparse_optim.py:624-626
        const float t = step[row[r]] + 1.0f;
        b1 = 1.0f - powf(p.beta1, t);
        b2 = 1.0f - powf(p.beta2, t);
        cc = cnt ? (float)__ldg(cnt + i) : 1.0f;  // grad / cnt, sparse_optim.py:608-611
      }
      bias1[r] = __shfl_sync(0xffffffffu, b1, leader);
      bias2[r] = __shfl_sync(0xffffffffu, b2, leader);
      c[r] = __shfl_sync(0xffffffffu, cc, leader);
    }
    if (VEC4) {
      for (int64_t k = sub; k < (dim >> 2); k += G) {
        float4 gg[kOptRows], mm[kOptRows], vv[kOptRows], ee[kOptRows];
#pragma unroll
        for (int r = 0; r < kOptRows; ++r)
          if (row[r] >= 0) {
            gg[r] = __ldg(reinterpret_cast<const float4*>(grads + (i0 + r * ngroups) * dim) + k);
            mm[r] = reinterpret_cast<const float4*>(mem + row[r] * dim)[k];
            vv[r] = reinterpret_cast<const float4*>(power + row[r] * dim)[k];
            ee[r] = EmbIO<E>::load4(emb + row[r] * dim + 4 * k);
          }
#pragma unroll
        for (int r = 0; r < kOptRows; ++r)
          if (row[r] >= 0) {
            if (cnt) { gg[r].x /= c[r]; gg[r].y /= c[r]; gg[r].z /= c[r]; gg[r].w /= c[r]; }
            ee[r].x -= adam_elem(gg[r].x, mm[r].x, vv[r].x, bias1[r], bias2[r], p);
            ee[r].y -= adam_elem(gg[r].y, mm[r].y, vv[r].y, bias1[r], bias2[r], p);
            ee[r].z -= adam_elem(gg[r].z, mm[r].z, vv[r].z, bias1[r], bias2[r], p);
            ee[r].w -= adam_elem(gg[r].w, mm[r].w, vv[r].w, bias1[r], bias2[r], p);
            reinterpret_cast<float4*>(mem + row[r] * dim)[k] = mm[r];
            reinterpret_cast<float4*>(power + row[r] * dim)[k] = vv[r];
            EmbIO<E>::store4(emb + row[r] * dim + 4 * k, ee[r]);
          }
      }
    } else {
      for (int64_t k = sub; k < dim; k += G) {
#pragma unroll
        for (int r = 0; r < kOptRows; ++r)
          if (row[r] >= 0) {
            float gg = __ldg(grads + (i0 + r * ngroups) * dim + k);
            if (cnt) gg /= c[r];
            float mm = mem[row[r] * dim + k], vv = power[row[r] * dim + k];
            const float upd = adam_elem(gg, mm, vv, bias1[r], bias2[r], p);
            mem[row[r] * dim + k] = mm;
            power[row[r] * dim + k] = vv;
            E* e = emb + row[r] * dim + k;
            EmbIO<E>::store(e, EmbIO<E>::load(e) - upd);
          }
      }
    }
  }
}

// The vector path of both update rules (dim % 4 == 0, 16-byte aligned rows).  A warp takes 32
// rows per round: lane l works out the per-row scalars of row l once (for Adam the two bias
// corrections, whose powf would otherwise be issued for every 16 bytes of the row), then the
// warp walks the rows, G lanes per row and kOptRows rows in flight, taking the scalars by
// shuffle.  Divisions by per-row scalars are multiplications by their reciprocals (one ulp,
// far inside the 1e-5 the parity tests allow); the element-wise division and the square root
// are IEEE.
template <typename E, bool ADAM>
__global__ void __launch_bounds__(kBlock, 3) sparse_update_vec_kernel(
    const int64_t* __restrict__ ids, const float* __restrict__ grads,
    const int64_t* __restrict__ cnt, int64_t n, const int64_t* __restrict__ n_dev, int64_t dim,
    RowMap map, const float* __restrict__ step, float* __restrict__ s0, float* __restrict__ s1,
    E* __restrict__ emb, AdamParams p, int glog2, int rpw) {
  // rpw: rows a warp takes per round (32, or fewer so that a short list still fills the GPU)
  n = effective_n(n, n_dev);
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int G = 1 << glog2, rpp = 32 >> glog2;
  const int sub = lane & (G - 1), which = lane >> glog2;
  const int64_t vpr = dim >> 2;
  for (int64_t base = warp * rpw; base < n; base += nwarps * rpw) {
    const int64_t i = base + lane;
    const int64_t row = (lane < rpw && i < n) ? map(__ldg(ids + i)) : -1;
    float ra = 1.0f, rb = 1.0f, rc = 1.0f;
    if (row >= 0) {
      if (ADAM) {
        // state_step = state_step + 1 (per row), sparse_optim.py:624-626
        const float t = step[row] + 1.0f;
        ra = 1.0f / (1.0f - powf(p.beta1, t));
        rb = 1.0f / (1.0f - powf(p.beta2, t));
      }
      if (cnt) rc = 1.0f / (float)__ldg(cnt + i);  // grad / cnt, sparse_optim.py:608-611
    }
    for (int pass = 0; pass * rpp < rpw; pass += kOptRows) {
      int64_t rw[kOptRows];
      float a[kOptRows], b[kOptRows], c[kOptRows];
      const float4* gp[kOptRows];
#pragma unroll
      for (int u = 0; u < kOptRows; ++u) {
        const int q = ((pass + u) * rpp + which) & 31;
        rw[u] = __shfl_sync(0xffffffffu, row, q);
        a[u] = __shfl_sync(0xffffffffu, ra, q);
        b[u] = __shfl_sync(0xffffffffu, rb, q);
        c[u] = __shfl_sync(0xffffffffu, rc, q);
        if ((pass + u) * rpp + which >= rpw) rw[u] = -1;
        gp[u] = reinterpret_cast<const float4*>(grads + (base + q) * dim);
      }
      for (int64_t k = sub; k < vpr; k += G) {
        float4 gg[kOptRows], mm[kOptRows], vv[kOptRows], ee[kOptRows];
#pragma unroll
        for (int u = 0; u < kOptRows; ++u)
          if (rw[u] >= 0) {
            gg[u] = __ldg(gp[u] + k);
            mm[u] = reinterpret_cast<const float4*>(s0 + rw[u] * dim)[k];
            if (ADAM) vv[u] = reinterpret_cast<const float4*>(s1 + rw[u] * dim)[k];
            ee[u] = EmbIO<E>::load4(emb + rw[u] * dim + 4 * k);
          }
#pragma unroll
        for (int u = 0; u < kOptRows; ++u)
          if (rw[u] >= 0) {
            float* g4 = reinterpret_cast<float*>(&gg[u]);
            float* m4 = reinterpret_cast<float*>(&mm[u]);
            float* v4 = reinterpret_cast<float*>(&vv[u]);
            float* e4 = reinterpret_cast<float*>(&ee[u]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float g = cnt ? g4[j] * c[u] : g4[j];
              if (ADAM) {
                m4[j] = p.beta1 * m4[j] + p.one_minus_beta1 * g;
                v4[j] = p.beta2 * v4[j] + p.one_minus_beta2 * (g * g);
                e4[j] -= p.lr * (m4[j] * a[u]) / (sqrtf(v4[j] * b[u]) + p.eps);  // sparse_optim.py:654-655
              } else {
                m4[j] += g * g;
                e4[j] -= p.lr * g / (sqrtf(m4[j]) + p.eps);
              }
            }
            reinterpret_cast<float4*>(s0 + rw[u] * dim)[k] = mm[u];
            if (ADAM) reinterpret_cast<float4*>(s1 + rw[u] * dim)[k] = vv[u];
            EmbIO<E>::store4(emb + rw[u] * dim + 4 * k, ee[u]);
          }
      }
    }
  }
}

// rows per warp and round: 32 unless that leaves the GPU short of warps (a list of 84k rows is
// only 2.6k rounds of 32)
int rows_per_warp_for(int64_t n, int glog2) {
  const int min_rows = 32 >> glog2 > 4 ? 32 >> glog2 : 4;  // at least one pass of whole row groups
  int rpw = 32;
  while (rpw > min_rows && ceil_div(n, rpw) < (int64_t)sm_count() * 48) rpw >>= 1;
  return rpw;
}

int grid_for_warps(int64_t n, int rpw) {
  int64_t blocks = ceil_div(ceil_div(n, rpw) * 32, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}

// step[row] += 1 for every updated row; a launch of its own so that no lane of
// the update kernel can see the new step of its own row.
__global__ void bump_step_kernel(const int64_t* __restrict__ ids, int64_t n,
                                 const int64_t* __restrict__ n_dev, RowMap map,
                                 float* __restrict__ step) {
  n = effective_n(n, n_dev);
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int64_t row = map(__ldg(ids + i));
  if (row >= 0) step[row] += 1.0f;
}

template <typename E, bool VEC4>
__global__ void __launch_bounds__(kBlock) sparse_adagrad_kernel(
    const int64_t* __restrict__ ids, const float* __restrict__ grads,
    const int64_t* __restrict__ cnt, int64_t n, const int64_t* __restrict__ n_dev, int64_t dim,
    RowMap map, float* __restrict__ state_sum, E* __restrict__ emb, float lr, float eps, int glog2) {
  n = effective_n(n, n_dev);
  const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t group = tid >> glog2;
  const int sub = (int)(tid & ((1 << glog2) - 1));
  const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) >> glog2;
  const int G = 1 << glog2;
  for (int64_t i = group; i < n; i += ngroups) {
    const int64_t row = map(__ldg(ids + i));
    if (row < 0) continue;
    const float c = cnt ? (float)__ldg(cnt + i) : 1.0f;
    const float* g = grads + i * dim;
    float* s = state_sum + row * dim;
    E* e = emb + row * dim;
    if (VEC4) {
      for (int64_t k = sub; k < (dim >> 2); k += G) {
        float4 gg = __ldg(reinterpret_cast<const float4*>(g) + k);
        if (cnt) { gg.x /= c; gg.y /= c; gg.z /= c; gg.w /= c; }
        float4 ss = reinterpret_cast<float4*>(s)[k];
        float4 ee = EmbIO<E>::load4(e + 4 * k);
        ss.x += gg.x * gg.x; ss.y += gg.y * gg.y; ss.z += gg.z * gg.z; ss.w += gg.w * gg.w;
        ee.x -= lr * gg.x / (sqrtf(ss.x) + eps);
        ee.y -= lr * gg.y / (sqrtf(ss.y) + eps);
        ee.z -= lr * gg.z / (sqrtf(ss.z) + eps);
        ee.w -= lr * gg.w / (sqrtf(ss.w) + eps);
        reinterpret_cast<float4*>(s)[k] = ss;
        EmbIO<E>::store4(e + 4 * k, ee);
      }
    } else {
      for (int64_t k = sub; k < dim; k += G) {
        float gg = __ldg(g + k);
        if (cnt) gg /= c;
        const float ss = s[k] + gg * gg;
        s[k] = ss;
        EmbIO<E>::store(e + k, EmbIO<E>::load(e + k) - lr * gg / (sqrtf(ss) + eps));
      }
    }
  }
}

int group_log2_for(int64_t units) {
  int g = 0;
  while ((1 << g) < units && g < 5) ++g;
  return g;
}

int grid_for_groups(int64_t n, int glog2) {
  int64_t blocks = ceil_div(ceil_div(n, kOptRows) << glog2, kBlock);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace
}  // namespace hb

using namespace hb;

extern "C" {

int hb_sparse_adam(const int64_t* ids, const float* grads, const int64_t* cnt, int64_t n,
                   const int64_t* n_dev, int64_t dim, int64_t id_offset, int64_t id_stride,
                   int64_t rows, float* step, float* mem, float* power, void* emb, int emb_elem_bytes,
                   double lr, double beta1, double beta2, double eps, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && dim > 0 && rows > 0 && id_stride > 0, "hb_sparse_adam: bad sizes");
  HB_CHECK_ARG(emb_elem_bytes == 4 || emb_elem_bytes == 2,
               "hb_sparse_adam: embedding must be fp32 (4) or fp16 (2)");
  HB_CHECK_ARG(n == 0 || (ids && grads && step && mem && power && emb), "hb_sparse_adam: null argument");
  if (n == 0) return HB_OK;
  const AdamParams p{(float)lr, (float)beta1, (float)beta2, (float)eps, (float)(1.0 - beta1),
                     (float)(1.0 - beta2)};
  const RowMap map{id_offset, id_stride, rows};
  const uintptr_t bits = (uintptr_t)grads | (uintptr_t)mem | (uintptr_t)power | (uintptr_t)emb;
  const bool vec4 = dim % 4 == 0 && (bits & 15) == 0;
  const int glog2 = group_log2_for(vec4 ? dim / 4 : dim);
  const int grid = grid_for_groups(n, glog2);
  const int rpw = rows_per_warp_for(n, glog2);
  cudaStream_t st = (cudaStream_t)stream;
#define HB_ADAM(E, V)                                                                          \
  HB_LAUNCH((sparse_adam_kernel<E, V>), grid, kBlock, 0, st, ids, grads, cnt, n, n_dev, dim, map, \
            step, mem, power, (E*)emb, p, glog2)
#define HB_ADAM_VEC(E)                                                                         \
  HB_LAUNCH((sparse_update_vec_kernel<E, true>), grid_for_warps(n, rpw), kBlock, 0, st, ids, grads, cnt, n, \
            n_dev, dim, map, step, mem, power, (E*)emb, p, glog2, rpw)
  if (emb_elem_bytes == 4) {
    if (vec4) HB_ADAM_VEC(float); else HB_ADAM(float, false);
  } else {
    if (vec4) HB_ADAM_VEC(__half); else HB_ADAM(__half, false);
  }
#undef HB_ADAM_VEC
#undef HB_ADAM
  HB_LAUNCH(bump_step_kernel, (int)ceil_div(n, kBlock), kBlock, 0, st, ids, n, n_dev, map, step);
  return HB_OK;
}

int hb_sparse_adagrad(const int64_t* ids, const float* grads, const int64_t* cnt, int64_t n,
                      const int64_t* n_dev, int64_t dim, int64_t id_offset, int64_t id_stride,
                      int64_t rows, float* state_sum, void* emb, int emb_elem_bytes, double lr,
                      double eps, hb_stream_t stream) {
  HB_CHECK_ARG(n >= 0 && dim > 0 && rows > 0 && id_stride > 0, "hb_sparse_adagrad: bad sizes");
  HB_CHECK_ARG(emb_elem_bytes == 4 || emb_elem_bytes == 2,
               "hb_sparse_adagrad: embedding must be fp32 (4) or fp16 (2)");
  HB_CHECK_ARG(n == 0 || (ids && grads && state_sum && emb), "hb_sparse_adagrad: null argument");
  if (n == 0) return HB_OK;
  const RowMap map{id_offset, id_stride, rows};
  const uintptr_t bits = (uintptr_t)grads | (uintptr_t)state_sum | (uintptr_t)emb;
  // fp16 rows are read 8 bytes at a time on the vector path
  const bool vec4 = dim % 4 == 0 && (bits & 15) == 0;
  const int glog2 = group_log2_for(vec4 ? dim / 4 : dim);
  const int grid = grid_for_groups(n, glog2);
  const int rpw = rows_per_warp_for(n, glog2);
  cudaStream_t st = (cudaStream_t)stream;
#define HB_ADAGRAD(E, V)                                                                        \
  HB_LAUNCH((sparse_adagrad_kernel<E, V>), grid, kBlock, 0, st, ids, grads, cnt, n, n_dev, dim, \
            map, state_sum, (E*)emb, (float)lr, (float)eps, glog2)
  const AdamParams p{(float)lr, 0.f, 0.f, (float)eps, 0.f, 0.f};
#define HB_ADAGRAD_VEC(E)                                                                       \
  HB_LAUNCH((sparse_update_vec_kernel<E, false>), grid_for_warps(n, rpw), kBlock, 0, st, ids, grads, cnt, n, \
            n_dev, dim, map, nullptr, state_sum, nullptr, (E*)emb, p, glog2, rpw)
  if (emb_elem_bytes == 4) {
    if (vec4) HB_ADAGRAD_VEC(float); else HB_ADAGRAD(float, false);
  } else {
    if (vec4) HB_ADAGRAD_VEC(__half); else HB_ADAGRAD(__half, false);
  }
#undef HB_ADAGRAD_VEC
#undef HB_ADAGRAD
  return HB_OK;
}

}  // extern "C"
