// Key search and point interpolation on an octree level:
//   Octree.search_key / search_xyzb          ocnn/octree/octree.py:448-488
//   octree_nearest_pts, octree_linear_pts    ocnn/nn/octree_interp.py:16-98
// The reference runs torch.searchsorted, builds a sparse COO matrix of the 8 corner weights
// per point and multiplies it with the features (cuSPARSE); here a binary search kernel,
// one kernel that finds the 8 corners and their weights, and warp-per-point gather /
// scatter kernels.  Gradients with respect to the features only.
#include "oc_common.cuh"

namespace oc {

// position of `q` in the ascending array keys[0..n), or -1
__device__ __forceinline__ int64_t find_key(const int64_t* __restrict__ keys, int64_t n, int64_t q) {
  int64_t lo = 0, hi = n;                 // first position with keys[pos] >= q
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (keys[mid] < q) lo = mid + 1; else hi = mid;
  }
  return (lo < n && keys[lo] == q) ? lo : -1;
}

__global__ void search_key_kernel(const int64_t* __restrict__ keys, int64_t n,
                                  const int64_t* __restrict__ query, int64_t m, int64_t* __restrict__ idx) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x)
    idx[i] = find_key(keys, n, query[i]);
}

// xyz2key of the reference for integer coordinates (shuffled_key.py:60-90): coordinates are
// taken modulo 2^depth (also negative ones: two's complement and the bit mask), the batch
// index goes to bit 48.
__device__ __forceinline__ int64_t key_of(int64_t x, int64_t y, int64_t z, int64_t b, int depth) {
  const uint64_t mask = (1ULL << depth) - 1ULL;
  const uint64_t k = morton3((uint64_t)x & mask, (uint64_t)y & mask, (uint64_t)z & mask);
  return (int64_t)(((uint64_t)b << 48) | k);
}

// One thread per (point, corner): the 8 cell centres around a point (ocnn/nn/octree_interp.py:63-88).
//   idx8[p, j] = row of corner j or -1;  w8[p, j] = | prod_d ((1 - g_jd) - frac_d) |
__global__ void interp_corners_kernel(const int64_t* __restrict__ keys, int64_t n, const float* __restrict__ pts,
                                      int64_t m, int depth, int bound_check, int64_t* __restrict__ idx8,
                                      float* __restrict__ w8) {
  const float bound = (float)(1 << depth);
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < m * 8; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = t >> 3;
    const int j = (int)(t & 7);
    const float g[3] = {(float)((j >> 2) & 1), (float)((j >> 1) & 1), (float)(j & 1)};
    float w = 1.f;
    int64_t c[3];
    bool inside = true;
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      const float f = __fsub_rn(pts[p * 4 + d], 0.5f);     // values sit at the cell centres
      const float fi = floorf(f);
      const float frac = __fsub_rn(f, fi);
      const float cn = __fadd_rn(fi, g[d]);
      w = __fmul_rn(w, __fsub_rn(__fsub_rn(1.0f, g[d]), frac));
      inside = inside && cn >= 0.f && cn < bound;
      c[d] = (int64_t)cn;
    }
    int64_t r = find_key(keys, n, key_of(c[0], c[1], c[2], (int64_t)pts[p * 4 + 3], depth));
    if (bound_check && !inside) r = -1;
    idx8[t] = r;
    w8[t] = fabsf(w);
  }
}

template <typename T>
__device__ __forceinline__ float ld(const T* p) { return to_f32<T>(*p); }

// out[p, :] = data[idx[p], :] or 0      (one warp per point, lanes over channels)
template <typename T>
__global__ void rows_gather_kernel(const T* __restrict__ data, const int64_t* __restrict__ idx, int64_t m, int C,
                                   T* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < m; p += nw) {
    const int64_t r = idx[p];
    for (int c = lane; c < C; c += 32) out[p * C + c] = r >= 0 ? data[r * C + c] : from_f32<T>(0.f);
  }
}

// acc[idx[p], :] += grad[p, :]          (fp32 accumulator, atomics: points share rows)
template <typename T>
__global__ void rows_scatter_add_kernel(const T* __restrict__ grad, const int64_t* __restrict__ idx, int64_t m, int C,
                                        float* __restrict__ acc) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < m; p += nw) {
    const int64_t r = idx[p];
    if (r < 0) continue;
    for (int c = lane; c < C; c += 32) atomicAdd(acc + r * C + c, ld<T>(grad + p * C + c));
  }
}

// FWD: out[p] = sum_j w_j data[idx_j] / (sum_j w_j + 1e-12) over the corners that exist
// !FWD: acc[idx_j] += w_j / (sum + 1e-12) * grad[p]
template <typename T, bool FWD>
__global__ void interp_linear_kernel(const T* __restrict__ src, const int64_t* __restrict__ idx8,
                                     const float* __restrict__ w8, int64_t m, int C, T* __restrict__ out,
                                     float* __restrict__ acc) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < m; p += nw) {
    int64_t my_r = -1;
    float my_w = 0.f;
    if (lane < 8) {
      my_r = idx8[p * 8 + lane];
      my_w = my_r >= 0 ? w8[p * 8 + lane] : 0.f;
    }
    int64_t r[8];
    float w[8];
    float norm = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      r[j] = __shfl_sync(0xffffffffu, my_r, j);
      w[j] = __shfl_sync(0xffffffffu, my_w, j);
      norm += w[j];
    }
    const float inv = 1.0f / (norm + 1e-12f);
    for (int c = lane; c < C; c += 32) {
      if (FWD) {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r[j] >= 0) a = fmaf(w[j], ld<T>(src + r[j] * C + c), a);
        out[p * C + c] = from_f32<T>(a * inv);
      } else {
        const float gsc = ld<T>(src + p * C + c) * inv;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r[j] >= 0) atomicAdd(acc + r[j] * C + c, w[j] * gsc);
      }
    }
  }
}

static inline unsigned warp_grid(int64_t m) {   // one warp per item, 8 warps per block
  int64_t blocks = cdiv(m, 8);
  const int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

static inline bool dtype_ok(int dtype) { return dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16; }

}  // namespace oc

using namespace oc;

#define OC_BY_DTYPE(dtype, stmt)                                  \
  do {                                                            \
    if ((dtype) == OC_F32) { using T = float; stmt; }             \
    else if ((dtype) == OC_F16) { using T = __half; stmt; }       \
    else { using T = __nv_bfloat16; stmt; }                       \
  } while (0)

extern "C" int oc_search_key(const int64_t* keys, int64_t n, const int64_t* query, int64_t m, int64_t* idx,
                             void* stream) {
  OC_REQUIRE(n >= 0 && m >= 0, OC_EINVAL, "oc_search_key: negative size");
  if (m == 0) return OC_OK;
  OC_REQUIRE((keys || n == 0) && query && idx, OC_EINVAL, "oc_search_key: null pointer");
  search_key_kernel<<<grid_1d(m, 256, 16), 256, 0, (cudaStream_t)stream>>>(keys, n, query, m, idx);
  OC_LAUNCH_OK("search_key_kernel");
  return OC_OK;
}

extern "C" int oc_interp_corners(const int64_t* keys, int64_t n, const float* pts, int64_t m, int depth,
                                 int bound_check, int64_t* idx8, float* w8, void* stream) {
  OC_REQUIRE(depth >= 0 && depth <= 16, OC_EINVAL, "oc_interp_corners: depth %d not in [0,16]", depth);
  OC_REQUIRE(n >= 0 && m >= 0, OC_EINVAL, "oc_interp_corners: negative size");
  if (m == 0) return OC_OK;
  OC_REQUIRE((keys || n == 0) && pts && idx8 && w8, OC_EINVAL, "oc_interp_corners: null pointer");
  interp_corners_kernel<<<grid_1d(m * 8, 256, 16), 256, 0, (cudaStream_t)stream>>>(keys, n, pts, m, depth,
                                                                                    bound_check, idx8, w8);
  OC_LAUNCH_OK("interp_corners_kernel");
  return OC_OK;
}

extern "C" int oc_rows_gather(const void* data, const int64_t* idx, int64_t m, int C, int dtype, void* out,
                              void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_rows_gather: bad dtype %d", dtype);
  OC_REQUIRE(m >= 0 && C >= 1, OC_EINVAL, "oc_rows_gather: bad sizes");
  if (m == 0) return OC_OK;
  OC_REQUIRE(idx && out, OC_EINVAL, "oc_rows_gather: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_DTYPE(dtype, (rows_gather_kernel<T><<<warp_grid(m), 256, 0, s>>>((const T*)data, idx, m, C, (T*)out)));
  OC_LAUNCH_OK("rows_gather_kernel");
  return OC_OK;
}

extern "C" int oc_rows_scatter_add(const void* grad, const int64_t* idx, int64_t m, int C, int dtype, float* acc,
                                   void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_rows_scatter_add: bad dtype %d", dtype);
  OC_REQUIRE(m >= 0 && C >= 1, OC_EINVAL, "oc_rows_scatter_add: bad sizes");
  if (m == 0) return OC_OK;
  OC_REQUIRE(grad && idx && acc, OC_EINVAL, "oc_rows_scatter_add: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_DTYPE(dtype, (rows_scatter_add_kernel<T><<<warp_grid(m), 256, 0, s>>>((const T*)grad, idx, m, C, acc)));
  OC_LAUNCH_OK("rows_scatter_add_kernel");
  return OC_OK;
}

extern "C" int oc_interp_linear_fwd(const void* data, const int64_t* idx8, const float* w8, int64_t m, int C,
                                    int dtype, void* out, void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_interp_linear_fwd: bad dtype %d", dtype);
  OC_REQUIRE(m >= 0 && C >= 1, OC_EINVAL, "oc_interp_linear_fwd: bad sizes");
  if (m == 0) return OC_OK;
  OC_REQUIRE(idx8 && w8 && out, OC_EINVAL, "oc_interp_linear_fwd: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_DTYPE(dtype, (interp_linear_kernel<T, true><<<warp_grid(m), 256, 0, s>>>((const T*)data, idx8, w8, m, C,
                                                                                 (T*)out, nullptr)));
  OC_LAUNCH_OK("interp_linear_kernel");
  return OC_OK;
}

extern "C" int oc_interp_linear_bwd(const void* grad_out, const int64_t* idx8, const float* w8, int64_t m, int C,
                                    int dtype, float* acc, void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_interp_linear_bwd: bad dtype %d", dtype);
  OC_REQUIRE(m >= 0 && C >= 1, OC_EINVAL, "oc_interp_linear_bwd: bad sizes");
  if (m == 0) return OC_OK;
  OC_REQUIRE(grad_out && idx8 && w8 && acc, OC_EINVAL, "oc_interp_linear_bwd: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_DTYPE(dtype, (interp_linear_kernel<T, false><<<warp_grid(m), 256, 0, s>>>((const T*)grad_out, idx8, w8, m,
                                                                                  C, nullptr, acc)));
  OC_LAUNCH_OK("interp_linear_kernel");
  return OC_OK;
}
