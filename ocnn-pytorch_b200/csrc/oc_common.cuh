// Shared helpers for the octree hot-path kernels (sm_100a only).
//
// Everything in this library is reached through the extern "C" entry points
// declared in include/octconv.h.  Entry points never allocate device memory:
// callers pass outputs and workspaces.  Errors are reported as negative status
// codes plus a thread-local message (oc_last_error()).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/octconv.h"

namespace oc {

void set_error(const char* fmt, ...);

#define OC_REQUIRE(cond, code, ...)            \
  do {                                         \
    if (!(cond)) {                             \
      oc::set_error(__VA_ARGS__);              \
      return (code);                           \
    }                                          \
  } while (0)

#define OC_CUDA_OK(expr)                                                     \
  do {                                                                       \
    cudaError_t e__ = (expr);                                                \
    if (e__ != cudaSuccess) {                                                \
      oc::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));        \
      return OC_ECUDA;                                                       \
    }                                                                        \
  } while (0)

#define OC_LAUNCH_OK(name)                                                   \
  do {                                                                       \
    cudaError_t e__ = cudaGetLastError();                                    \
    if (e__ != cudaSuccess) {                                                \
      oc::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__)); \
      return OC_ECUDA;                                                       \
    }                                                                        \
  } while (0)

static inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static inline size_t dtype_size(int dtype) {
  return dtype == OC_F32 ? 4 : 2;
}

// Number of SMs of the current device (cached per process; B200 = 148).
int sm_count();


// Tap list passed by value to kernels: column of the neighbour table per tap.
struct TapList { int t[OC_MAX_TAPS]; };

static inline int make_taps(const int* h_taps, int K, int ncols, TapList* out, const char* who) {
  OC_REQUIRE(K >= 1 && K <= OC_MAX_TAPS, OC_EINVAL, "%s: K %d not in [1,27]", who, K);
  OC_REQUIRE(h_taps, OC_EINVAL, "%s: null tap list", who);
  for (int k = 0; k < OC_MAX_TAPS; ++k) out->t[k] = 0;
  for (int k = 0; k < K; ++k) {
    OC_REQUIRE(h_taps[k] >= 0 && h_taps[k] < ncols, OC_EINVAL, "%s: tap %d column %d out of range",
               who, k, h_taps[k]);
    out->t[k] = h_taps[k];
  }
  return OC_OK;
}

static inline unsigned grid_1d(int64_t n, int threads = 256, int per_sm = 16) {
  int64_t blocks = cdiv(n, threads);
  int64_t cap = (int64_t)sm_count() * per_sm;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// ---------------------------------------------------------------------------
// Element conversion helpers
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Generic index load: neighbour tables are int64 at the reference boundary and
// int32 in the library's own shadow copies.
template <typename I> __device__ __forceinline__ int load_idx(const I* p) { return (int)(*p); }

// ---------------------------------------------------------------------------
// Morton ("shuffled") key bit tricks: x -> bit 3i+2, y -> 3i+1, z -> 3i.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint64_t spread3(uint64_t v) {
  v &= 0x1fffffULL;
  v = (v | (v << 32)) & 0x001f00000000ffffULL;
  v = (v | (v << 16)) & 0x001f0000ff0000ffULL;
  v = (v | (v << 8)) & 0x100f00f00f00f00fULL;
  v = (v | (v << 4)) & 0x10c30c30c30c30c3ULL;
  v = (v | (v << 2)) & 0x1249249249249249ULL;
  return v;
}

__host__ __device__ __forceinline__ uint64_t compact3(uint64_t v) {
  v &= 0x1249249249249249ULL;
  v = (v | (v >> 2)) & 0x10c30c30c30c30c3ULL;
  v = (v | (v >> 4)) & 0x100f00f00f00f00fULL;
  v = (v | (v >> 8)) & 0x001f0000ff0000ffULL;
  v = (v | (v >> 16)) & 0x001f00000000ffffULL;
  v = (v | (v >> 32)) & 0x1fffffULL;
  return v;
}

__host__ __device__ __forceinline__ uint64_t morton3(uint64_t x, uint64_t y, uint64_t z) {
  return (spread3(x) << 2) | (spread3(y) << 1) | spread3(z);
}

// ---------------------------------------------------------------------------
// Device-wide exclusive scan of int32 flags produced by a functor.
//   excl[i] = sum_{j<i} f(j),  *total = sum_j f(j)       (i < n)
// n is either a host value or read from device memory (n_dev != nullptr, in
// which case the launch is sized by n_max and surplus blocks exit).
// Three kernels (block reduce, single-block scan of block sums, block scan);
// no inter-block spinning.
// ---------------------------------------------------------------------------
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

static inline size_t scan_workspace_bytes(int64_t n_max) {
  return align_up((size_t)(cdiv(n_max, SCAN_TILE) + 1) * sizeof(int32_t), 256);
}

__device__ __forceinline__ int warp_incl_scan(int v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// Block-wide exclusive scan over SCAN_THREADS values; returns exclusive prefix
// and writes the block total to *total (valid for all threads after return).
__device__ __forceinline__ int block_excl_scan(int v, int* total) {
  __shared__ int warp_sums[SCAN_THREADS / 32];
  __shared__ int block_total;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = warp_incl_scan(v);
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
    int wi = warp_incl_scan(w);
    if (lane < SCAN_THREADS / 32) warp_sums[lane] = wi - w;
    if (lane == SCAN_THREADS / 32 - 1) block_total = wi;
  }
  __syncthreads();
  int r = incl - v + warp_sums[warp];
  *total = block_total;
  __syncthreads();
  return r;
}

template <typename F>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_reduce_kernel(F f, int64_t n_host, const int64_t* n_dev, int32_t* block_sums) {
  const int64_t n = n_dev ? *n_dev : n_host;
  const int64_t base = (int64_t)blockIdx.x * SCAN_TILE;
  if (base >= n) { if (threadIdx.x == 0) block_sums[blockIdx.x] = 0; return; }
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    if (i < n) s += f(i, n);
  }
  int total;
  block_excl_scan(s, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// Single block: exclusive scan of block_sums[0..nb) in place; total -> *total64.
static __global__ void __launch_bounds__(SCAN_THREADS)
scan_blocksums_kernel(int32_t* block_sums, int64_t nb, int64_t* total64) {
  int carry = 0;
  for (int64_t base = 0; base < nb; base += SCAN_THREADS) {
    int64_t i = base + threadIdx.x;
    int v = i < nb ? block_sums[i] : 0;
    int total;
    int ex = block_excl_scan(v, &total);
    if (i < nb) block_sums[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0 && total64) *total64 = carry;
}

// Calls sink(i, n, flag, exclusive_prefix) for every i < n.
template <typename F, typename S>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(F f, S sink, int64_t n_host, const int64_t* n_dev, const int32_t* block_sums) {
  const int64_t n = n_dev ? *n_dev : n_host;
  const int64_t base = (int64_t)blockIdx.x * SCAN_TILE;
  if (base >= n) return;
  int fl[SCAN_ITEMS];
  int s = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    fl[k] = (i < n) ? f(i, n) : 0;
    s += fl[k];
  }
  int total;
  int ex = block_excl_scan(s, &total) + block_sums[blockIdx.x];
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; ++k) {
    int64_t i = base + (int64_t)threadIdx.x * SCAN_ITEMS + k;
    if (i < n) sink(i, n, fl[k], ex);
    ex += fl[k];
  }
}

template <typename F, typename S>
static inline cudaError_t device_scan(F f, S sink, int64_t n_max, const int64_t* n_dev,
                                      int32_t* block_sums, int64_t* total_dev,
                                      cudaStream_t stream) {
  if (n_max <= 0) {
    if (total_dev) return cudaMemsetAsync(total_dev, 0, sizeof(int64_t), stream);
    return cudaSuccess;
  }
  const int64_t nb = cdiv(n_max, SCAN_TILE);
  scan_reduce_kernel<<<(unsigned)nb, SCAN_THREADS, 0, stream>>>(f, n_max, n_dev, block_sums);
  scan_blocksums_kernel<<<1, SCAN_THREADS, 0, stream>>>(block_sums, nb, total_dev);
  scan_apply_kernel<<<(unsigned)nb, SCAN_THREADS, 0, stream>>>(f, sink, n_max, n_dev, block_sums);
  return cudaGetLastError();
}

}  // namespace oc
