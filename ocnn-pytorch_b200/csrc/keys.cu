// Morton ("shuffled") key encode / decode.
//
// The reference encodes with 256-entry look-up tables and decodes with 512-entry
// tables (ocnn/octree/shuffled_key.py:12-115).  Here both directions are pure
// bit arithmetic in registers: one coalesced read per coordinate and one
// coalesced write per key, i.e. the kernels are HBM-streaming.
#include "oc_common.cuh"

namespace oc {

template <typename T> __device__ __forceinline__ long long coord_to_i64(T v) { return (long long)v; }

template <typename T>
__global__ void xyz2key_kernel(const T* __restrict__ x, const T* __restrict__ y,
                               const T* __restrict__ z, const T* __restrict__ b, int64_t n,
                               int depth, int64_t* __restrict__ key) {
  const uint64_t mask = (1ULL << depth) - 1ULL;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    // `.long()` truncates toward zero; negative values wrap through the mask.
    uint64_t xi = (uint64_t)coord_to_i64(x[i]) & mask;
    uint64_t yi = (uint64_t)coord_to_i64(y[i]) & mask;
    uint64_t zi = (uint64_t)coord_to_i64(z[i]) & mask;
    uint64_t k = morton3(xi, yi, zi);
    if (b) k |= ((uint64_t)coord_to_i64(b[i])) << 48;
    key[i] = (int64_t)k;
  }
}

__global__ void key2xyz_kernel(const int64_t* __restrict__ key, int64_t n, int nbits,
                               int64_t* __restrict__ x, int64_t* __restrict__ y,
                               int64_t* __restrict__ z, int64_t* __restrict__ b) {
  const uint64_t kmask = nbits >= 16 ? ((1ULL << 48) - 1ULL) : ((1ULL << (3 * nbits)) - 1ULL);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t kk = key[i];
    const uint64_t k = ((uint64_t)kk & ((1ULL << 48) - 1ULL)) & kmask;
    x[i] = (int64_t)compact3(k >> 2);
    y[i] = (int64_t)compact3(k >> 1);
    z[i] = (int64_t)compact3(k);
    if (b) b[i] = kk >> 48;  // arithmetic shift, like torch's `key >> 48`
  }
}

static inline unsigned grid_for(int64_t n, int threads) {
  int64_t blocks = cdiv(n, threads);
  int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace oc

using namespace oc;

extern "C" int oc_xyz2key(const void* x, const void* y, const void* z, const void* b,
                          int coord_dtype, int64_t n, int depth, int64_t* key, void* stream) {
  OC_REQUIRE(depth >= 0 && depth <= 16, OC_EINVAL, "oc_xyz2key: depth %d not in [0,16]", depth);
  OC_REQUIRE(n >= 0, OC_EINVAL, "oc_xyz2key: negative n");
  if (n == 0) return OC_OK;
  OC_REQUIRE(x && y && z && key, OC_EINVAL, "oc_xyz2key: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned g = grid_for(n, 256);
  switch (coord_dtype) {
    case OC_I64:
      xyz2key_kernel<int64_t><<<g, 256, 0, s>>>((const int64_t*)x, (const int64_t*)y,
                                                (const int64_t*)z, (const int64_t*)b, n, depth, key);
      break;
    case OC_I32:
      xyz2key_kernel<int32_t><<<g, 256, 0, s>>>((const int32_t*)x, (const int32_t*)y,
                                                (const int32_t*)z, (const int32_t*)b, n, depth, key);
      break;
    case OC_I16:
      xyz2key_kernel<int16_t><<<g, 256, 0, s>>>((const int16_t*)x, (const int16_t*)y,
                                                (const int16_t*)z, (const int16_t*)b, n, depth, key);
      break;
    case OC_COORD_F32:
      xyz2key_kernel<float><<<g, 256, 0, s>>>((const float*)x, (const float*)y, (const float*)z,
                                              (const float*)b, n, depth, key);
      break;
    case OC_COORD_F64:
      xyz2key_kernel<double><<<g, 256, 0, s>>>((const double*)x, (const double*)y,
                                               (const double*)z, (const double*)b, n, depth, key);
      break;
    default:
      OC_REQUIRE(false, OC_EINVAL, "oc_xyz2key: unsupported coordinate dtype %d", coord_dtype);
  }
  OC_LAUNCH_OK("xyz2key_kernel");
  return OC_OK;
}

extern "C" int oc_key2xyz(const int64_t* key, int64_t n, int depth, int64_t* x, int64_t* y,
                          int64_t* z, int64_t* b, void* stream) {
  OC_REQUIRE(depth >= 0 && depth <= 16, OC_EINVAL, "oc_key2xyz: depth %d not in [0,16]", depth);
  OC_REQUIRE(n >= 0, OC_EINVAL, "oc_key2xyz: negative n");
  if (n == 0) return OC_OK;
  OC_REQUIRE(key && x && y && z, OC_EINVAL, "oc_key2xyz: null pointer");
  // The reference decodes (depth + 2) / 3 chunks of 9 key bits = 3 bits per axis.
  const int nbits = ((depth + 2) / 3) * 3;
  key2xyz_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(key, n, nbits, x, y, z, b);
  OC_LAUNCH_OK("key2xyz_kernel");
  return OC_OK;
}
