// Average pooling over a neighbour table, per-octree (global) mean, and per-octree row scaling:
//   octree_avg_pool, octree_global_pool      ocnn/nn/octree_pool.py:68-124
//   OctreeDropPath (the per-octree mask)     ocnn/nn/octree_drop.py:14-60
// The reference builds a sparse COO matrix per call (avg pool) and uses atomic scatter_add
// (global pool); here a warp gathers one output row, and rows of one octree are contiguous
// (keys sort batch-major), so the global mean is a column sum over a row range.
#include "oc_common.cuh"
#include "conv_internal.cuh"

namespace oc {

// out[p, :] = v_p * sum_k data[table[p, taps[k]], :],  v_p = 1 / (#valid + 1e-8); val[p] = v_p
template <typename T, typename I>
__global__ void avgpool_fwd_kernel(const T* __restrict__ data, const I* __restrict__ table, int table_cols,
                                   TapList taps, int K, int64_t n_out, int C, T* __restrict__ out,
                                   float* __restrict__ val) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; p < n_out; p += nw) {
    const int64_t mine = lane < K ? (int64_t)table[p * table_cols + taps.t[lane]] : -1;
    const int cnt = __popc(__ballot_sync(0xffffffffu, mine >= 0));
    const float v = 1.0f / ((float)cnt + 1e-8f);
    if (val && lane == 0) val[p] = v;
    for (int c0 = 0; c0 < C; c0 += 32) {
      const int c = c0 + lane;
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const int64_t idx = __shfl_sync(0xffffffffu, mine, k);
        if (idx >= 0 && c < C) acc = fmaf(v, to_f32<T>(data[idx * C + c]), acc);
      }
      if (c < C) out[p * C + c] = from_f32<T>(acc);
    }
  }
}

// grad_in[n, :] = sum_k val[t] * grad_out[t, :],  t = table_t[n, taps[k]] (the scatter direction as a gather)
template <typename T, typename I>
__global__ void avgpool_bwd_kernel(const T* __restrict__ gout, const float* __restrict__ val,
                                   const I* __restrict__ table_t, int table_cols, TapList taps, int K,
                                   int64_t n_in, int C, T* __restrict__ gin) {
  const int lane = threadIdx.x & 31;
  const int64_t nw = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; n < n_in; n += nw) {
    const int64_t mine = lane < K ? (int64_t)table_t[n * table_cols + taps.t[lane]] : -1;
    const float vm = mine >= 0 ? val[mine] : 0.f;
    for (int c0 = 0; c0 < C; c0 += 32) {
      const int c = c0 + lane;
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const int64_t t = __shfl_sync(0xffffffffu, mine, k);
        const float v = __shfl_sync(0xffffffffu, vm, k);
        if (t >= 0 && c < C) acc = fmaf(v, to_f32<T>(gout[t * C + c]), acc);
      }
      if (c < C) gin[n * C + c] = from_f32<T>(acc);
    }
  }
}

struct SegOffsets { int64_t o[65]; };  // up to 64 octrees per launch

// mean[b, c] = sums[b, c] / max(count_b, 1)
__global__ void segment_mean_kernel(const float* __restrict__ sums, SegOffsets offs, int nb, int C,
                                    float* __restrict__ mean) {
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < nb * C; t += gridDim.x * blockDim.x) {
    const int b = t / C;
    const int64_t cnt = offs.o[b + 1] - offs.o[b];
    mean[t] = sums[t] / (float)(cnt < 1 ? 1 : cnt);
  }
}

// out[r, :] = data[r, :] * scale[b] for the rows r of octree b (grid.y = octree)
template <typename T>
__global__ void scale_segments_kernel(const T* __restrict__ data, SegOffsets offs, const float* __restrict__ scale,
                                      int C, T* __restrict__ out) {
  const int b = blockIdx.y;
  const float sc = scale[b];
  const int64_t e0 = offs.o[b] * C, e1 = offs.o[b + 1] * C;
  for (int64_t e = e0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < e1; e += (int64_t)gridDim.x * blockDim.x)
    out[e] = from_f32<T>(to_f32<T>(data[e]) * sc);
}

static inline unsigned warp_rows_grid(int64_t rows) {
  int64_t blocks = cdiv(rows, 8);
  const int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

static inline bool dtype_ok(int dtype) { return dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16; }

static int check_table(const char* who, int idx_bytes, int table_cols, int K, const int* h_taps, TapList* taps) {
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "%s: idx_bytes must be 4 or 8", who);
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "%s: table_cols %d not in [1,27]", who, table_cols);
  OC_REQUIRE(K >= 1 && K <= OC_MAX_TAPS, OC_EINVAL, "%s: K %d not in [1,27]", who, K);
  return make_taps(h_taps, K, table_cols, taps, who);
}

}  // namespace oc

using namespace oc;

#define OC_BY_TI(dtype, idx_bytes, stmt)                                              \
  do {                                                                                \
    if ((idx_bytes) == 8) {                                                           \
      using I = int64_t;                                                              \
      if ((dtype) == OC_F32) { using T = float; stmt; }                               \
      else if ((dtype) == OC_F16) { using T = __half; stmt; }                         \
      else { using T = __nv_bfloat16; stmt; }                                         \
    } else {                                                                          \
      using I = int32_t;                                                              \
      if ((dtype) == OC_F32) { using T = float; stmt; }                               \
      else if ((dtype) == OC_F16) { using T = __half; stmt; }                         \
      else { using T = __nv_bfloat16; stmt; }                                         \
    }                                                                                 \
  } while (0)

extern "C" int oc_avgpool_fwd(const void* data, const void* table, int idx_bytes, int table_cols,
                              const int* h_taps, int K, int64_t n_out, int C, int dtype, void* out, float* val,
                              void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_avgpool_fwd: bad dtype %d", dtype);
  OC_REQUIRE(n_out >= 0 && C >= 1, OC_EINVAL, "oc_avgpool_fwd: bad sizes");
  TapList taps;
  int rc = check_table("oc_avgpool_fwd", idx_bytes, table_cols, K, h_taps, &taps);
  if (rc) return rc;
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(table && out, OC_EINVAL, "oc_avgpool_fwd: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_TI(dtype, idx_bytes, (avgpool_fwd_kernel<T, I><<<warp_rows_grid(n_out), 256, 0, s>>>(
                                 (const T*)data, (const I*)table, table_cols, taps, K, n_out, C, (T*)out, val)));
  OC_LAUNCH_OK("avgpool_fwd_kernel");
  return OC_OK;
}

extern "C" int oc_avgpool_bwd(const void* grad_out, const float* val, const void* table_t, int idx_bytes,
                              int table_cols, const int* h_taps, int K, int64_t n_in, int C, int dtype,
                              void* grad_in, void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_avgpool_bwd: bad dtype %d", dtype);
  OC_REQUIRE(n_in >= 0 && C >= 1, OC_EINVAL, "oc_avgpool_bwd: bad sizes");
  TapList taps;
  int rc = check_table("oc_avgpool_bwd", idx_bytes, table_cols, K, h_taps, &taps);
  if (rc) return rc;
  if (n_in == 0) return OC_OK;
  OC_REQUIRE(val && table_t && grad_in, OC_EINVAL, "oc_avgpool_bwd: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  OC_BY_TI(dtype, idx_bytes, (avgpool_bwd_kernel<T, I><<<warp_rows_grid(n_in), 256, 0, s>>>(
                                 (const T*)grad_out, val, (const I*)table_t, table_cols, taps, K, n_in, C, (T*)grad_in)));
  OC_LAUNCH_OK("avgpool_bwd_kernel");
  return OC_OK;
}

extern "C" size_t oc_global_pool_workspace_bytes(int64_t n, int batch, int C) {
  if (n < 0 || batch < 1 || C < 1) return 0;
  return colstats_workspace_bytes(n, C) + align_up((size_t)batch * C * sizeof(float), 256);
}

extern "C" int oc_global_pool_fwd(const void* data, const int64_t* h_offsets, int batch, int C, int dtype,
                                  float* mean, void* workspace, size_t workspace_bytes, void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_global_pool_fwd: bad dtype %d", dtype);
  OC_REQUIRE(batch >= 1 && C >= 1 && h_offsets && mean && workspace, OC_EINVAL, "oc_global_pool_fwd: bad arguments");
  for (int b = 0; b < batch; ++b)
    OC_REQUIRE(h_offsets[b + 1] >= h_offsets[b], OC_EINVAL, "oc_global_pool_fwd: offsets must not decrease");
  const int64_t n = h_offsets[batch] - h_offsets[0];
  OC_REQUIRE(workspace_bytes >= oc_global_pool_workspace_bytes(n, batch, C), OC_ENOMEM,
             "oc_global_pool_fwd: workspace too small");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t cs_bytes = colstats_workspace_bytes(n, C);
  float* sums = (float*)((char*)workspace + cs_bytes);
  const size_t es = dtype == OC_F32 ? 4 : 2;
  for (int b = 0; b < batch; ++b) {       // rows of one octree are a contiguous range
    const int64_t rows = h_offsets[b + 1] - h_offsets[b];
    int rc = launch_colstats((const char*)data + (size_t)h_offsets[b] * C * es, nullptr, rows, C, dtype,
                             sums + (size_t)b * C, nullptr, workspace, cs_bytes, s);
    if (rc) return rc;
  }
  for (int b0 = 0; b0 < batch; b0 += 64) {
    const int nb = batch - b0 < 64 ? batch - b0 : 64;
    SegOffsets o;
    for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
    segment_mean_kernel<<<(unsigned)cdiv((int64_t)nb * C, 256), 256, 0, s>>>(sums + (size_t)b0 * C, o, nb, C,
                                                                             mean + (size_t)b0 * C);
  }
  OC_LAUNCH_OK("segment_mean_kernel");
  return OC_OK;
}

extern "C" int oc_scale_segments(const void* data, const int64_t* h_offsets, int batch, const float* scale, int C,
                                 int dtype, void* out, void* stream) {
  OC_REQUIRE(dtype_ok(dtype), OC_EINVAL, "oc_scale_segments: bad dtype %d", dtype);
  OC_REQUIRE(batch >= 1 && C >= 1 && h_offsets && scale, OC_EINVAL, "oc_scale_segments: bad arguments");
  for (int b = 0; b < batch; ++b)
    OC_REQUIRE(h_offsets[b + 1] >= h_offsets[b], OC_EINVAL, "oc_scale_segments: offsets must not decrease");
  if (h_offsets[batch] == h_offsets[0]) return OC_OK;
  OC_REQUIRE(data && out, OC_EINVAL, "oc_scale_segments: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  for (int b0 = 0; b0 < batch; b0 += 64) {
    const int nb = batch - b0 < 64 ? batch - b0 : 64;
    SegOffsets o;
    for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
    const int64_t per = cdiv((o.o[nb] - o.o[0]) * C, (int64_t)nb * 256 * 8);
    const dim3 grid((unsigned)(per < 1 ? 1 : (per > 4096 ? 4096 : per)), (unsigned)nb);
    if (dtype == OC_F32) scale_segments_kernel<float><<<grid, 256, 0, s>>>((const float*)data, o, scale + b0, C, (float*)out);
    else if (dtype == OC_F16) scale_segments_kernel<__half><<<grid, 256, 0, s>>>((const __half*)data, o, scale + b0, C, (__half*)out);
    else scale_segments_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)data, o, scale + b0, C, (__nv_bfloat16*)out);
  }
  OC_LAUNCH_OK("scale_segments_kernel");
  return OC_OK;
}
