// Octree convolution on FMA units: fp32 data (parity within 1e-4 of the
// reference's fp32 arithmetic needs true fp32 products, which the tensor cores
// do not provide) and channel counts the tensor-core tiles do not cover.
//
// Restates forward_gemm / backward_gemm / weight_gemm of
// ocnn/nn/octree_conv.py:115-202 without the im2col buffer: rows are gathered
// straight into shared-memory tiles.
#include "oc_common.cuh"
#include "conv_internal.cuh"

namespace oc {

// ---------------------------------------------------------------------------
// weight preparation: any (dtype, orientation) -> fp32 [K][Cin][Cout]
// ---------------------------------------------------------------------------
template <typename W>
__global__ void prep_weights_f32_kernel(const W* __restrict__ w, int K, int Cin, int Cout,
                                        int transposed, float* __restrict__ out) {
  const int64_t total = (int64_t)K * Cin * Cout;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int co = (int)(t % Cout);
    const int ci = (int)((t / Cout) % Cin);
    const int k = (int)(t / ((int64_t)Cout * Cin));
    const int64_t src = transposed ? ((int64_t)k * Cout + co) * Cin + ci : t;
    out[t] = to_f32<W>(w[src]);
  }
}

int prep_weights_f32(const void* w, int w_dtype, int K, int Cin, int Cout, int transposed,
                     float* out, cudaStream_t s) {
  const int64_t total = (int64_t)K * Cin * Cout;
  const unsigned g = (unsigned)(cdiv(total, 256) > 1184 ? 1184 : cdiv(total, 256));
  if (w_dtype == OC_F32)
    prep_weights_f32_kernel<float><<<g, 256, 0, s>>>((const float*)w, K, Cin, Cout, transposed, out);
  else if (w_dtype == OC_F16)
    prep_weights_f32_kernel<__half><<<g, 256, 0, s>>>((const __half*)w, K, Cin, Cout, transposed, out);
  else
    prep_weights_f32_kernel<__nv_bfloat16><<<g, 256, 0, s>>>((const __nv_bfloat16*)w, K, Cin, Cout, transposed, out);
  OC_LAUNCH_OK("prep_weights_f32_kernel");
  return OC_OK;
}

// ---------------------------------------------------------------------------
// gather-GEMM forward (also input gradient with a mirrored / inverse table)
// ---------------------------------------------------------------------------
constexpr int FM = 64, FN = 64, FK = 16, FT = 256;

template <typename T, typename I>
__global__ void __launch_bounds__(FT)
conv_fma_kernel(const T* __restrict__ data, const float* __restrict__ W, const T* __restrict__ bias,
                const I* __restrict__ table, int table_cols, TapList taps, int K, int64_t n_out,
                int Cin, int Cout, T* __restrict__ out) {
  __shared__ float As[FK][FM + 4];
  __shared__ float Ws[FK][FN + 4];
  __shared__ int sidx[FM];
  const int tid = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * FM;
  const int n0 = blockIdx.y * FN;
  const int ty = tid / 16, tx = tid % 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k = 0; k < K; ++k) {
    int any = 0;
    if (tid < FM) {
      const int64_t r = row0 + tid;
      const int v = r < n_out ? (int)table[r * table_cols + taps.t[k]] : -1;
      sidx[tid] = v;
      any = v >= 0;
    }
    if (!__syncthreads_or(any)) continue;  // whole tile has no neighbour at this tap
    const float* Wk = W + (int64_t)k * Cin * Cout;
    for (int c0 = 0; c0 < Cin; c0 += FK) {
      {  // A: 64 rows x 16 channels
        const int r = tid / 4, cq = (tid % 4) * 4;
        const int idx = sidx[r];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + cq + j;
          As[cq + j][r] = (idx >= 0 && c < Cin) ? to_f32<T>(data[(int64_t)idx * Cin + c]) : 0.f;
        }
      }
      {  // W: 16 channels x 64 outputs
        const int kk = tid / 16, co = (tid % 16) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c0 + kk, n = n0 + co + j;
          Ws[kk][co + j] = (c < Cin && n < Cout) ? Wk[(int64_t)c * Cout + n] : 0.f;
        }
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < FK; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t r = row0 + ty * 4 + i;
    if (r >= n_out) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < Cout) {
        float v = acc[i][j];
        // the reference rounds the product to the data dtype, then adds the bias
        if (bias) v = to_f32<T>(from_f32<T>(v)) + to_f32<T>(bias[n]);
        out[r * Cout + n] = from_f32<T>(v);
      }
    }
  }
}

template <typename T, typename I>
static int launch_conv_fma_t(const ConvArgs& a, const float* Wf, cudaStream_t s) {
  dim3 grid((unsigned)cdiv(a.n_out, FM), (unsigned)cdiv(a.Cout, FN));
  conv_fma_kernel<T, I><<<grid, FT, 0, s>>>((const T*)a.data, Wf, (const T*)a.bias, (const I*)a.table,
                                            a.table_cols, a.taps, a.K, a.n_out, a.Cin, a.Cout, (T*)a.out);
  OC_LAUNCH_OK("conv_fma_kernel");
  return OC_OK;
}

int launch_conv_fma(const ConvArgs& a, const float* Wf, cudaStream_t s) {
  if (a.n_out == 0) return OC_OK;
  if (a.idx_bytes == 8) {
    if (a.dtype == OC_F32) return launch_conv_fma_t<float, int64_t>(a, Wf, s);
    if (a.dtype == OC_F16) return launch_conv_fma_t<__half, int64_t>(a, Wf, s);
    return launch_conv_fma_t<__nv_bfloat16, int64_t>(a, Wf, s);
  }
  if (a.dtype == OC_F32) return launch_conv_fma_t<float, int32_t>(a, Wf, s);
  if (a.dtype == OC_F16) return launch_conv_fma_t<__half, int32_t>(a, Wf, s);
  return launch_conv_fma_t<__nv_bfloat16, int32_t>(a, Wf, s);
}

// ---------------------------------------------------------------------------
// weight gradient: partial[s][k][ci][co] over row slices, then a fixed-order sum
// ---------------------------------------------------------------------------
template <typename T, typename I>
__global__ void __launch_bounds__(FT)
wgrad_fma_kernel(const T* __restrict__ data, const T* __restrict__ gout, const I* __restrict__ table,
                 int table_cols, TapList taps, int K, int64_t n_out, int Cin, int Cout,
                 int64_t rows_per_split, float* __restrict__ partial) {
  __shared__ float As[FK][FM + 4];  // [row][ci]
  __shared__ float Gs[FK][FN + 4];  // [row][co]
  __shared__ int sidx[FK];
  const int tid = threadIdx.x;
  const int ci_tiles = (Cin + FM - 1) / FM, co_tiles = (Cout + FN - 1) / FN;
  int b = blockIdx.x;
  const int cot = b % co_tiles; b /= co_tiles;
  const int cit = b % ci_tiles; b /= ci_tiles;
  const int k = b;
  const int c0 = cit * FM, n0 = cot * FN;
  const int64_t r_begin = (int64_t)blockIdx.y * rows_per_split;
  int64_t r_end = r_begin + rows_per_split;
  if (r_end > n_out) r_end = n_out;
  const int ty = tid / 16, tx = tid % 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int64_t r0 = r_begin; r0 < r_end; r0 += FK) {
    int any = 0;
    if (tid < FK) {
      const int64_t r = r0 + tid;
      const int v = r < r_end ? (int)table[r * table_cols + taps.t[k]] : -1;
      sidx[tid] = v;
      any = v >= 0;
    }
    if (!__syncthreads_or(any)) continue;
    {  // 16 rows x 64 channels each for A (gathered) and G (dense)
      const int rr = tid / 16, cq = (tid % 16) * 4;
      const int idx = sidx[rr];
      const int64_t r = r0 + rr;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + cq + j;
        As[rr][cq + j] = (idx >= 0 && c < Cin) ? to_f32<T>(data[(int64_t)idx * Cin + c]) : 0.f;
        const int n = n0 + cq + j;
        Gs[rr][cq + j] = (idx >= 0 && r < r_end && n < Cout) ? to_f32<T>(gout[r * Cout + n]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < FK; ++rr) {
      float a[4], g[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[rr][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) g[j] = Gs[rr][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], g[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* P = partial + ((int64_t)blockIdx.y * K + k) * Cin * Cout;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = c0 + ty * 4 + i;
    if (c >= Cin) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < Cout) P[(int64_t)c * Cout + n] = acc[i][j];
    }
  }
}

__global__ void reduce_partials_kernel(const float* __restrict__ partial, int splits, int64_t n,
                                       float* __restrict__ out) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n;
       t += (int64_t)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int i = 0; i < splits; ++i) s += partial[(int64_t)i * n + t];
    out[t] = s;
  }
}

int reduce_partials(const float* partial, int splits, int64_t n, float* out, cudaStream_t s) {
  int64_t blocks = cdiv(n, 256);
  if (blocks > 1184) blocks = 1184;
  reduce_partials_kernel<<<(unsigned)blocks, 256, 0, s>>>(partial, splits, n, out);
  OC_LAUNCH_OK("reduce_partials_kernel");
  return OC_OK;
}

int wgrad_fma_splits(int K, int Cin, int Cout, int64_t n_out) {
  const int tiles = K * (int)cdiv(Cin, FM) * (int)cdiv(Cout, FN);
  int splits = (int)cdiv((int64_t)sm_count() * 4, tiles);
  const int64_t max_by_rows = cdiv(n_out > 0 ? n_out : 1, 256);
  if (splits > max_by_rows) splits = (int)max_by_rows;
  if (splits < 1) splits = 1;
  if (splits > 256) splits = 256;
  return splits;
}

template <typename T, typename I>
static int launch_wgrad_fma_t(const WgradArgs& a, float* partial, int splits, cudaStream_t s) {
  const int tiles = a.K * (int)cdiv(a.Cin, FM) * (int)cdiv(a.Cout, FN);
  int64_t rps = cdiv(a.n_out, splits);
  rps = cdiv(rps, FK) * FK;
  dim3 grid((unsigned)tiles, (unsigned)splits);
  wgrad_fma_kernel<T, I><<<grid, FT, 0, s>>>((const T*)a.data, (const T*)a.grad_out, (const I*)a.table,
                                             a.table_cols, a.taps, a.K, a.n_out, a.Cin, a.Cout, rps, partial);
  OC_LAUNCH_OK("wgrad_fma_kernel");
  return OC_OK;
}

int launch_wgrad_fma(const WgradArgs& a, float* partial, int splits, cudaStream_t s) {
  if (a.idx_bytes == 8) {
    if (a.dtype == OC_F32) return launch_wgrad_fma_t<float, int64_t>(a, partial, splits, s);
    if (a.dtype == OC_F16) return launch_wgrad_fma_t<__half, int64_t>(a, partial, splits, s);
    return launch_wgrad_fma_t<__nv_bfloat16, int64_t>(a, partial, splits, s);
  }
  if (a.dtype == OC_F32) return launch_wgrad_fma_t<float, int32_t>(a, partial, splits, s);
  if (a.dtype == OC_F16) return launch_wgrad_fma_t<__half, int32_t>(a, partial, splits, s);
  return launch_wgrad_fma_t<__nv_bfloat16, int32_t>(a, partial, splits, s);
}

}  // namespace oc
