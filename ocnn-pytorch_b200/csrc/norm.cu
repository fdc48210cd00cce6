// Normalisation kernels for (N, C) octree features.
//
// BatchNorm (torch.nn.BatchNorm1d as aliased by ocnn/nn/octree_norm.py:16) is
// split into column statistics + a fused affine pass so that the statistics can
// be all-reduced across GPUs between the two.  GroupNorm restates
// OctreeGroupNorm.forward (ocnn/nn/octree_norm.py:45-65) with per-octree row
// ranges instead of three atomic scatter_adds.  All reductions are two-stage
// (per-block partials in a workspace, then a fixed-order sum): no atomics, so
// results are reproducible run to run.
#include <mutex>

#include "oc_common.cuh"
#include "conv_internal.cuh"

namespace oc {

constexpr int CS_THREADS = 256;

// Block layout: CT channel-threads x RL row-lanes (CT * RL = 256).  Each block
// owns a row slice and loops over channel tiles of CT.
static inline int cs_ct(int C) { return C >= 64 ? 64 : (C >= 32 ? 32 : (C >= 16 ? 16 : (C >= 8 ? 8 : 4))); }

static inline int cs_splits(int64_t n) {
  int64_t s = cdiv(n > 0 ? n : 1, 512);
  const int64_t cap = (int64_t)sm_count() * 4;
  if (s > cap) s = cap;
  if (s < 1) s = 1;
  return (int)s;
}

template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
colstats_kernel(const T* __restrict__ a, const T* __restrict__ b, int64_t row_begin, int64_t row_end,
                int64_t rows_per_split, int C, int CT, float* __restrict__ part_a,
                float* __restrict__ part_ab) {
  __shared__ float sa[CS_THREADS], sab[CS_THREADS];
  const int RL = CS_THREADS / CT;
  const int ct = threadIdx.x % CT, rl = threadIdx.x / CT;
  const int64_t r0 = row_begin + (int64_t)blockIdx.x * rows_per_split;
  int64_t r1 = r0 + rows_per_split;
  if (r1 > row_end) r1 = row_end;
  for (int c0 = 0; c0 < C; c0 += CT) {
    const int c = c0 + ct;
    float s1 = 0.f, s2 = 0.f;
    if (c < C) {
      for (int64_t r = r0 + rl; r < r1; r += RL) {
        const float x = to_f32<T>(a[r * C + c]);
        const float y = b ? to_f32<T>(b[r * C + c]) : x;
        s1 += x;
        s2 = fmaf(x, y, s2);
      }
    }
    sa[threadIdx.x] = s1;
    sab[threadIdx.x] = s2;
    __syncthreads();
    if (rl == 0 && c < C) {
      for (int i = 1; i < RL; ++i) { s1 += sa[i * CT + ct]; s2 += sab[i * CT + ct]; }
      part_a[(int64_t)blockIdx.x * C + c] = s1;
      part_ab[(int64_t)blockIdx.x * C + c] = s2;
    }
    __syncthreads();
  }
}

__global__ void colstats_final_kernel(const float* __restrict__ part_a, const float* __restrict__ part_ab,
                                      int splits, int C, float* __restrict__ sum_a,
                                      float* __restrict__ sum_ab) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s1 = 0.f, s2 = 0.f;
  for (int i = 0; i < splits; ++i) { s1 += part_a[(int64_t)i * C + c]; s2 += part_ab[(int64_t)i * C + c]; }
  if (sum_a) sum_a[c] = s1;
  if (sum_ab) sum_ab[c] = s2;
}


// ---- 16-byte vectorised variants (C a multiple of 16 / sizeof(T), aligned pointers) ----
template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[16 / sizeof(T)]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) v[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[16 / sizeof(T)]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < (int)(16 / sizeof(T)); ++i) e[i] = from_f32<T>(v[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Thread (rl, v) sums the 16-byte vector v of the rows rl, rl + RL, ... of the block's
// slice; row lanes are then folded through shared memory.  VPR = vectors per row.
template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
colstats_vec_kernel(const T* __restrict__ a, const T* __restrict__ b, int64_t n, int64_t rows_per_split, int C,
                    float* __restrict__ part_a, float* __restrict__ part_ab) {
  constexpr int N = 16 / sizeof(T);
  extern __shared__ float sm[];                 // [2][RL][VW * N]
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;   // vectors handled per pass
  const int RL = CS_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  const bool active = rl < RL;
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_split;
  int64_t r1 = r0 + rows_per_split;
  if (r1 > n) r1 = n;
  for (int v0 = 0; v0 < VPR; v0 += VW) {
    const int vv = v0 + v;
    float s1[N], s2[N];
#pragma unroll
    for (int i = 0; i < N; ++i) { s1[i] = 0.f; s2[i] = 0.f; }
    if (active && vv < VPR) {
      for (int64_t r = r0 + rl; r < r1; r += RL) {
        float x[N], y[N];
        load_vec<T>(a + r * C + vv * N, x);
        if (b) load_vec<T>(b + r * C + vv * N, y);
#pragma unroll
        for (int i = 0; i < N; ++i) { s1[i] += x[i]; s2[i] = fmaf(x[i], b ? y[i] : x[i], s2[i]); }
      }
    }
    if (active) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        sm[(rl * VW + v) * N + i] = s1[i];
        sm[(RL * VW + rl * VW + v) * N + i] = s2[i];
      }
    }
    __syncthreads();
    // fold the RL row lanes: one thread per channel of this pass
    for (int c = threadIdx.x; c < VW * N; c += CS_THREADS) {
      const int ch = v0 * N + c;
      if (ch < C) {
        float t1 = 0.f, t2 = 0.f;
        for (int l = 0; l < RL; ++l) { t1 += sm[l * VW * N + c]; t2 += sm[(RL + l) * VW * N + c]; }
        part_a[(int64_t)blockIdx.x * C + ch] = t1;
        part_ab[(int64_t)blockIdx.x * C + ch] = t2;
      }
    }
    __syncthreads();
  }
}

// Apply kernels: a block owns the rows [r0, r1); thread (rl, v) handles the 16-byte vector v of
// the rows r0 + rl, r0 + rl + RL, ...  The column of a thread never changes, so its per-channel
// constants are read once into registers and the row loop is load / fma / store only (a division
// or modulo per vector to find the column costs more than the memory traffic it accompanies).
// Four rows are in flight per thread.
template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
affine_cols_vec_kernel(const T* __restrict__ x, const float* __restrict__ scale, const float* __restrict__ shift,
                       int64_t n, int64_t rows_per_block, int C, T* __restrict__ out) {
  constexpr int N = 16 / sizeof(T);
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
  const int RL = CS_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  if (rl >= RL) return;
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  int64_t r1 = r0 + rows_per_block;
  if (r1 > n) r1 = n;
  for (int vv = v; vv < VPR; vv += VW) {
    float sc[N], sh[N];
#pragma unroll
    for (int i = 0; i < N; ++i) { sc[i] = scale[vv * N + i]; sh[i] = shift[vv * N + i]; }
    const T* xp = x + (int64_t)vv * N;
    T* op = out + (int64_t)vv * N;
    int64_t r = r0 + rl;
    for (; r + 3 * RL < r1; r += 4 * RL) {
      float a[4][N];
#pragma unroll
      for (int u = 0; u < 4; ++u) load_vec<T>(xp + (r + u * RL) * C, a[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
#pragma unroll
        for (int i = 0; i < N; ++i) a[u][i] = fmaf(a[u][i], sc[i], sh[i]);
        store_vec<T>(op + (r + u * RL) * C, a[u]);
      }
    }
    for (; r < r1; r += RL) {
      float a[N];
      load_vec<T>(xp + r * C, a);
#pragma unroll
      for (int i = 0; i < N; ++i) a[i] = fmaf(a[i], sc[i], sh[i]);
      store_vec<T>(op + r * C, a);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
bn_bwd_apply_vec_kernel(const T* __restrict__ g, const T* __restrict__ x, const float* __restrict__ ka,
                        const float* __restrict__ kb, const float* __restrict__ kc, int64_t n,
                        int64_t rows_per_block, int C, T* __restrict__ gin) {
  constexpr int N = 16 / sizeof(T);
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
  const int RL = CS_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  if (rl >= RL) return;
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  int64_t r1 = r0 + rows_per_block;
  if (r1 > n) r1 = n;
  for (int vv = v; vv < VPR; vv += VW) {
    float a[N], b[N], c[N];
#pragma unroll
    for (int i = 0; i < N; ++i) { a[i] = ka[vv * N + i]; b[i] = kb[vv * N + i]; c[i] = kc[vv * N + i]; }
    const T* gp = g + (int64_t)vv * N;
    const T* xp = x + (int64_t)vv * N;
    T* op = gin + (int64_t)vv * N;
    int64_t r = r0 + rl;
    for (; r + RL < r1; r += 2 * RL) {
      float gv[2][N], xv[2][N];
#pragma unroll
      for (int u = 0; u < 2; ++u) { load_vec<T>(gp + (r + u * RL) * C, gv[u]); load_vec<T>(xp + (r + u * RL) * C, xv[u]); }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int i = 0; i < N; ++i) gv[u][i] = gv[u][i] * a[i] + xv[u][i] * b[i] + c[i];
        store_vec<T>(op + (r + u * RL) * C, gv[u]);
      }
    }
    for (; r < r1; r += RL) {
      float gv[N], xv[N];
      load_vec<T>(gp + r * C, gv);
      load_vec<T>(xp + r * C, xv);
#pragma unroll
      for (int i = 0; i < N; ++i) gv[i] = gv[i] * a[i] + xv[i] * b[i] + c[i];
      store_vec<T>(op + r * C, gv);
    }
  }
}

static inline bool vec16_ok(int C, int dtype, const void* p0, const void* p1, const void* p2) {
  const int N = (int)(16 / dtype_size(dtype));
  return C % N == 0 && ((uintptr_t)p0 % 16) == 0 && ((uintptr_t)p1 % 16) == 0 && ((uintptr_t)p2 % 16) == 0;
}

// blocks for an apply kernel over n rows: enough to fill the GPU, at least 64 rows each
static inline void apply_split(int64_t n, int* blocks, int64_t* rows_per_block) {
  int64_t nb = cdiv(n, 64);
  const int64_t cap = (int64_t)sm_count() * 16;
  if (nb > cap) nb = cap;
  if (nb < 1) nb = 1;
  *rows_per_block = cdiv(n, nb);
  *blocks = (int)cdiv(n, *rows_per_block);
}

template <typename T>
static void launch_colstats_vec(const void* a, const void* b, int64_t n, int C, int splits, int64_t rps, float* pa,
                                float* pab, cudaStream_t s) {
  constexpr int N = 16 / sizeof(T);
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
  const int RL = CS_THREADS / VW;
  const size_t smem = (size_t)2 * RL * VW * N * sizeof(float);
  colstats_vec_kernel<T><<<splits, CS_THREADS, smem, s>>>((const T*)a, (const T*)b, n, rps, C, pa, pab);
}

size_t colstats_workspace_bytes(int64_t n, int C) {
  return align_up((size_t)cs_splits(n) * C * 2 * sizeof(float), 256);
}

int launch_colstats(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                    float* sum_ab, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  if (n == 0) {
    if (sum_a) OC_CUDA_OK(cudaMemsetAsync(sum_a, 0, (size_t)C * 4, s));
    if (sum_ab) OC_CUDA_OK(cudaMemsetAsync(sum_ab, 0, (size_t)C * 4, s));
    return OC_OK;
  }
  const int splits = cs_splits(n);
  OC_REQUIRE(workspace && workspace_bytes >= (size_t)splits * C * 2 * 4, OC_ENOMEM,
             "colstats: workspace too small");
  float* pa = (float*)workspace;
  float* pab = pa + (size_t)splits * C;
  const int64_t rps = cdiv(n, splits);
  const int CT = cs_ct(C);
  if (vec16_ok(C, dtype, a, b, nullptr) && C <= 8192) {
    if (dtype == OC_F32) launch_colstats_vec<float>(a, b, n, C, splits, rps, pa, pab, s);
    else if (dtype == OC_F16) launch_colstats_vec<__half>(a, b, n, C, splits, rps, pa, pab, s);
    else launch_colstats_vec<__nv_bfloat16>(a, b, n, C, splits, rps, pa, pab, s);
  } else if (dtype == OC_F32)
    colstats_kernel<float><<<splits, CS_THREADS, 0, s>>>((const float*)a, (const float*)b, 0, n, rps, C, CT, pa, pab);
  else if (dtype == OC_F16)
    colstats_kernel<__half><<<splits, CS_THREADS, 0, s>>>((const __half*)a, (const __half*)b, 0, n, rps, C, CT, pa, pab);
  else
    colstats_kernel<__nv_bfloat16><<<splits, CS_THREADS, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, 0, n, rps, C, CT, pa, pab);
  colstats_final_kernel<<<(unsigned)cdiv(C, 128), 128, 0, s>>>(pa, pab, splits, C, sum_a, sum_ab);
  OC_LAUNCH_OK("colstats kernels");
  return OC_OK;
}

// out = x * scale[c] + shift[c]
template <typename T>
__global__ void affine_cols_kernel(const T* __restrict__ x, const float* __restrict__ scale,
                                   const float* __restrict__ shift, int64_t total, int C,
                                   T* __restrict__ out) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(t % C);
    out[t] = from_f32<T>(fmaf(to_f32<T>(x[t]), scale[c], shift[c]));
  }
}

template <typename T>
__global__ void bn_bwd_apply_kernel(const T* __restrict__ g, const T* __restrict__ x,
                                    const float* __restrict__ ka, const float* __restrict__ kb,
                                    const float* __restrict__ kc, int64_t total, int C,
                                    T* __restrict__ gin) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(t % C);
    gin[t] = from_f32<T>(to_f32<T>(g[t]) * ka[c] + to_f32<T>(x[t]) * kb[c] + kc[c]);
  }
}

// ---------------------------------------------------------------------------
// GroupNorm
// ---------------------------------------------------------------------------
// Stage A partials: per (octree b, split s, channel c) sums of x (pass 1) or of
// (x - mean)^2 (pass 2) / of g*w and g*w*(x-mean) (backward).  SPLITS blocks per
// octree keep the grid busy for small batches.
constexpr int GN_SPLITS = 32;

struct GnOffsets { int64_t o[65]; };  // up to 64 octrees per launch chunk

template <typename T, int MODE>
// MODE 0: sum x ; MODE 1: sum (x-mean)^2 ; MODE 2: (sum g*w, sum g*w*(x-mean)) ; MODE 3: (sum g, sum g*(x-mean)*inv_std) per channel
__global__ void __launch_bounds__(CS_THREADS)
gn_partial_kernel(const T* __restrict__ x, const T* __restrict__ g, GnOffsets offs, int b0, int C,
                  int cpg, int CT, const float* __restrict__ mean, const float* __restrict__ inv_std,
                  const float* __restrict__ weight, float* __restrict__ p1, float* __restrict__ p2) {
  __shared__ float s1s[CS_THREADS], s2s[CS_THREADS];
  const int bl = blockIdx.y;
  const int b = b0 + bl;
  const int G = C / cpg;
  const int64_t rb = offs.o[bl], re = offs.o[bl + 1];
  const int64_t rps = (re - rb + GN_SPLITS - 1) / GN_SPLITS;
  const int64_t r0 = rb + (int64_t)blockIdx.x * rps;
  int64_t r1 = r0 + rps;
  if (r1 > re) r1 = re;
  const int RL = CS_THREADS / CT;
  const int ct = threadIdx.x % CT, rl = threadIdx.x / CT;
  for (int c0 = 0; c0 < C; c0 += CT) {
    const int c = c0 + ct;
    float s1 = 0.f, s2 = 0.f;
    if (c < C) {
      const float m = MODE >= 1 ? mean[b * G + c / cpg] : 0.f;
      const float is = MODE == 3 ? inv_std[b * G + c / cpg] : 0.f;
      const float w = MODE == 2 ? weight[c] : 0.f;
      for (int64_t r = r0 + rl; r < r1; r += RL) {
        const float xv = to_f32<T>(x[r * C + c]);
        if (MODE == 0) s1 += xv;
        if (MODE == 1) { const float d = xv - m; s1 = fmaf(d, d, s1); }
        if (MODE == 2) { const float gw = to_f32<T>(g[r * C + c]) * w; s1 += gw; s2 = fmaf(gw, xv - m, s2); }
        if (MODE == 3) { const float gv = to_f32<T>(g[r * C + c]); s1 += gv; s2 = fmaf(gv, (xv - m) * is, s2); }
      }
    }
    s1s[threadIdx.x] = s1;
    s2s[threadIdx.x] = s2;
    __syncthreads();
    if (rl == 0 && c < C) {
      for (int i = 1; i < RL; ++i) { s1 += s1s[i * CT + ct]; s2 += s2s[i * CT + ct]; }
      const int64_t o = ((int64_t)b * GN_SPLITS + blockIdx.x) * C + c;
      p1[o] = s1;
      if (p2) p2[o] = s2;
    }
    __syncthreads();
  }
}

// One thread per (b, group): fold the per-channel partials.
// STAGE 0: mean ; STAGE 1: inv_std ; STAGE 2: backward coefficients.
__global__ void gn_finalize_kernel(const float* __restrict__ p1, const float* __restrict__ p2,
                                   GnOffsets offs_all, int batch, int C, int cpg, float eps,
                                   int stage, float* __restrict__ mean, float* __restrict__ inv_std,
                                   float* __restrict__ coef_a, float* __restrict__ coef_b) {
  const int G = C / cpg;
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= batch * G) return;
  const int b = t / G, gi = t % G;
  float s1 = 0.f, s2 = 0.f;
  for (int sp = 0; sp < GN_SPLITS; ++sp)
    for (int c = gi * cpg; c < (gi + 1) * cpg; ++c) {
      s1 += p1[((int64_t)b * GN_SPLITS + sp) * C + c];
      if (p2) s2 += p2[((int64_t)b * GN_SPLITS + sp) * C + c];
    }
  const float cnt = (float)(offs_all.o[b + 1] - offs_all.o[b]) * (float)cpg;
  const float inv_count = 1.0f / (cnt + eps);
  if (stage == 0) {
    mean[t] = s1 * inv_count;
  } else if (stage == 1) {
    inv_std[t] = 1.0f / sqrtf(s1 * inv_count + eps);
  } else {
    // y = x - m, m = s*sum(x), v = s*sum(y^2), r = (v+eps)^-1/2, out = y*r*w + b.
    // With gw = grad_out * w:  dx = gw*r + y*coef_a + coef_b, where
    //   dv = -0.5 r^3 sum(gw*y),  coef_a = 2 s dv,
    //   coef_b = -s * (r*sum(gw) + 2 s dv sum(y)),  sum(y) = (m/s) * (1 - cnt*s).
    const float r = inv_std[t], m = mean[t];
    const float dv = -0.5f * r * r * r * s2;
    const float sum_y = (m / inv_count) * (1.0f - cnt * inv_count);
    coef_a[t] = 2.0f * inv_count * dv;
    coef_b[t] = -inv_count * (r * s1 + 2.0f * inv_count * dv * sum_y);
  }
}

template <typename T>
__global__ void gn_apply_kernel(const T* __restrict__ x, GnOffsets offs, int b0, int nb, int C, int cpg,
                                const float* __restrict__ mean, const float* __restrict__ inv_std,
                                const float* __restrict__ weight, const float* __restrict__ bias,
                                T* __restrict__ out) {
  const int G = C / cpg;
  const int64_t rb = offs.o[0], re = offs.o[nb];
  for (int64_t t = rb * C + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < re * C;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / C;
    const int c = (int)(t - r * C);
    int bl = 0;
    while (bl + 1 < nb && r >= offs.o[bl + 1]) ++bl;
    const int gi = (b0 + bl) * G + c / cpg;
    const float y = (to_f32<T>(x[t]) - mean[gi]) * inv_std[gi];
    out[t] = from_f32<T>(y * weight[c] + bias[c]);
  }
}

template <typename T>
__global__ void gn_bwd_apply_kernel(const T* __restrict__ g, const T* __restrict__ x, GnOffsets offs,
                                    int b0, int nb, int C, int cpg, const float* __restrict__ mean,
                                    const float* __restrict__ inv_std, const float* __restrict__ weight,
                                    const float* __restrict__ coef_a, const float* __restrict__ coef_b,
                                    T* __restrict__ gin) {
  const int G = C / cpg;
  const int64_t rb = offs.o[0], re = offs.o[nb];
  for (int64_t t = rb * C + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < re * C;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / C;
    const int c = (int)(t - r * C);
    int bl = 0;
    while (bl + 1 < nb && r >= offs.o[bl + 1]) ++bl;
    const int gi = (b0 + bl) * G + c / cpg;
    const float y = to_f32<T>(x[t]) - mean[gi];
    gin[t] = from_f32<T>(to_f32<T>(g[t]) * weight[c] * inv_std[gi] + y * coef_a[gi] + coef_b[gi]);
  }
}


// 16-byte vectorised GroupNorm kernels (same arithmetic as the scalar ones above).
template <typename T, int MODE>
__global__ void __launch_bounds__(CS_THREADS)
gn_partial_vec_kernel(const T* __restrict__ x, const T* __restrict__ g, GnOffsets offs, int b0, int C, int cpg,
                      const float* __restrict__ mean, const float* __restrict__ inv_std,
                      const float* __restrict__ weight, float* __restrict__ p1, float* __restrict__ p2) {
  constexpr int N = 16 / sizeof(T);
  extern __shared__ float sm[];                 // [2][RL][VW * N]
  const int bl = blockIdx.y;
  const int b = b0 + bl;
  const int G = C / cpg;
  const int64_t rb = offs.o[bl], re = offs.o[bl + 1];
  const int64_t rps = (re - rb + GN_SPLITS - 1) / GN_SPLITS;
  const int64_t r0 = rb + (int64_t)blockIdx.x * rps;
  int64_t r1 = r0 + rps;
  if (r1 > re) r1 = re;
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
  const int RL = CS_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  const bool active = rl < RL;
  for (int v0 = 0; v0 < VPR; v0 += VW) {
    const int vv = v0 + v;
    float s1[N], s2[N], m[N], is[N], w[N];
#pragma unroll
    for (int i = 0; i < N; ++i) { s1[i] = 0.f; s2[i] = 0.f; m[i] = 0.f; is[i] = 0.f; w[i] = 0.f; }
    if (active && vv < VPR) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const int c = vv * N + i;
        if (MODE >= 1) m[i] = mean[b * G + c / cpg];
        if (MODE == 3) is[i] = inv_std[b * G + c / cpg];
        if (MODE == 2) w[i] = weight[c];
      }
      for (int64_t r = r0 + rl; r < r1; r += RL) {
        float xv[N], gv[N];
        load_vec<T>(x + r * C + vv * N, xv);
        if (MODE >= 2) load_vec<T>(g + r * C + vv * N, gv);
#pragma unroll
        for (int i = 0; i < N; ++i) {
          if (MODE == 0) s1[i] += xv[i];
          if (MODE == 1) { const float d = xv[i] - m[i]; s1[i] = fmaf(d, d, s1[i]); }
          if (MODE == 2) { const float gw = gv[i] * w[i]; s1[i] += gw; s2[i] = fmaf(gw, xv[i] - m[i], s2[i]); }
          if (MODE == 3) { s1[i] += gv[i]; s2[i] = fmaf(gv[i], (xv[i] - m[i]) * is[i], s2[i]); }
        }
      }
    }
    if (active) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        sm[(rl * VW + v) * N + i] = s1[i];
        sm[(RL * VW + rl * VW + v) * N + i] = s2[i];
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < VW * N; c += CS_THREADS) {
      const int ch = v0 * N + c;
      if (ch < C) {
        float t1 = 0.f, t2 = 0.f;
        for (int l = 0; l < RL; ++l) { t1 += sm[l * VW * N + c]; t2 += sm[(RL + l) * VW * N + c]; }
        const int64_t o = ((int64_t)b * GN_SPLITS + blockIdx.x) * C + ch;
        p1[o] = t1;
        if (p2) p2[o] = t2;
      }
    }
    __syncthreads();
  }
}

// MODE 0: out = (x - mean) * inv_std * weight + bias ; MODE 1: grad_in (see gn_bwd_apply_kernel).
// grid = (row chunks, octrees of this launch): a block works inside one octree, so the statistics
// of a thread's channels are fixed and live in registers (same layout as the BatchNorm apply kernels).
template <typename T, int MODE>
__global__ void __launch_bounds__(CS_THREADS)
gn_apply_vec_kernel(const T* __restrict__ x, const T* __restrict__ g, GnOffsets offs, int b0, int C, int cpg,
                    const float* __restrict__ mean, const float* __restrict__ inv_std,
                    const float* __restrict__ weight, const float* __restrict__ bias,
                    const float* __restrict__ coef_a, const float* __restrict__ coef_b, T* __restrict__ out) {
  constexpr int N = 16 / sizeof(T);
  const int G = C / cpg;
  const int VPR = C / N;
  const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
  const int RL = CS_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  if (rl >= RL) return;
  const int bl = blockIdx.y;
  const int64_t rb = offs.o[bl], re = offs.o[bl + 1];
  const int64_t rpb = (re - rb + gridDim.x - 1) / gridDim.x;
  const int64_t r0 = rb + (int64_t)blockIdx.x * rpb;
  int64_t r1 = r0 + rpb;
  if (r1 > re) r1 = re;
  for (int vv = v; vv < VPR; vv += VW) {
    float m[N], is[N], w[N], bs[N], ca[N], cb[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int c = vv * N + i;
      const int gi = (b0 + bl) * G + c / cpg;
      m[i] = mean[gi]; is[i] = inv_std[gi]; w[i] = weight[c];
      bs[i] = MODE == 0 ? bias[c] : 0.f;
      ca[i] = MODE == 1 ? coef_a[gi] : 0.f;
      cb[i] = MODE == 1 ? coef_b[gi] : 0.f;
    }
    const T* xp = x + (int64_t)vv * N;
    const T* gp = MODE == 1 ? g + (int64_t)vv * N : nullptr;
    T* op = out + (int64_t)vv * N;
    int64_t r = r0 + rl;
    for (; r + RL < r1; r += 2 * RL) {
      float xv[2][N], gv[2][N];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        load_vec<T>(xp + (r + u * RL) * C, xv[u]);
        if (MODE == 1) load_vec<T>(gp + (r + u * RL) * C, gv[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
#pragma unroll
        for (int i = 0; i < N; ++i) {
          const float y = xv[u][i] - m[i];
          if (MODE == 0) xv[u][i] = y * is[i] * w[i] + bs[i];
          else xv[u][i] = gv[u][i] * w[i] * is[i] + y * ca[i] + cb[i];
        }
        store_vec<T>(op + (r + u * RL) * C, xv[u]);
      }
    }
    for (; r < r1; r += RL) {
      float xv[N], gv[N];
      load_vec<T>(xp + r * C, xv);
      if (MODE == 1) load_vec<T>(gp + r * C, gv);
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const float y = xv[i] - m[i];
        if (MODE == 0) xv[i] = y * is[i] * w[i] + bs[i];
        else xv[i] = gv[i] * w[i] * is[i] + y * ca[i] + cb[i];
      }
      store_vec<T>(op + r * C, xv);
    }
  }
}

// grad_weight[c] = sum_b sum_splits p2, grad_bias[c] = ... p1 (MODE 3 partials)
__global__ void gn_param_grad_kernel(const float* __restrict__ p1, const float* __restrict__ p2,
                                     int batch, int C, float* __restrict__ gw, float* __restrict__ gb) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s1 = 0.f, s2 = 0.f;
  for (int i = 0; i < batch * GN_SPLITS; ++i) { s1 += p1[(int64_t)i * C + c]; s2 += p2[(int64_t)i * C + c]; }
  if (gb) gb[c] = s1;
  if (gw) gw[c] = s2;
}

struct GnPlan {
  float *p1, *p2, *coef_a, *coef_b;
  size_t total;
};

static GnPlan gn_plan(void* ws, int batch, int C) {
  GnPlan p;
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  const size_t part = (size_t)batch * GN_SPLITS * C * 4;
  size_t o1 = take(part), o2 = take(part), oa = take((size_t)batch * C * 4), ob = take((size_t)batch * C * 4);
  char* base = (char*)ws;
  p.p1 = (float*)(base + o1);
  p.p2 = (float*)(base + o2);
  p.coef_a = (float*)(base + oa);
  p.coef_b = (float*)(base + ob);
  p.total = off;
  return p;
}

template <typename T, int MODE>
static void gn_partials(const void* x, const void* g, const int64_t* h_offsets, int batch, int C, int cpg,
                        const float* mean, const float* inv_std, const float* weight, float* p1, float* p2,
                        cudaStream_t s) {
  const int CT = cs_ct(C);
  for (int b0 = 0; b0 < batch; b0 += 64) {
    const int nb = batch - b0 < 64 ? batch - b0 : 64;
    GnOffsets o;
    for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
    dim3 grid(GN_SPLITS, nb);
    constexpr int N = 16 / sizeof(T);
    if (C % N == 0 && C <= 8192 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)g % 16) == 0) {
      const int VPR = C / N;
      const int VW = VPR < CS_THREADS ? VPR : CS_THREADS;
      const size_t smem = (size_t)2 * (CS_THREADS / VW) * VW * N * sizeof(float);
      gn_partial_vec_kernel<T, MODE><<<grid, CS_THREADS, smem, s>>>((const T*)x, (const T*)g, o, b0, C, cpg, mean,
                                                                    inv_std, weight, p1, p2);
    } else
    gn_partial_kernel<T, MODE><<<grid, CS_THREADS, 0, s>>>((const T*)x, (const T*)g, o, b0, C, cpg, CT, mean,
                                                           inv_std, weight, p1, p2);
  }
}

// row chunks per octree for the apply kernels: fill the GPU, at least 64 rows per chunk on average
static inline int gn_apply_chunks(int64_t rows, int nb) {
  int64_t per = cdiv(cdiv(rows, nb > 0 ? nb : 1), 64);
  const int64_t cap = cdiv((int64_t)sm_count() * 16, nb > 0 ? nb : 1);
  if (per > cap) per = cap;
  return (int)(per < 1 ? 1 : per);
}

static void gn_finalize(const float* p1, const float* p2, const int64_t* h_offsets, int batch, int C, int cpg,
                        float eps, int stage, float* mean, float* inv_std, float* ca, float* cb, cudaStream_t s) {
  // offsets are only used for per-octree counts: pass them in chunks of 64
  const int G = C / cpg;
  for (int b0 = 0; b0 < batch; b0 += 64) {
    const int nb = batch - b0 < 64 ? batch - b0 : 64;
    GnOffsets o;
    for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
    const int n = nb * G;
    gn_finalize_kernel<<<(unsigned)cdiv(n, 128), 128, 0, s>>>(
        p1 + (size_t)b0 * GN_SPLITS * C, p2 ? p2 + (size_t)b0 * GN_SPLITS * C : nullptr, o, nb, C, cpg, eps,
        stage, mean + (size_t)b0 * G, inv_std + (size_t)b0 * G, ca ? ca + (size_t)b0 * G : nullptr,
        cb ? cb + (size_t)b0 * G : nullptr);
  }
}

}  // namespace oc

using namespace oc;

extern "C" size_t oc_colstats_workspace_bytes(int64_t n, int C) {
  if (C < 1) return 0;
  return colstats_workspace_bytes(n, C);
}

extern "C" int oc_colstats(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                           float* sum_ab, void* workspace, size_t workspace_bytes, void* stream) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "oc_colstats: bad dtype");
  OC_REQUIRE(n >= 0 && C >= 1 && (n == 0 || a), OC_EINVAL, "oc_colstats: bad argument");
  return launch_colstats(a, b, n, C, dtype, sum_a, sum_ab, workspace, workspace_bytes, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Column statistics without any workspace: the per-block partial sums live in a
// fixed array that is part of the library image.
//
// Meant for hosts that hand the whole device to an arena of their own at start-up
// (an inference server, a trainer with a locked pool) and for plugin callers that
// are handed raw pointers and no allocator at all: there a cudaMalloc inside the
// step either fails or stalls every stream of the process, and there is nobody to
// ask for a workspace.  The price is a hard size limit and one shared buffer.
// ---------------------------------------------------------------------------
constexpr int STATIC_STATS_MAX_C = 4096;
constexpr size_t STATIC_STATS_FLOATS = 512 * 1024;   // 2 MiB, resident on every GPU that loads the library
static __device__ __align__(256) float g_static_stats[STATIC_STATS_FLOATS];

// The array name is only a host-side handle; kernels need its device address, which
// differs per GPU.  Resolved once per device, with that device current.
static int static_stats_address(float** out) {
  static std::mutex mu;
  static float* per_device[64] = {nullptr};
  int dev = 0;
  OC_CUDA_OK(cudaGetDevice(&dev));
  OC_REQUIRE(dev >= 0 && dev < 64, OC_EINVAL, "oc_colstats_static: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    void* p = nullptr;
    OC_CUDA_OK(cudaGetSymbolAddress(&p, g_static_stats));
    OC_REQUIRE(p != nullptr, OC_ECUDA, "oc_colstats_static: null symbol address");
    per_device[dev] = (float*)p;
  }
  *out = per_device[dev];
  return OC_OK;
}

extern "C" int oc_colstats_static(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                                  float* sum_ab, void* stream) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "oc_colstats_static: bad dtype");
  OC_REQUIRE(C >= 1 && C <= STATIC_STATS_MAX_C, OC_EINVAL,
             "oc_colstats_static: C = %d exceeds the built-in scratch limit of %d channels; use oc_colstats with "
             "a caller-provided workspace", C, STATIC_STATS_MAX_C);
  OC_REQUIRE(n >= 0 && n < (1LL << 40), OC_EINVAL, "oc_colstats_static: row count out of range");
  OC_REQUIRE(n == 0 || a, OC_EINVAL, "oc_colstats_static: null input");
  cudaStream_t s = (cudaStream_t)stream;
  if (n == 0) {
    if (sum_a) OC_CUDA_OK(cudaMemsetAsync(sum_a, 0, (size_t)C * 4, s));
    if (sum_ab) OC_CUDA_OK(cudaMemsetAsync(sum_ab, 0, (size_t)C * 4, s));
    return OC_OK;
  }
  float* scratch = nullptr;
  int rc = static_stats_address(&scratch);
  if (rc) return rc;
  // As many row slices as fit: two partial rows of C floats per slice.  Every slot
  // that the final pass reads is written by this launch, so stale contents of the
  // shared array never matter and nothing has to be cleared.
  int splits = cs_splits(n);
  const int64_t cap = (int64_t)(STATIC_STATS_FLOATS / (2 * (size_t)C));
  if (splits > cap) splits = (int)cap;
  float* pa = scratch;
  float* pab = scratch + (size_t)splits * C;
  const int64_t rps = cdiv(n, splits);
  const int CT = cs_ct(C);
  if (dtype == OC_F32)
    colstats_kernel<float><<<splits, CS_THREADS, 0, s>>>((const float*)a, (const float*)b, 0, n, rps, C, CT, pa, pab);
  else if (dtype == OC_F16)
    colstats_kernel<__half><<<splits, CS_THREADS, 0, s>>>((const __half*)a, (const __half*)b, 0, n, rps, C, CT, pa, pab);
  else
    colstats_kernel<__nv_bfloat16><<<splits, CS_THREADS, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, 0, n, rps, C, CT, pa, pab);
  colstats_final_kernel<<<(unsigned)cdiv(C, 128), 128, 0, s>>>(pa, pab, splits, C, sum_a, sum_ab);
  OC_LAUNCH_OK("colstats kernels (static scratch)");
  return OC_OK;
}

extern "C" int oc_affine_cols(const void* x, const float* scale, const float* shift, int64_t n, int C,
                              int dtype, void* out, void* stream) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "oc_affine_cols: bad dtype");
  OC_REQUIRE(n >= 0 && C >= 1, OC_EINVAL, "oc_affine_cols: bad sizes");
  if (n == 0) return OC_OK;
  OC_REQUIRE(x && scale && shift && out, OC_EINVAL, "oc_affine_cols: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = n * C;
  const unsigned g = grid_1d(total, 256, 32);
  if (vec16_ok(C, dtype, x, out, nullptr)) {
    int gv; int64_t rpb;
    apply_split(n, &gv, &rpb);
    if (dtype == OC_F32) affine_cols_vec_kernel<float><<<gv, CS_THREADS, 0, s>>>((const float*)x, scale, shift, n, rpb, C, (float*)out);
    else if (dtype == OC_F16) affine_cols_vec_kernel<__half><<<gv, CS_THREADS, 0, s>>>((const __half*)x, scale, shift, n, rpb, C, (__half*)out);
    else affine_cols_vec_kernel<__nv_bfloat16><<<gv, CS_THREADS, 0, s>>>((const __nv_bfloat16*)x, scale, shift, n, rpb, C, (__nv_bfloat16*)out);
  } else
  if (dtype == OC_F32) affine_cols_kernel<float><<<g, 256, 0, s>>>((const float*)x, scale, shift, total, C, (float*)out);
  else if (dtype == OC_F16) affine_cols_kernel<__half><<<g, 256, 0, s>>>((const __half*)x, scale, shift, total, C, (__half*)out);
  else affine_cols_kernel<__nv_bfloat16><<<g, 256, 0, s>>>((const __nv_bfloat16*)x, scale, shift, total, C, (__nv_bfloat16*)out);
  OC_LAUNCH_OK("affine_cols_kernel");
  return OC_OK;
}

extern "C" int oc_bn_bwd_apply(const void* g, const void* x, const float* ka, const float* kb,
                               const float* kc, int64_t n, int C, int dtype, void* grad_in, void* stream) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "oc_bn_bwd_apply: bad dtype");
  OC_REQUIRE(n >= 0 && C >= 1, OC_EINVAL, "oc_bn_bwd_apply: bad sizes");
  if (n == 0) return OC_OK;
  OC_REQUIRE(g && x && ka && kb && kc && grad_in, OC_EINVAL, "oc_bn_bwd_apply: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t total = n * C;
  const unsigned gr = grid_1d(total, 256, 32);
  if (vec16_ok(C, dtype, g, x, grad_in)) {
    int gv; int64_t rpb;
    apply_split(n, &gv, &rpb);
    if (dtype == OC_F32) bn_bwd_apply_vec_kernel<float><<<gv, CS_THREADS, 0, s>>>((const float*)g, (const float*)x, ka, kb, kc, n, rpb, C, (float*)grad_in);
    else if (dtype == OC_F16) bn_bwd_apply_vec_kernel<__half><<<gv, CS_THREADS, 0, s>>>((const __half*)g, (const __half*)x, ka, kb, kc, n, rpb, C, (__half*)grad_in);
    else bn_bwd_apply_vec_kernel<__nv_bfloat16><<<gv, CS_THREADS, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, ka, kb, kc, n, rpb, C, (__nv_bfloat16*)grad_in);
  } else
  if (dtype == OC_F32) bn_bwd_apply_kernel<float><<<gr, 256, 0, s>>>((const float*)g, (const float*)x, ka, kb, kc, total, C, (float*)grad_in);
  else if (dtype == OC_F16) bn_bwd_apply_kernel<__half><<<gr, 256, 0, s>>>((const __half*)g, (const __half*)x, ka, kb, kc, total, C, (__half*)grad_in);
  else bn_bwd_apply_kernel<__nv_bfloat16><<<gr, 256, 0, s>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)x, ka, kb, kc, total, C, (__nv_bfloat16*)grad_in);
  OC_LAUNCH_OK("bn_bwd_apply_kernel");
  return OC_OK;
}

extern "C" size_t oc_gn_workspace_bytes(int batch, int C) {
  if (batch < 1 || C < 1) return 0;
  return gn_plan(nullptr, batch, C).total;
}

static int gn_check(const int64_t* h_offsets, int batch, int C, int groups, int dtype, const char* who) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "%s: bad dtype", who);
  OC_REQUIRE(batch >= 1 && C >= 1 && groups >= 1 && C % groups == 0, OC_EINVAL,
             "%s: bad batch/channels/groups (%d, %d, %d)", who, batch, C, groups);
  OC_REQUIRE(h_offsets, OC_EINVAL, "%s: null offsets", who);
  for (int b = 0; b < batch; ++b)
    OC_REQUIRE(h_offsets[b] <= h_offsets[b + 1], OC_EINVAL, "%s: offsets must be non-decreasing", who);
  return OC_OK;
}

#define GN_T(dtype, ...)                                            \
  do {                                                              \
    if ((dtype) == OC_F32) { using T = float; __VA_ARGS__; }        \
    else if ((dtype) == OC_F16) { using T = __half; __VA_ARGS__; }  \
    else { using T = __nv_bfloat16; __VA_ARGS__; }                  \
  } while (0)

extern "C" int oc_gn_fwd(const void* x, const int64_t* h_offsets, int batch, int C, int groups,
                         float eps, const float* weight, const float* bias, int dtype, void* out,
                         float* mean, float* inv_std, void* workspace, size_t workspace_bytes,
                         void* stream) {
  int rc = gn_check(h_offsets, batch, C, groups, dtype, "oc_gn_fwd");
  if (rc) return rc;
  OC_REQUIRE(weight && bias && mean && inv_std && workspace, OC_EINVAL, "oc_gn_fwd: null pointer");
  const GnPlan P = gn_plan(workspace, batch, C);
  OC_REQUIRE(workspace_bytes >= P.total, OC_ENOMEM, "oc_gn_fwd: workspace %zu < %zu", workspace_bytes, P.total);
  const int64_t n = h_offsets[batch] - h_offsets[0];
  if (n > 0) OC_REQUIRE(x && out, OC_EINVAL, "oc_gn_fwd: null data");
  cudaStream_t s = (cudaStream_t)stream;
  const int cpg = C / groups;
  GN_T(dtype, (gn_partials<T, 0>(x, nullptr, h_offsets, batch, C, cpg, nullptr, nullptr, nullptr, P.p1, nullptr, s)));
  gn_finalize(P.p1, nullptr, h_offsets, batch, C, cpg, eps, 0, mean, inv_std, nullptr, nullptr, s);
  GN_T(dtype, (gn_partials<T, 1>(x, nullptr, h_offsets, batch, C, cpg, mean, nullptr, nullptr, P.p1, nullptr, s)));
  gn_finalize(P.p1, nullptr, h_offsets, batch, C, cpg, eps, 1, mean, inv_std, nullptr, nullptr, s);
  for (int b0 = 0; b0 < batch && n > 0; b0 += 64) {
    const int nb = batch - b0 < 64 ? batch - b0 : 64;
    GnOffsets o;
    for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
    const int64_t total = (o.o[nb] - o.o[0]) * C;
    if (total == 0) continue;
    if (vec16_ok(C, dtype, x, out, nullptr)) {
      const dim3 ga((unsigned)gn_apply_chunks(o.o[nb] - o.o[0], nb), (unsigned)nb);
      GN_T(dtype, (gn_apply_vec_kernel<T, 0><<<ga, CS_THREADS, 0, s>>>((const T*)x, nullptr, o, b0, C, cpg, mean, inv_std, weight, bias, nullptr, nullptr, (T*)out)));
    } else
    GN_T(dtype, (gn_apply_kernel<T><<<grid_1d(total, 256, 32), 256, 0, s>>>((const T*)x, o, b0, nb, C, cpg, mean, inv_std, weight, bias, (T*)out)));
  }
  OC_LAUNCH_OK("group norm forward kernels");
  return OC_OK;
}

extern "C" int oc_gn_bwd(const void* grad_out, const void* x, const int64_t* h_offsets, int batch,
                         int C, int groups, float eps, const float* weight, const float* mean,
                         const float* inv_std, int dtype, void* grad_in, float* grad_weight,
                         float* grad_bias, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = gn_check(h_offsets, batch, C, groups, dtype, "oc_gn_bwd");
  if (rc) return rc;
  OC_REQUIRE(weight && mean && inv_std && workspace, OC_EINVAL, "oc_gn_bwd: null pointer");
  const GnPlan P = gn_plan(workspace, batch, C);
  OC_REQUIRE(workspace_bytes >= P.total, OC_ENOMEM, "oc_gn_bwd: workspace %zu < %zu", workspace_bytes, P.total);
  const int64_t n = h_offsets[batch] - h_offsets[0];
  if (n > 0) OC_REQUIRE(x && grad_out, OC_EINVAL, "oc_gn_bwd: null data");
  cudaStream_t s = (cudaStream_t)stream;
  const int cpg = C / groups;
  if (grad_weight || grad_bias) {
    GN_T(dtype, (gn_partials<T, 3>(x, grad_out, h_offsets, batch, C, cpg, mean, inv_std, nullptr, P.p1, P.p2, s)));
    gn_param_grad_kernel<<<(unsigned)cdiv(C, 128), 128, 0, s>>>(P.p1, P.p2, batch, C, grad_weight, grad_bias);
  }
  if (grad_in) {
    GN_T(dtype, (gn_partials<T, 2>(x, grad_out, h_offsets, batch, C, cpg, mean, nullptr, weight, P.p1, P.p2, s)));
    gn_finalize(P.p1, P.p2, h_offsets, batch, C, cpg, eps, 2, const_cast<float*>(mean),
                const_cast<float*>(inv_std), P.coef_a, P.coef_b, s);
    for (int b0 = 0; b0 < batch && n > 0; b0 += 64) {
      const int nb = batch - b0 < 64 ? batch - b0 : 64;
      GnOffsets o;
      for (int i = 0; i <= nb; ++i) o.o[i] = h_offsets[b0 + i];
      const int64_t total = (o.o[nb] - o.o[0]) * C;
      if (total == 0) continue;
      if (vec16_ok(C, dtype, x, grad_out, grad_in)) {
        const dim3 ga((unsigned)gn_apply_chunks(o.o[nb] - o.o[0], nb), (unsigned)nb);
        GN_T(dtype, (gn_apply_vec_kernel<T, 1><<<ga, CS_THREADS, 0, s>>>((const T*)x, (const T*)grad_out, o, b0, C, cpg, mean, inv_std, weight, nullptr, P.coef_a, P.coef_b, (T*)grad_in)));
      } else
      GN_T(dtype, (gn_bwd_apply_kernel<T><<<grid_1d(total, 256, 32), 256, 0, s>>>((const T*)grad_out, (const T*)x, o, b0, nb, C, cpg, mean, inv_std, weight, P.coef_a, P.coef_b, (T*)grad_in)));
    }
  }
  OC_LAUNCH_OK("group norm backward kernels");
  return OC_OK;
}
