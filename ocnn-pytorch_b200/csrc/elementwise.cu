// Bandwidth-bound companions of the octree convolution: depth-wise conv,
// pad / depad, 8-sibling max pooling and nearest upsampling.
//
// Restates ocnn/nn/octree_dwconv.py:30-118, ocnn/nn/octree_pad.py:13-39,
// ocnn/nn/octree_pool.py:17-38 and ocnn/nn/octree_interp.py:140-162 as single
// fused kernels: the reference's pad -> op -> depad chains and its (N, K, C)
// gather buffers never touch HBM.  One thread handles one 16-byte slice of a
// row, so a warp reads and writes full 128-byte lines.
#include "oc_common.cuh"

namespace oc {

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

// 16-byte chunk of N elements of T, loaded / stored as one transaction.
template <typename T>
struct Chunk {
  static constexpr int N = 16 / sizeof(T);
  uint4 raw;
  __device__ __forceinline__ T get(int i) const { return reinterpret_cast<const T*>(&raw)[i]; }
  __device__ __forceinline__ void set(int i, T v) { reinterpret_cast<T*>(&raw)[i] = v; }
};

template <typename T, bool VEC>
struct RowIO;

template <typename T>
struct RowIO<T, true> {
  static constexpr int N = 16 / sizeof(T);
  __device__ static __forceinline__ void load(const T* p, float* v) {
    Chunk<T> c;
    c.raw = *reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = to_f32<T>(c.get(i));
  }
  __device__ static __forceinline__ void store(T* p, const float* v) {
    Chunk<T> c;
#pragma unroll
    for (int i = 0; i < N; ++i) c.set(i, from_f32<T>(v[i]));
    *reinterpret_cast<uint4*>(p) = c.raw;
  }
};

template <typename T>
struct RowIO<T, false> {
  static constexpr int N = 1;
  __device__ static __forceinline__ void load(const T* p, float* v) { v[0] = to_f32<T>(*p); }
  __device__ static __forceinline__ void store(T* p, const float* v) { *p = from_f32<T>(v[0]); }
};

// Grid-stride walk over (row, 16-byte chunk of the row) pairs without a division per step:
// the pair advances by (stride / cpr, stride % cpr) with one carry.
struct RowChunkIter {
  int64_t row, drow;
  int col, dcol, cpr;
  __device__ __forceinline__ explicit RowChunkIter(int cpr_) : cpr(cpr_) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    drow = stride / cpr;
    dcol = (int)(stride % cpr);
    row = t0 / cpr;
    col = (int)(t0 % cpr);
  }
  __device__ __forceinline__ void next() {
    row += drow;
    col += dcol;
    if (col >= cpr) { col -= cpr; ++row; }
  }
};

// ---------------------------------------------------------------------------
// depth-wise convolution
// ---------------------------------------------------------------------------
template <typename T, typename I, bool VEC>
__global__ void dwconv_kernel(const T* __restrict__ data, const float* __restrict__ w,
                              const I* __restrict__ table, int table_cols, TapList taps, int K,
                              int64_t n_out, int C, T* __restrict__ out) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;  // chunks per row
  for (RowChunkIter it(cpr); it.row < n_out; it.next()) {
    const int64_t r = it.row;
    const int c0 = it.col * N;
    float acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.f;
    for (int k = 0; k < K; ++k) {
      const int64_t idx = (int64_t)table[r * table_cols + taps.t[k]];
      if (idx < 0) continue;
      float v[N];
      RowIO<T, VEC>::load(data + idx * C + c0, v);
#pragma unroll
      for (int i = 0; i < N; ++i) acc[i] = fmaf(v[i], w[k * C + c0 + i], acc[i]);
    }
    RowIO<T, VEC>::store(out + r * C + c0, acc);
  }
}


// Same computation with the per-block staging that makes it bandwidth-efficient:
// the (K, C) weights sit in shared memory as fp32 for the whole block, the K neighbour
// indices of the block's rows are fetched once (coalesced) instead of once per thread,
// and each thread then streams its 16-byte channel slice of every valid neighbour row.
// A thread works on DW_ROWS rows at once: the kernel is bound by L1 wavefronts (91 % of peak
// with one row per thread, two thirds of them the weight reads from shared memory), and a
// tap's 8 weights are then read once for DW_ROWS rows; the rows' loads are independent.
constexpr int DW_ROWS = 4;

template <typename T, typename I>
__global__ void __launch_bounds__(256)
dwconv_staged_kernel(const T* __restrict__ data, const float* __restrict__ w, const I* __restrict__ table,
                     int table_cols, TapList taps, int K, int64_t n_out, int C, int rows_per_block,
                     T* __restrict__ out) {
  constexpr int N = 16 / sizeof(T);
  extern __shared__ __align__(16) float dsm[];
  float* sw = dsm;                               // [K][C]
  int* sidx = (int*)(dsm + (size_t)K * C);       // [rows_per_block][K]
  for (int i = threadIdx.x; i < K * C; i += blockDim.x) sw[i] = w[i];
  const int cpr = C / N;
  const int slots = rows_per_block / DW_ROWS;    // row slots of the block; slot s owns rows s, s + slots, ...
  const int r_local = threadIdx.x / cpr;
  const int c0 = (threadIdx.x % cpr) * N;
  const bool active = r_local < slots;
  const int64_t n_blocks = (n_out + rows_per_block - 1) / rows_per_block;
  for (int64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
    const int64_t row_base = blk * rows_per_block;
    __syncthreads();                             // weights ready / previous indices consumed
    {
      int rr = threadIdx.x / K, kk = threadIdx.x % K;        // (row, tap) of entry threadIdx.x, advanced without division
      const int drr = blockDim.x / K, dkk = blockDim.x % K;
      for (int i = threadIdx.x; i < rows_per_block * K; i += blockDim.x) {
        const int64_t r = row_base + rr;
        sidx[i] = r < n_out ? (int)table[r * table_cols + taps.t[kk]] : -1;
        rr += drr; kk += dkk;
        if (kk >= K) { kk -= K; ++rr; }
      }
    }
    __syncthreads();
    if (!active) continue;
    float acc[DW_ROWS][N];
#pragma unroll
    for (int j = 0; j < DW_ROWS; ++j)
#pragma unroll
      for (int i = 0; i < N; ++i) acc[j][i] = 0.f;
    for (int k = 0; k < K; ++k) {
      float wv[N];
#pragma unroll
      for (int q = 0; q < N / 4; ++q) {
        const float4 t = reinterpret_cast<const float4*>(sw + k * C + c0)[q];
        wv[4 * q + 0] = t.x; wv[4 * q + 1] = t.y; wv[4 * q + 2] = t.z; wv[4 * q + 3] = t.w;
      }
      uint4 raw[DW_ROWS];
      bool ok[DW_ROWS];
#pragma unroll
      for (int j = 0; j < DW_ROWS; ++j) {
        const int idx = sidx[(r_local + j * slots) * K + k];
        ok[j] = idx >= 0;
        raw[j] = ok[j] ? *reinterpret_cast<const uint4*>(data + (int64_t)idx * C + c0) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < DW_ROWS; ++j) {
        if (!ok[j]) continue;
        const T* e = reinterpret_cast<const T*>(&raw[j]);
#pragma unroll
        for (int i = 0; i < N; ++i) acc[j][i] = fmaf(to_f32<T>(e[i]), wv[i], acc[j][i]);
      }
    }
#pragma unroll
    for (int j = 0; j < DW_ROWS; ++j) {
      const int64_t r = row_base + r_local + j * slots;
      if (r < n_out) RowIO<T, true>::store(out + r * C + c0, acc[j]);
    }
  }
}

template <typename T, typename I>
static bool launch_dwconv_staged(const void* data, const float* weights, const void* table, int table_cols,
                                 const TapList& taps, int K, int64_t n_out, int C, void* out, cudaStream_t s) {
  constexpr int N = 16 / sizeof(T);
  const int cpr = C / N;
  if (cpr > 256) return false;
  const int rpb = (256 / cpr) * DW_ROWS;
  const size_t smem = (size_t)K * C * 4 + (size_t)rpb * K * 4;
  if (smem > 200 * 1024) return false;
  auto kern = dwconv_staged_kernel<T, I>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int64_t n_blocks = (n_out + rpb - 1) / rpb;
  const int64_t cap = (int64_t)sm_count() * (smem > 64 * 1024 ? 2 : 6);
  kern<<<(unsigned)(n_blocks < cap ? n_blocks : cap), 256, smem, s>>>((const T*)data, weights, (const I*)table, table_cols,
                                                                     taps, K, n_out, C, rpb, (T*)out);
  return true;
}

// grad_w partials: block (x = channel block, y = row split); thread = channel.
template <typename T, typename I>
__global__ void dwconv_wgrad_kernel(const T* __restrict__ data, const T* __restrict__ gout,
                                    const I* __restrict__ table, int table_cols, TapList taps,
                                    int K, int64_t n_out, int C, int64_t rows_per_split,
                                    float* __restrict__ partial) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t r_begin = (int64_t)blockIdx.y * rows_per_split;
  int64_t r_end = r_begin + rows_per_split;
  if (r_end > n_out) r_end = n_out;
  float acc[OC_MAX_TAPS];
#pragma unroll
  for (int k = 0; k < OC_MAX_TAPS; ++k) acc[k] = 0.f;
  if (c < C) {
    for (int64_t r = r_begin; r < r_end; ++r) {
      const float g = to_f32<T>(gout[r * C + c]);
#pragma unroll
      for (int k = 0; k < OC_MAX_TAPS; ++k) {
        if (k < K) {
          const int64_t idx = (int64_t)table[r * table_cols + taps.t[k]];
          if (idx >= 0) acc[k] = fmaf(to_f32<T>(data[idx * C + c]), g, acc[k]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < OC_MAX_TAPS; ++k)
      if (k < K) partial[((int64_t)blockIdx.y * K + k) * C + c] = acc[k];
  }
}

// Vector form of the weight gradient: block = (row split, group of DWG_TAPS taps); thread
// (row lane rl, 16-byte channel vector v) walks the rows rl, rl + RL, ... of the split, loads
// grad_out once per row and the gathered row once per tap (16 bytes each), and keeps the
// DWG_TAPS x N partial sums of its channels in registers; row lanes are folded through
// shared memory tap by tap.  The blocks of one row split (one per tap group) run together and
// share the split's rows through L2.  Measured on the 4 M-row, C = 256 case with 1 / 2 / 3 / 5 / 9
// taps per block: 11.2 / 6.6 / 7.5 / 10.5 / 16.9 ms - few taps keep the accumulators small and many
// warps resident, one tap reads grad_out 27 times.  (The scalar kernel above issues one 2-byte
// load per channel, tap and row: 35 ms.)
#ifndef OC_DWG_TAPS
#define OC_DWG_TAPS 2
#endif
constexpr int DWG_TAPS = OC_DWG_TAPS;
constexpr int DWG_THREADS = 256;

template <typename T, typename I>
__global__ void __launch_bounds__(DWG_THREADS)
dwconv_wgrad_vec_kernel(const T* __restrict__ data, const T* __restrict__ gout, const I* __restrict__ table,
                        int table_cols, TapList taps, int K, int64_t n_out, int C, int64_t rows_per_split,
                        float* __restrict__ partial) {
  constexpr int N = 16 / sizeof(T);
  extern __shared__ float wsm[];                 // [RL][VW * N]
  const int VPR = C / N;
  const int VW = VPR < DWG_THREADS ? VPR : DWG_THREADS;
  const int RL = DWG_THREADS / VW;
  const int v = threadIdx.x % VW, rl = threadIdx.x / VW;
  const bool active = rl < RL;
  // blockIdx.x (the fast index of the block order) = tap group, blockIdx.y = row split: the blocks that
  // stream the same rows for different taps run at the same time and share them through L2.  With the
  // tap group as the slow index every group streamed both feature matrices from DRAM again (9.8 GB
  // of DRAM reads for 1.2 GB of data at 1 M rows, C = 256).
  const int split = blockIdx.y;
  const int k_lo = blockIdx.x * DWG_TAPS;
  const int nk = min(DWG_TAPS, K - k_lo);
  const int64_t r0 = (int64_t)split * rows_per_split;
  int64_t r1 = r0 + rows_per_split;
  if (r1 > n_out) r1 = n_out;
  int col[DWG_TAPS];
#pragma unroll
  for (int k = 0; k < DWG_TAPS; ++k) col[k] = taps.t[k_lo + (k < nk ? k : 0)];
  for (int v0 = 0; v0 < VPR; v0 += VW) {
    const int vv = v0 + v;
    float acc[DWG_TAPS][N];
#pragma unroll
    for (int k = 0; k < DWG_TAPS; ++k)
#pragma unroll
      for (int i = 0; i < N; ++i) acc[k][i] = 0.f;
    if (active && vv < VPR) {
      for (int64_t r = r0 + rl; r < r1; r += RL) {
        float g[N];
        RowIO<T, true>::load(gout + r * C + vv * N, g);
        const I* trow = table + r * table_cols;
        // all index loads first, then all row loads: DWG_TAPS independent requests in flight per thread
        int64_t idx[DWG_TAPS];
#pragma unroll
        for (int k = 0; k < DWG_TAPS; ++k) idx[k] = k < nk ? (int64_t)trow[col[k]] : -1;
        uint4 raw[DWG_TAPS];
#pragma unroll
        for (int k = 0; k < DWG_TAPS; ++k)
          raw[k] = idx[k] >= 0 ? *reinterpret_cast<const uint4*>(data + idx[k] * C + vv * N) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < DWG_TAPS; ++k) {
          if (idx[k] < 0) continue;
          const T* e = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
          for (int i = 0; i < N; ++i) acc[k][i] = fmaf(to_f32<T>(e[i]), g[i], acc[k][i]);
        }
      }
    }
    // fold the row lanes, one tap at a time
#pragma unroll
    for (int k = 0; k < DWG_TAPS; ++k) {
      if (k >= nk) break;                         // block-uniform
      if (active) {
#pragma unroll
        for (int i = 0; i < N; ++i) wsm[(rl * VW + v) * N + i] = acc[k][i];
      }
      __syncthreads();
      for (int c = threadIdx.x; c < VW * N; c += DWG_THREADS) {
        const int ch = v0 * N + c;
        if (ch < C) {
          float t = 0.f;
          for (int l = 0; l < RL; ++l) t += wsm[l * VW * N + c];
          partial[((int64_t)split * K + k_lo + k) * C + ch] = t;
        }
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------
// pad / depad
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void fill_rows_kernel(T* __restrict__ out, int64_t n_chunks, float fill) {
  constexpr int N = RowIO<T, VEC>::N;
  float v[N];
#pragma unroll
  for (int i = 0; i < N; ++i) v[i] = fill;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_chunks;
       t += (int64_t)gridDim.x * blockDim.x)
    RowIO<T, VEC>::store(out + t * N, v);
}

// scatter == true : out[index[j]] = data[j];  false : out[j] = data[index[j]]
template <typename T, bool VEC, bool SCATTER>
__global__ void index_rows_kernel(const T* __restrict__ data, const int64_t* __restrict__ index,
                                  int64_t n, int C, T* __restrict__ out) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;
  for (RowChunkIter it(cpr); it.row < n; it.next()) {
    const int64_t j = it.row;
    const int c0 = it.col * N;
    const int64_t q = index[j];
    float v[N];
    RowIO<T, VEC>::load(data + (SCATTER ? j : q) * C + c0, v);
    RowIO<T, VEC>::store(out + (SCATTER ? q : j) * C + c0, v);
  }
}

// ---------------------------------------------------------------------------
// max pool over the 8 siblings
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void maxpool_fwd_kernel(const T* __restrict__ data, const int32_t* __restrict__ child_in,
                                   const int32_t* __restrict__ child_out, int64_t n_out, int C,
                                   T* __restrict__ out, int64_t* __restrict__ argmax) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;
  for (RowChunkIter it(cpr); it.row < n_out; it.next()) {
    const int64_t p = it.row;
    const int c0 = it.col * N;
    const int64_t j = child_out ? (int64_t)child_out[p] : p;
    float best[N];
    int arg[N];
    if (j < 0) {
#pragma unroll
      for (int i = 0; i < N; ++i) best[i] = 0.f;
      RowIO<T, VEC>::store(out + p * C + c0, best);
      continue;
    }
#pragma unroll
    for (int i = 0; i < N; ++i) { best[i] = -INFINITY; arg[i] = 0; }
    for (int s = 0; s < 8; ++s) {
      const int64_t src = child_in ? (int64_t)child_in[j * 8 + s] : j * 8 + s;
      if (src < 0) continue;  // padded with -inf in the reference: never a strict maximum
      float v[N];
      RowIO<T, VEC>::load(data + src * C + c0, v);
#pragma unroll
      for (int i = 0; i < N; ++i)
        if (v[i] > best[i]) { best[i] = v[i]; arg[i] = s; }
    }
    RowIO<T, VEC>::store(out + p * C + c0, best);
    if (argmax) {
#pragma unroll
      for (int i = 0; i < N; ++i) argmax[j * C + c0 + i] = arg[i];
    }
  }
}

// One thread per (fine row, chunk): grad_in[src(8j+s)] = argmax == s ? g : 0.
template <typename T, bool VEC>
__global__ void maxpool_bwd_kernel(const T* __restrict__ gout, const int64_t* __restrict__ argmax,
                                   const int32_t* __restrict__ child_in,
                                   const int32_t* __restrict__ child_out, int64_t n_out, int C,
                                   T* __restrict__ gin) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;
  for (RowChunkIter it(cpr); it.row < n_out; it.next()) {
    const int64_t p = it.row;
    const int c0 = it.col * N;
    const int64_t j = child_out ? (int64_t)child_out[p] : p;
    if (j < 0) continue;
    float g[N];
    RowIO<T, VEC>::load(gout + p * C + c0, g);
    for (int s = 0; s < 8; ++s) {
      const int64_t dst = child_in ? (int64_t)child_in[j * 8 + s] : j * 8 + s;
      if (dst < 0) continue;
      float v[N];
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] = (argmax[j * C + c0 + i] == s) ? g[i] : 0.f;
      RowIO<T, VEC>::store(gin + dst * C + c0, v);
    }
  }
}

// ---------------------------------------------------------------------------
// nearest upsample
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void upsample_fwd_kernel(const T* __restrict__ data, const int64_t* __restrict__ idx_coarse,
                                    const int64_t* __restrict__ idx_fine, int64_t n_out, int C,
                                    T* __restrict__ out) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;
  for (RowChunkIter it(cpr); it.row < n_out; it.next()) {
    const int64_t m = it.row;
    const int c0 = it.col * N;
    const int64_t src = idx_coarse ? idx_coarse[m >> 3] : (idx_fine[m] >> 3);
    float v[N];
    RowIO<T, VEC>::load(data + src * C + c0, v);
    RowIO<T, VEC>::store(out + m * C + c0, v);
  }
}

template <typename T, bool VEC>
__global__ void upsample_bwd_kernel(const T* __restrict__ gout, const int32_t* __restrict__ child_coarse,
                                    const int32_t* __restrict__ child_fine, int64_t n_in, int C,
                                    T* __restrict__ gin) {
  constexpr int N = RowIO<T, VEC>::N;
  const int cpr = C / N;
  for (RowChunkIter it(cpr); it.row < n_in; it.next()) {
    const int64_t q = it.row;
    const int c0 = it.col * N;
    float acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.f;
    const int64_t j = child_coarse ? (int64_t)child_coarse[q] : q;
    if (j >= 0) {
      for (int s = 0; s < 8; ++s) {
        const int64_t src = child_fine ? (int64_t)child_fine[j * 8 + s] : j * 8 + s;
        if (src < 0) continue;
        float v[N];
        RowIO<T, VEC>::load(gout + src * C + c0, v);
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] += v[i];
      }
    }
    RowIO<T, VEC>::store(gin + q * C + c0, acc);
  }
}

// ---------------------------------------------------------------------------
// dispatch helpers
// ---------------------------------------------------------------------------
static inline bool vec_ok(int C, int dtype, const void* a, const void* b) {
  const size_t es = dtype_size(dtype);
  return ((size_t)C * es) % 16 == 0 && ((uintptr_t)a % 16) == 0 && ((uintptr_t)b % 16) == 0;
}

#define OC_DISPATCH_T(dtype, ...)                                   \
  do {                                                              \
    if ((dtype) == OC_F32) { using T = float; __VA_ARGS__; }        \
    else if ((dtype) == OC_F16) { using T = __half; __VA_ARGS__; }  \
    else { using T = __nv_bfloat16; __VA_ARGS__; }                  \
  } while (0)

#define OC_DISPATCH_TV(dtype, vec, ...)                                           \
  do {                                                                            \
    if (vec) { constexpr bool V = true; OC_DISPATCH_T(dtype, __VA_ARGS__); }      \
    else { constexpr bool V = false; OC_DISPATCH_T(dtype, __VA_ARGS__); }         \
  } while (0)

static inline int chunk_elems(int dtype, bool vec) { return vec ? (int)(16 / dtype_size(dtype)) : 1; }

static inline int check_dtype(int dtype, const char* who) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "%s: bad dtype %d", who, dtype);
  return OC_OK;
}

}  // namespace oc

using namespace oc;

extern "C" int oc_dwconv_fwd(const void* data, int64_t n_in, const float* weights, const void* table,
                             int idx_bytes, int table_cols, const int* h_taps, int K, int64_t n_out,
                             int C, int dtype, void* out, void* stream) {
  int rc = check_dtype(dtype, "oc_dwconv_fwd");
  if (rc) return rc;
  TapList taps;
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "oc_dwconv_fwd: bad table_cols");
  rc = make_taps(h_taps, K, table_cols, &taps, "oc_dwconv_fwd");
  if (rc) return rc;
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "oc_dwconv_fwd: idx_bytes must be 4 or 8");
  OC_REQUIRE(C >= 1 && n_out >= 0 && n_in >= 0, OC_EINVAL, "oc_dwconv_fwd: bad sizes");
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(data && weights && table && out, OC_EINVAL, "oc_dwconv_fwd: null pointer");
  const bool vec = vec_ok(C, dtype, data, out);
  const int64_t work = n_out * (C / chunk_elems(dtype, vec));
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned g = grid_1d(work, 256, 32);
  if (vec && ((uintptr_t)weights % 16) == 0) {
    bool done = false;
    if (idx_bytes == 8)
      OC_DISPATCH_T(dtype, (done = launch_dwconv_staged<T, int64_t>(data, weights, table, table_cols, taps, K, n_out, C, out, s)));
    else
      OC_DISPATCH_T(dtype, (done = launch_dwconv_staged<T, int32_t>(data, weights, table, table_cols, taps, K, n_out, C, out, s)));
    if (done) {
      OC_LAUNCH_OK("dwconv_staged_kernel");
      return OC_OK;
    }
  }
  if (idx_bytes == 8)
    OC_DISPATCH_TV(dtype, vec, (dwconv_kernel<T, int64_t, V><<<g, 256, 0, s>>>((const T*)data, weights, (const int64_t*)table, table_cols, taps, K, n_out, C, (T*)out)));
  else
    OC_DISPATCH_TV(dtype, vec, (dwconv_kernel<T, int32_t, V><<<g, 256, 0, s>>>((const T*)data, weights, (const int32_t*)table, table_cols, taps, K, n_out, C, (T*)out)));
  OC_LAUNCH_OK("dwconv_kernel");
  return OC_OK;
}

static int dw_splits(int C, int64_t n_out) {
  const int cblocks = (int)cdiv(C, 128);
  int splits = (int)cdiv((int64_t)sm_count() * 8, cblocks);
  const int64_t by_rows = cdiv(n_out > 0 ? n_out : 1, 64);
  if (splits > by_rows) splits = (int)by_rows;
  if (splits < 1) splits = 1;
  if (splits > 2048) splits = 2048;
  return splits;
}

extern "C" size_t oc_dwconv_wgrad_workspace_bytes(int K, int C, int64_t n_out) {
  if (K < 1 || C < 1) return 0;
  return align_up((size_t)dw_splits(C, n_out) * K * C * sizeof(float), 256);
}

namespace oc { int reduce_partials(const float*, int, int64_t, float*, cudaStream_t); }

extern "C" int oc_dwconv_wgrad(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                               const void* table, int idx_bytes, int table_cols, const int* h_taps,
                               int K, int C, int dtype, float* grad_w, void* workspace,
                               size_t workspace_bytes, void* stream) {
  int rc = check_dtype(dtype, "oc_dwconv_wgrad");
  if (rc) return rc;
  TapList taps;
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "oc_dwconv_wgrad: bad table_cols");
  rc = make_taps(h_taps, K, table_cols, &taps, "oc_dwconv_wgrad");
  if (rc) return rc;
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "oc_dwconv_wgrad: idx_bytes must be 4 or 8");
  OC_REQUIRE(C >= 1 && n_out >= 0 && n_in >= 0 && grad_w, OC_EINVAL, "oc_dwconv_wgrad: bad argument");
  cudaStream_t s = (cudaStream_t)stream;
  if (n_out == 0) {
    OC_CUDA_OK(cudaMemsetAsync(grad_w, 0, (size_t)K * C * 4, s));
    return OC_OK;
  }
  OC_REQUIRE(data && grad_out && table && workspace, OC_EINVAL, "oc_dwconv_wgrad: null pointer");
  const int splits = dw_splits(C, n_out);
  OC_REQUIRE(workspace_bytes >= (size_t)splits * K * C * 4, OC_ENOMEM, "oc_dwconv_wgrad: workspace too small");
  const int64_t rps = cdiv(n_out, splits);
  dim3 grid((unsigned)cdiv(C, 128), (unsigned)splits);
  float* partial = (float*)workspace;
  if (vec_ok(C, dtype, data, grad_out) && C * (int)dtype_size(dtype) / 16 <= 4096) {
    const int N = 16 / (int)dtype_size(dtype);
    const int VPR = C / N, VW = VPR < DWG_THREADS ? VPR : DWG_THREADS, RL = DWG_THREADS / VW;
    const size_t smem = (size_t)RL * VW * N * sizeof(float);
    const dim3 gv((unsigned)cdiv(K, DWG_TAPS), (unsigned)splits);
    if (idx_bytes == 8)
      OC_DISPATCH_T(dtype, (dwconv_wgrad_vec_kernel<T, int64_t><<<gv, DWG_THREADS, smem, s>>>((const T*)data, (const T*)grad_out, (const int64_t*)table, table_cols, taps, K, n_out, C, rps, partial)));
    else
      OC_DISPATCH_T(dtype, (dwconv_wgrad_vec_kernel<T, int32_t><<<gv, DWG_THREADS, smem, s>>>((const T*)data, (const T*)grad_out, (const int32_t*)table, table_cols, taps, K, n_out, C, rps, partial)));
    OC_LAUNCH_OK("dwconv_wgrad_vec_kernel");
    return reduce_partials(partial, splits, (int64_t)K * C, grad_w, s);
  }
  if (idx_bytes == 8)
    OC_DISPATCH_T(dtype, (dwconv_wgrad_kernel<T, int64_t><<<grid, 128, 0, s>>>((const T*)data, (const T*)grad_out, (const int64_t*)table, table_cols, taps, K, n_out, C, rps, partial)));
  else
    OC_DISPATCH_T(dtype, (dwconv_wgrad_kernel<T, int32_t><<<grid, 128, 0, s>>>((const T*)data, (const T*)grad_out, (const int32_t*)table, table_cols, taps, K, n_out, C, rps, partial)));
  OC_LAUNCH_OK("dwconv_wgrad_kernel");
  return reduce_partials(partial, splits, (int64_t)K * C, grad_w, s);
}

extern "C" int oc_pad(const void* data, const int64_t* index, int64_t n_nempty, int64_t n_all, int C,
                      int dtype, float fill, void* out, void* stream) {
  int rc = check_dtype(dtype, "oc_pad");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_nempty >= 0 && n_all >= n_nempty, OC_EINVAL, "oc_pad: bad sizes");
  if (n_all == 0) return OC_OK;
  OC_REQUIRE(out && (n_nempty == 0 || (data && index)), OC_EINVAL, "oc_pad: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = vec_ok(C, dtype, data ? data : out, out);
  const int ce = chunk_elems(dtype, vec);
  OC_DISPATCH_TV(dtype, vec, (fill_rows_kernel<T, V><<<grid_1d(n_all * C / ce, 256, 32), 256, 0, s>>>((T*)out, n_all * C / ce, fill)));
  if (n_nempty > 0)
    OC_DISPATCH_TV(dtype, vec, (index_rows_kernel<T, V, true><<<grid_1d(n_nempty * (C / ce), 256, 32), 256, 0, s>>>((const T*)data, index, n_nempty, C, (T*)out)));
  OC_LAUNCH_OK("pad kernels");
  return OC_OK;
}

extern "C" int oc_depad(const void* data, const int64_t* index, int64_t n_nempty, int C, int dtype,
                        void* out, void* stream) {
  int rc = check_dtype(dtype, "oc_depad");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_nempty >= 0, OC_EINVAL, "oc_depad: bad sizes");
  if (n_nempty == 0) return OC_OK;
  OC_REQUIRE(data && index && out, OC_EINVAL, "oc_depad: null pointer");
  const bool vec = vec_ok(C, dtype, data, out);
  const int ce = chunk_elems(dtype, vec);
  cudaStream_t s = (cudaStream_t)stream;
  OC_DISPATCH_TV(dtype, vec, (index_rows_kernel<T, V, false><<<grid_1d(n_nempty * (C / ce), 256, 32), 256, 0, s>>>((const T*)data, index, n_nempty, C, (T*)out)));
  OC_LAUNCH_OK("depad kernel");
  return OC_OK;
}

extern "C" int oc_maxpool_fwd(const void* data, const int32_t* children_in, const int32_t* children_out,
                              int64_t n_out, int C, int dtype, void* out, int64_t* argmax, void* stream) {
  int rc = check_dtype(dtype, "oc_maxpool_fwd");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_out >= 0, OC_EINVAL, "oc_maxpool_fwd: bad sizes");
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(data && out, OC_EINVAL, "oc_maxpool_fwd: null pointer");
  const bool vec = vec_ok(C, dtype, data, out);
  const int ce = chunk_elems(dtype, vec);
  cudaStream_t s = (cudaStream_t)stream;
  OC_DISPATCH_TV(dtype, vec, (maxpool_fwd_kernel<T, V><<<grid_1d(n_out * (C / ce), 256, 32), 256, 0, s>>>((const T*)data, children_in, children_out, n_out, C, (T*)out, argmax)));
  OC_LAUNCH_OK("maxpool_fwd_kernel");
  return OC_OK;
}

extern "C" int oc_maxpool_bwd(const void* grad_out, const int64_t* argmax, const int32_t* children_in,
                              const int32_t* children_out, int64_t n_out, int64_t n_in, int C,
                              int dtype, void* grad_in, void* stream) {
  int rc = check_dtype(dtype, "oc_maxpool_bwd");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_out >= 0 && n_in >= 0, OC_EINVAL, "oc_maxpool_bwd: bad sizes");
  if (n_in == 0) return OC_OK;
  OC_REQUIRE(grad_in, OC_EINVAL, "oc_maxpool_bwd: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  // Every fine row with a non-empty parent is written exactly once; with
  // children_in == NULL that is every row, otherwise exactly the non-empty rows,
  // so no pre-clear is needed.  Rows are cleared only in the degenerate n_out = 0 case.
  if (n_out == 0) {
    OC_CUDA_OK(cudaMemsetAsync(grad_in, 0, (size_t)n_in * C * dtype_size(dtype), s));
    return OC_OK;
  }
  OC_REQUIRE(grad_out && argmax, OC_EINVAL, "oc_maxpool_bwd: null pointer");
  const bool vec = vec_ok(C, dtype, grad_out, grad_in);
  const int ce = chunk_elems(dtype, vec);
  OC_DISPATCH_TV(dtype, vec, (maxpool_bwd_kernel<T, V><<<grid_1d(n_out * (C / ce), 256, 32), 256, 0, s>>>((const T*)grad_out, argmax, children_in, children_out, n_out, C, (T*)grad_in)));
  OC_LAUNCH_OK("maxpool_bwd_kernel");
  return OC_OK;
}

extern "C" int oc_upsample_fwd(const void* data, const int64_t* index_coarse, const int64_t* index_fine,
                               int64_t n_out, int C, int dtype, void* out, void* stream) {
  int rc = check_dtype(dtype, "oc_upsample_fwd");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_out >= 0, OC_EINVAL, "oc_upsample_fwd: bad sizes");
  OC_REQUIRE((index_coarse != nullptr) != (index_fine != nullptr), OC_EINVAL,
             "oc_upsample_fwd: exactly one index array must be given");
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(data && out, OC_EINVAL, "oc_upsample_fwd: null pointer");
  const bool vec = vec_ok(C, dtype, data, out);
  const int ce = chunk_elems(dtype, vec);
  cudaStream_t s = (cudaStream_t)stream;
  OC_DISPATCH_TV(dtype, vec, (upsample_fwd_kernel<T, V><<<grid_1d(n_out * (C / ce), 256, 32), 256, 0, s>>>((const T*)data, index_coarse, index_fine, n_out, C, (T*)out)));
  OC_LAUNCH_OK("upsample_fwd_kernel");
  return OC_OK;
}

extern "C" int oc_upsample_bwd(const void* grad_out, const int32_t* children_coarse,
                               const int32_t* children_fine, int64_t n_in, int C, int dtype,
                               void* grad_in, void* stream) {
  int rc = check_dtype(dtype, "oc_upsample_bwd");
  if (rc) return rc;
  OC_REQUIRE(C >= 1 && n_in >= 0, OC_EINVAL, "oc_upsample_bwd: bad sizes");
  OC_REQUIRE((children_coarse != nullptr) != (children_fine != nullptr), OC_EINVAL,
             "oc_upsample_bwd: exactly one children array must be given");
  if (n_in == 0) return OC_OK;
  OC_REQUIRE(grad_out && grad_in, OC_EINVAL, "oc_upsample_bwd: null pointer");
  const bool vec = vec_ok(C, dtype, grad_out, grad_in);
  const int ce = chunk_elems(dtype, vec);
  cudaStream_t s = (cudaStream_t)stream;
  OC_DISPATCH_TV(dtype, vec, (upsample_bwd_kernel<T, V><<<grid_1d(n_in * (C / ce), 256, 32), 256, 0, s>>>((const T*)grad_out, children_coarse, children_fine, n_in, C, (T*)grad_in)));
  OC_LAUNCH_OK("upsample_bwd_kernel");
  return OC_OK;
}
