// 3x3x3 neighbour tables and their variants.
//
// Restates Octree.construct_neigh / get_neigh / nempty_index / remap_nempty_neigh
// (ocnn/octree/octree.py:160-199, 404-439, 490-523).  The reference materialises
// three (N, 8, 27) int64 temporaries per depth; here each table is produced by a
// single kernel whose only HBM traffic is the 27 parent entries read and the 216
// entries written per non-empty parent (coalesced, one warp per parent).
#include "oc_common.cuh"

namespace oc {

// Column k = (dx+1)*9 + (dy+1)*3 + (dz+1); child i = cx*4 + cy*2 + cz.
__global__ void neigh_full_kernel(int depth, int64_t n_local, int64_t total,
                                  int64_t* __restrict__ neigh) {
  const int bound = 1 << depth;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total * 27;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t node = t / 27;
    const int k = (int)(t - node * 27);
    const int64_t b = node / n_local;
    const uint64_t m = (uint64_t)(node - b * n_local);
    const int x = (int)compact3(m >> 2) + k / 9 - 1;
    const int y = (int)compact3(m >> 1) + (k / 3) % 3 - 1;
    const int z = (int)compact3(m) + k % 3 - 1;
    int64_t v = -1;
    if (x >= 0 && y >= 0 && z >= 0 && x < bound && y < bound && z < bound)
      v = (int64_t)morton3((uint64_t)x, (uint64_t)y, (uint64_t)z) + b * n_local;
    neigh[t] = v;
  }
}

// One warp per NON-EMPTY parent node p of depth d-1 (most parents of a deep level are empty:
// a block first compacts the non-empty parents of a chunk of 256 nodes with one coalesced read
// of `children`, then its 8 warps take them in turn).  Lanes 0..26 fetch the parent's 27
// neighbours q and their child pointers c = children[q]; the 8 x 27 outputs of the parent's
// octet are then assembled with shuffles:
//   t = (cx,cy,cz) + (kx,ky,kz) + 1 in [1,4]^3, parent tap = t >> 1, child = t & 1
// (the reference's lut_parent / lut_child, octree.py:86-95).
// Each lane writes two consecutive entries (16 bytes) per step; which parent tap / child they
// come from depends only on the lane and the step, and is computed once per thread.
__global__ void __launch_bounds__(256)
neigh_from_parent_kernel(const int64_t* __restrict__ neigh_p, const int32_t* __restrict__ children_p,
                         int64_t nnum_p, int64_t* __restrict__ neigh, int32_t* __restrict__ neigh32) {
  __shared__ int s_p[256], s_j[256], s_wcnt[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // entries o = 2 (32 it + lane) and o + 1 of the octet's 216, it = 0..3
  int kp0[4], kp1[4], ch0[4], ch1[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int o = 2 * (it * 32 + lane) + e;
      const int i = o / 27, k = o - i * 27;
      const int tx = ((i >> 2) & 1) + k / 9 + 1;
      const int ty = ((i >> 1) & 1) + (k / 3) % 3 + 1;
      const int tz = (i & 1) + k % 3 + 1;
      const int kp = o < 216 ? (tx >> 1) * 9 + (ty >> 1) * 3 + (tz >> 1) : 0;
      const int ch = ((tx & 1) << 2) | ((ty & 1) << 1) | (tz & 1);
      if (e == 0) { kp0[it] = kp; ch0[it] = ch; } else { kp1[it] = kp; ch1[it] = ch; }
    }
  }
  const int64_t n_chunks = (nnum_p + 255) / 256;
  for (int64_t chunk = blockIdx.x; chunk < n_chunks; chunk += gridDim.x) {
    const int64_t p_mine = chunk * 256 + threadIdx.x;
    const int j_mine = p_mine < nnum_p ? children_p[p_mine] : -1;
    const unsigned ballot = __ballot_sync(0xffffffffu, j_mine >= 0);
    if (lane == 0) s_wcnt[warp] = __popc(ballot);
    __syncthreads();
    int base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int c = s_wcnt[w];
      if (w < warp) base += c;
      total += c;
    }
    if (j_mine >= 0) {
      const int pos = base + __popc(ballot & ((1u << lane) - 1u));
      s_p[pos] = (int)threadIdx.x;
      s_j[pos] = j_mine;
    }
    __syncthreads();
    // two parents per step, so that their dependent loads overlap
    for (int e = warp; e < total; e += 16) {
      const bool two = e + 8 < total;
      const int64_t pa = chunk * 256 + s_p[e], pb = chunk * 256 + s_p[two ? e + 8 : e];
      const int ja = s_j[e], jb = s_j[two ? e + 8 : e];
      int64_t qa = -1, qb = -1;
      if (lane < 27) {
        qa = neigh_p[pa * 27 + lane];
        qb = neigh_p[pb * 27 + lane];
      }
      const int ca = qa >= 0 ? children_p[qa] : -1;
      const int cb = qb >= 0 ? children_p[qb] : -1;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half == 1 && !two) break;             // warp-uniform
        const int c = half ? cb : ca;
        const int j = half ? jb : ja;
        longlong2* out = reinterpret_cast<longlong2*>(neigh + (int64_t)j * 216);
        int2* out32 = neigh32 ? reinterpret_cast<int2*>(neigh32 + (int64_t)j * 216) : nullptr;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int c0 = __shfl_sync(0xffffffffu, c, kp0[it]);
          const int c1 = __shfl_sync(0xffffffffu, c, kp1[it]);
          const int o2 = it * 32 + lane;          // pair index, valid < 108
          if (o2 < 108) {
            const int64_t v0 = c0 < 0 ? -1 : (int64_t)c0 * 8 + ch0[it];
            const int64_t v1 = c1 < 0 ? -1 : (int64_t)c1 * 8 + ch1[it];
            out[o2] = make_longlong2(v0, v1);
            if (out32) out32[o2] = make_int2((int)v0, (int)v1);
          }
        }
      }
    }
    __syncthreads();     // the lists are rewritten by the next chunk
  }
}

// masks[r] = bit k set iff table[r, taps[k]] >= 0
template <typename I>
__global__ void tap_mask_kernel(const I* __restrict__ table, int table_cols, TapList taps, int K, int64_t n_rows,
                                int32_t* __restrict__ masks) {
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < n_rows; r += (int64_t)gridDim.x * blockDim.x) {
    const I* row = table + r * table_cols;
    uint32_t m = 0;
    for (int k = 0; k < K; ++k) m |= (row[taps.t[k]] >= 0 ? 1u : 0u) << k;
    masks[r] = (int32_t)m;
  }
}

struct NemptyFlag {
  const int32_t* children;
  __device__ int operator()(int64_t i, int64_t) const { return children[i] >= 0 ? 1 : 0; }
};
struct NemptySink {
  int64_t* index;
  __device__ void operator()(int64_t i, int64_t, int flag, int ex) const {
    if (flag) index[ex] = i;
  }
};

template <typename O>
__global__ void neigh_variant_kernel(const int64_t* __restrict__ neigh,
                                     const int32_t* __restrict__ children,
                                     const int64_t* __restrict__ rows, int64_t row_stride,
                                     int64_t n_rows, TapList taps, int K, O* __restrict__ out) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_rows * K;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / K;
    const int k = (int)(t - r * K);
    const int64_t row = rows ? rows[r] : r * row_stride;
    int64_t e = neigh[row * 27 + taps.t[k]];
    if (children && e >= 0) e = (int64_t)children[e];
    out[t] = (O)e;
  }
}

template <typename I>
__global__ void neigh_inverse_kernel(const I* __restrict__ table, int64_t n_rows, int table_cols,
                                     TapList taps, int K, int32_t* __restrict__ inv) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < n_rows * K;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = t / K;
    const int k = (int)(t - r * K);
    const int64_t e = (int64_t)table[r * table_cols + taps.t[k]];
    // For a fixed tap the map row -> neighbour is injective (a fixed spatial
    // offset), so every (target, tap) slot has at most one writer.
    if (e >= 0) inv[e * K + k] = (int32_t)r;
  }
}

__global__ void fill_i32_kernel2(int32_t* __restrict__ p, int64_t n, int32_t v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// offsets[b] = first row whose batch id (key >> 48) is >= b; rank within the
// non-empty rows when children != NULL (prefix count of children >= 0).
__global__ void batch_lower_bound_kernel(const int64_t* __restrict__ keys, int64_t nnum, int batch,
                                         int64_t* __restrict__ offs) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b > batch) return;
  int64_t lo = 0, hi = nnum;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if ((keys[mid] >> 48) < b) lo = mid + 1; else hi = mid;
  }
  offs[b] = lo;
}

struct OffsetSink {
  const int64_t* keys;
  int64_t* offs_ne;
  int batch;
  __device__ void operator()(int64_t i, int64_t n, int flag, int ex) const {
    // Row i opens every batch id in (id of row i-1, id of row i].
    const int64_t bi = keys[i] >> 48;
    const int64_t bp = i > 0 ? (keys[i - 1] >> 48) : -1;
    for (int64_t b = bp + 1; b <= bi && b <= batch; ++b) offs_ne[b] = ex;
    if (i == n - 1)
      for (int64_t b = bi + 1; b <= batch; ++b) offs_ne[b] = ex + flag;
  }
};

static inline unsigned grid1d(int64_t n, int threads = 256) {
  int64_t blocks = cdiv(n, threads);
  int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace oc

using namespace oc;

extern "C" int oc_neigh_full(int depth, int batch_size, int64_t* neigh, void* stream) {
  OC_REQUIRE(depth >= 0 && depth <= 9 && batch_size >= 1, OC_EINVAL, "oc_neigh_full: bad depth/batch");
  const int64_t n_local = 1LL << (3 * depth);
  const int64_t total = n_local * batch_size;
  OC_REQUIRE(total < (1LL << 31), OC_EINVAL, "oc_neigh_full: layer too large");
  OC_REQUIRE(neigh, OC_EINVAL, "oc_neigh_full: null output");
  neigh_full_kernel<<<grid1d(total * 27), 256, 0, (cudaStream_t)stream>>>(depth, n_local, total, neigh);
  OC_LAUNCH_OK("neigh_full_kernel");
  return OC_OK;
}

extern "C" int oc_neigh_from_parent(const int64_t* neigh_p, const int32_t* children_p,
                                    int64_t nnum_p, int64_t* neigh, int32_t* neigh32, void* stream) {
  OC_REQUIRE(nnum_p >= 0, OC_EINVAL, "oc_neigh_from_parent: negative size");
  if (nnum_p == 0) return OC_OK;
  OC_REQUIRE(neigh_p && children_p && neigh, OC_EINVAL, "oc_neigh_from_parent: null pointer");
  int64_t blocks = cdiv(nnum_p, 256);            // chunks of 256 parents
  const int64_t cap = (int64_t)sm_count() * 8;   // 8 resident blocks of 256 threads per SM
  if (blocks > cap) blocks = cap;
  neigh_from_parent_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(neigh_p, children_p, nnum_p, neigh, neigh32);
  OC_LAUNCH_OK("neigh_from_parent_kernel");
  return OC_OK;
}

extern "C" int oc_tap_masks(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                            int64_t n_rows, int32_t* masks, void* stream) {
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "oc_tap_masks: idx_bytes must be 4 or 8");
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27 && K >= 1 && K <= OC_MAX_TAPS && n_rows >= 0, OC_EINVAL,
             "oc_tap_masks: bad sizes");
  TapList taps;
  int rc = make_taps(h_taps, K, table_cols, &taps, "oc_tap_masks");
  if (rc) return rc;
  if (n_rows == 0) return OC_OK;
  OC_REQUIRE(table && masks, OC_EINVAL, "oc_tap_masks: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (idx_bytes == 8)
    tap_mask_kernel<int64_t><<<grid1d(n_rows), 256, 0, s>>>((const int64_t*)table, table_cols, taps, K, n_rows, masks);
  else
    tap_mask_kernel<int32_t><<<grid1d(n_rows), 256, 0, s>>>((const int32_t*)table, table_cols, taps, K, n_rows, masks);
  OC_LAUNCH_OK("tap_mask_kernel");
  return OC_OK;
}

extern "C" size_t oc_nempty_index_workspace_bytes(int64_t nnum) {
  return scan_workspace_bytes(nnum > 0 ? nnum : 1);
}

extern "C" int oc_nempty_index(const int32_t* children, int64_t nnum, int64_t* index,
                               void* workspace, size_t workspace_bytes, void* stream) {
  OC_REQUIRE(nnum >= 0, OC_EINVAL, "oc_nempty_index: negative size");
  if (nnum == 0) return OC_OK;
  OC_REQUIRE(children && index && workspace, OC_EINVAL, "oc_nempty_index: null pointer");
  OC_REQUIRE(workspace_bytes >= scan_workspace_bytes(nnum), OC_ENOMEM, "oc_nempty_index: workspace too small");
  OC_CUDA_OK(device_scan(NemptyFlag{children}, NemptySink{index}, nnum, nullptr, (int32_t*)workspace,
                         nullptr, (cudaStream_t)stream));
  return OC_OK;
}

extern "C" int oc_neigh_variant(const int64_t* neigh, const int32_t* children, const int64_t* rows,
                                int64_t row_stride, int64_t n_rows, const int* h_taps, int K,
                                void* out, int out_bytes, void* stream) {
  TapList taps;
  int rc = make_taps(h_taps, K, 27, &taps, "oc_neigh_variant");
  if (rc) return rc;
  OC_REQUIRE(n_rows >= 0, OC_EINVAL, "oc_neigh_variant: negative rows");
  OC_REQUIRE(out_bytes == 8 || out_bytes == 4, OC_EINVAL, "oc_neigh_variant: out_bytes must be 4 or 8");
  if (n_rows == 0) return OC_OK;
  OC_REQUIRE(neigh && out, OC_EINVAL, "oc_neigh_variant: null pointer");
  const unsigned g = grid1d(n_rows * K);
  if (out_bytes == 8)
    neigh_variant_kernel<int64_t><<<g, 256, 0, (cudaStream_t)stream>>>(neigh, children, rows, row_stride, n_rows, taps, K, (int64_t*)out);
  else
    neigh_variant_kernel<int32_t><<<g, 256, 0, (cudaStream_t)stream>>>(neigh, children, rows, row_stride, n_rows, taps, K, (int32_t*)out);
  OC_LAUNCH_OK("neigh_variant_kernel");
  return OC_OK;
}

extern "C" int oc_neigh_inverse(const void* table, int idx_bytes, int64_t n_rows, int table_cols,
                                const int* h_taps, int K, int64_t n_targets, int32_t* inv,
                                void* stream) {
  TapList taps;
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "oc_neigh_inverse: bad table_cols");
  int rc = make_taps(h_taps, K, table_cols, &taps, "oc_neigh_inverse");
  if (rc) return rc;
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "oc_neigh_inverse: idx_bytes must be 4 or 8");
  OC_REQUIRE(n_rows >= 0 && n_targets >= 0, OC_EINVAL, "oc_neigh_inverse: negative size");
  OC_REQUIRE(n_rows < (1LL << 31), OC_EINVAL, "oc_neigh_inverse: too many rows for int32");
  if (n_targets == 0) return OC_OK;
  OC_REQUIRE(inv, OC_EINVAL, "oc_neigh_inverse: null output");
  cudaStream_t s = (cudaStream_t)stream;
  fill_i32_kernel2<<<grid1d(n_targets * K), 256, 0, s>>>(inv, n_targets * K, -1);
  if (n_rows > 0) {
    OC_REQUIRE(table, OC_EINVAL, "oc_neigh_inverse: null table");
    const unsigned g = grid1d(n_rows * K);
    if (idx_bytes == 8)
      neigh_inverse_kernel<int64_t><<<g, 256, 0, s>>>((const int64_t*)table, n_rows, table_cols, taps, K, inv);
    else
      neigh_inverse_kernel<int32_t><<<g, 256, 0, s>>>((const int32_t*)table, n_rows, table_cols, taps, K, inv);
  }
  OC_LAUNCH_OK("neigh_inverse_kernel");
  return OC_OK;
}

extern "C" int oc_batch_offsets(const int64_t* keys, const int32_t* children, int64_t nnum,
                                int batch, int64_t* h_offsets, void* workspace,
                                size_t workspace_bytes, void* stream) {
  OC_REQUIRE(batch >= 1 && batch < 32768, OC_EINVAL, "oc_batch_offsets: bad batch");
  OC_REQUIRE(nnum >= 1 && keys && h_offsets && workspace, OC_EINVAL, "oc_batch_offsets: bad argument");
  const size_t need = align_up((size_t)(batch + 1) * 8, 256) * 2 + scan_workspace_bytes(nnum);
  OC_REQUIRE(workspace_bytes >= need, OC_ENOMEM, "oc_batch_offsets: workspace %zu < %zu", workspace_bytes, need);
  cudaStream_t s = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  int64_t* offs = (int64_t*)ws;
  int64_t* offs_ne = (int64_t*)(ws + align_up((size_t)(batch + 1) * 8, 256));
  int32_t* scan_tmp = (int32_t*)(ws + 2 * align_up((size_t)(batch + 1) * 8, 256));
  batch_lower_bound_kernel<<<(unsigned)cdiv(batch + 1, 128), 128, 0, s>>>(keys, nnum, batch, offs);
  OC_LAUNCH_OK("batch_lower_bound_kernel");
  const int64_t* src = offs;
  if (children) {
    OC_CUDA_OK(device_scan(NemptyFlag{children}, OffsetSink{keys, offs_ne, batch}, nnum, nullptr,
                           scan_tmp, nullptr, s));
    src = offs_ne;
  }
  OC_CUDA_OK(cudaMemcpyAsync(h_offsets, src, (size_t)(batch + 1) * 8, cudaMemcpyDeviceToHost, s));
  OC_CUDA_OK(cudaStreamSynchronize(s));
  return OC_OK;
}
