// Octree construction on the device.
//
// Restates Octree.build_octree (ocnn/octree/octree.py:201-287) as a fixed
// sequence of streaming kernels with a single device->host read of the node
// counts:
//   1. keygen     : scale points, truncate, interleave -> "compact" keys
//                   (batch << 3*depth | morton), identity permutation
//   2. radix sort : stable LSD sort over the live key bits only
//   3. unique     : head flags + scan -> leaf keys, leaf starts, point->leaf rank
//   4. per depth  : parent = key >> 3, head flags + scan -> parent keys, parent rank
//   5. emit       : keys / children of every depth, averaged leaf signals
// Compact keys make the parent of a node `key >> 3` for every batch element and
// the node index inside a dense layer the key itself.
#include "oc_common.cuh"

namespace oc {

// ---------------------------------------------------------------------------
// Workspace layout
// ---------------------------------------------------------------------------
constexpr int SORT_WARPS = 8;
constexpr int SORT_THREADS = SORT_WARPS * 32;
constexpr int SORT_ITEMS = 8;                       // keys per thread
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;  // keys per block
constexpr int RADIX_BITS = 8;
constexpr int RADIX = 1 << RADIX_BITS;

struct BuildLayout {
  size_t key_a, key_b, val_a, val_b, hist, scan_tmp, leaf_rank, leaf_start, counts;
  size_t level_keys;  // (depth - full_depth + 1) arrays of npts u64, index 0 = depth
  size_t level_pidx;  // (depth - full_depth) arrays of npts i32, index 0 = depth
  size_t level_first; // (depth - full_depth) arrays of npts + 1 i32: first node of every parent, index 0 = depth
  size_t total;
  int64_t sort_blocks;
};

static BuildLayout build_layout(int64_t npts, int depth, int full_depth) {
  BuildLayout L;
  const size_t P = (size_t)(npts > 0 ? npts : 1);
  size_t off = 0;
  auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
  L.sort_blocks = cdiv((int64_t)P, SORT_TILE);
  L.key_a = take(P * 8);
  L.key_b = take(P * 8);
  L.val_a = take(P * 4);
  L.val_b = take(P * 4);
  L.hist = take((size_t)RADIX * L.sort_blocks * 4);
  size_t scan_n = (size_t)RADIX * L.sort_blocks;
  if (scan_n < P) scan_n = P;
  L.scan_tmp = take(scan_workspace_bytes((int64_t)scan_n));
  L.leaf_rank = take(P * 4);
  L.leaf_start = take((P + 1) * 4);
  L.counts = take(32 * 8);
  const int nlev = depth - full_depth + 1;
  L.level_keys = take((size_t)nlev * P * 8);
  L.level_pidx = take((size_t)(nlev > 1 ? nlev - 1 : 1) * P * 4);
  L.level_first = take((size_t)(nlev > 1 ? nlev - 1 : 1) * (P + 1) * 4);
  L.total = off;
  return L;
}

// ---------------------------------------------------------------------------
// 1. key generation
// ---------------------------------------------------------------------------
template <typename B>
__global__ void keygen_kernel(const float* __restrict__ pts, const B* __restrict__ bid,
                              int64_t n, int depth, float bx, float by, float bz, float mul,
                              uint64_t* __restrict__ key, uint32_t* __restrict__ val) {
  const uint64_t mask = (1ULL << depth) - 1ULL;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    // (p - bbmin) * mul with two separate fp32 roundings (no FMA contraction),
    // matching Points.normalize (ocnn/octree/points.py:241).
    const float fx = __fmul_rn(__fsub_rn(pts[3 * i + 0], bx), mul);
    const float fy = __fmul_rn(__fsub_rn(pts[3 * i + 1], by), mul);
    const float fz = __fmul_rn(__fsub_rn(pts[3 * i + 2], bz), mul);
    const uint64_t xi = (uint64_t)(long long)fx & mask;
    const uint64_t yi = (uint64_t)(long long)fy & mask;
    const uint64_t zi = (uint64_t)(long long)fz & mask;
    uint64_t k = morton3(xi, yi, zi);
    if (bid) k |= ((uint64_t)(long long)bid[i]) << (3 * depth);
    key[i] = k;
    val[i] = (uint32_t)i;
  }
}

// ---------------------------------------------------------------------------
// 2. stable LSD radix sort, 8 bits per pass
// ---------------------------------------------------------------------------
// Each block owns a contiguous tile; each warp a contiguous slice of the tile;
// a warp walks its slice 32 keys at a time, so "earlier" always means lower
// (warp, round, lane) and ranks can be made stable with match_any + popc.
__device__ __forceinline__ void warp_digit_count(int* hist_row, int digit, bool valid) {
  const unsigned peers = __match_any_sync(0xffffffffu, valid ? digit : RADIX);
  const int lane = threadIdx.x & 31;
  if (valid && (__ffs(peers) - 1) == lane) hist_row[digit] += __popc(peers);
  __syncwarp();
}

__global__ void __launch_bounds__(SORT_THREADS)
radix_hist_kernel(const uint64_t* __restrict__ key, int64_t n, int shift,
                  uint32_t* __restrict__ hist, int64_t nblocks) {
  __shared__ int wh[SORT_WARPS][RADIX];
  for (int i = threadIdx.x; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&wh[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t base = (int64_t)blockIdx.x * SORT_TILE + (int64_t)warp * (32 * SORT_ITEMS);
#pragma unroll
  for (int r = 0; r < SORT_ITEMS; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool valid = i < n;
    const int d = valid ? (int)((key[i] >> shift) & (RADIX - 1)) : 0;
    warp_digit_count(wh[warp], d, valid);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < RADIX; d += SORT_THREADS) {
    int s = 0;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) s += wh[w][d];
    hist[(int64_t)d * nblocks + blockIdx.x] = (uint32_t)s;
  }
}

// Scatter pass.  The block first orders its own tile by digit in shared memory (stable: warp,
// round, lane), then copies it out position by position: position j of the ordered tile, digit
// d, goes to (start of the block's run of digit d in the output) + (j - start of digit d in the
// tile), so consecutive threads write consecutive addresses within a run instead of 256 scattered
// buckets per warp.
__global__ void __launch_bounds__(SORT_THREADS)
radix_scatter_kernel(const uint64_t* __restrict__ key_in, const uint32_t* __restrict__ val_in,
                     int64_t n, int shift, const uint32_t* __restrict__ hist_scanned,
                     int64_t nblocks, uint64_t* __restrict__ key_out,
                     uint32_t* __restrict__ val_out) {
  __shared__ int wh[SORT_WARPS][RADIX];
  __shared__ int64_t gdelta[RADIX];            // output position of tile position j with digit d = gdelta[d] + j
  __shared__ int wsum[SORT_WARPS];
  __shared__ uint64_t skey[SORT_TILE];
  __shared__ uint32_t sval[SORT_TILE];
  static_assert(RADIX == SORT_THREADS, "one thread per digit in the offset step");
  for (int i = threadIdx.x; i < SORT_WARPS * RADIX; i += SORT_THREADS) (&wh[0][0])[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tile0 = (int64_t)blockIdx.x * SORT_TILE;
  const int64_t base = tile0 + (int64_t)warp * (32 * SORT_ITEMS);
  uint64_t k[SORT_ITEMS];
#pragma unroll
  for (int r = 0; r < SORT_ITEMS; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool valid = i < n;
    k[r] = valid ? key_in[i] : 0;
    warp_digit_count(wh[warp], (int)((k[r] >> shift) & (RADIX - 1)), valid);
  }
  __syncthreads();
  {
    // thread d: the tile's count of digit d, its exclusive prefix over the digits (start of digit d in
    // the ordered tile), then the start of every warp's share
    const int d = threadIdx.x;
    int total = 0;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) total += wh[w][d];
    int incl = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    int before = 0;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) before += w < warp ? wsum[w] : 0;
    int run = before + incl - total;             // start of digit d in the ordered tile
    gdelta[d] = (int64_t)hist_scanned[(int64_t)d * nblocks + blockIdx.x] - run;
#pragma unroll
    for (int w = 0; w < SORT_WARPS; ++w) {
      const int c = wh[w][d];
      wh[w][d] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < SORT_ITEMS; ++r) {
    const int64_t i = base + r * 32 + lane;
    const bool valid = i < n;
    const int d = (int)((k[r] >> shift) & (RADIX - 1));
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? d : RADIX);
    if (valid) {
      const int pos = wh[warp][d] + __popc(peers & ((1u << lane) - 1u));
      skey[pos] = k[r];
      sval[pos] = val_in[i];
    }
    __syncwarp();
    if (valid && (__ffs(peers) - 1) == lane) wh[warp][d] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  const int64_t left = n - tile0;
  const int cnt = (int)(left < SORT_TILE ? left : SORT_TILE);
  for (int j = threadIdx.x; j < cnt; j += SORT_THREADS) {
    const uint64_t kk = skey[j];
    const int64_t pos = gdelta[(int)((kk >> shift) & (RADIX - 1))] + j;
    key_out[pos] = kk;
    val_out[pos] = sval[j];
  }
}

struct HistFlag {
  const uint32_t* h;
  __device__ int operator()(int64_t i, int64_t) const { return (int)h[i]; }
};
struct HistSink {
  uint32_t* h;
  __device__ void operator()(int64_t i, int64_t, int, int ex) const { h[i] = (uint32_t)ex; }
};

// ---------------------------------------------------------------------------
// 3./4. unique via head flags + scan
// ---------------------------------------------------------------------------
struct LeafHead {
  const uint64_t* key;
  __device__ int operator()(int64_t i, int64_t) const { return (i == 0 || key[i] != key[i - 1]) ? 1 : 0; }
};
struct LeafSink {
  const uint64_t* key;
  uint64_t* uniq;
  int32_t* rank;
  int32_t* start;
  __device__ void operator()(int64_t i, int64_t n, int flag, int ex) const {
    const int r = ex + flag - 1;
    rank[i] = r;
    if (flag) { uniq[r] = key[i]; start[r] = (int32_t)i; }
    if (i == n - 1) start[r + 1] = (int32_t)n;
  }
};
struct ParentHead {
  const uint64_t* key;
  __device__ int operator()(int64_t i, int64_t) const {
    return (i == 0 || (key[i] >> 3) != (key[i - 1] >> 3)) ? 1 : 0;
  }
};
struct ParentSink {
  const uint64_t* key;
  uint64_t* pkey;
  int32_t* pidx;
  int32_t* pfirst;   // pfirst[r] = first node of parent r, pfirst[#parents] = n
  __device__ void operator()(int64_t i, int64_t n, int flag, int ex) const {
    const int r = ex + flag - 1;
    pidx[i] = r;
    if (flag) { pkey[r] = key[i] >> 3; pfirst[r] = (int32_t)i; }
    if (i == n - 1) pfirst[r + 1] = (int32_t)n;
  }
};

// ---------------------------------------------------------------------------
// 5. emit
// ---------------------------------------------------------------------------
__device__ __forceinline__ int64_t expand_key(uint64_t ck, int depth) {
  const uint64_t m = ck & ((1ULL << (3 * depth)) - 1ULL);
  const uint64_t b = ck >> (3 * depth);
  return (int64_t)((b << 48) | m);
}

__global__ void full_layer_kernel(int depth, int64_t n, int64_t* __restrict__ keys,
                                  int32_t* __restrict__ children) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    if (keys) keys[i] = expand_key((uint64_t)i, depth);
    if (children) children[i] = (int32_t)i;
  }
}

__global__ void fill_i32_kernel(int32_t* __restrict__ p, int64_t n, int32_t v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// children of the deepest dense layer: node index == compact key
__global__ void full_children_kernel(const uint64_t* __restrict__ lk, int64_t n,
                                     int32_t* __restrict__ children) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    children[lk[i]] = (int32_t)i;
}

// A sparse layer in one pass: node t is child (t & 7) of the (t >> 3)-th non-empty parent; its
// key follows from the parent's key, and it is non-empty if one of the parent's (at most 8,
// key-sorted) nodes lk[first[p] .. first[p+1]) has that child index - its rank is the position.
__global__ void level_emit_kernel(const uint64_t* __restrict__ pkeys, const uint64_t* __restrict__ lk,
                                  const int32_t* __restrict__ first, int64_t nnum, int depth,
                                  int64_t* __restrict__ keys, int32_t* __restrict__ children) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nnum;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = t >> 3;
    const uint64_t c = (uint64_t)(t & 7);
    keys[t] = expand_key((pkeys[p] << 3) | c, depth);
    int32_t child = -1;
    const int32_t e = first[p + 1];
    for (int32_t i = first[p]; i < e; ++i)
      if ((lk[i] & 7) == c) child = i;
    children[t] = child;
  }
}

__global__ void point_rank_kernel(const uint32_t* __restrict__ perm,
                                  const int32_t* __restrict__ rank, int64_t n,
                                  int64_t* __restrict__ idx) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    idx[perm[i]] = (int64_t)rank[i];
}

// One thread per leaf; points of a leaf are consecutive in the sorted order and,
// because the sort is stable, in their original order — the same summation order
// as a sequential scatter_add, so the result does not vary run to run.
__global__ void leaf_average_kernel(const float* __restrict__ pts, const float* __restrict__ nrm,
                                    const float* __restrict__ feat, int nfeat,
                                    const uint32_t* __restrict__ perm,
                                    const int32_t* __restrict__ start, int64_t nleaf, float bx,
                                    float by, float bz, float mul, float* __restrict__ out_pts,
                                    float* __restrict__ out_nrm, float* __restrict__ out_feat) {
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < nleaf;
       r += (int64_t)gridDim.x * blockDim.x) {
    const int s = start[r], e = start[r + 1];
    const float cnt = (float)(e - s);
    if (out_pts) {
      float ax = 0.f, ay = 0.f, az = 0.f;
      for (int j = s; j < e; ++j) {
        const int64_t p = perm[j];
        ax = __fadd_rn(ax, __fmul_rn(__fsub_rn(pts[3 * p + 0], bx), mul));
        ay = __fadd_rn(ay, __fmul_rn(__fsub_rn(pts[3 * p + 1], by), mul));
        az = __fadd_rn(az, __fmul_rn(__fsub_rn(pts[3 * p + 2], bz), mul));
      }
      out_pts[3 * r + 0] = __fdiv_rn(ax, cnt);
      out_pts[3 * r + 1] = __fdiv_rn(ay, cnt);
      out_pts[3 * r + 2] = __fdiv_rn(az, cnt);
    }
    if (out_nrm) {
      float ax = 0.f, ay = 0.f, az = 0.f;
      for (int j = s; j < e; ++j) {
        const int64_t p = perm[j];
        ax = __fadd_rn(ax, nrm[3 * p + 0]);
        ay = __fadd_rn(ay, nrm[3 * p + 1]);
        az = __fadd_rn(az, nrm[3 * p + 2]);
      }
      // F.normalize: v / max(||v||_2, 1e-12)
      float nn = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(ax, ax), __fmul_rn(ay, ay)), __fmul_rn(az, az)));
      nn = fmaxf(nn, 1e-12f);
      out_nrm[3 * r + 0] = __fdiv_rn(ax, nn);
      out_nrm[3 * r + 1] = __fdiv_rn(ay, nn);
      out_nrm[3 * r + 2] = __fdiv_rn(az, nn);
    }
    if (out_feat) {
      for (int c = 0; c < nfeat; ++c) {
        float a = 0.f;
        for (int j = s; j < e; ++j) a = __fadd_rn(a, feat[(int64_t)perm[j] * nfeat + c]);
        out_feat[r * nfeat + c] = __fdiv_rn(a, cnt);
      }
    }
  }
}

__global__ void grow_layer_kernel(const int64_t* __restrict__ keys_p,
                                  const int32_t* __restrict__ children_p, int64_t nnum_p,
                                  int64_t* __restrict__ keys, int32_t* __restrict__ children) {
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nnum_p * 8;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = t >> 3;
    const int c = children_p[p];
    if (c < 0) continue;
    const int64_t kp = keys_p[p];
    const int64_t b = (kp >> 48) << 48;
    const int64_t k = ((kp & ((1LL << 48) - 1)) << 3) | b;
    const int64_t o = ((int64_t)c << 3) | (t & 7);
    keys[o] = k + (t & 7);
    children[o] = (int32_t)o;
  }
}

static inline unsigned grid1d(int64_t n, int threads = 256) {
  int64_t blocks = cdiv(n, threads);
  int64_t cap = (int64_t)sm_count() * 16;
  return (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

}  // namespace oc

using namespace oc;

extern "C" size_t oc_build_workspace_bytes(int64_t npts, int depth, int full_depth, int batch_size) {
  (void)batch_size;
  if (depth < 1 || depth > 16 || full_depth < 0 || full_depth > depth) return 0;
  return build_layout(npts, depth, full_depth).total;
}

extern "C" int oc_build_octree_count(const float* points, const void* batch_id, int bid_dtype,
                                     int64_t npts, int depth, int full_depth, int batch_size,
                                     const float* h_bbmin3, float mul, void* workspace,
                                     size_t workspace_bytes, int64_t* h_nnum_nempty, void* stream) {
  OC_REQUIRE(depth >= 1 && depth <= 16, OC_EINVAL, "build: depth %d not in [1,16]", depth);
  OC_REQUIRE(full_depth >= 0 && full_depth <= depth, OC_EINVAL,
             "build: full_depth %d not in [0,depth]", full_depth);
  OC_REQUIRE(batch_size >= 1 && batch_size < 32768, OC_EINVAL, "build: bad batch_size %d", batch_size);
  OC_REQUIRE(npts >= 1 && npts < (1LL << 31), OC_EINVAL, "build: npts %lld not in [1, 2^31)", (long long)npts);
  OC_REQUIRE(points && h_bbmin3 && workspace && h_nnum_nempty, OC_EINVAL, "build: null pointer");
  OC_REQUIRE(batch_size == 1 || batch_id, OC_EINVAL, "build: batch_id required when batch_size > 1");
  int bbits = 0;
  while ((1 << bbits) < batch_size) ++bbits;
  OC_REQUIRE(3 * depth + bbits <= 63, OC_EINVAL, "build: key does not fit in 63 bits");
  OC_REQUIRE((int64_t)batch_size << (3 * full_depth) < (1LL << 31), OC_EINVAL,
             "build: dense layer too large");
  const BuildLayout L = build_layout(npts, depth, full_depth);
  OC_REQUIRE(workspace_bytes >= L.total, OC_ENOMEM, "build: workspace %zu < %zu bytes",
             workspace_bytes, L.total);
  cudaStream_t s = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  uint64_t* key_a = (uint64_t*)(ws + L.key_a);
  uint64_t* key_b = (uint64_t*)(ws + L.key_b);
  uint32_t* val_a = (uint32_t*)(ws + L.val_a);
  uint32_t* val_b = (uint32_t*)(ws + L.val_b);
  uint32_t* hist = (uint32_t*)(ws + L.hist);
  int32_t* scan_tmp = (int32_t*)(ws + L.scan_tmp);
  int64_t* counts = (int64_t*)(ws + L.counts);

  const float bx = h_bbmin3[0], by = h_bbmin3[1], bz = h_bbmin3[2];
  const unsigned g = grid1d(npts);
  if (!batch_id || batch_size == 1) {
    keygen_kernel<float><<<g, 256, 0, s>>>(points, nullptr, npts, depth, bx, by, bz, mul, key_a, val_a);
  } else if (bid_dtype == OC_COORD_F32) {
    keygen_kernel<float><<<g, 256, 0, s>>>(points, (const float*)batch_id, npts, depth, bx, by, bz, mul, key_a, val_a);
  } else if (bid_dtype == OC_I64) {
    keygen_kernel<int64_t><<<g, 256, 0, s>>>(points, (const int64_t*)batch_id, npts, depth, bx, by, bz, mul, key_a, val_a);
  } else if (bid_dtype == OC_I32) {
    keygen_kernel<int32_t><<<g, 256, 0, s>>>(points, (const int32_t*)batch_id, npts, depth, bx, by, bz, mul, key_a, val_a);
  } else {
    OC_REQUIRE(false, OC_EINVAL, "build: unsupported batch_id dtype %d", bid_dtype);
  }
  OC_LAUNCH_OK("keygen_kernel");

  // LSD radix sort over the live bits only.
  const int live_bits = 3 * depth + (batch_size > 1 ? bbits : 0);
  const int64_t nb = L.sort_blocks;
  uint64_t *kin = key_a, *kout = key_b;
  uint32_t *vin = val_a, *vout = val_b;
  for (int shift = 0; shift < live_bits; shift += RADIX_BITS) {
    radix_hist_kernel<<<(unsigned)nb, SORT_THREADS, 0, s>>>(kin, npts, shift, hist, nb);
    OC_CUDA_OK(device_scan(HistFlag{hist}, HistSink{hist}, (int64_t)RADIX * nb, nullptr, scan_tmp,
                           nullptr, s));
    radix_scatter_kernel<<<(unsigned)nb, SORT_THREADS, 0, s>>>(kin, vin, npts, shift, hist, nb, kout, vout);
    OC_LAUNCH_OK("radix_scatter_kernel");
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  // The emit call must find the sorted permutation without re-deriving the
  // ping-pong parity: keep it in val_a.
  if (vin != val_a) {
    OC_CUDA_OK(cudaMemcpyAsync(val_a, vin, (size_t)npts * 4, cudaMemcpyDeviceToDevice, s));
  }

  uint64_t* lk = (uint64_t*)(ws + L.level_keys);
  int32_t* lp = (int32_t*)(ws + L.level_pidx);
  int32_t* leaf_rank = (int32_t*)(ws + L.leaf_rank);
  int32_t* leaf_start = (int32_t*)(ws + L.leaf_start);
  OC_CUDA_OK(cudaMemsetAsync(counts, 0, 32 * 8, s));
  OC_CUDA_OK(device_scan(LeafHead{kin}, LeafSink{kin, lk, leaf_rank, leaf_start}, npts, nullptr,
                         scan_tmp, counts + depth, s));
  for (int d = depth; d > full_depth; --d) {
    const uint64_t* cur = lk + (size_t)(depth - d) * npts;
    uint64_t* par = lk + (size_t)(depth - d + 1) * npts;
    int32_t* pidx = lp + (size_t)(depth - d) * npts;
    int32_t* pfirst = (int32_t*)(ws + L.level_first) + (size_t)(depth - d) * (npts + 1);
    OC_CUDA_OK(device_scan(ParentHead{cur}, ParentSink{cur, par, pidx, pfirst}, npts, counts + d, scan_tmp,
                           counts + d - 1, s));
  }
  int64_t h_counts[32];
  OC_CUDA_OK(cudaMemcpyAsync(h_counts, counts, 32 * 8, cudaMemcpyDeviceToHost, s));
  OC_CUDA_OK(cudaStreamSynchronize(s));
  for (int d = 0; d <= depth; ++d)
    h_nnum_nempty[d] = d < full_depth ? ((int64_t)batch_size << (3 * d)) : h_counts[d];
  return OC_OK;
}

extern "C" int oc_build_octree_emit(const float* points, const float* normals, const float* features,
                                    int nfeat, int64_t npts, int depth, int full_depth,
                                    int batch_size, const float* h_bbmin3, float mul,
                                    const void* workspace, const int64_t* h_nnum_nempty,
                                    int64_t* const* h_keys, int32_t* const* h_children,
                                    float* out_points, float* out_normals, float* out_features,
                                    int64_t* out_idx, void* stream) {
  OC_REQUIRE(depth >= 1 && depth <= 16 && full_depth >= 0 && full_depth <= depth, OC_EINVAL,
             "emit: bad depth/full_depth");
  OC_REQUIRE(points && workspace && h_nnum_nempty && h_keys && h_children && h_bbmin3, OC_EINVAL,
             "emit: null pointer");
  OC_REQUIRE((out_normals == nullptr) || normals, OC_EINVAL, "emit: normals output without input");
  OC_REQUIRE((out_features == nullptr) || (features && nfeat > 0), OC_EINVAL,
             "emit: features output without input");
  const BuildLayout L = build_layout(npts, depth, full_depth);
  cudaStream_t s = (cudaStream_t)stream;
  const char* ws = (const char*)workspace;
  const uint32_t* perm = (const uint32_t*)(ws + L.val_a);
  const uint64_t* lk = (const uint64_t*)(ws + L.level_keys);
  const int32_t* lf = (const int32_t*)(ws + L.level_first);
  const int32_t* leaf_rank = (const int32_t*)(ws + L.leaf_rank);
  const int32_t* leaf_start = (const int32_t*)(ws + L.leaf_start);

  for (int d = 0; d <= full_depth; ++d) {
    const int64_t n = (int64_t)batch_size << (3 * d);
    OC_REQUIRE(h_keys[d] && h_children[d], OC_EINVAL, "emit: null output at depth %d", d);
    full_layer_kernel<<<grid1d(n), 256, 0, s>>>(d, n, h_keys[d], d < full_depth ? h_children[d] : nullptr);
  }
  {
    const int d = full_depth;
    const int64_t n = (int64_t)batch_size << (3 * d);
    fill_i32_kernel<<<grid1d(n), 256, 0, s>>>(h_children[d], n, -1);
    const int64_t nne = h_nnum_nempty[d];
    full_children_kernel<<<grid1d(nne), 256, 0, s>>>(lk + (size_t)(depth - d) * npts, nne, h_children[d]);
  }
  for (int d = full_depth + 1; d <= depth; ++d) {
    const int64_t nnum = 8 * h_nnum_nempty[d - 1];
    const int64_t nne = h_nnum_nempty[d];
    OC_REQUIRE(h_keys[d] && h_children[d], OC_EINVAL, "emit: null output at depth %d", d);
    (void)nne;
    level_emit_kernel<<<grid1d(nnum), 256, 0, s>>>(lk + (size_t)(depth - d + 1) * npts, lk + (size_t)(depth - d) * npts,
                                                   lf + (size_t)(depth - d) * (npts + 1), nnum, d, h_keys[d],
                                                   h_children[d]);
  }
  OC_LAUNCH_OK("octree emit kernels");
  if (out_idx) point_rank_kernel<<<grid1d(npts), 256, 0, s>>>(perm, leaf_rank, npts, out_idx);
  if (out_points || out_normals || out_features) {
    const int64_t nleaf = h_nnum_nempty[depth];
    leaf_average_kernel<<<grid1d(nleaf, 128), 128, 0, s>>>(
        points, normals, features, nfeat, perm, leaf_start, nleaf, h_bbmin3[0], h_bbmin3[1],
        h_bbmin3[2], mul, out_points, out_normals, out_features);
  }
  OC_LAUNCH_OK("octree signal kernels");
  return OC_OK;
}

// ---------------------------------------------------------------------------
// Row order by tap mask: rows of a neighbour table sorted (stably) by the bit mask of
// their valid taps, with the radix sort of the octree build (mask = key, row = value).
// ---------------------------------------------------------------------------
extern "C" int oc_tap_masks(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                            int64_t n_rows, int32_t* masks, void* stream);

namespace oc {
struct OrderLayout {
  size_t key_a, key_b, val_a, val_b, masks, hist, scan_tmp, counts, bitpos, total;
  int64_t sort_blocks;
};
static OrderLayout order_layout(int64_t n) {
  OrderLayout L;
  size_t off = 0;
  auto take = [&](size_t b) { size_t o = off; off += align_up(b, 256); return o; };
  const int64_t m = n > 0 ? n : 1;
  L.sort_blocks = cdiv(m, SORT_TILE);
  L.key_a = take((size_t)m * 8);
  L.key_b = take((size_t)m * 8);
  L.val_a = take((size_t)m * 4);
  L.val_b = take((size_t)m * 4);
  L.masks = take((size_t)m * 4);
  L.hist = take((size_t)RADIX * L.sort_blocks * 4);
  L.scan_tmp = take(scan_workspace_bytes((int64_t)RADIX * L.sort_blocks));
  L.counts = take(32 * sizeof(unsigned long long));
  L.bitpos = take(32 * sizeof(int));
  L.total = off;
  return L;
}
// counts[k] = rows whose mask has bit k: lane k of every warp keeps the count of bit k
__global__ void tap_count_kernel(const int32_t* __restrict__ masks, int64_t n, unsigned long long* __restrict__ counts) {
  const int lane = threadIdx.x & 31;
  unsigned long long mine = 0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t n_round = (n + 31) / 32 * 32;                       // whole warps take part in the ballots
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_round; i += stride) {
    const uint32_t m = i < n ? (uint32_t)masks[i] : 0u;
#pragma unroll
    for (int k = 0; k < OC_MAX_TAPS; ++k) {
      const unsigned b = __ballot_sync(0xffffffffu, (m >> k) & 1u);
      if (lane == k) mine += __popc(b);
    }
  }
  if (lane < OC_MAX_TAPS && mine) atomicAdd(&counts[lane], mine);
}

// Bit position of every tap in the sort key: the taps whose frequency is farthest from one half
// take the most significant bits (ties: the lower tap is more significant).  Rows that hold a
// rare tap then sit together and the other tiles skip it; the taps that about half of the rows
// have vary inside a tile, where they waste least.
__global__ void tap_bitpos_kernel(const unsigned long long* __restrict__ counts, int64_t n, int K, int* __restrict__ bitpos) {
  const int t = threadIdx.x;
  if (t >= K) return;
  auto score = [&](int k) { const long long d = 2 * (long long)counts[k] - (long long)n; return d < 0 ? -d : d; };
  const long long mine = score(t);
  int rank = 0;                                      // taps that are more significant than t
  for (int k = 0; k < K; ++k) {
    const long long o = score(k);
    rank += (o > mine || (o == mine && k < t)) ? 1 : 0;
  }
  bitpos[t] = K - 1 - rank;
}

__global__ void mask_key_kernel(const int32_t* __restrict__ masks, int64_t n, int K, int chunk_shift,
                                const int* __restrict__ bitpos, uint64_t* __restrict__ key,
                                uint32_t* __restrict__ val) {
  __shared__ int spos[OC_MAX_TAPS];
  if (threadIdx.x < OC_MAX_TAPS) spos[threadIdx.x] = threadIdx.x < K ? bitpos[threadIdx.x] : 0;
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    // grid1d caps the grid: a grid-stride loop.  Key = (chunk of the row, mask with its bits reordered).
    const uint32_t m = (uint32_t)masks[i];
    uint32_t pm = 0;
    for (int k = 0; k < K; ++k) pm |= ((m >> k) & 1u) << spos[k];
    key[i] = ((uint64_t)(i >> chunk_shift) << K) | (uint64_t)pm;
    val[i] = (uint32_t)i;
  }
}
}  // namespace oc

extern "C" size_t oc_tap_order_workspace_bytes(int64_t n_rows) { return oc::order_layout(n_rows).total; }

extern "C" int oc_tap_order(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                            int64_t n_rows, int chunk_log2, int32_t* perm, void* workspace, size_t workspace_bytes,
                            void* stream) {
  using namespace oc;
  cudaStream_t s = (cudaStream_t)stream;
  OC_REQUIRE(n_rows >= 0 && n_rows < INT32_MAX, OC_EINVAL, "tap_order: n_rows %lld", (long long)n_rows);
  if (n_rows == 0) return OC_OK;
  const OrderLayout L = order_layout(n_rows);
  OC_REQUIRE(perm && workspace && workspace_bytes >= L.total, OC_ENOMEM, "tap_order: workspace %zu < %zu",
             workspace_bytes, L.total);
  uint8_t* ws = (uint8_t*)workspace;
  uint64_t *kin = (uint64_t*)(ws + L.key_a), *kout = (uint64_t*)(ws + L.key_b);
  uint32_t *vin = (uint32_t*)(ws + L.val_a), *vout = (uint32_t*)(ws + L.val_b);
  int32_t* masks = (int32_t*)(ws + L.masks);
  uint32_t* hist = (uint32_t*)(ws + L.hist);
  int32_t* scan_tmp = (int32_t*)(ws + L.scan_tmp);
  int rc = oc_tap_masks(table, idx_bytes, table_cols, h_taps, K, n_rows, masks, stream);
  if (rc) return rc;
  OC_REQUIRE(chunk_log2 >= 0 && chunk_log2 < 32, OC_EINVAL, "tap_order: chunk_log2 %d", chunk_log2);
  const int chunk_shift = chunk_log2 > 0 ? chunk_log2 : 31;         // 0: one chunk (n_rows < 2^31)
  int key_bits = K;
  while (((n_rows - 1) >> chunk_shift) >> (key_bits - K)) ++key_bits;   // + bits of the last chunk's number
  unsigned long long* counts = (unsigned long long*)(ws + L.counts);
  int* bitpos = (int*)(ws + L.bitpos);
  OC_CUDA_OK(cudaMemsetAsync(counts, 0, 32 * sizeof(unsigned long long), s));
  tap_count_kernel<<<grid1d(n_rows), 256, 0, s>>>(masks, n_rows, counts);
  tap_bitpos_kernel<<<1, 32, 0, s>>>(counts, n_rows, K, bitpos);
  mask_key_kernel<<<grid1d(n_rows), 256, 0, s>>>(masks, n_rows, K, chunk_shift, bitpos, kin, vin);
  OC_LAUNCH_OK("mask_key_kernel");
  const int64_t nb = L.sort_blocks;
  for (int shift = 0; shift < key_bits; shift += RADIX_BITS) {
    radix_hist_kernel<<<(unsigned)nb, SORT_THREADS, 0, s>>>(kin, n_rows, shift, hist, nb);
    OC_CUDA_OK(device_scan(HistFlag{hist}, HistSink{hist}, (int64_t)RADIX * nb, nullptr, scan_tmp, nullptr, s));
    radix_scatter_kernel<<<(unsigned)nb, SORT_THREADS, 0, s>>>(kin, vin, n_rows, shift, hist, nb, kout, vout);
    OC_LAUNCH_OK("radix_scatter_kernel");
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  OC_CUDA_OK(cudaMemcpyAsync(perm, vin, (size_t)n_rows * 4, cudaMemcpyDeviceToDevice, s));
  return OC_OK;
}

extern "C" int oc_full_layer(int depth, int batch_size, int64_t* keys, int32_t* children, void* stream) {
  OC_REQUIRE(depth >= 0 && depth <= 10 && batch_size >= 1, OC_EINVAL, "oc_full_layer: bad depth/batch");
  const int64_t n = (int64_t)batch_size << (3 * depth);
  OC_REQUIRE(n < (1LL << 31), OC_EINVAL, "oc_full_layer: layer too large");
  OC_REQUIRE(keys || children, OC_EINVAL, "oc_full_layer: null outputs");
  full_layer_kernel<<<grid1d(n), 256, 0, (cudaStream_t)stream>>>(depth, n, keys, children);
  OC_LAUNCH_OK("full_layer_kernel");
  return OC_OK;
}

extern "C" int oc_grow_layer(const int64_t* keys_p, const int32_t* children_p, int64_t nnum_p,
                             int64_t* keys, int32_t* children, void* stream) {
  OC_REQUIRE(nnum_p >= 0, OC_EINVAL, "oc_grow_layer: negative size");
  if (nnum_p == 0) return OC_OK;
  OC_REQUIRE(keys_p && children_p && keys && children, OC_EINVAL, "oc_grow_layer: null pointer");
  grow_layer_kernel<<<grid1d(nnum_p * 8), 256, 0, (cudaStream_t)stream>>>(keys_p, children_p, nnum_p, keys, children);
  OC_LAUNCH_OK("grow_layer_kernel");
  return OC_OK;
}
