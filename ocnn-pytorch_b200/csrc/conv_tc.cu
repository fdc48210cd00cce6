// Octree convolution on the 5th-generation tensor cores (tcgen05 + TMEM), fp16 /
// bf16 data with fp32 accumulation.
//
// Gather implicit GEMM (forward, and input gradient through a mirrored / inverse
// table): out[r, :] = sum_k data[table[r, taps[k]], :] . Wk.  It replaces the
// reference's Triton kernels conv_fwd_implicit_gemm(_splitk) and
// conv_bwd_input_implicit_gemm(_splitk) (ocnn/nn/kernels/*.py) and the im2col +
// torch.mm path of ocnn/nn/octree_conv.py:115-168.
//
// One persistent CTA per SM walks output tiles of H x 128 rows (H = 1, or 2 when a tile
// table is given and Cout <= 128).  Warp roles:
//   warps 0-3  epilogue : TMEM -> registers -> (+bias, cast) -> global
//   warp 4     MMA issuer: all 32 lanes run the loop, an elected lane issues tcgen05.mma
//                         128 x Cout x 16 per K step; accumulators double-buffered in TMEM
//                         so the epilogue of tile i overlaps the main loop of tile i+1.
//   warp 8     loader   : one bulk copy per 128-row half brings that half's block of the tile
//                         table (tap mask + tap-major int32 indices) into shared memory.
//   warps 5-7, 9-11, 13-14 producers: a stage = one reduction block (a tap x 64 channels, or
//                         2 / 4 whole taps when Cin = 32 / 16): per half the 128 gathered
//                         input rows, copied by cp.async (16 B per lane, 8 lanes per row,
//                         zero-fill for missing neighbours) into the 128-byte-swizzled
//                         K-major layout the MMA reads, plus the matching block of the
//                         pre-swizzled weight image (one bulk copy).  Whole blocks are dealt
//                         to the warps round-robin; each lane's completion arrives on the
//                         stage barrier, nobody waits.  Blocks whose taps have no valid
//                         neighbour in the whole tile are skipped.  Given a plain table
//                         (H = 1) the producers prefetch and publish the indices themselves.
// Stages flow through a ring of full/empty mbarriers; the header of a tile's first stage
// tells the MMA warp how many stages the tile has.  Every wait is bounded.
#include <cuda.h>
#include <stdlib.h>

#include "oc_common.cuh"
#include "conv_internal.cuh"
#include "tc_ptx.cuh"

namespace oc {

__device__ int g_tc_status = 0;  // sticky: non-zero after any abandoned wait
// Profiling build (-DOC_PROF): every role accumulates clock64() intervals (time waiting on
// each barrier, time issuing copies / MMAs) and adds them to g_prof at exit; oc_debug_prof
// reads the totals.  -DOC_NOCOPY drops the gather copies and -DOC_NOMMA the MMAs, which
// shows how fast each side of the pipeline runs alone (results are then meaningless).
// None of this is compiled into the shipped library.
#ifdef OC_PROF
__device__ unsigned long long g_prof[64];
#define PROF_T(v) const long long v = clock64()
#define PROF_ADD(i, d) pr[i] += (d)
#define PROF_DECL long long pr[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_FLUSH(base, n) if (lane == 0) { for (int _i = 0; _i < (n); ++_i) atomicAdd(&g_prof[(base) + _i], (unsigned long long)pr[_i]); }
#else
#define PROF_T(v)
#define PROF_ADD(i, d)
#define PROF_DECL
#define PROF_FLUSH(base, n)
#endif

namespace tc {

constexpr int TILE_M = 128;
constexpr int KBLK = 64;                 // channels per K block = one 128-byte swizzle row
constexpr int A_BYTES = TILE_M * 128;    // 16 KB
constexpr int PROD_WARPS = 8;             // gathering warps
constexpr int PROD_THREADS = PROD_WARPS * 32;
constexpr int FSPLIT = PROD_THREADS / TILE_M;    // threads that share the index prefetch of one row
// Warp roles by index: 0-3 epilogue, 4 MMA issuer, producers = the warps > 4 whose index is
// not a multiple of 4.  The MMA warp then shares its SM sub-partition (warp % 4 == 0) with no
// producer: tcgen05.mma and cp.async leave through the same per-partition memory-instruction
// queue, and behind a producer's slowly draining cp.async an MMA took ~3x longer to issue.
constexpr int MMA_WARP = 4;
constexpr int N_WARPS = 5 + PROD_WARPS + (PROD_WARPS + 2) / 3;   // producers plus the skipped multiples of 4
constexpr int THREADS = N_WARPS * 32;
constexpr int MAX_STAGES = 8;
constexpr int MAX_NT = 256;
// Index buffer of one tile in shared memory: a 16-byte header (word 0 = mask of the taps that
// have a valid row in this tile) followed by one 512-byte row of 128 int32 indices per tap.
// A tile table (oc_tile_table_build) stores the tiles of a neighbour table in exactly this form,
// so that one bulk copy per tile fetches them.
constexpr int IDX_HDR_BYTES = 16;
constexpr int IDX_BUF_BYTES = IDX_HDR_BYTES + OC_MAX_TAPS * TILE_M * 4;
constexpr int LOADER_WARP = 8;            // fetches tile-table blocks (idle when a plain table is given)

struct Params {
  const void* data;
  const void* wimg;    // [n_tiles_n][K][KB][NT x 128 B] swizzled weight image
  const void* bias;
  const void* table;
  const void* tiled;   // tile table (then `table` is unused) or null
  const int32_t* perm; // tile-table position -> output row (null: identity); see oc_tile_table_build
  uint32_t tiled_block_bytes;
  void* out;
  int64_t n_out;
  int table_cols;
  int K, Cin, Cout;
  int KB;              // 64-channel blocks per tap (1 when Cin <= 64)
  int PACK;            // taps per block: 64 / Cin when Cin is 16 or 32, else 1
  int NBLK;            // blocks of the reduction = weight blocks per N tile
  int NT;              // output channels per CTA tile (multiple of 16, <= 256)
  int stages;
  int tmem_cols;       // power of two >= 2 * H * NT
  int tma;             // gathered rows come by TMA (tile::gather4 through the kernel's tensor map)
  int oob_row;         // a row index outside the tensor map: stands for "no neighbour", reads zeros
  TapList taps;
};

struct SmemLayout {
  uint32_t stage_bytes, ring, sidx, bias, bars, hdr, misc, total;
};

__host__ __device__ inline SmemLayout smem_layout(int NT, int stages, int H) {
  SmemLayout L;
  L.stage_bytes = H * A_BYTES + NT * 128;      // H gathered blocks, then the weight block
  L.ring = 0;
  L.sidx = L.ring + stages * L.stage_bytes;
  L.bias = L.sidx + 2 * H * IDX_BUF_BYTES;
  L.bars = L.bias + MAX_NT * 4;
  L.hdr = L.bars + (2 * MAX_STAGES + 9) * 8;
  L.misc = L.hdr + MAX_STAGES * 4;
  L.total = L.misc + 256;
  return L;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b, float ba, float bb, bool has_bias) {
  if (BF16) {
    __nv_bfloat16 x = __float2bfloat16_rn(a), y = __float2bfloat16_rn(b);
    if (has_bias) {
      x = __float2bfloat16_rn(__bfloat162float(x) + ba);
      y = __float2bfloat16_rn(__bfloat162float(y) + bb);
    }
    return (uint32_t)__bfloat16_as_ushort(x) | ((uint32_t)__bfloat16_as_ushort(y) << 16);
  } else {
    __half x = __float2half_rn(a), y = __float2half_rn(b);
    if (has_bias) {
      x = __float2half_rn(__half2float(x) + ba);
      y = __float2half_rn(__half2float(y) + bb);
    }
    return (uint32_t)__half_as_ushort(x) | ((uint32_t)__half_as_ushort(y) << 16);
  }
}

// H = 128-row halves per tile (1 or 2).  With H = 2 a stage holds the gathered blocks of both
// halves next to ONE weight block: the weight traffic from L2 (8 KB per 16 KB gathered at
// C = 64) and the per-stage bookkeeping of the MMA warp are shared by 256 rows.
template <bool BF16, typename I, int H>
__global__ void __launch_bounds__(THREADS, 1)
conv_tc_kernel(const Params p, const __grid_constant__ CUtensorMap data_map) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: swizzle atoms are 8 rows x 128 B
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const SmemLayout L = smem_layout(p.NT, p.stages, H);
  const uint32_t s_base = smem_u32(smem);
  float* sbias = (float*)(smem + L.bias);
  const uint32_t bars = pin_reg(s_base + L.bars);
  volatile uint32_t* hdr = (volatile uint32_t*)(smem + L.hdr);
  uint32_t* misc = (uint32_t*)(smem + L.misc);   // [0] tmem base, [1] abort flag, [2..] warp masks (2 buffers x PROD_WARPS)
  volatile int* abort_flag = (volatile int*)(misc + 1);

  const int S = p.stages;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * MAX_STAGES + 2 + a); };
  const uint32_t psync_bar = bars + 8u * (2 * MAX_STAGES + 4);   // producers-only rendezvous
  auto ifull_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 5 + b); };    // tile-table blocks of buffer b have landed
  auto iempty_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 7 + b); };   // every producer warp is done with them
  // index buffer b, half h: header word 0 = tap mask, then K rows of 128 int32
  auto idx_hdr = [&](int b, int h) { return (volatile uint32_t*)(smem + L.sidx + (b * H + h) * IDX_BUF_BYTES); };
  auto idx_rows = [&](int b, int h) { return (int*)(smem + L.sidx + (b * H + h) * IDX_BUF_BYTES + IDX_HDR_BYTES); };
  const bool tiled = p.tiled != nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * p.NT;                       // first output channel of this CTA
  const int64_t n_tiles = ((p.n_out + TILE_M - 1) / TILE_M + H - 1) / H;   // tiles of H x 128 rows

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 32 * H + 1);   // the lanes of the H owning warps + 1 arrive.expect_tx (weights)
      mbar_init(empty_bar(s), 1);           // one tcgen05.commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 128);
    }
    mbar_init(psync_bar, PROD_THREADS);
    for (int b = 0; b < 2; ++b) {
      mbar_init(ifull_bar(b), 1);             // one arrive.expect_tx of the loader
      mbar_init(iempty_bar(b), PROD_WARPS);   // lane 0 of every producer warp
    }
    misc[1] = 0;
    fence_mbar_init();
  }
  for (int i = threadIdx.x; i < p.NT; i += THREADS) {
    float b = 0.f;
    if (p.bias && n0 + i < p.Cout)
      b = BF16 ? __bfloat162float(((const __nv_bfloat16*)p.bias)[n0 + i]) : __half2float(((const __half*)p.bias)[n0 + i]);
    sbias[i] = b;
  }
  if (warp == 0) {
    tmem_alloc(s_base + L.misc, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];

  const int pw_raw = (warp - 5) - ((warp - 5) >> 2);     // producer number of warps 5,6,7,9,10,11,13,14,...
  if (warp > 4 && (warp & 3) != 0 && pw_raw < PROD_WARPS) {
    // ===================================================================== producers
    const int pw = pw_raw;
    const int pt = pw * 32 + lane;             // 0..255
    const int frow = pt & (TILE_M - 1);        // index prefetch: row `frow`, taps k = fpart (mod FSPLIT)
    const int fpart = pt >> 7;
    const I* table = (const I*)p.table;
    const uint8_t* data = pin_reg((const uint8_t*)p.data);
    const uint32_t row_bytes = pin_reg((uint32_t)p.Cin * 2);
    const uint8_t* wimg = pin_reg((const uint8_t*)p.wimg + (size_t)blockIdx.y * p.NBLK * (size_t)(p.NT * 128));
    const uint32_t b_bytes = pin_reg((uint32_t)p.NT * 128);
    // loop bounds and strides of the stage loop, pinned in registers
    const int KB = pin_reg(p.KB), Cin = pin_reg(p.Cin), NS = pin_reg(S), PACK = pin_reg(p.PACK), K = pin_reg(p.K);
    const uint32_t pmask = (1u << PACK) - 1u;      // tap bits of one block
    const uint32_t ring0 = pin_reg(s_base + L.ring), stage_bytes = pin_reg(L.stage_bytes);
    bool bad_index = false;                    // the tile table names taps >= K (built for another K)
    // A stage = one valid tap x one 64-channel block: H gathered blocks (128 rows x 8 chunks of
    // 16 B each) + the weight block.  Whole blocks are dealt to the producer warps round-robin,
    // so the per-block bookkeeping (slot wait, header, weight copy, barrier arrival) is paid by
    // one warp while the others work on their own blocks.  8 lanes copy one 128-byte row; lane
    // group g = lane / 8 owns the rows 32 g .. 32 g + 31 of the block, fetched 4 indices at a time.
    const int chunk = lane & 7;
    const int grp = lane >> 3;
    // Cin = 16 / 32: a 128-byte row holds 4 / 2 taps; this lane's 16-byte chunk belongs to tap
    // (first tap of the block) + sub and to bytes ch_off.. of that tap's row.  Otherwise one tap.
    const int cpt = PACK > 1 ? Cin >> 3 : 8;       // chunks per tap
    const int sub = PACK > 1 ? chunk / cpt : 0;
    const int ch_off = (PACK > 1 ? chunk % cpt : chunk) * 16;
    const int n_own = pin_reg(S * H < PROD_WARPS ? S * H : PROD_WARPS);   // warps that own blocks (a warp needs a slot of its own)
    int owner = 0;                             // producer warp that owns the next block
    int s = 0;                                 // ring slot of the next stage
    uint32_t ring_phase = 0;                   // flips each time the ring wraps
    constexpr int NF = (OC_MAX_TAPS + FSPLIT - 1) / FSPLIT;
    int nidx[NF];
    bool ok = true;
    uint32_t psync_phase = 0;
    PROF_DECL;
    PROF_T(p_start);

    // plain table (H == 1 only): every thread prefetches half a row of the next tile's indices
    auto fetch_indices = [&](int64_t tile) {
      const int64_t r = tile * TILE_M + frow;
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        const int k = FSPLIT * i + fpart;
        nidx[i] = (k < p.K && r < p.n_out) ? (int)table[r * p.table_cols + p.taps.t[k < OC_MAX_TAPS ? k : 0]] : -1;
      }
    };
    auto publish_indices = [&](int buf) -> uint32_t {
      uint32_t m = 0;
      int* dst = idx_rows(buf, 0);
#pragma unroll
      for (int i = 0; i < NF; ++i) {
        const int k = FSPLIT * i + fpart;
        if (k < OC_MAX_TAPS) {
          dst[k * TILE_M + frow] = nidx[i];
          m |= (nidx[i] >= 0 ? 1u : 0u) << k;
        }
      }
      m = __reduce_or_sync(0xffffffffu, m);
      if (lane == 0) misc[2 + pw + PROD_WARPS * buf] = m;
      // rendezvous of the producer threads on an mbarrier, so that even this wait
      // is bounded (a plain bar.sync would hang if one thread had given up)
      mbar_arrive(psync_bar);
      if (!mbar_wait(psync_bar, psync_phase, abort_flag, &g_tc_status, 5)) ok = false;
      psync_phase ^= 1u;
      uint32_t all = 0;
#pragma unroll
      for (int w = 0; w < PROD_WARPS; ++w) all |= misc[2 + w + PROD_WARPS * buf];
      return all;
    };
    int64_t tile = blockIdx.x;
    int buf = 0;
    uint32_t mask = 0;
    uint32_t it = 0;                           // tiles done by this CTA
    if (H == 1 && !tiled && tile < n_tiles) {
      fetch_indices(tile);
      mask = publish_indices(buf);
    }
    for (; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int64_t next = tile + gridDim.x;
      PROF_T(pf0);
      if (H > 1 || tiled) {
        buf = (int)(it & 1u);
        if (!mbar_wait(ifull_bar(buf), (it >> 1) & 1u, abort_flag, &g_tc_status, 6)) { ok = false; break; }
        mask = 0;
#pragma unroll
        for (int h = 0; h < H; ++h) mask |= *idx_hdr(buf, h);
        if (mask >> p.K) { mask &= (1u << p.K) - 1u; bad_index = true; }   // not a tile table of K taps
      } else if (next < n_tiles) {
        fetch_indices(next);   // loads stay in flight during this tile
      }
      PROF_T(pf1); PROF_ADD(3, pf1 - pf0);
      if (mask == 0) mask = 1;                   // nothing valid: one all-zero stage keeps the flow uniform
      PROF_T(pl0);
      // Candidate blocks in order: (tap k .. k + PACK - 1, channel block kb); candidate number cb
      // is also the block's place in the weight image.  A block is a stage if one of its taps
      // has a valid row in this tile.
      uint32_t n_st = (uint32_t)__popc(mask) * (uint32_t)KB;
      if (PACK > 1) {
        n_st = 0;
        for (int k = 0; k < K; k += PACK) n_st += ((mask >> k) & pmask) ? 1u : 0u;
      }
      bool first = true;
      int k = 0, kb = 0;
      for (int cb = 0; k < K && ok; ++cb) {
        const int k_blk = k, kb_blk = kb;
        if (++kb == KB) { kb = 0; k += PACK; }
        if (!((mask >> k_blk) & pmask)) continue;
        {
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const bool mine = owner == pw;            // blocks are dealt round-robin
            if (++owner == n_own) owner = 0;
            if (mine) {
              PROF_T(pw0);
              if (!mbar_wait(empty_bar(s), ring_phase ^ 1u, abort_flag, &g_tc_status, 1)) { ok = false; break; }
              PROF_T(pw1); PROF_ADD(0, pw1 - pw0);
              const uint32_t a_dst = ring0 + s * stage_bytes + h * A_BYTES;
              if (h == 0 && lane == 0) {
                if (first) hdr[s] = n_st;               // the first stage of a tile carries its stage count
#ifdef OC_NOCOPY
                mbar_arrive(full_bar(s));
#else
                mbar_arrive_expect_tx(full_bar(s), b_bytes);
                bulk_g2s(ring0 + s * stage_bytes + H * A_BYTES, wimg + (size_t)cb * b_bytes, b_bytes, full_bar(s));
#endif
              }
#ifndef OC_NOCOPY
              if (p.tma) {
                // TMA path (64-channel blocks of whole taps): lane l asks for the rows 4 l .. 4 l + 3
                // of the block with one tile::gather4 copy; the TMA unit applies the 128-byte
                // swizzle and completes 512 bytes on the stage's barrier.
                const int4 r4 = *reinterpret_cast<const int4*>(idx_rows(buf, h) + k_blk * TILE_M + 4 * lane);
                const int oob = p.oob_row;
                mbar_arrive_expect_tx(full_bar(s), 512u);
                tma_gather4(a_dst + (uint32_t)lane * 512u, &data_map, kb_blk * KBLK, r4.x < 0 ? oob : r4.x,
                            r4.y < 0 ? oob : r4.y, r4.z < 0 ? oob : r4.z, r4.w < 0 ? oob : r4.w, full_bar(s));
                PROF_T(pw2); PROF_ADD(1, pw2 - pw1); PROF_ADD(2, 1);
                continue;
              }
              const int k_lane = k_blk + sub;            // this lane's tap
              const bool live = PACK > 1 ? k_lane < K : chunk * 8 < min(KBLK, Cin - kb_blk * KBLK);
              {
                const uint8_t* lane_src = data + (size_t)kb_blk * 128 + ch_off;
                const int* irow = idx_rows(buf, h) + (live ? k_lane : 0) * TILE_M + grp * 32;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const int4 r4 = *reinterpret_cast<const int4*>(irow + 4 * q);
                  const int rid[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    const int r = grp * 32 + 4 * q + j;            // (r & 7) == (4 q + j) & 7: known at compile time
                    const int idx = live ? rid[j] : -1;            // dead chunk (past Cin or past the last tap): zeros
                    cp_async_16(a_dst + r * 128 + ((chunk ^ ((4 * q + j) & 7)) << 4),
                                lane_src + (size_t)(idx < 0 ? 0 : idx) * row_bytes, idx >= 0 ? 16u : 0u);
                  }
                }
              }
#endif
              // arrives on the stage's barrier once this lane's copies have landed; the lane
              // itself does not wait, so every warp keeps a whole block in flight
              cp_async_arrive_noinc(full_bar(s));
              PROF_T(pw2); PROF_ADD(1, pw2 - pw1); PROF_ADD(2, 1);
            }
          }
          first = false;
          if (++s == NS) { s = 0; ring_phase ^= 1u; }
        }
      }
      PROF_T(pl1); PROF_ADD(6, pl1 - pl0);
      if (H > 1 || tiled) {
        __syncwarp();                                   // every lane has read its indices of this tile
        if (lane == 0) mbar_arrive(iempty_bar(buf));
      } else if (next < n_tiles) {
        PROF_T(pp0);
        buf ^= 1;
        mask = publish_indices(buf);
        PROF_T(pp1); PROF_ADD(4, pp1 - pp0);
      }
    }
    PROF_T(p_end); PROF_ADD(5, p_end - p_start);
    PROF_FLUSH(0, 12);
    if (bad_index) atomicMax(&g_tc_status, 90);
    cp_async_wait_all();   // nothing of this thread may still be writing shared memory at exit
  } else if (warp == LOADER_WARP) {
    // ===================================================================== tile-table loader
    // One bulk copy per 128-row half brings header + indices into one of two buffers.
    if (tiled && lane == 0) {
      const uint8_t* src = (const uint8_t*)p.tiled;
      uint32_t it = 0;
      for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
        const int b = (int)(it & 1u);
        if (it >= 2 && !mbar_wait(iempty_bar(b), ((it >> 1) - 1u) & 1u, abort_flag, &g_tc_status, 7)) break;
        // the tile table is padded to a whole number of tiles, so both halves always exist
        mbar_arrive_expect_tx(ifull_bar(b), H * p.tiled_block_bytes);
#pragma unroll
        for (int h = 0; h < H; ++h)
          bulk_g2s(s_base + L.sidx + (b * H + h) * IDX_BUF_BYTES, src + (size_t)(tile * H + h) * p.tiled_block_bytes,
                   p.tiled_block_bytes, ifull_bar(b));
      }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    // ===================================================================== MMA issuer
    // All 32 lanes run the loop (waits, header reads, address arithmetic) so that it is
    // warp-uniform; one elected lane issues the tcgen05 instructions.
    {
      // Descriptors are formed incrementally: the low word of a descriptor holds the start
      // address >> 4, so slot s / half h / K step ks only add s * (stage_bytes / 16) +
      // h * (A_BYTES / 16) + 2 * ks to the low word of the descriptor of slot 0.  Rebuilding the
      // 64-bit descriptor from a run-time address for every MMA makes this loop about twice as slow.
      const uint32_t idesc = make_idesc(BF16 ? 1 : 0, 0, 0, TILE_M, p.NT);
      const uint64_t da0 = make_desc_sw128(s_base + L.ring, 16, 1024);
      const uint64_t desc_hi = da0 & 0xffffffff00000000ull;
      const uint32_t la0 = (uint32_t)da0;
      const uint32_t sb16 = L.stage_bytes >> 4;
      const bool nk4 = p.PACK > 1 || (p.Cin & (KBLK - 1)) == 0;   // every K block is full (or zero-padded): 4 MMAs per block
      int s = 0;
      uint32_t ring_phase = 0, acc = 0, acc_phase = 0;  // acc_phase: bit a = phase of accumulator set a
      bool ok = true;
      PROF_DECL;
      PROF_T(m_start);
      for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        PROF_T(mt0);
        ok = mbar_wait(tempty_bar(acc), ((acc_phase >> acc) & 1u) ^ 1u, abort_flag, &g_tc_status, 2);
        if (__any_sync(0xffffffffu, !ok)) break;
        tc_fence_after();
        PROF_T(mt1); PROF_ADD(0, mt1 - mt0);
        const uint32_t d_tmem = tmem_base + acc * (uint32_t)(H * p.NT);
        uint32_t n_st = 1;
        int kb = 0;
        for (uint32_t st = 0; st < n_st; ++st) {
          PROF_T(mf0);
          ok = mbar_wait(full_bar(s), ring_phase, abort_flag, &g_tc_status, 3);
          if (__any_sync(0xffffffffu, !ok)) break;
          tc_fence_after();
          PROF_T(mf1); PROF_ADD(1, mf1 - mf0);
          // the first stage of a tile carries the tile's stage count
          if (st == 0) n_st = __reduce_or_sync(0xffffffffu, hdr[s]);
          const uint32_t la = la0 + (uint32_t)s * sb16, lb = la + H * (A_BYTES >> 4);
#ifndef OC_NOMMA
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const uint32_t lah = la + h * (A_BYTES >> 4);
            const uint32_t dh = d_tmem + h * (uint32_t)p.NT;
            if (nk4) {
#pragma unroll
              for (uint32_t ks = 0; ks < 4; ++ks)
                if (elect_one())
                  umma_f16(dh, desc_hi | (lah + 2 * ks), desc_hi | (lb + 2 * ks), idesc, (st == 0 && ks == 0) ? 0u : 1u);
            } else {
              const uint32_t nk = (uint32_t)min(KBLK, p.Cin - kb * KBLK) >> 4;
              for (uint32_t ks = 0; ks < nk; ++ks)
                if (elect_one())
                  umma_f16(dh, desc_hi | (lah + 2 * ks), desc_hi | (lb + 2 * ks), idesc, (st == 0 && ks == 0) ? 0u : 1u);
            }
          }
#endif
          if (elect_one()) umma_commit(empty_bar(s));         // slot reusable once these MMAs have read it
          if (++s == S) { s = 0; ring_phase ^= 1u; }
          if (++kb == p.KB) kb = 0;
          PROF_T(mf2); PROF_ADD(2, mf2 - mf1); PROF_ADD(3, 1);
        }
        if (!ok) break;
        if (elect_one()) umma_commit(tfull_bar(acc));         // accumulators complete
        acc_phase ^= 1u << acc;
        acc ^= 1u;
      }
      PROF_T(m_end); PROF_ADD(4, m_end - m_start);
      PROF_FLUSH(16, 5);
    }
    __syncwarp();
  } else if (warp < 4) {
    // ===================================================================== epilogue (warps 0-3)
    uint32_t acc = 0, acc_phase = 0;
    const bool has_bias = p.bias != nullptr;
    uint16_t* out = (uint16_t*)p.out;
    PROF_DECL;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
      PROF_T(e0);
      if (!mbar_wait(tfull_bar(acc), (acc_phase >> acc) & 1u, abort_flag, &g_tc_status, 4, 256)) break;
      tc_fence_after();
      PROF_T(e1); PROF_ADD(0, e1 - e0);
#pragma unroll
      for (int h = 0; h < H; ++h) {
        int64_t row = (tile * H + h) * TILE_M + warp * 32 + lane;     // position in the tile table
        if (p.perm && row < p.n_out) {                                // -> output row
          row = p.perm[row];
          if (row < 0) row = p.n_out;                                 // not a row number: nothing is written
        }
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (acc * H + h) * (uint32_t)p.NT;
        for (int c0 = 0; c0 < p.NT; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
          if (row < p.n_out && n0 + c0 < p.Cout) {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = pack2<BF16>(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]), sbias[c0 + 2 * j],
                                 sbias[c0 + 2 * j + 1], has_bias);
            uint4* dst = (uint4*)(out + row * p.Cout + n0 + c0);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(tempty_bar(acc));
      PROF_T(e2); PROF_ADD(1, e2 - e1); PROF_ADD(2, 1);
      acc_phase ^= 1u << acc;
      acc ^= 1u;
    }
    if (warp == 0) { PROF_FLUSH(24, 3); }
  }

  // ------------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // Something gave up: give copies and MMAs still in flight time to land before
    // the shared memory and TMEM of this CTA are released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {}
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ---------------------------------------------------------------------------
// weight image: [nt][k][kb] blocks of NT rows x 128 B, row = output channel,
// 16-byte chunk c of a row holds input channels kb*64 + c*8 .. +7 and is stored
// at chunk position c ^ (row & 7) (the 128-byte swizzle the MMA descriptor names).
// ---------------------------------------------------------------------------
template <typename W, bool BF16>
__global__ void prep_weights_tc_kernel(const W* __restrict__ w, int K, int Cin, int Cout, int transposed,
                                       int KB, int PACK, int NBLK, int NT, int n_tiles_n, uint16_t* __restrict__ img) {
  const int64_t total = (int64_t)n_tiles_n * NBLK * NT * 64;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total;
       t += (int64_t)gridDim.x * blockDim.x) {
    const int e = (int)(t % 64);                  // element of the 64-wide reduction block
    const int row = (int)((t / 64) % NT);
    const int64_t blk = t / (64 * (int64_t)NT);
    const int cb = (int)(blk % NBLK);             // block within the N tile
    const int nt = (int)(blk / NBLK);
    int k, ci;
    if (PACK > 1) { k = cb * PACK + e / Cin; ci = e % Cin; }      // several taps per block
    else { k = cb / KB; ci = (cb % KB) * 64 + e; }
    const int chunk = e >> 3, within = e & 7;
    const int co = nt * NT + row;
    float v = 0.f;
    if (k < K && ci < Cin && co < Cout) {
      const int64_t src = transposed ? ((int64_t)k * Cout + co) * Cin + ci : ((int64_t)k * Cin + ci) * Cout + co;
      v = to_f32<W>(w[src]);
    }
    const int64_t dst = blk * ((int64_t)NT * 64) + (int64_t)row * 64 + ((chunk ^ (row & 7)) << 3) + within;
    img[dst] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
  }
}

struct Plan {
  int KB, PACK, NBLK, NT, n_tiles_n, stages, tmem_cols, H;
  uint32_t smem_bytes;
  bool ok;
};

// H = 128-row halves per tile (see the kernel).
static Plan make_plan(int K, int Cin, int Cout, int dtype, int H = 1) {
  Plan P = {};
  P.ok = false;
  P.H = H;
  if (!(dtype == OC_F16 || dtype == OC_BF16)) return P;
  if (Cin < 16 || Cin % 16 != 0 || Cout < 16 || Cout % 16 != 0) return P;
  if (K < 1 || K > OC_MAX_TAPS) return P;
  P.KB = (Cin + KBLK - 1) / KBLK;
  P.PACK = (Cin == 16 || Cin == 32) ? KBLK / Cin : 1;     // taps that share one 64-wide block
  P.NBLK = P.PACK > 1 ? (K + P.PACK - 1) / P.PACK : K * P.KB;
  P.n_tiles_n = (Cout + MAX_NT - 1) / MAX_NT;
  P.NT = ((Cout + P.n_tiles_n - 1) / P.n_tiles_n + 15) / 16 * 16;
  P.tmem_cols = 32;
  while (P.tmem_cols < 2 * H * P.NT) P.tmem_cols *= 2;
  if (P.tmem_cols > 512) return P;
  const uint32_t budget = 227 * 1024 - 1024;
  int stages = MAX_STAGES;
  while (stages > 2 && smem_layout(P.NT, stages, H).total > budget) --stages;
  if (smem_layout(P.NT, stages, H).total > budget) return P;
  P.stages = stages;
  P.smem_bytes = smem_layout(P.NT, stages, H).total + 1024;
  P.ok = true;
  return P;
}

// Two halves per tile pay when the weight block is re-fetched for many tiles and enough
// stages still fit: tile table given, at least 4 stages, at least 4 tiles per SM.
static Plan choose_plan(int K, int Cin, int Cout, int dtype, int64_t n_out, bool tiled) {
  if (tiled && n_out >= (int64_t)8 * TILE_M * sm_count()) {
    const Plan P2 = make_plan(K, Cin, Cout, dtype, 2);
    if (P2.ok && P2.stages >= 4) return P2;
  }
  return make_plan(K, Cin, Cout, dtype, 1);
}

}  // namespace tc

bool conv_tc_supported(int K, int Cin, int Cout, int dtype) { return tc::make_plan(K, Cin, Cout, dtype).ok; }

// ---------------------------------------------------------------------------
// tile table: the neighbour table regrouped for the tensor-core kernels.  Block t (one
// per 128 output rows) = 16-byte header (word 0: mask of the taps with a valid entry in
// this tile) + K rows of 128 int32 indices, row k = column taps[k] of table rows
// 128 t .. 128 t + 127 (-1 past the end).  The kernels fetch a block with one bulk copy.
// ---------------------------------------------------------------------------
size_t tile_table_block_bytes(int K) { return (size_t)tc::IDX_HDR_BYTES + (size_t)K * tc::TILE_M * 4; }

// padded to an even number of blocks: the kernels may walk the table two blocks at a time
static int64_t tile_table_blocks(int64_t n_out) { return (cdiv(n_out, tc::TILE_M) + 1) / 2 * 2; }

size_t tile_table_bytes(int64_t n_out, int K) { return (size_t)tile_table_blocks(n_out) * tile_table_block_bytes(K); }

template <typename I>
__global__ void __launch_bounds__(tc::TILE_M)
tile_table_kernel(const I* __restrict__ table, int table_cols, TapList taps, int K, int64_t n_out, int64_t n_in,
                  const int32_t* __restrict__ perm, uint8_t* __restrict__ out, uint32_t block_bytes) {
  __shared__ uint32_t smask;
  if (threadIdx.x == 0) smask = 0;
  __syncthreads();
  const int64_t tile = blockIdx.x;
  const int64_t pos = tile * tc::TILE_M + threadIdx.x;        // position in the tile table
  int64_t r = (perm && pos < n_out) ? (int64_t)perm[pos] : pos;   // row of the plain table
  if (r < 0 || (pos < n_out && r >= n_out)) {                     // not a permutation of the rows: reported
    atomicMax(&g_tc_status, 90);
    r = n_out;
  }
  uint8_t* blk = out + (size_t)tile * block_bytes;
  int* rows = (int*)(blk + tc::IDX_HDR_BYTES);
  uint32_t m = 0;
  for (int k = 0; k < K; ++k) {
    int64_t v64 = (pos < n_out && r < n_out) ? (int64_t)table[r * table_cols + taps.t[k]] : -1;
    if (n_in > 0 && v64 >= n_in) {   // would read past the feature rows: dropped and reported
      v64 = -1;
      atomicMax(&g_tc_status, 90);
    }
    const int v = v64 < 0 ? -1 : (int)v64;
    rows[k * tc::TILE_M + threadIdx.x] = v;
    m |= (v >= 0 ? 1u : 0u) << k;
  }
  m = __reduce_or_sync(0xffffffffu, m);
  if ((threadIdx.x & 31) == 0 && m) atomicOr(&smask, m);
  __syncthreads();
  if (threadIdx.x < 4) ((uint32_t*)blk)[threadIdx.x] = threadIdx.x == 0 ? smask : 0u;
}

int launch_tile_table(const void* table, int idx_bytes, int table_cols, const TapList& taps, int K,
                      int64_t n_out, int64_t n_in, const int32_t* perm, void* out, cudaStream_t s) {
  if (n_out == 0) return OC_OK;
  const unsigned grid = (unsigned)tile_table_blocks(n_out);   // a padding block holds -1 only
  const uint32_t bb = (uint32_t)tile_table_block_bytes(K);
  if (idx_bytes == 8)
    tile_table_kernel<int64_t><<<grid, tc::TILE_M, 0, s>>>((const int64_t*)table, table_cols, taps, K, n_out, n_in, perm, (uint8_t*)out, bb);
  else
    tile_table_kernel<int32_t><<<grid, tc::TILE_M, 0, s>>>((const int32_t*)table, table_cols, taps, K, n_out, n_in, perm, (uint8_t*)out, bb);
  OC_LAUNCH_OK("tile_table_kernel");
  return OC_OK;
}

size_t conv_tc_weight_bytes(int K, int Cin, int Cout) {
  const tc::Plan P = tc::make_plan(K, Cin, Cout, OC_F16);
  return (size_t)P.n_tiles_n * P.NBLK * P.NT * 128;
}

int prep_weights_tc(const void* w, int w_dtype, int K, int Cin, int Cout, int transposed, int dtype,
                    void* out, cudaStream_t s) {
  const tc::Plan P = tc::make_plan(K, Cin, Cout, dtype);
  OC_REQUIRE(P.ok, OC_EINVAL, "conv_tc: unsupported shape");
  const int64_t total = (int64_t)P.n_tiles_n * P.NBLK * P.NT * 64;
  const unsigned g = grid_1d(total, 256, 8);
  uint16_t* img = (uint16_t*)out;
  const bool bf = dtype == OC_BF16;
  if (w_dtype == OC_F32) {
    if (bf) tc::prep_weights_tc_kernel<float, true><<<g, 256, 0, s>>>((const float*)w, K, Cin, Cout, transposed, P.KB, P.PACK, P.NBLK, P.NT, P.n_tiles_n, img);
    else tc::prep_weights_tc_kernel<float, false><<<g, 256, 0, s>>>((const float*)w, K, Cin, Cout, transposed, P.KB, P.PACK, P.NBLK, P.NT, P.n_tiles_n, img);
  } else if (bf) {
    tc::prep_weights_tc_kernel<__nv_bfloat16, true><<<g, 256, 0, s>>>((const __nv_bfloat16*)w, K, Cin, Cout, transposed, P.KB, P.PACK, P.NBLK, P.NT, P.n_tiles_n, img);
  } else {
    tc::prep_weights_tc_kernel<__half, false><<<g, 256, 0, s>>>((const __half*)w, K, Cin, Cout, transposed, P.KB, P.PACK, P.NBLK, P.NT, P.n_tiles_n, img);
  }
  OC_LAUNCH_OK("prep_weights_tc_kernel");
  return OC_OK;
}

// Tensor map of a (rows, C) fp16 / bf16 matrix for tile::gather4: box = 64 channels x 1 row,
// 128-byte swizzle, rows outside the matrix read as zeros.
static int make_rows_map(const void* base, int64_t rows, int C, int dtype, CUtensorMap* map) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  if (!encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    OC_CUDA_OK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    OC_REQUIRE(fn && q == cudaDriverEntryPointSuccess, OC_ECUDA, "cuTensorMapEncodeTiled is not available");
    encode = (EncodeFn)fn;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)C, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)C * 2};
  const cuuint32_t box[2] = {64, 1};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, dtype == OC_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                            const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  OC_REQUIRE(r == CUDA_SUCCESS, OC_ECUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return OC_OK;
}

// Whether the gathered rows come by TMA (tile::gather4) instead of per-lane cp.async: whole
// 64-channel blocks and 32-bit row numbers, and the environment variable OC_TMA_GATHER=1 (read at
// every launch).  Both paths give the same bits and, measured on B200, the same speed within 3 %
// (the gather is bound by the latency of the rows in flight, not by how they are requested), so
// the cp.async path, which also serves Cin = 16 / 32 and partial blocks, is the default.
static bool tma_gather_ok(int64_t n_in, int Cin, int pack) {
  const char* e = getenv("OC_TMA_GATHER");
  return e && atoi(e) != 0 && pack == 1 && Cin % 64 == 0 && n_in > 0 && n_in < INT32_MAX;
}

template <bool BF16, typename I, int H>
static int launch_conv_tc_t(const tc::Params& prm, const tc::Plan& P, const CUtensorMap& map, cudaStream_t s) {
  auto kern = tc::conv_tc_kernel<BF16, I, H>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  OC_CUDA_OK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    OC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_dev = dev;
  }
  const int64_t n_tiles = cdiv(cdiv(prm.n_out, tc::TILE_M), H);
  const int sms = sm_count();
  dim3 grid((unsigned)(n_tiles < sms ? n_tiles : sms), (unsigned)P.n_tiles_n);
  kern<<<grid, tc::THREADS, P.smem_bytes, s>>>(prm, map);
  OC_LAUNCH_OK("conv_tc_kernel");
  return OC_OK;
}

int launch_conv_tc(const ConvArgs& a, const void* Wimg, int* status_dev, cudaStream_t s) {
  (void)status_dev;
  const tc::Plan P = tc::choose_plan(a.K, a.Cin, a.Cout, a.dtype, a.n_out, a.tiled != nullptr);
  OC_REQUIRE(P.ok, OC_EINVAL, "conv_tc: unsupported shape");
  OC_REQUIRE(((uintptr_t)a.data % 16) == 0 && ((uintptr_t)a.out % 16) == 0 && ((uintptr_t)Wimg % 16) == 0,
             OC_EINVAL, "conv_tc: data, out and workspace must be 16-byte aligned");
  if (a.n_out == 0) return OC_OK;
  tc::Params prm;
  prm.data = a.data; prm.wimg = Wimg; prm.bias = a.bias; prm.table = a.table; prm.out = a.out;
  prm.perm = a.tiled ? a.perm : nullptr;
  prm.tiled = a.tiled; prm.tiled_block_bytes = (uint32_t)tile_table_block_bytes(a.K);
  OC_REQUIRE(((uintptr_t)a.tiled % 16) == 0, OC_EINVAL, "conv_tc: the tile table must be 16-byte aligned");
  prm.n_out = a.n_out; prm.table_cols = a.table_cols; prm.K = a.K; prm.Cin = a.Cin; prm.Cout = a.Cout;
  prm.KB = P.KB; prm.PACK = P.PACK; prm.NBLK = P.NBLK; prm.NT = P.NT; prm.stages = P.stages; prm.tmem_cols = P.tmem_cols; prm.taps = a.taps;
  alignas(64) CUtensorMap map;
  memset(&map, 0, sizeof(map));
  prm.tma = tma_gather_ok(a.n_in, a.Cin, P.PACK) ? 1 : 0;
  prm.oob_row = (int)a.n_in;
  if (prm.tma) {
    int rc = make_rows_map(a.data, a.n_in, a.Cin, a.dtype, &map);
    if (rc) return rc;
  }
  const bool bf = a.dtype == OC_BF16;
  if (P.H == 2) return bf ? launch_conv_tc_t<true, int32_t, 2>(prm, P, map, s) : launch_conv_tc_t<false, int32_t, 2>(prm, P, map, s);
  if (a.idx_bytes == 8) return bf ? launch_conv_tc_t<true, int64_t, 1>(prm, P, map, s) : launch_conv_tc_t<false, int64_t, 1>(prm, P, map, s);
  return bf ? launch_conv_tc_t<true, int32_t, 1>(prm, P, map, s) : launch_conv_tc_t<false, int32_t, 1>(prm, P, map, s);
}

int read_tc_status(cudaStream_t s, int* h_status) {
  int v = 0, zero = 0;
  OC_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, g_tc_status, sizeof(int), 0, cudaMemcpyDeviceToHost, s));
  OC_CUDA_OK(cudaStreamSynchronize(s));
  if (v != 0) OC_CUDA_OK(cudaMemcpyToSymbolAsync(g_tc_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s));
  *h_status = v;
  return OC_OK;
}

}  // namespace oc

#ifdef OC_PROF
extern "C" int oc_debug_prof(unsigned long long* host64, int reset) {
  if (reset) { unsigned long long z[64] = {0}; return (int)cudaMemcpyToSymbol(oc::g_prof, z, sizeof(z)); }
  return (int)cudaMemcpyFromSymbol(host64, oc::g_prof, 64 * sizeof(unsigned long long));
}
#endif
#include "wgrad_tc.cuh"
