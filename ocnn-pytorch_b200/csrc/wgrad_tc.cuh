// Weight gradient of the octree convolution on tcgen05 tensor cores (fp16 / bf16
// data, fp32 accumulation in TMEM):
//     grad_w[k, ci, co] = sum_r data[table[r, taps[k]], ci] * grad_out[r, co]
// It replaces weight_gemm of ocnn/nn/octree_conv.py:170-202 and the Triton
// kernels conv_bwd_weight_implicit_gemm(_splitk) of the reference.
//
// As a GEMM the reduction runs over the rows r, so both operands are "MN-major"
// for the MMA: a gathered tile (128 rows x 64 channels, one 128-byte swizzled
// line per row — byte for byte the A tile of the forward kernel) is read
// transposed as a 64 x 128 block of the M x K operand, and a dense tile of
// grad_out rows is the K x N operand.  Two 64-channel blocks (two taps, or the
// two halves of one tap when Cin > 64) form one 128-row M tile.
//
// Work split: grid = (row slices, M-tile groups, N tiles).  A CTA walks the 128-row
// tiles of its slice; per tile it loads grad_out once and, for every M tile of its
// group with at least one valid neighbour, gathers the two blocks and issues
// 8 MMAs (K = 16 rows each) into that M tile's own TMEM accumulator, which stays
// resident for the whole slice.
// Roles: a loader warp brings in, per row tile, the tile-table block's header and the index rows
// of this CTA's taps (two bulk copies); four
// warps load the grad_out tile, a quarter each (with one warp this load bounds the kernel when
// Cout >= 128); eight producer warps gather, each owning whole 64-channel blocks
// dealt round-robin (so a warp keeps a block of its own in flight while the others work
// on theirs); one warp issues the MMAs.  The neighbour table always comes as a tile table
// (oc_tile_table_build); the entry point builds one in the workspace when given a plain table.  At the end every accumulator is written to a
// per-slice fp32 partial and a second kernel adds the slices in a fixed order
// (no atomics: the result does not vary from run to run).
// (Included at the end of conv_tc.cu: both kernels share the sticky status word,
// and the library is built without relocatable device code.)
#pragma once

namespace oc {

namespace wg {

using namespace tc;

constexpr int TILE_R = 128;               // rows (the MMA K extent) per tile
constexpr int BLK_BYTES = TILE_R * 128;   // one 64-channel block of 128 rows
constexpr int PROD_WARPS = 8;
constexpr int PROD_THREADS = PROD_WARPS * 32;
// Warp 4: MMA issuer; warp 8: tile-table loader; producers: warps > 4 whose index is not a
// multiple of 4, so that the MMA warp's SM sub-partition holds no copying warp; warps 1-3 and 15
// load the grad_out tile (a quarter each); warps 0-11 run the epilogue at the end.
constexpr int MMA_WARP = 4;
constexpr int LOADER_WARP = 8;
constexpr int N_WARPS = 5 + PROD_WARPS + (PROD_WARPS + 2) / 3;
constexpr int THREADS = N_WARPS * 32;
static_assert(N_WARPS == 16, "warp roles are laid out for 16 warps");
constexpr int MAX_STAGES = 6;
constexpr int MAX_MT = 16;                // M tiles (accumulators) per CTA

struct Params {
  const void* data;
  const void* gout;
  const void* tiled;    // tile table of the K taps
  const int32_t* perm;  // tile-table position -> row of grad_out (null: identity)
  uint32_t tiled_block_bytes;
  float* partial;       // [row slices][K][Cin][Cout]
  int64_t n_out;
  int64_t tiles_per_slice;
  int K, Cin, Cout;
  int KB;               // 64-channel blocks per tap (1 when Cin <= 64)
  int PACK;             // taps per block: 64 / Cin when Cin is 16 or 32, else 1
  int nblk;             // blocks of the M extent: K * KB, or ceil(K / PACK)
  int NTW;              // output channels per CTA (multiple of 16, <= 128)
  int GB;               // 64-column blocks of grad_out per tile = ceil(NTW / 64)
  int mt_per_cta;
  int stages;
  int tmem_cols;
};

struct SmemLayout {
  uint32_t ring, gbuf, sidx, bars, hdr, misc, total;
};

__host__ __device__ inline SmemLayout smem_layout(int GB, int stages) {
  SmemLayout L;
  L.ring = 0;                                     // stages x 2 blocks
  L.gbuf = L.ring + stages * 2 * BLK_BYTES;       // 2 buffers x GB blocks
  L.sidx = L.gbuf + 2 * GB * BLK_BYTES;
  L.bars = L.sidx + 2 * IDX_BUF_BYTES;
  L.hdr = L.bars + (2 * MAX_STAGES + 9) * 8;
  L.misc = L.hdr + MAX_STAGES * 4;
  L.total = L.misc + 128;
  return L;
}

template <bool BF16>
__global__ void __launch_bounds__(THREADS, 1) wgrad_tc_kernel(const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const SmemLayout L = smem_layout(p.GB, p.stages);
  const uint32_t s_base = smem_u32(smem);
  const uint32_t bars = pin_reg(s_base + L.bars);
  volatile uint32_t* hdr = (volatile uint32_t*)(smem + L.hdr);
  uint32_t* misc = (uint32_t*)(smem + L.misc);   // [0] tmem base, [1] abort, [18] touched
  volatile int* abort_flag = (volatile int*)(misc + 1);

  const int S = p.stages;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (MAX_STAGES + s); };
  auto gfull_bar = [&](int g) { return bars + 8u * (2 * MAX_STAGES + g); };
  auto gempty_bar = [&](int g) { return bars + 8u * (2 * MAX_STAGES + 2 + g); };
  auto ifull_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 4 + b); };    // tile-table block b has landed
  auto iempty_bar = [&](int b) { return bars + 8u * (2 * MAX_STAGES + 6 + b); };   // every producer warp is done with it
  const uint32_t done_bar = bars + 8u * (2 * MAX_STAGES + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slice = blockIdx.x;
  const int m_lo = blockIdx.y * p.mt_per_cta;                     // first M tile of this CTA
  const int n_mt_all = (p.nblk + 1) / 2;
  const int m_cnt = min(p.mt_per_cta, n_mt_all - m_lo);
  const int n0 = blockIdx.z * p.NTW;
  const int64_t n_tiles = (p.n_out + TILE_R - 1) / TILE_R;
  // slice s walks tiles s, s + slices, s + 2 slices, ...: equal work per slice whatever the
  // row order of the tile table (tiles ordered by tap mask get more expensive towards the end)
  const int64_t t_begin = slice, t_end = n_tiles, t_step = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full_bar(s), 64 + 1);   // the lanes of the two warps that own the stage's blocks + the header writer
      mbar_init(empty_bar(s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(gfull_bar(g), 128);     // the lanes of the four grad_out loader warps
      mbar_init(gempty_bar(g), 1);
      mbar_init(ifull_bar(g), 1);
      mbar_init(iempty_bar(g), PROD_WARPS);
    }
    mbar_init(done_bar, 1);
    misc[1] = 0;
    misc[18] = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(s_base + L.misc, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = misc[0];

  const int pw_raw = (warp - 5) - ((warp - 5) >> 2);
  const int gq = warp == 15 ? 0 : (warp >= 1 && warp <= 3 ? warp : -1);   // quarter of the grad_out tile this warp loads
  if (warp > 4 && (warp & 3) != 0 && pw_raw < PROD_WARPS) {
    // ===================================================================== producers
    const int pw = pw_raw;
    const uint8_t* data = pin_reg((const uint8_t*)p.data);
    const uint32_t row_bytes = pin_reg((uint32_t)p.Cin * 2);
    const int KB = pin_reg(p.KB), Cin = pin_reg(p.Cin), NS = pin_reg(S), nblk = pin_reg(p.nblk);
    const int PACK = pin_reg(p.PACK), K = pin_reg(p.K);
    const uint32_t pmask = (1u << PACK) - 1u;      // tap bits of one block
    bool bad_index = false;        // the tile table names taps >= K (built for another K)
    const uint32_t ring0 = pin_reg(s_base + L.ring);
    const int chunk = lane & 7;
    const int grp = lane >> 3;
    // Cin = 16 / 32: a 128-byte row holds 4 / 2 taps; this lane's 16-byte chunk belongs to tap
    // (first tap of the block) + sub and to bytes ch_off.. of that tap's row.  Otherwise one tap.
    const int cpt = PACK > 1 ? Cin >> 3 : 8;       // chunks per tap
    const int sub = PACK > 1 ? chunk / cpt : 0;
    const int ch_off = (PACK > 1 ? chunk % cpt : chunk) * 16;
    // block b = (first tap, channel block): (b / KB, b % KB), or (b * PACK, 0) when taps are packed;
    // (k_lo, kb_lo) = that of this CTA's first block; group_taps = taps that feed its M tiles
    const int k_lo = pin_reg(PACK > 1 ? 2 * m_lo * PACK : (2 * m_lo) / KB);
    const int kb_lo = pin_reg(PACK > 1 ? 0 : (2 * m_lo) % KB);
    uint32_t group_taps = 0;
    {
      int k = k_lo, kb = kb_lo;
      for (int b = 2 * m_lo; b < 2 * (m_lo + m_cnt) && b < nblk; ++b) {
        group_taps |= pmask << k;
        if (++kb == KB) { kb = 0; k += PACK; }
      }
    }
    int s = 0;
    uint32_t ring_phase = 0;
    int owner = 0;                 // producer warp that owns the next block
    bool ok = true;
    uint32_t touched = 0;

    // Copies one block (128 rows x 128 bytes) whose first tap is k (k < 0: no valid row, zeros):
    // 8 lanes copy one row; lane group `grp` owns rows 32 grp .. 32 grp + 31.
    auto gather_block = [&](uint32_t dst, const int* cur, int k, int kb) {
      const int k_lane = k + sub;                        // this lane's tap
      const bool live = k >= 0 && (PACK > 1 ? k_lane < K : chunk * 8 < min(64, Cin - kb * 64));
      const uint8_t* lane_src = data + (size_t)kb * 128 + ch_off;
      const int* irow = cur + (live ? k_lane : 0) * TILE_R + grp * 32;
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        int4 r4 = make_int4(-1, -1, -1, -1);
        if (live) r4 = *reinterpret_cast<const int4*>(irow + 4 * q);
        const int rid[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int r = grp * 32 + 4 * q + j;
          const int idx = rid[j];
#ifndef OC_NOCOPY
          cp_async_16(dst + r * 128 + ((chunk ^ ((4 * q + j) & 7)) << 4),
                      lane_src + (size_t)(idx < 0 ? 0 : idx) * row_bytes, idx >= 0 ? 16u : 0u);
#endif
        }
      }
    };

    uint32_t it = 0;
    for (int64_t tile = t_begin; tile < t_end && ok; tile += t_step, ++it) {
      const int buf = (int)(it & 1u);
      if (!mbar_wait(ifull_bar(buf), (it >> 1) & 1u, abort_flag, &g_tc_status, 14)) { ok = false; break; }
      const uint32_t mask_all = *(volatile uint32_t*)(smem + L.sidx + buf * IDX_BUF_BYTES);
      if (mask_all >> p.K) bad_index = true;            // not a tile table of K taps
      const uint32_t mask = mask_all & group_taps;
      const int* cur = (const int*)(smem + L.sidx + buf * IDX_BUF_BYTES + IDX_HDR_BYTES);
      // one stage per M tile that has a valid tap in this row tile; a row tile without any
      // still gets one (all-zero) stage, so that the grad_out buffers are handed over uniformly.
      // Block b = (tap b / KB, channel block b % KB); the pair is advanced by counting, a
      // division by the run-time KB in this loop costs as much as the copies themselves.
      int last_m = 0;
      {
        int k = k_lo, kb = kb_lo;
        for (int m = 0; m < m_cnt; ++m) {
          const bool v0 = ((mask >> k) & pmask) != 0;
          if (++kb == KB) { kb = 0; k += PACK; }
          const bool v1 = 2 * (m_lo + m) + 1 < nblk && ((mask >> k) & pmask) != 0;
          if (++kb == KB) { kb = 0; k += PACK; }
          if (v0 || v1) last_m = m;
        }
      }
      bool first = true;
      int k0 = k_lo, kb0 = kb_lo;
      for (int m = 0; m <= last_m && ok; ++m) {
        int k1 = k0, kb1 = kb0 + 1;               // second block of the M tile
        if (kb1 == KB) { kb1 = 0; k1 += PACK; }
        const bool has1 = 2 * (m_lo + m) + 1 < nblk;
        const bool v0 = ((mask >> k0) & pmask) != 0;
        const bool v1 = has1 && ((mask >> k1) & pmask) != 0;
        const int ck0 = k0, ckb0 = kb0;           // this M tile's first block
        k0 = k1; kb0 = kb1 + 1;                   // first block of the next M tile
        if (kb0 == KB) { kb0 = 0; k0 += PACK; }
        if (!(v0 || v1) && !(mask == 0 && m == 0)) continue;
        const bool mine0 = owner == pw;
        if (++owner == PROD_WARPS) owner = 0;
        const bool mine1 = owner == pw;
        if (++owner == PROD_WARPS) owner = 0;
        if (mine0 || mine1) {
          if (!mbar_wait(empty_bar(s), ring_phase ^ 1u, abort_flag, &g_tc_status, 12)) { ok = false; break; }
          const uint32_t a_dst = ring0 + s * (uint32_t)(2 * BLK_BYTES);
          if (mine0) {
            if (lane == 0) {
              hdr[s] = (first ? 1u : 0u) | (m == last_m ? 2u : 0u) | (((touched >> m) & 1u) ? 0u : 8u) |
                       ((uint32_t)m << 8);
              mbar_arrive(full_bar(s));
            }
            gather_block(a_dst, cur, v0 ? ck0 : -1, ckb0);
          } else {
            gather_block(a_dst + BLK_BYTES, cur, v1 ? k1 : -1, has1 ? kb1 : 0);
          }
          cp_async_arrive_noinc(full_bar(s));
        }
        touched |= 1u << m;
        first = false;
        if (++s == NS) { s = 0; ring_phase ^= 1u; }
      }
      __syncwarp();                                   // every lane has read its indices of this tile
      if (lane == 0) mbar_arrive(iempty_bar(buf));
    }
    // end marker for the MMA warp: a stage without copies whose header says END
    {
      const bool mine0 = owner == pw;
      if (++owner == PROD_WARPS) owner = 0;
      const bool mine1 = owner == pw;
      if ((mine0 || mine1) && ok && mbar_wait(empty_bar(s), ring_phase ^ 1u, abort_flag, &g_tc_status, 13)) {
        if (mine0 && lane == 0) {
          hdr[s] = 4u;
          misc[18] = touched;
          mbar_arrive(full_bar(s));
        }
        cp_async_arrive_noinc(full_bar(s));
      }
    }
    if (bad_index) atomicMax(&g_tc_status, 90);
    cp_async_wait_all();
  } else if (warp == LOADER_WARP) {
    // ===================================================================== index loader
    // Per row tile: the header of the tile-table block and the index rows of the taps this CTA's
    // M tiles cover (a contiguous range of taps), two bulk copies issued by lane 0.
    const uint8_t* src = (const uint8_t*)p.tiled;
    const int b_lo = 2 * m_lo, b_hi = min(p.nblk, 2 * (m_lo + m_cnt));      // blocks of this CTA
    const int k_first = p.PACK > 1 ? b_lo * p.PACK : b_lo / p.KB;
    const int k_end = min(p.K, p.PACK > 1 ? b_hi * p.PACK : (b_hi + p.KB - 1) / p.KB);
    const uint32_t rows_off = IDX_HDR_BYTES + (uint32_t)k_first * TILE_R * 4;
    const uint32_t rows_len = (uint32_t)(k_end - k_first) * TILE_R * 4;
    uint32_t it = 0;
    for (int64_t tile = t_begin; tile < t_end; tile += t_step, ++it) {
      const int b = (int)(it & 1u);
      if (it >= 2 && !mbar_wait(iempty_bar(b), ((it >> 1) - 1u) & 1u, abort_flag, &g_tc_status, 10)) break;
      if (lane == 0) {
        const uint8_t* blk = src + (size_t)tile * p.tiled_block_bytes;
        const uint32_t dst = s_base + L.sidx + b * IDX_BUF_BYTES;
        mbar_arrive_expect_tx(ifull_bar(b), IDX_HDR_BYTES + rows_len);
        bulk_g2s(dst, blk, IDX_HDR_BYTES, ifull_bar(b));
        bulk_g2s(dst + rows_off, blk + rows_off, rows_len, ifull_bar(b));
      }
      __syncwarp();
    }
  } else if (gq >= 0) {
    // ===================================================================== grad_out loaders
    // Four warps, each 32 rows of the tile: dense rows, NTW columns, as GB swizzled 64-column
    // blocks; 8 lanes copy one row.  Lane l first reads which row of grad_out stands at
    // position 32 gq + l of the tile (the row order of the tile table, or the position itself).
    const uint8_t* gout = (const uint8_t*)p.gout;
    const uint32_t grow_bytes = (uint32_t)p.Cout * 2;
    const int chunk = lane & 7, rsub = lane >> 3;
    uint32_t it = 0;
    for (int64_t tile = t_begin; tile < t_end; tile += t_step, ++it) {
      const int b = (int)(it & 1u);
      const int64_t pos = tile * TILE_R + gq * 32 + lane;
      int my_row = -1;
      if (pos < p.n_out) my_row = p.perm ? p.perm[pos] : (int)pos;
      if (my_row >= p.n_out) my_row = -1;                   // not a row number: zeros
      if (!mbar_wait(gempty_bar(b), ((it >> 1) & 1u) ^ 1u, abort_flag, &g_tc_status, 11)) break;
      const uint32_t g_dst = s_base + L.gbuf + b * (uint32_t)(p.GB * BLK_BYTES) + (uint32_t)gq * 32u * 128u;
      for (int gb = 0; gb < p.GB; ++gb) {
        const int col = n0 + gb * 64 + chunk * 8;
        const bool col_ok = col < p.Cout && gb * 64 + chunk * 8 < p.NTW;
        const uint8_t* col_src = gout + (size_t)col * 2;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + rsub;                       // row of this warp's quarter
          const int row = __shfl_sync(0xffffffffu, my_row, r);
          const bool v = col_ok && row >= 0;
          cp_async_16(g_dst + gb * BLK_BYTES + r * 128 + ((chunk ^ (r & 7)) << 4),
                      v ? col_src + (size_t)row * grow_bytes : gout, v ? 16u : 0u);
        }
      }
      cp_async_arrive_noinc(gfull_bar(b));
    }
    cp_async_wait_all();
  } else if (warp == MMA_WARP) {
    // ===================================================================== MMA issuer
    // (all 32 lanes run the loop so that it stays warp-uniform; one elected lane issues)
    {
      const uint32_t idesc = make_idesc(BF16 ? 1 : 0, 1, 1, 128, p.NTW);   // both operands MN-major
      // MN-major, 128-byte swizzle: 64-element atoms along M / N are BLK_BYTES apart (leading
      // offset), groups of 8 rows along K are 1024 B apart (stride offset).  Descriptors are
      // formed by adding (offset >> 4) to the low word of the descriptor of slot 0, which
      // issues about twice as fast as rebuilding them from a run-time address.
      const uint64_t da0 = make_desc_sw128(s_base + L.ring, BLK_BYTES, 1024);
      const uint64_t dg0 = make_desc_sw128(s_base + L.gbuf, BLK_BYTES, 1024);
      const uint64_t desc_hi = da0 & 0xffffffff00000000ull;
      const uint32_t la0 = (uint32_t)da0, lg0 = (uint32_t)dg0;
      const uint32_t a_step = (uint32_t)(2 * BLK_BYTES) >> 4, g_step = (uint32_t)(p.GB * BLK_BYTES) >> 4;
      int s = 0;
      uint32_t ring_phase = 0;
      uint32_t gb_sel = 0, g_phase = 0;   // g_phase: bit b = phase of grad_out buffer b
      for (;;) {
        if (!mbar_wait(full_bar(s), ring_phase, abort_flag, &g_tc_status, 16)) break;
        tc_fence_after();
        const uint32_t h = hdr[s];
        if (h & 4u) break;
        if (h & 1u) {   // first stage of a row tile: its grad_out block must have landed
          if (!mbar_wait(gfull_bar(gb_sel), (g_phase >> gb_sel) & 1u, abort_flag, &g_tc_status, 17)) break;
          tc_fence_after();
        }
        const uint32_t m = h >> 8;
        const uint32_t la = la0 + (uint32_t)s * a_step, lg = lg0 + gb_sel * g_step;
        const uint32_t d_tmem = tmem_base + m * (uint32_t)p.NTW;
#pragma unroll
        for (uint32_t ks = 0; ks < TILE_R / 16; ++ks)
#ifndef OC_NOMMA
          if (elect_one())
            umma_f16(d_tmem, desc_hi | (la + ks * 128), desc_hi | (lg + ks * 128), idesc, ((h & 8u) && ks == 0) ? 0u : 1u);
#endif
        if (elect_one()) umma_commit(empty_bar(s));
        if (h & 2u) {   // last stage of the row tile: release the grad_out buffer
          if (elect_one()) umma_commit(gempty_bar(gb_sel));
          g_phase ^= 1u << gb_sel;
          gb_sel ^= 1u;
        }
        if (++s == S) { s = 0; ring_phase ^= 1u; }
      }
      __syncwarp();
      if (elect_one()) umma_commit(done_bar);
      mbar_wait(done_bar, 0, abort_flag, &g_tc_status, 18);   // all MMAs retired
    }
    __syncwarp();
  }
  // warps 0-3 have no role in the main loop: they wait here without polling.

  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {}
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  // ------------------------------------------------------------------------ epilogue
  // Warp w reads TMEM lanes 32*(w%4).. of the M tiles m = w/4, w/4 + 3, ... (warps 0-11).
  if (warp < 12 && !*abort_flag) {
    const uint32_t touched = misc[18];
    const int q = warp & 3;
    const int mrow = q * 32 + lane;                    // row of the M tile = (block half, channel)
    for (int m = warp >> 2; m < m_cnt; m += 3) {
      const int b = 2 * (m_lo + m) + (mrow >> 6);
      const int e = mrow & 63;                           // element of the block: (tap, channel) when packed
      const int k = p.PACK > 1 ? b * p.PACK + e / p.Cin : b / p.KB;
      const int ci = p.PACK > 1 ? e % p.Cin : (b % p.KB) * 64 + e;
      const bool row_ok = b < p.nblk && k < p.K && ci < p.Cin;
      const bool has = (touched >> m) & 1u;
      float* dst = p.partial + (((int64_t)slice * p.K + (row_ok ? k : 0)) * p.Cin + (row_ok ? ci : 0)) * p.Cout + n0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + m * (uint32_t)p.NTW;
      for (int c0 = 0; c0 < p.NTW; c0 += 16) {
        uint32_t r[16];
        if (has) {          // warp-uniform
          tmem_ld16(taddr + c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) r[j] = 0u;
        }
        if (row_ok && n0 + c0 < p.Cout) {
          float4* d4 = (float4*)(dst + c0);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            d4[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                __uint_as_float(r[4 * j + 3]));
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

struct Plan {
  int KB, PACK, nblk, n_mt, NTW, GB, n_tiles_n, mt_per_cta, groups, stages, tmem_cols, slices;
  int64_t tiles_per_slice;
  uint32_t smem_bytes;
  bool ok;
};

static Plan make_plan(int K, int Cin, int Cout, int64_t n_out, int dtype) {
  Plan P = {};
  P.ok = false;
  if (!(dtype == OC_F16 || dtype == OC_BF16)) return P;
  if (Cin < 16 || Cin % 16 != 0 || Cout < 16 || Cout % 16 != 0) return P;
  if (K < 1 || K > OC_MAX_TAPS) return P;
  P.KB = (Cin + 63) / 64;
  P.PACK = (Cin == 16 || Cin == 32) ? 64 / Cin : 1;        // taps that share one 64-wide block
  P.nblk = P.PACK > 1 ? (K + P.PACK - 1) / P.PACK : K * P.KB;
  P.n_mt = (P.nblk + 1) / 2;
  P.n_tiles_n = (Cout + 127) / 128;
  P.NTW = Cout <= 128 ? Cout : 128;
  P.GB = (P.NTW + 63) / 64;
  P.mt_per_cta = 512 / P.NTW;
  if (P.mt_per_cta > MAX_MT) P.mt_per_cta = MAX_MT;
  if (P.mt_per_cta > P.n_mt) P.mt_per_cta = P.n_mt;
  P.groups = (P.n_mt + P.mt_per_cta - 1) / P.mt_per_cta;
  // balance the groups
  P.mt_per_cta = (P.n_mt + P.groups - 1) / P.groups;
  P.tmem_cols = 32;
  while (P.tmem_cols < P.mt_per_cta * P.NTW) P.tmem_cols *= 2;
  if (P.tmem_cols > 512) return P;
  const uint32_t budget = 227 * 1024 - 1024;
  int stages = MAX_STAGES;
  while (stages > 2 && smem_layout(P.GB, stages).total > budget) --stages;
  if (smem_layout(P.GB, stages).total > budget) return P;
  P.stages = stages;
  P.smem_bytes = smem_layout(P.GB, stages).total + 1024;
  const int64_t n_tiles = cdiv(n_out > 0 ? n_out : 1, TILE_R);
  int64_t slices = sm_count() / (P.groups * P.n_tiles_n);
  if (slices < 1) slices = 1;
  if (slices > n_tiles) slices = n_tiles;
  P.tiles_per_slice = cdiv(n_tiles, slices);
  P.slices = (int)cdiv(n_tiles, P.tiles_per_slice);
  P.ok = true;
  return P;
}

}  // namespace wg

bool wgrad_tc_supported(int K, int Cin, int Cout, int dtype) { return wg::make_plan(K, Cin, Cout, 1, dtype).ok; }

// workspace = per-slice partials, then room for a tile table (used when the caller has none)
static size_t wgrad_tc_partial_bytes(const wg::Plan& P, int K, int Cin, int Cout) {
  return align_up((size_t)P.slices * K * Cin * Cout * sizeof(float), 256);
}

size_t wgrad_tc_workspace_bytes(int K, int Cin, int Cout, int64_t n_out) {
  const wg::Plan P = wg::make_plan(K, Cin, Cout, n_out, OC_F16);
  return wgrad_tc_partial_bytes(P, K, Cin, Cout) + align_up(tile_table_bytes(n_out, K), 256);
}

template <bool BF16>
static int launch_wgrad_tc_t(const wg::Params& prm, const wg::Plan& P, cudaStream_t s) {
  auto kern = wg::wgrad_tc_kernel<BF16>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  OC_CUDA_OK(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    OC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured_dev = dev;
  }
  dim3 grid((unsigned)P.slices, (unsigned)P.groups, (unsigned)P.n_tiles_n);
  kern<<<grid, wg::THREADS, P.smem_bytes, s>>>(prm);
  OC_LAUNCH_OK("wgrad_tc_kernel");
  return OC_OK;
}

int launch_wgrad_tc(const WgradArgs& a, float* grad_w, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  const wg::Plan P = wg::make_plan(a.K, a.Cin, a.Cout, a.n_out, a.dtype);
  OC_REQUIRE(P.ok, OC_EINVAL, "wgrad_tc: unsupported shape");
  OC_REQUIRE(a.n_out <= INT32_MAX, OC_EINVAL, "wgrad_tc: more than 2^31 - 1 rows");
  const size_t partial_bytes = wgrad_tc_partial_bytes(P, a.K, a.Cin, a.Cout);
  const size_t need = partial_bytes + (a.tiled ? 0 : tile_table_bytes(a.n_out, a.K));
  OC_REQUIRE(workspace && workspace_bytes >= need, OC_ENOMEM, "wgrad_tc: workspace %zu < %zu", workspace_bytes, need);
  OC_REQUIRE(((uintptr_t)a.data % 16) == 0 && ((uintptr_t)a.grad_out % 16) == 0 && ((uintptr_t)workspace % 16) == 0 &&
                 ((uintptr_t)a.tiled % 16) == 0,
             OC_EINVAL, "wgrad_tc: data, grad_out, tile table and workspace must be 16-byte aligned");
  const void* tiled = a.tiled;
  if (!tiled) {   // plain table: regroup it first (one pass over the table)
    void* tt = (char*)workspace + partial_bytes;
    int rc = launch_tile_table(a.table, a.idx_bytes, a.table_cols, a.taps, a.K, a.n_out, a.n_in, nullptr, tt, s);
    if (rc) return rc;
    tiled = tt;
  }
  wg::Params prm;
  prm.data = a.data; prm.gout = a.grad_out; prm.tiled = tiled; prm.perm = a.tiled ? a.perm : nullptr;
  prm.tiled_block_bytes = (uint32_t)tile_table_block_bytes(a.K); prm.partial = (float*)workspace;
  prm.n_out = a.n_out; prm.tiles_per_slice = P.tiles_per_slice;
  prm.K = a.K; prm.Cin = a.Cin; prm.Cout = a.Cout; prm.KB = P.KB; prm.PACK = P.PACK; prm.nblk = P.nblk; prm.NTW = P.NTW;
  prm.GB = P.GB; prm.mt_per_cta = P.mt_per_cta; prm.stages = P.stages; prm.tmem_cols = P.tmem_cols;
  int rc = a.dtype == OC_BF16 ? launch_wgrad_tc_t<true>(prm, P, s) : launch_wgrad_tc_t<false>(prm, P, s);
  if (rc) return rc;
  return reduce_partials((const float*)workspace, P.slices, (int64_t)a.K * a.Cin * a.Cout, grad_w, s);
}

}  // namespace oc
