/* liboctconv — C ABI of the B200 (sm_100a) octree sparse-convolution hot path.
 *
 * The reference project (octree-nn/ocnn-pytorch) is pure Python and has no FFI;
 * its plug-in seams for this path are Python callables.  Each entry point below
 * names the reference interface (file:line inside the reference project) whose
 * work it replaces.  Conventions shared by every entry point:
 *
 *  - All pointers are raw device pointers unless the name starts with `h_`
 *    (host memory).  Tensors are row-major and contiguous.
 *  - `stream` is a cudaStream_t passed as void*; work is enqueued on it.
 *  - Nothing allocates device memory (except where stated): the caller passes
 *    outputs and, where an `*_workspace_bytes` query exists, a workspace.
 *  - Return value: OC_OK (0) or a negative OC_E* code; oc_last_error() returns
 *    a thread-local message for the last failure on the calling thread.
 *  - Feature dtypes use the OC_F32 / OC_F16 / OC_BF16 codes.  Index tables are
 *    int64 (the reference dtype, `idx_bytes` = 8) or int32 (`idx_bytes` = 4).
 *  - A neighbour table is addressed as table[row * table_cols + taps[k]] for
 *    tap k; `h_taps` is a host array of K column numbers.  This covers the
 *    reference's sub-kernels (column subsets, ocnn/octree/octree.py:98-106,517-523)
 *    and the mirrored taps of the stride-1 input gradient without materialising
 *    a second table.
 */
#ifndef OCTCONV_H_
#define OCTCONV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  OC_OK = 0,
  OC_EINVAL = -1,   /* bad argument (shape, dtype, null pointer, unsupported size) */
  OC_ENOMEM = -2,   /* workspace too small */
  OC_ECUDA = -3,    /* CUDA runtime error */
  OC_ETIMEOUT = -4  /* a bounded device-side wait expired; results are invalid */
};

enum { OC_F32 = 0, OC_F16 = 1, OC_BF16 = 2 };

/* coordinate / batch-id element types accepted by oc_xyz2key and the build */
enum { OC_I64 = 10, OC_I32 = 11, OC_COORD_F32 = 12, OC_COORD_F64 = 13, OC_I16 = 14 };

#define OC_MAX_TAPS 27

int oc_version(void);
const char* oc_last_error(void);

/* Device-side waits in the tensor-core kernels are bounded; a wait that expires
 * makes the kernel unwind and sets a sticky per-device status word.  This call
 * synchronises `stream`, returns OC_ETIMEOUT if the word is set (and clears it),
 * OC_OK otherwise.  No counterpart in the reference (its kernels cannot time out). */
int oc_status_check(void* stream);

/* ---- Morton ("shuffled") keys ------------------------------------------- */

/* ocnn/octree/shuffled_key.py:60-90 (xyz2key).  x,y,z (and b, may be NULL) are
 * arrays of `coord_dtype`; values are truncated toward zero like `.long()`,
 * masked to `depth` bits and interleaved; key = (b << 48) | morton. */
int oc_xyz2key(const void* x, const void* y, const void* z, const void* b,
               int coord_dtype, int64_t n, int depth, int64_t* key, void* stream);

/* ocnn/octree/shuffled_key.py:93-115 (key2xyz).  Decodes ceil(depth/3)*3 bits
 * per axis exactly as the reference's 9-bit chunk loop does. */
int oc_key2xyz(const int64_t* key, int64_t n, int depth, int64_t* x, int64_t* y,
               int64_t* z, int64_t* b, void* stream);

/* ---- Octree construction ------------------------------------------------- */

/* ocnn/octree/octree.py:201-287 (Octree.build_octree) + points.py:223-244
 * (Points.normalize), in two calls so that the caller can allocate exact-size
 * outputs after a single device->host read of the node counts.
 *
 * oc_build_octree_count: scales points ((p - bbmin) * mul, two fp32 roundings),
 * makes keys, radix-sorts them, and derives the unique node keys of every
 * depth in `workspace`.  Writes nnum_nempty[d] for d = full_depth..depth into
 * h_nnum_nempty[d] (host array of depth+1 entries; entries below full_depth are
 * set to batch_size * 8^d) and synchronises `stream` once.
 * batch_id may be NULL (batch_size 1); bid_dtype is OC_COORD_F32, OC_I64 or OC_I32. */
size_t oc_build_workspace_bytes(int64_t npts, int depth, int full_depth, int batch_size);
int oc_build_octree_count(const float* points, const void* batch_id, int bid_dtype,
                          int64_t npts, int depth, int full_depth, int batch_size,
                          const float* h_bbmin3, float mul, void* workspace,
                          size_t workspace_bytes, int64_t* h_nnum_nempty, void* stream);

/* oc_build_octree_emit: fills keys[d] (int64, nnum[d]) and children[d] (int32,
 * nnum[d]) for d = 0..depth (h_keys / h_children are host arrays of depth+1
 * device pointers), the averaged leaf signals (octree.py:273-281: points in
 * [0, 2^depth] units, L2-normalised normal sums, feature means; any of the
 * three outputs may be NULL together with its input) and idx (int64, npts:
 * point -> rank of its non-empty leaf).  Must follow oc_build_octree_count on
 * the same workspace and arguments. */
int oc_build_octree_emit(const float* points, const float* normals, const float* features,
                         int nfeat, int64_t npts, int depth, int full_depth, int batch_size,
                         const float* h_bbmin3, float mul, const void* workspace,
                         const int64_t* h_nnum_nempty, int64_t* const* h_keys,
                         int32_t* const* h_children, float* out_points, float* out_normals,
                         float* out_features, int64_t* out_idx, void* stream);

/* ocnn/octree/octree.py:289-321 (octree_grow_full): keys = (b << 48) | m,
 * children = arange, for one dense layer of batch_size * 8^depth nodes. */
int oc_full_layer(int depth, int batch_size, int64_t* keys, int32_t* children, void* stream);

/* ocnn/octree/octree.py:353-402 (octree_grow): keys of depth d from the keys of
 * the non-empty nodes of depth d-1 (children_p >= 0), children = arange. */
int oc_grow_layer(const int64_t* keys_p, const int32_t* children_p, int64_t nnum_p,
                  int64_t* keys, int32_t* children, void* stream);

/* ---- Neighbour tables ---------------------------------------------------- */

/* ocnn/octree/octree.py:411-428 (construct_neigh, dense branch): table of
 * batch_size * 8^depth rows x 27 int64, -1 outside the grid. */
int oc_neigh_full(int depth, int batch_size, int64_t* neigh, void* stream);

/* ocnn/octree/octree.py:430-439 (construct_neigh, parent-derived branch):
 * neigh_p (nnum_p, 27) and children_p (nnum_p) of depth d-1 -> neigh (8 *
 * nnum_nempty_p, 27) of depth d.  If neigh32 is non-NULL an int32 copy of the
 * table is written too. */
int oc_neigh_from_parent(const int64_t* neigh_p, const int32_t* children_p, int64_t nnum_p,
                         int64_t* neigh, int32_t* neigh32, void* stream);

/* ocnn/octree/octree.py:160-172 (nempty_index): indices of the nodes with
 * children >= 0, ascending.  `count` = number expected by the caller
 * (nnum_nempty); a mismatch is reported as OC_EINVAL only in debug builds. */
size_t oc_nempty_index_workspace_bytes(int64_t nnum);
int oc_nempty_index(const int32_t* children, int64_t nnum, int64_t* index,
                    void* workspace, size_t workspace_bytes, void* stream);

/* ocnn/octree/octree.py:188-199, 490-523 (remap_nempty_neigh / get_neigh):
 * out[r, j] = remap(neigh[row(r), h_taps[j]]), row(r) = rows ? rows[r] :
 * r * row_stride, remap(e) = (children && e >= 0) ? children[e] : e.
 * out is (n_rows, K) with out_bytes-wide integers (8 or 4). */
int oc_neigh_variant(const int64_t* neigh, const int32_t* children, const int64_t* rows,
                     int64_t row_stride, int64_t n_rows, const int* h_taps, int K,
                     void* out, int out_bytes, void* stream);

/* Inverse of a neighbour table (no reference counterpart as a function; it
 * replaces the atomics of scatter_add in ocnn/nn/octree_conv.py:145-168 by a
 * gather): inv[table[r, h_taps[k]], k] = r, all other entries -1.  inv is
 * (n_targets, K) int32 and must be pre-filled by this call (it is). */
int oc_neigh_inverse(const void* table, int idx_bytes, int64_t n_rows, int table_cols,
                     const int* h_taps, int K, int64_t n_targets, int32_t* inv, void* stream);

/* ---- Average / global pooling, per-octree scaling ------------------------------ */

/* octree_avg_pool, ocnn/nn/octree_pool.py:68-103 (the reference multiplies a sparse COO matrix):
 *   out[r] = v_r * sum_k data[table[r, taps[k]]],  v_r = 1 / (#entries >= 0 + 1e-8);  val[r] = v_r
 * (fp32, may be NULL).  Gradient: grad_in[n] = sum_k val[t] * grad_out[t], t = table_t[n, taps_t[k]],
 * with the mirrored / inverse table of the scatter direction (as for oc_conv_fwd). */
int oc_avgpool_fwd(const void* data, const void* table, int idx_bytes, int table_cols,
                   const int* h_taps, int K, int64_t n_out, int C, int dtype, void* out, float* val,
                   void* stream);
int oc_avgpool_bwd(const void* grad_out, const float* val, const void* table_t, int idx_bytes,
                   int table_cols, const int* h_taps, int K, int64_t n_in, int C, int dtype,
                   void* grad_in, void* stream);

/* octree_global_pool, ocnn/nn/octree_pool.py:106-124: mean[b] = sum of the rows of octree b /
 * max(count_b, 1), fp32 (batch, C).  h_offsets (batch+1, host): row ranges of the octrees
 * (oc_batch_offsets); rows of one octree are contiguous. */
size_t oc_global_pool_workspace_bytes(int64_t n, int batch, int C);
int oc_global_pool_fwd(const void* data, const int64_t* h_offsets, int batch, int C, int dtype,
                       float* mean, void* workspace, size_t workspace_bytes, void* stream);

/* out[r] = data[r] * scale[b] for the rows of octree b: the per-octree mask of OctreeDropPath
 * (ocnn/nn/octree_drop.py:14-60) and the gradient of the global mean; scale: device, fp32 (batch). */
int oc_scale_segments(const void* data, const int64_t* h_offsets, int batch, const float* scale, int C,
                      int dtype, void* out, void* stream);

/* ---- Key search and point interpolation ------------------------------------ */

/* Octree.search_key, ocnn/octree/octree.py:464-488: idx[i] = position of query[i] in the
 * ascending node keys keys[0..n) (all nodes of a depth, or its non-empty nodes), -1 if absent.
 * Octree.search_xyzb (:448-462) = oc_xyz2key on the query coordinates, then this. */
int oc_search_key(const int64_t* keys, int64_t n, const int64_t* query, int64_t m, int64_t* idx,
                  void* stream);

/* Steps 1-2 of octree_linear_pts, ocnn/nn/octree_interp.py:63-88, for points pts (m,4) =
 * (x, y, z, batch) already scaled to [0, 2^depth): the 8 cell centres around each point,
 * idx8 (m,8) = their rows among `keys` or -1 (also outside [0, 2^depth) when bound_check;
 * without it coordinates wrap modulo 2^depth exactly as xyz2key does), w8 (m,8) fp32 =
 * |prod_d ((1 - g_d) - frac_d)|. */
int oc_interp_corners(const int64_t* keys, int64_t n, const float* pts, int64_t m, int depth,
                      int bound_check, int64_t* idx8, float* w8, void* stream);

/* octree_nearest_pts, ocnn/nn/octree_interp.py:16-48: out[p] = data[idx[p]] or 0 where
 * idx[p] < 0; and its gradient acc[idx[p]] += grad[p] (fp32 accumulator of the caller,
 * zeroed by the caller, atomics because points share rows: order of summation not fixed,
 * as in the reference's index_add). */
int oc_rows_gather(const void* data, const int64_t* idx, int64_t m, int C, int dtype, void* out,
                   void* stream);
int oc_rows_scatter_add(const void* grad, const int64_t* idx, int64_t m, int C, int dtype, float* acc,
                        void* stream);

/* Step 3 of octree_linear_pts (:90-98, the reference multiplies a sparse COO matrix):
 *   out[p] = sum_j w8[p,j] data[idx8[p,j]] / (sum_j w8[p,j] + 1e-12)  over the corners with idx >= 0,
 * and the gradient with respect to data, acc[idx8[p,j]] += w8[p,j] / (sum + 1e-12) * grad_out[p]
 * (fp32 accumulator as above). */
int oc_interp_linear_fwd(const void* data, const int64_t* idx8, const float* w8, int64_t m, int C,
                         int dtype, void* out, void* stream);
int oc_interp_linear_bwd(const void* grad_out, const int64_t* idx8, const float* w8, int64_t m, int C,
                         int dtype, float* acc, void* stream);

/* ---- Octree convolution -------------------------------------------------- */

/* Gather-GEMM, the forward of ocnn/nn/octree_conv.py:115-143 (forward_gemm) and
 * of ocnn/nn/kernels/conv_fwd_implicit_gemm_splitk.py:118-150:
 *   out[r, :] = sum_k data[table[r, taps[k]], :] . Wk  (+ bias),  r < n_out
 * Wk = weights[k] (Cin x Cout) when w_transposed == 0 with weights (K,Cin,Cout);
 * Wk = weights[k]^T when w_transposed == 1 with weights (K,Cout,Cin).  Entries
 * < 0 contribute zero.  weights are `w_dtype` (OC_F32 or `dtype`), data/out/bias
 * are `dtype`; accumulation is fp32.  The same call serves the input gradient
 * (octree_conv.py:145-168, kernels/conv_bwd_implicit_gemm_splitk.py:204-244)
 * when given the mirrored or inverse table and w_transposed = 1. */
size_t oc_conv_workspace_bytes(int K, int Cin, int Cout, int dtype);
int oc_conv_fwd(const void* data, int64_t n_in, const void* weights, int w_dtype,
                int w_transposed, const void* bias, const void* table, int idx_bytes,
                int table_cols, const int* h_taps, int K, int64_t n_out, int Cin, int Cout,
                int dtype, void* out, void* workspace, size_t workspace_bytes, void* stream);

/* Tile table: the neighbour table of one convolution (the (n_out, table_cols) table that
 * Octree.get_neigh returns, ocnn/octree/octree.py:490-523, restricted to `taps`) regrouped
 * for the tensor-core kernel, which then fetches the indices of 128 output rows with one
 * bulk copy instead of 27 strided loads per row.  Block t covers rows 128 t .. 128 t + 127:
 * a 16-byte header (word 0 = bit mask of the taps that have an entry >= 0 in the block)
 * followed by K rows of 128 int32, row k = column taps[k] (-1 = none, also past n_out).
 * Build it once per (depth, kernel, stride, nempty) and reuse it for every layer and
 * step on that octree level, like the reference caches `neigh`.  The reference has no
 * counterpart; it is optional: oc_conv_fwd with the plain table gives the same result.
 * oc_conv_tiled_supported: 1 where oc_conv_fwd_tiled accepts the shape (fp16 / bf16,
 * Cin and Cout multiples of 16). */
int oc_conv_tiled_supported(int K, int Cin, int Cout, int dtype);
/* masks[r] (int32) = bit k set iff table[r, taps[k]] >= 0: the sort key for row_perm below. */
int oc_tap_masks(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                 int64_t n_rows, int32_t* masks, void* stream);
/* perm (device int32 (n_rows)) = the rows of the table sorted, stably, by oc_tap_masks: the
 * row_perm of oc_tile_table_build below.  An 8-bit LSD radix sort over the K mask bits, the same
 * kernels that sort the point keys in oc_build_octree_count.  The sort key is the mask with its
 * bits reordered: the taps whose frequency over the table is farthest from one half are the most
 * significant (ties: the lower tap first), so rows with a rare tap sit together.  chunk_log2 > 0: the rows are sorted
 * within consecutive chunks of 2^chunk_log2 rows only (key = chunk number, then mask), which keeps
 * the rows of a tile within one neighbourhood of the octree; 0: one sort over all rows. */
size_t oc_tap_order_workspace_bytes(int64_t n_rows);
int oc_tap_order(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                 int64_t n_rows, int chunk_log2, int32_t* perm, void* workspace, size_t workspace_bytes,
                 void* stream);
size_t oc_tile_table_bytes(int64_t n_out, int K);
/* n_in > 0: number of feature rows the table indexes; an entry >= n_in is stored as -1 and
 * the next oc_status_check returns OC_EINVAL (the kernels do not re-check indices).  n_in = 0: no check.
 * The table holds an even number of blocks (a padding block of -1 if needed). */
/* row_perm (device int32 (n_out), a permutation of 0 .. n_out-1, or NULL): position j of the tile
 * table then holds table row row_perm[j].  Grouping rows that share their valid taps makes whole
 * taps empty in a tile, and empty taps are skipped: the inverse table of a stride-2 convolution
 * (oc_neigh_inverse) has 1 to 8 valid taps of 27 per row and which ones depends only on the
 * node's child index, so rows ordered by child index run 3.4 instead of 27 taps per tile.
 * More generally, rows sorted by the bit mask of their valid taps leave every tile with few distinct
 * taps (16.8 instead of 27 stages per tile on the depth-8 benchmark batch, 11 instead of 27 with
 * nempty).  The same array must be given to oc_conv_fwd_tiled / oc_conv_wgrad_tiled. */
int oc_tile_table_build(const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                        int64_t n_out, int64_t n_in, const int32_t* row_perm, void* tiles,
                        size_t tiles_bytes, void* stream);
/* oc_conv_fwd with the table given as a tile table (same K and tap order as at build; out[row_perm[j]]
 * receives position j when the table was built with a row permutation). */
int oc_conv_fwd_tiled(const void* data, int64_t n_in, const void* weights, int w_dtype,
                      int w_transposed, const void* bias, const void* tiles, const int32_t* row_perm,
                      int K, int64_t n_out, int Cin, int Cout, int dtype, void* out, void* workspace,
                      size_t workspace_bytes, void* stream);

/* Weight gradient, ocnn/nn/octree_conv.py:170-202 (weight_gemm) and
 * kernels/conv_bwd_implicit_gemm_splitk.py:246-306:
 *   grad_w[k, ci, co] = sum_r data[table[r, taps[k]], ci] * grad_out[r, co]
 * grad_w is fp32 (K,Cin,Cout).  If grad_bias is non-NULL it receives the column
 * sums of grad_out (fp32, Cout) (conv_bwd_implicit_gemm_splitk.py:344-345). */
size_t oc_conv_wgrad_workspace_bytes(int K, int Cin, int Cout, int64_t n_out, int dtype);
int oc_conv_wgrad(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                  const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                  int Cin, int Cout, int dtype, float* grad_w, float* grad_bias,
                  void* workspace, size_t workspace_bytes, void* stream);
/* oc_conv_wgrad with the table given as a tile table (see oc_tile_table_build); same
 * workspace size.  Given a plain table, oc_conv_wgrad regroups it into the workspace on
 * every call where the tensor-core kernel applies, so the tile table saves that pass. */
int oc_conv_wgrad_tiled(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                        const void* tiles, const int32_t* row_perm, int K, int Cin, int Cout, int dtype,
                        float* grad_w, float* grad_bias, void* workspace, size_t workspace_bytes,
                        void* stream);

/* Depth-wise convolution, ocnn/nn/octree_dwconv.py:30-118:
 *   out[r, c] = sum_k data[table[r, taps[k]], c] * w[k, c]     (weights fp32 (K,C))
 * (also its input gradient, given the mirrored / inverse table), and
 *   grad_w[k, c] = sum_r data[table[r, taps[k]], c] * grad_out[r, c]. */
int oc_dwconv_fwd(const void* data, int64_t n_in, const float* weights, const void* table,
                  int idx_bytes, int table_cols, const int* h_taps, int K, int64_t n_out,
                  int C, int dtype, void* out, void* stream);
size_t oc_dwconv_wgrad_workspace_bytes(int K, int C, int64_t n_out);
int oc_dwconv_wgrad(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                    const void* table, int idx_bytes, int table_cols, const int* h_taps, int K,
                    int C, int dtype, float* grad_w, void* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- Pad / pool / upsample ---------------------------------------------- */

/* ocnn/nn/octree_pad.py:13-39.  pad: out (n_all, C) = fill everywhere, then
 * out[index[j]] = data[j];  depad: out[j] = data[index[j]]  (j < n_nempty). */
int oc_pad(const void* data, const int64_t* index, int64_t n_nempty, int64_t n_all, int C,
           int dtype, float fill, void* out, void* stream);
int oc_depad(const void* data, const int64_t* index, int64_t n_nempty, int C, int dtype,
             void* out, void* stream);

/* ocnn/nn/octree_pool.py:17-38 (octree_max_pool) fused with its pad/depad.
 * For every node p < n_out: j = children_out ? children_out[p] : p; if j < 0 the
 * output row is 0; else out[p] = max_i data[src(8j+i)], src(t) = children_in ?
 * children_in[t] (skipped when < 0, i.e. -inf) : t.  argmax (int64, row j,
 * may be NULL) holds the sibling number 0..7 of the first maximum.
 * nempty=False: children_in = NULL, children_out = children[d-1];
 * nempty=True : children_in = children[d], children_out = NULL. */
int oc_maxpool_fwd(const void* data, const int32_t* children_in, const int32_t* children_out,
                   int64_t n_out, int C, int dtype, void* out, int64_t* argmax, void* stream);
/* Gradient of the above: grad_in (n_in, C) is fully written (zeros elsewhere). */
int oc_maxpool_bwd(const void* grad_out, const int64_t* argmax, const int32_t* children_in,
                   const int32_t* children_out, int64_t n_out, int64_t n_in, int C, int dtype,
                   void* grad_in, void* stream);

/* ocnn/nn/octree_interp.py:140-162 (octree_nearest_upsample) fused with depad:
 * out[m] = data[src(m)], m < n_out.  nempty=False: src(m) = index_coarse[m >> 3]
 * (index_coarse = nempty_index(depth)); nempty=True: src(m) = index_fine[m] >> 3
 * (index_fine = nempty_index(depth+1)).  Exactly one of the two is non-NULL. */
int oc_upsample_fwd(const void* data, const int64_t* index_coarse, const int64_t* index_fine,
                    int64_t n_out, int C, int dtype, void* out, void* stream);
/* Gradient: grad_in[q] = sum of grad_out over the (up to 8) fine rows that copied
 * row q.  nempty=False: children_coarse = children[depth] (rows q with
 * children < 0 get 0); nempty=True: children_fine = children[depth+1]. */
int oc_upsample_bwd(const void* grad_out, const int32_t* children_coarse,
                    const int32_t* children_fine, int64_t n_in, int C, int dtype,
                    void* grad_in, void* stream);

/* ---- Normalisation ------------------------------------------------------- */

/* torch.nn.BatchNorm1d as used by ocnn/nn/octree_norm.py:16 on (N, C) data.
 * oc_colstats: sums[0:C] = sum_n x[n,c] * (w ? w[n,c] : 1) ... two column
 * reductions in one pass: sum_a[c] = sum_n a[n,c], sum_ab[c] = sum_n a[n,c]*b[n,c]
 * (b = a when b is NULL).  Used for (sum x, sum x^2) forward and (sum g, sum g*x)
 * backward.  fp32 outputs, deterministic two-stage reduction. */
size_t oc_colstats_workspace_bytes(int64_t n, int C);
int oc_colstats(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                float* sum_ab, void* workspace, size_t workspace_bytes, void* stream);
/* Same sums as oc_colstats, for callers that have no way to supply a workspace
 * and must not trigger an allocation: hosts whose start-up code reserved the whole
 * GPU for their own arena, or plugin code that only ever sees raw pointers.  The
 * per-block partials go to a 2 MiB array built into the library (every GPU that
 * loads the library keeps that array until the process exits).  Nothing here calls
 * cudaMalloc / cudaFree or any allocating routine.
 *   - Limit: C <= 4096; a larger C is refused with OC_EINVAL and a message that
 *     points to oc_colstats.  The number of row slices shrinks as C grows.
 *   - The first call on each device looks up the array's device address (with
 *     that device current); make that first call outside any stream capture.
 *   - All calls share the one array, which still holds the previous call's
 *     partials; each call overwrites every slot it later reads, so no clearing is
 *     needed, but two calls that overlap on the GPU (different streams) race.
 * No counterpart in the reference: it exists only for these callers. */
int oc_colstats_static(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                       float* sum_ab, void* stream);
/* out[n,c] = x[n,c] * scale[c] + shift[c]   (scale/shift fp32) */
int oc_affine_cols(const void* x, const float* scale, const float* shift, int64_t n, int C,
                   int dtype, void* out, void* stream);
/* grad_in[n,c] = g[n,c] * ka[c] + x[n,c] * kb[c] + kc[c]   (BatchNorm backward) */
int oc_bn_bwd_apply(const void* g, const void* x, const float* ka, const float* kb,
                    const float* kc, int64_t n, int C, int dtype, void* grad_in, void* stream);

/* ocnn/nn/octree_norm.py:19-80 (OctreeGroupNorm).  Rows of octree b are the
 * contiguous range [h_offsets[b], h_offsets[b+1]) (host array, batch+1 entries).
 * stats: mean/inv_std per (b, group) with the reference's eps placement
 * (inv_count = 1/(n_b*cpg + eps), var from centred values, 1/sqrt(var + eps)).
 * fwd: out = (x - mean) * inv_std * weight + bias. */
size_t oc_gn_workspace_bytes(int batch, int C);
int oc_gn_fwd(const void* x, const int64_t* h_offsets, int batch, int C, int groups, float eps,
              const float* weight, const float* bias, int dtype, void* out, float* mean,
              float* inv_std, void* workspace, size_t workspace_bytes, void* stream);
int oc_gn_bwd(const void* grad_out, const void* x, const int64_t* h_offsets, int batch, int C,
              int groups, float eps, const float* weight, const float* mean,
              const float* inv_std, int dtype, void* grad_in, float* grad_weight,
              float* grad_bias, void* workspace, size_t workspace_bytes, void* stream);

/* ocnn/octree/octree.py:133-145 (batch_id): row offsets of each octree at one
 * depth, from the sorted keys (key >> 48) — optionally over non-empty nodes only
 * (children != NULL).  h_offsets: host array of batch+1 entries; synchronises. */
int oc_batch_offsets(const int64_t* keys, const int32_t* children, int64_t nnum, int batch,
                     int64_t* h_offsets, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* OCTCONV_H_ */
