// C-ABI glue: error reporting, device queries and the convolution entry points
// (argument validation, workspace carving and kernel selection).
#include <stdarg.h>

#include "oc_common.cuh"
#include "conv_internal.cuh"

namespace oc {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) cached = n;
    cached_dev = dev;
  }
  return cached;
}

struct ConvPlan {
  bool tc;
  size_t w_off, w_bytes, status_off, total;
};

static ConvPlan conv_plan(int K, int Cin, int Cout, int dtype) {
  ConvPlan p;
  p.tc = conv_tc_supported(K, Cin, Cout, dtype);
  p.w_off = 0;
  p.w_bytes = p.tc ? conv_tc_weight_bytes(K, Cin, Cout) : (size_t)K * Cin * Cout * sizeof(float);
  p.status_off = align_up(p.w_bytes, 256);
  p.total = p.status_off + 256;
  return p;
}

struct WgradPlan {
  bool tc;
  int splits;
  size_t partial_off, partial_bytes, stats_off, stats_bytes, total;
};

static WgradPlan wgrad_plan(int K, int Cin, int Cout, int64_t n_out, int dtype) {
  WgradPlan p;
  p.tc = wgrad_tc_supported(K, Cin, Cout, dtype);
  p.splits = p.tc ? 0 : wgrad_fma_splits(K, Cin, Cout, n_out);
  p.partial_off = 0;
  p.partial_bytes = p.tc ? wgrad_tc_workspace_bytes(K, Cin, Cout, n_out)
                         : (size_t)p.splits * K * Cin * Cout * sizeof(float);
  p.stats_off = align_up(p.partial_bytes, 256);
  p.stats_bytes = colstats_workspace_bytes(n_out, Cout);
  p.total = p.stats_off + p.stats_bytes;
  return p;
}

static int check_conv_common(const char* who, int K, int Cin, int Cout, int dtype, int idx_bytes,
                             int table_cols, int64_t n_in, int64_t n_out) {
  OC_REQUIRE(dtype == OC_F32 || dtype == OC_F16 || dtype == OC_BF16, OC_EINVAL, "%s: bad dtype %d", who, dtype);
  OC_REQUIRE(K >= 1 && K <= OC_MAX_TAPS, OC_EINVAL, "%s: K %d not in [1,27]", who, K);
  OC_REQUIRE(Cin >= 1 && Cout >= 1 && Cin <= 65536 && Cout <= 65536, OC_EINVAL, "%s: bad channels (%d, %d)", who, Cin, Cout);
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "%s: idx_bytes must be 4 or 8", who);
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "%s: table_cols %d not in [1,27]", who, table_cols);
  OC_REQUIRE(n_in >= 0 && n_out >= 0 && n_in < (1LL << 31) && n_out < (1LL << 31), OC_EINVAL,
             "%s: row counts must be in [0, 2^31)", who);
  return OC_OK;
}

}  // namespace oc

using namespace oc;

extern "C" int oc_version(void) { return 100; }

extern "C" const char* oc_last_error(void) { return g_err; }

extern "C" int oc_status_check(void* stream) {
  int v = 0;
  int rc = read_tc_status((cudaStream_t)stream, &v);
  if (rc) return rc;
  OC_REQUIRE(v != 90, OC_EINVAL,
             "a neighbour index >= n_in was met while building a tile table, or a kernel was given a tile "
             "table built for another K; such entries were treated as -1, so results of kernels launched "
             "since the last check are wrong");
  OC_REQUIRE(v == 0, OC_ETIMEOUT,
             "a bounded device-side wait expired in a tensor-core kernel (role code %d); results of "
             "kernels launched since the last check are invalid", v);
  return OC_OK;
}

extern "C" size_t oc_conv_workspace_bytes(int K, int Cin, int Cout, int dtype) {
  if (K < 1 || K > OC_MAX_TAPS || Cin < 1 || Cout < 1) return 0;
  return conv_plan(K, Cin, Cout, dtype).total;
}

// `tiles` non-null: the table comes as a tile table (tensor-core shapes only).
static int conv_fwd_impl(const char* who, const void* data, int64_t n_in, const void* weights, int w_dtype,
                         int w_transposed, const void* bias, const void* table, int idx_bytes,
                         int table_cols, const int* h_taps, const void* tiles, const int32_t* perm, int K,
                         int64_t n_out, int Cin, int Cout, int dtype, void* out, void* workspace,
                         size_t workspace_bytes, void* stream) {
  int rc = check_conv_common(who, K, Cin, Cout, dtype, idx_bytes, table_cols, n_in, n_out);
  if (rc) return rc;
  OC_REQUIRE(w_dtype == OC_F32 || w_dtype == dtype, OC_EINVAL, "%s: weights must be fp32 or the data dtype", who);
  ConvArgs a;
  if (tiles) {
    for (int k = 0; k < K; ++k) a.taps.t[k] = k;   // the tile table already holds the chosen taps, in order
  } else {
    rc = make_taps(h_taps, K, table_cols, &a.taps, who);
    if (rc) return rc;
  }
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(weights && (table || tiles) && out && workspace, OC_EINVAL, "%s: null pointer", who);
  OC_REQUIRE(data || n_in == 0, OC_EINVAL, "%s: null data", who);
  const ConvPlan P = conv_plan(K, Cin, Cout, dtype);
  OC_REQUIRE(P.tc || !tiles, OC_EINVAL,
             "%s: a tile table needs fp16/bf16 data and channel counts that are multiples of 16 "
             "(ask oc_conv_tiled_supported); use oc_conv_fwd with the plain table", who);
  OC_REQUIRE(workspace_bytes >= P.total, OC_ENOMEM, "%s: workspace %zu < %zu bytes", who, workspace_bytes, P.total);
  a.data = data; a.n_in = n_in; a.bias = bias; a.table = table; a.tiled = tiles; a.perm = perm; a.idx_bytes = idx_bytes;
  a.table_cols = table_cols; a.K = K; a.n_out = n_out; a.Cin = Cin; a.Cout = Cout; a.dtype = dtype;
  a.out = out;
  cudaStream_t s = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  if (P.tc) {
    rc = prep_weights_tc(weights, w_dtype, K, Cin, Cout, w_transposed, dtype, ws + P.w_off, s);
    if (rc) return rc;
    return launch_conv_tc(a, ws + P.w_off, (int*)(ws + P.status_off), s);
  }
  rc = prep_weights_f32(weights, w_dtype, K, Cin, Cout, w_transposed, (float*)(ws + P.w_off), s);
  if (rc) return rc;
  return launch_conv_fma(a, (const float*)(ws + P.w_off), s);
}

extern "C" int oc_conv_fwd(const void* data, int64_t n_in, const void* weights, int w_dtype,
                           int w_transposed, const void* bias, const void* table, int idx_bytes,
                           int table_cols, const int* h_taps, int K, int64_t n_out, int Cin,
                           int Cout, int dtype, void* out, void* workspace, size_t workspace_bytes,
                           void* stream) {
  return conv_fwd_impl("oc_conv_fwd", data, n_in, weights, w_dtype, w_transposed, bias, table, idx_bytes,
                       table_cols, h_taps, nullptr, nullptr, K, n_out, Cin, Cout, dtype, out, workspace,
                       workspace_bytes, stream);
}

extern "C" int oc_conv_tiled_supported(int K, int Cin, int Cout, int dtype) {
  return (K >= 1 && K <= OC_MAX_TAPS && conv_tc_supported(K, Cin, Cout, dtype)) ? 1 : 0;
}

extern "C" size_t oc_tile_table_bytes(int64_t n_out, int K) {
  if (K < 1 || K > OC_MAX_TAPS || n_out < 0) return 0;
  return tile_table_bytes(n_out, K);
}

extern "C" int oc_tile_table_build(const void* table, int idx_bytes, int table_cols, const int* h_taps,
                                   int K, int64_t n_out, int64_t n_in, const int32_t* row_perm, void* tiles,
                                   size_t tiles_bytes, void* stream) {
  OC_REQUIRE(K >= 1 && K <= OC_MAX_TAPS, OC_EINVAL, "oc_tile_table_build: K %d not in [1,27]", K);
  OC_REQUIRE(idx_bytes == 8 || idx_bytes == 4, OC_EINVAL, "oc_tile_table_build: idx_bytes must be 4 or 8");
  OC_REQUIRE(table_cols >= 1 && table_cols <= 27, OC_EINVAL, "oc_tile_table_build: table_cols %d not in [1,27]", table_cols);
  OC_REQUIRE(n_out >= 0 && n_out < (1LL << 31), OC_EINVAL, "oc_tile_table_build: n_out must be in [0, 2^31)");
  OC_REQUIRE(n_in >= 0 && n_in < (1LL << 31), OC_EINVAL, "oc_tile_table_build: n_in must be in [0, 2^31)");
  TapList taps;
  int rc = make_taps(h_taps, K, table_cols, &taps, "oc_tile_table_build");
  if (rc) return rc;
  if (n_out == 0) return OC_OK;
  OC_REQUIRE(table && tiles, OC_EINVAL, "oc_tile_table_build: null pointer");
  OC_REQUIRE(((uintptr_t)tiles % 16) == 0, OC_EINVAL, "oc_tile_table_build: tiles must be 16-byte aligned");
  OC_REQUIRE(tiles_bytes >= tile_table_bytes(n_out, K), OC_ENOMEM, "oc_tile_table_build: tiles %zu < %zu bytes",
             tiles_bytes, tile_table_bytes(n_out, K));
  return launch_tile_table(table, idx_bytes, table_cols, taps, K, n_out, n_in, row_perm, tiles, (cudaStream_t)stream);
}

extern "C" int oc_conv_fwd_tiled(const void* data, int64_t n_in, const void* weights, int w_dtype,
                                 int w_transposed, const void* bias, const void* tiles, const int32_t* row_perm,
                                 int K, int64_t n_out, int Cin, int Cout, int dtype, void* out, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  OC_REQUIRE(tiles, OC_EINVAL, "oc_conv_fwd_tiled: null tile table");
  // no plain table: its width only has to pass the range check, the taps are 0 .. K-1
  return conv_fwd_impl("oc_conv_fwd_tiled", data, n_in, weights, w_dtype, w_transposed, bias, nullptr, 4,
                       K >= 1 && K <= OC_MAX_TAPS ? K : 1, nullptr, tiles, row_perm, K, n_out, Cin, Cout, dtype, out,
                       workspace, workspace_bytes, stream);
}

extern "C" size_t oc_conv_wgrad_workspace_bytes(int K, int Cin, int Cout, int64_t n_out, int dtype) {
  if (K < 1 || K > OC_MAX_TAPS || Cin < 1 || Cout < 1 || n_out < 0) return 0;
  return wgrad_plan(K, Cin, Cout, n_out, dtype).total;
}

static int conv_wgrad_impl(const char* who, const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                           const void* table, int idx_bytes, int table_cols, const int* h_taps, const void* tiles,
                           const int32_t* perm, int K, int Cin, int Cout, int dtype, float* grad_w, float* grad_bias,
                           void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_conv_common(who, K, Cin, Cout, dtype, idx_bytes, table_cols, n_in, n_out);
  if (rc) return rc;
  WgradArgs a;
  if (tiles) {
    for (int k = 0; k < K; ++k) a.taps.t[k] = k;
  } else {
    rc = make_taps(h_taps, K, table_cols, &a.taps, who);
    if (rc) return rc;
  }
  OC_REQUIRE(grad_w, OC_EINVAL, "%s: null grad_w", who);
  cudaStream_t s = (cudaStream_t)stream;
  if (n_out == 0) {
    OC_CUDA_OK(cudaMemsetAsync(grad_w, 0, (size_t)K * Cin * Cout * 4, s));
    if (grad_bias) OC_CUDA_OK(cudaMemsetAsync(grad_bias, 0, (size_t)Cout * 4, s));
    return OC_OK;
  }
  OC_REQUIRE(grad_out && (table || tiles) && workspace, OC_EINVAL, "%s: null pointer", who);
  OC_REQUIRE(data || n_in == 0, OC_EINVAL, "%s: null data", who);
  const WgradPlan P = wgrad_plan(K, Cin, Cout, n_out, dtype);
  OC_REQUIRE(P.tc || !tiles, OC_EINVAL,
             "%s: a tile table needs fp16/bf16 data and channel counts that are multiples of 16 "
             "(ask oc_conv_tiled_supported); use oc_conv_wgrad with the plain table", who);
  OC_REQUIRE(workspace_bytes >= P.total, OC_ENOMEM, "%s: workspace %zu < %zu bytes", who, workspace_bytes, P.total);
  a.data = data; a.n_in = n_in; a.grad_out = grad_out; a.n_out = n_out; a.table = table; a.tiled = tiles; a.perm = perm;
  a.idx_bytes = idx_bytes; a.table_cols = table_cols; a.K = K; a.Cin = Cin; a.Cout = Cout; a.dtype = dtype;
  char* ws = (char*)workspace;
  if (P.tc) {
    rc = launch_wgrad_tc(a, grad_w, ws + P.partial_off, P.partial_bytes, s);
  } else {
    rc = launch_wgrad_fma(a, (float*)(ws + P.partial_off), P.splits, s);
    if (rc) return rc;
    rc = reduce_partials((const float*)(ws + P.partial_off), P.splits, (int64_t)K * Cin * Cout, grad_w, s);
  }
  if (rc) return rc;
  if (grad_bias)
    rc = launch_colstats(grad_out, nullptr, n_out, Cout, dtype, grad_bias, nullptr, ws + P.stats_off,
                         P.stats_bytes, s);
  return rc;
}

extern "C" int oc_conv_wgrad(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                             const void* table, int idx_bytes, int table_cols, const int* h_taps,
                             int K, int Cin, int Cout, int dtype, float* grad_w, float* grad_bias,
                             void* workspace, size_t workspace_bytes, void* stream) {
  return conv_wgrad_impl("oc_conv_wgrad", data, n_in, grad_out, n_out, table, idx_bytes, table_cols, h_taps,
                         nullptr, nullptr, K, Cin, Cout, dtype, grad_w, grad_bias, workspace, workspace_bytes, stream);
}

extern "C" int oc_conv_wgrad_tiled(const void* data, int64_t n_in, const void* grad_out, int64_t n_out,
                                   const void* tiles, const int32_t* row_perm, int K, int Cin, int Cout, int dtype,
                                   float* grad_w, float* grad_bias, void* workspace, size_t workspace_bytes,
                                   void* stream) {
  OC_REQUIRE(tiles, OC_EINVAL, "oc_conv_wgrad_tiled: null tile table");
  return conv_wgrad_impl("oc_conv_wgrad_tiled", data, n_in, grad_out, n_out, nullptr, 4,
                         K >= 1 && K <= OC_MAX_TAPS ? K : 1, nullptr, tiles, row_perm, K, Cin, Cout, dtype, grad_w,
                         grad_bias, workspace, workspace_bytes, stream);
}
