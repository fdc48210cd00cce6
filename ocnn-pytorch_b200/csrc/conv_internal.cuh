// Argument bundles shared by the convolution launchers (FMA and tensor-core).
#pragma once
#include "oc_common.cuh"

namespace oc {

struct ConvArgs {
  const void* data;    // (n_in, Cin)
  int64_t n_in;
  const void* bias;    // (Cout) or null, same dtype as data
  const void* table;   // (n_out, table_cols) indices into data rows, < 0 = none
  const void* tiled = nullptr;   // the same table as a tile table (tensor-core kernels only); then `table` may be null
  const int32_t* perm = nullptr; // row order of the tile table (position -> output row), null = identity
  int idx_bytes;       // 8 or 4
  int table_cols;
  TapList taps;
  int K;
  int64_t n_out;
  int Cin, Cout;
  int dtype;
  void* out;           // (n_out, Cout)
};

struct WgradArgs {
  const void* data;      // (n_in, Cin)
  int64_t n_in;
  const void* grad_out;  // (n_out, Cout)
  int64_t n_out;
  const void* table;
  const void* tiled = nullptr;   // the same table as a tile table (tensor-core kernel only); then `table` may be null
  const int32_t* perm = nullptr; // row order of the tile table (position -> row of grad_out), null = identity
  int idx_bytes;
  int table_cols;
  TapList taps;
  int K;
  int Cin, Cout;
  int dtype;
};

// conv_fma.cu
int prep_weights_f32(const void* w, int w_dtype, int K, int Cin, int Cout, int transposed,
                     float* out, cudaStream_t s);
int launch_conv_fma(const ConvArgs& a, const float* Wf, cudaStream_t s);
int wgrad_fma_splits(int K, int Cin, int Cout, int64_t n_out);
int launch_wgrad_fma(const WgradArgs& a, float* partial, int splits, cudaStream_t s);
int reduce_partials(const float* partial, int splits, int64_t n, float* out, cudaStream_t s);

// conv_tc.cu (tcgen05 / TMEM path, fp16 and bf16)
bool conv_tc_supported(int K, int Cin, int Cout, int dtype);
size_t tile_table_block_bytes(int K);
size_t tile_table_bytes(int64_t n_out, int K);
int launch_tile_table(const void* table, int idx_bytes, int table_cols, const TapList& taps, int K,
                      int64_t n_out, int64_t n_in, const int32_t* perm, void* out, cudaStream_t s);
size_t conv_tc_weight_bytes(int K, int Cin, int Cout);
int prep_weights_tc(const void* w, int w_dtype, int K, int Cin, int Cout, int transposed, int dtype,
                    void* out, cudaStream_t s);
int launch_conv_tc(const ConvArgs& a, const void* Wimg, int* status_dev, cudaStream_t s);

int read_tc_status(cudaStream_t s, int* h_status);

bool wgrad_tc_supported(int K, int Cin, int Cout, int dtype);
size_t wgrad_tc_workspace_bytes(int K, int Cin, int Cout, int64_t n_out);
int launch_wgrad_tc(const WgradArgs& a, float* grad_w, void* workspace, size_t workspace_bytes,
                    cudaStream_t s);

// norm.cu
size_t colstats_workspace_bytes(int64_t n, int C);
int launch_colstats(const void* a, const void* b, int64_t n, int C, int dtype, float* sum_a,
                    float* sum_ab, void* workspace, size_t workspace_bytes, cudaStream_t s);

}  // namespace oc
