// placeholder; replaced by the tcgen05 implementation
#include "oc_common.cuh"
#include "conv_internal.cuh"
namespace oc {
bool conv_tc_supported(int, int, int, int) { return false; }
size_t conv_tc_weight_bytes(int, int, int) { return 0; }
int prep_weights_tc(const void*, int, int, int, int, int, int, void*, cudaStream_t) { return OC_EINVAL; }
int launch_conv_tc(const ConvArgs&, const void*, int*, cudaStream_t) { return OC_EINVAL; }
bool wgrad_tc_supported(int, int, int, int) { return false; }
size_t wgrad_tc_workspace_bytes(int, int, int, int64_t) { return 0; }
int launch_wgrad_tc(const WgradArgs&, float*, void*, size_t, cudaStream_t) { return OC_EINVAL; }
}
