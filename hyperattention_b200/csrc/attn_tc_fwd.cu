// placeholder replaced by the tcgen05 kernels
#include "attn_index.cuh"
namespace ha {
bool tc_supported(const ha_attn_params&) { return false; }
int tc_attn_fwd(const ha_attn_params&, cudaStream_t) { return HA_ERR_INVALID; }
int tc_attn_bwd(const ha_attn_params&, cudaStream_t) { return HA_ERR_INVALID; }
}
