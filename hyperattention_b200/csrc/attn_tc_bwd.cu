// placeholder until the tcgen05 backward lands
#include "attn_index.cuh"
namespace ha {
bool tc_bwd_supported(const ha_attn_params&) { return false; }
int tc_attn_bwd(const ha_attn_params&, cudaStream_t) { return HA_ERR_INVALID; }
}
