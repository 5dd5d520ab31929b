// Argument checking and dispatch for ha_attn_fwd / ha_attn_bwd.
#include "attn_index.cuh"

namespace ha {
int simt_attn_fwd(const ha_attn_params& p, cudaStream_t st);
int simt_attn_bwd(const ha_attn_params& p, cudaStream_t st);
int tc_attn_fwd(const ha_attn_params& p, cudaStream_t st);
bool tc_supported(const ha_attn_params& p);
bool tc_bwd_supported(const ha_attn_params& p);
int tc_attn_bwd(const ha_attn_params& p, cudaStream_t st);

static int check_common(const ha_attn_params& p, bool backward) {
  if (p.dtype != HA_BF16 && p.dtype != HA_FP16 && p.dtype != HA_FP32) return HA_ERR_DTYPE;
  if (p.B < 0 || p.H < 0 || p.n < 0 || p.d <= 0 || p.dv <= 0 || p.d > 256 || p.dv > 256) return HA_ERR_INVALID;
  if (p.segs_per_head < 1 || p.span < 0 || p.q_off < 0 || p.k_off < 0 || p.m_q < 0 || p.m_k < 0) return HA_ERR_INVALID;
  if ((long long)p.segs_per_head * p.span > p.n) return HA_ERR_INVALID;
  if (p.q_off + p.m_q > p.span) return HA_ERR_INVALID;
  // a single-segment exact-attention call may have more keys than queries (n describes the query side then)
  if (p.k_off + p.m_k > p.span && !(p.mode == HA_MODE_FLASH && p.segs_per_head == 1 && !backward)) return HA_ERR_INVALID;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse) return HA_ERR_INVALID;
  if (p.mode == HA_MODE_HYPER) {
    // the reference asserts: equal lengths, multiples of 128 (src/hyper_attn_triton.py:695, :911)
    if (p.m_q != p.m_k || p.m_q % TILE != 0) return HA_ERR_INVALID;
    if (p.block_size < 1 || p.sample_size < 0 || p.sample_size % TILE != 0) return HA_ERR_INVALID;
    if (p.sample_size > p.m_k) return HA_ERR_INVALID;   // the reference would read past the head here
    if (!p.q_idx || !p.k_idx) return HA_ERR_INVALID;
    if (p.flags & HA_FLAG_CAUSAL) return HA_ERR_INVALID;
    if ((p.sample_logw == nullptr) != (p.sample_mask == nullptr)) return HA_ERR_INVALID;
  } else if (p.mode == HA_MODE_FLASH) {
    if ((p.flags & HA_FLAG_CAUSAL) && p.m_q != p.m_k) return HA_ERR_INVALID;
    if (p.m_q > 0 && p.m_k == 0) return HA_ERR_INVALID;
  } else {
    return HA_ERR_INVALID;
  }
  if (backward) {
    if (!p.d_o || !p.delta || !p.dq_acc || !p.dk_acc || !p.dv_acc) return HA_ERR_INVALID;
  }
  return HA_OK;
}
}  // namespace ha

using namespace ha;

extern "C" {

int ha_attn_fwd(const ha_attn_params* p, void* stream) {
  if (!p) return HA_ERR_INVALID;
  int rc = check_common(*p, false);
  if (rc != HA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && tc_supported(*p)) return tc_attn_fwd(*p, st);
  return simt_attn_fwd(*p, st);
}

int ha_attn_bwd(const ha_attn_params* p, void* stream) {
  if (!p) return HA_ERR_INVALID;
  int rc = check_common(*p, true);
  if (rc != HA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && tc_bwd_supported(*p)) return tc_attn_bwd(*p, st);
  return simt_attn_bwd(*p, st);
}

}  // extern "C"
