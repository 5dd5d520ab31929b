// Argument checking and dispatch for ha_attn_fwd / ha_attn_bwd.
#include "attn_index.cuh"

namespace ha {
int simt_attn_fwd(const ha_attn_params& p, cudaStream_t st);
int simt_attn_bwd(const ha_attn_params& p, cudaStream_t st);
int tc_attn_fwd(const ha_attn_params& p, cudaStream_t st);
int ws_attn_fwd(const ha_attn_params& p, cudaStream_t st);
bool ws_fwd_supported(const ha_attn_params& p);
bool tc_supported(const ha_attn_params& p);
bool tc_bwd_supported(const ha_attn_params& p);
int tc_attn_bwd(const ha_attn_params& p, cudaStream_t st);
int ws_attn_bwd(const ha_attn_params& p, cudaStream_t st);
bool ws_bwd_supported(const ha_attn_params& p);
bool ws_bwd_shape_ok(const ha_attn_params& p);

static int check_common(const ha_attn_params& p, bool backward) {
  if (p.dtype != HA_BF16 && p.dtype != HA_FP16 && p.dtype != HA_FP32) return HA_ERR_DTYPE;
  if (p.B < 0 || p.H < 0 || p.n < 0 || p.d <= 0 || p.dv <= 0 || p.d > 256 || p.dv > 256) return HA_ERR_INVALID;
  if (p.segs_per_head < 1 || p.span < 0 || p.q_off < 0 || p.k_off < 0 || p.m_q < 0 || p.m_k < 0) return HA_ERR_INVALID;
  if ((long long)p.segs_per_head * p.span > p.n) return HA_ERR_INVALID;
  if (p.q_off + p.m_q > p.span) return HA_ERR_INVALID;
  // a single-segment exact-attention call may have more keys than queries (n describes the query side then)
  if (p.k_off + p.m_k > p.span && !(p.mode == HA_MODE_FLASH && p.segs_per_head == 1 && !backward)) return HA_ERR_INVALID;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse) return HA_ERR_INVALID;
  if (p.kv_group < 0 || (p.kv_group > 1 && p.H % p.kv_group != 0)) return HA_ERR_INVALID;
  if (p.kv_group > 1) {
    // a K/V row collects gradient terms from every query head of its group: fp32 accumulators only, nothing "stored once";
    // the per-tile sample weights are computed per query head and not offered together with shared K/V heads
    if (p.dk_out || p.dv_out || p.dq_out || (p.flags & HA_FLAG_BWD_KV_INIT) || p.sample_logw) return HA_ERR_INVALID;
  }
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
    if (!p.d_o || !p.delta || (!p.dq_acc && !p.dq_out)) return HA_ERR_INVALID;
    if (p.dk_out || p.dv_out) {
      // direct dK/dV: hyper pattern only (one work item owns a key tile's block part), both outputs, slot buffers if sampled
      if (!p.dk_out || !p.dv_out || p.mode != HA_MODE_HYPER) return HA_ERR_INVALID;
      if (p.sample_size > 0 && (!p.dk_sacc || !p.dv_sacc)) return HA_ERR_INVALID;
      if ((uintptr_t)p.dk_out % 16 != 0 || (uintptr_t)p.dv_out % 16 != 0) return HA_ERR_INVALID;
      if (p.dq_out && (uintptr_t)p.dq_out % 16 != 0) return HA_ERR_INVALID;
    } else if (!p.dk_acc || !p.dv_acc || p.dq_out) {
      return HA_ERR_INVALID;   // (dq_out comes with dk_out / dv_out only)
    }
  }
  return HA_OK;
}

template <typename T>
__global__ void bwd_finish_kernel(const ha_attn_params p, long long total, const bool tiled) {
  // one thread per (segment, slot, 8 elements of dk | dv)
  const int cpr_k = p.d / 8, cpr = cpr_k + p.dv / 8;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % cpr);
  const long long ss = i / cpr;
  const int slot = (int)(ss % p.sample_size), seg = (int)(ss / p.sample_size);
  const SegInfo si = seg_info(p, seg);
  const int row = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + slot] : slot;
  const long long out_row = ((long long)(si.b * p.H + si.h)) * p.n + si.k_row0 + row;
  const bool is_k = c < cpr_k;
  const int w = is_k ? p.d : p.dv, e0 = (is_k ? c : c - cpr_k) * 8;
  T* out = (is_k ? (T*)p.dk_out : (T*)p.dv_out) + out_row * w + e0;
  // Layout of the slot buffers: [slot][w] rows, or -- written by the warp-specialised kernel (w = 64) -- per tile of 128
  // slots two halves of [128 rows][32 floats], the 16-byte chunks of a row XOR-swizzled by the row: the layout of that
  // kernel's staging tile.
  const float* accb = (is_k ? p.dk_sacc : p.dv_sacc) + kseg_of(p, seg) * p.sample_size * w;
  float4 a0, a1;
  if (tiled) {
    const float* rowp = accb + (long long)(slot / TILE) * (TILE * 64) + (e0 / 32) * (TILE * 32) + (slot % TILE) * 32;
    const int c = (e0 % 32) / 4;
    a0 = *reinterpret_cast<const float4*>(rowp + ((c ^ (slot & 7)) << 2));
    a1 = *reinterpret_cast<const float4*>(rowp + (((c + 1) ^ (slot & 7)) << 2));
  } else {
    a0 = *reinterpret_cast<const float4*>(accb + (long long)slot * w + e0);
    a1 = *reinterpret_cast<const float4*>(accb + (long long)slot * w + e0 + 4);
  }
  uint4 raw = *reinterpret_cast<const uint4*>(out);
  T* v = reinterpret_cast<T*>(&raw);
  const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] = from_f32<T>(to_f32<T>(v[j]) + a[j]);
  *reinterpret_cast<uint4*>(out) = raw;
}

// HA_FLAG_CHECK_INDICES: every entry of an index array must be a row of its segment.
__global__ void index_check_kernel(const int32_t* __restrict__ idx, long long count, int limit, int32_t* status, int32_t* status_host) {
  bool bad = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const int v = idx[i];
    bad |= v < 0 || v >= limit;
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) {
    if (status) atomicExch(status, HA_DEV_BAD_INDEX);
    if (status_host) {
      *reinterpret_cast<volatile int32_t*>(status_host) = HA_DEV_BAD_INDEX;
      __threadfence_system();
    }
  }
}

static int check_indices(const ha_attn_params& p, cudaStream_t st) {
  if (!p.status) return HA_ERR_INVALID;
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const long long ksegs = p.kv_group > 1 ? segs / p.kv_group : segs;
  struct { const int32_t* ptr; long long count; int limit; } arr[3] = {
      {p.q_idx, segs * p.m_q, p.m_q}, {p.k_idx, ksegs * p.m_k, p.m_k}, {p.sample_idx, ksegs * p.sample_size, p.m_k}};
  for (auto& a : arr) {
    if (!a.ptr || a.count == 0) continue;
    const long long want = (a.count + 255) / 256;
    index_check_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, st>>>(a.ptr, a.count, a.limit, p.status, p.status_host);
    HA_LAUNCHED("ha_attn index check");
  }
  return HA_OK;
}

// One warp, one mbarrier that nobody arrives at: the wait runs out after `polls` polls and is reported like any other.
__global__ void wait_probe_kernel(int32_t* status, int32_t* status_host, int polls) {
  __shared__ uint64_t bar_mem;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  bool done = false;
  for (int i = 0; i < polls && !done; ++i) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(0u) : "memory");
    done = ok != 0;
  }
  if (!done && threadIdx.x == 0) report_timeout(status, status_host);
}
}  // namespace ha

using namespace ha;

extern "C" {

int ha_attn_fwd(const ha_attn_params* p, void* stream) {
  if (!p) return HA_ERR_INVALID;
  int rc = check_common(*p, false);
  if (rc != HA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((p->flags & HA_FLAG_CHECK_INDICES) && p->mode == HA_MODE_HYPER && (rc = check_indices(*p, st)) != HA_OK) return rc;
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && ws_fwd_supported(*p)) return ws_attn_fwd(*p, st);
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && tc_supported(*p)) return tc_attn_fwd(*p, st);
  return simt_attn_fwd(*p, st);
}

int ha_attn_bwd(const ha_attn_params* p, void* stream) {
  if (!p) return HA_ERR_INVALID;
  int rc = check_common(*p, true);
  if (rc != HA_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if ((p->flags & HA_FLAG_CHECK_INDICES) && p->mode == HA_MODE_HYPER && (rc = check_indices(*p, st)) != HA_OK) return rc;
  if (p->flags & HA_FLAG_BWD_KV_INIT) {
    // one work item must own a key tile's whole dK/dV: exact attention with a single chunk of query tiles
    if (p->mode != HA_MODE_FLASH || p->m_q > 16 * TILE || p->dk_out) return HA_ERR_INVALID;
  }
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && ws_bwd_supported(*p)) return ws_attn_bwd(*p, st);
  if (!(p->flags & HA_FLAG_FORCE_SIMT) && tc_bwd_supported(*p)) return tc_attn_bwd(*p, st);
  if (p->dk_out || (p->flags & HA_FLAG_BWD_KV_INIT)) return HA_ERR_INVALID;   // tensor-core kernel only
  return simt_attn_bwd(*p, st);
}

int ha_attn_bwd_direct_level(const ha_attn_params* p) {
  if (!p || !p->d_o || p->mode != HA_MODE_HYPER || p->kv_group > 1) return 0;
  if ((p->flags & HA_FLAG_FORCE_SIMT) || !tc_bwd_supported(*p)) return 0;
  if (ws_bwd_shape_ok(*p)) return 2;   // the warp-specialised kernel sums every query tile's dQ inside one work item
  const bool whole_blocks = !(p->flags & HA_FLAG_SMOOTH) && (p->block_size + TILE - 1) / TILE == 2 && p->m_k % (2 * TILE) == 0;
  if (p->d == 64 && p->dv == 64 && whole_blocks && (p->sample_size == 0 || p->sample_size == 2 * TILE)) return 2;
  return 1;
}

int ha_wait_probe(int32_t* status, int32_t* status_host, int32_t polls, void* stream) {
  if ((!status && !status_host) || polls < 1 || polls > SPIN_LIMIT) return HA_ERR_INVALID;
  wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, status_host, polls);
  HA_LAUNCHED("ha_wait_probe");
  return HA_OK;
}

int ha_attn_bwd_finish(const ha_attn_params* p, void* stream) {
  if (!p) return HA_ERR_INVALID;
  int rc = check_common(*p, true);
  if (rc != HA_OK) return rc;
  if (!p->dk_out || p->dtype == HA_FP32 || p->d % 8 || p->dv % 8) return HA_ERR_INVALID;
  const long long segs = (long long)p->B * p->H * p->segs_per_head;
  const long long total = segs * p->sample_size * (p->d / 8 + p->dv / 8);
  if (total == 0) return HA_OK;
  if ((total + 255) / 256 > 0x7fffffffLL) return HA_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const bool tiled = !(p->flags & HA_FLAG_FORCE_SIMT) && ws_bwd_supported(*p);     // which kernel filled the slot buffers
  if (p->dtype == HA_BF16) bwd_finish_kernel<__nv_bfloat16><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(*p, total, tiled);
  else bwd_finish_kernel<__half><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(*p, total, tiled);
  HA_LAUNCHED("ha_attn_bwd_finish");
  return HA_OK;
}

}  // extern "C"
