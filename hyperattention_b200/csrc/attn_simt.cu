// fp32 CUDA-core attention, forward and backward, for every element type and head dimension <= 256.
//
// This is the full-precision path: float32 inputs (where tensor cores would lose the 1e-4 agreement the float32
// configuration asks for) and head dimensions the tcgen05 kernels are not specialised for.  It implements the same
// two patterns as the tensor-core kernels (sorted block windows + sampled rows; exact attention with an optional
// causal mask) from the same index arithmetic.
//
// Forward: one warp per query.  Keys are taken 32 at a time, one key per lane for the q.k dot product (the query
// sits in shared memory), a warp-wide online softmax update, then the 32 weighted value rows are accumulated with
// the lanes splitting the value dimension.
// Backward: one warp per (key, chunk of queries).  One query per lane for the two dot products, then the lanes
// split the head dimension to accumulate dK/dV in registers and to add dQ rows into the fp32 accumulator with
// coalesced atomics.  All three gradients land in fp32 accumulators owned by the caller.
#include "attn_index.cuh"

namespace ha {

constexpr int SIMT_WARPS = 4;
constexpr int MAXD = 256;
constexpr int QCHUNK = 256;   // queries per backward work item

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ a_smem, const T* __restrict__ row, int d) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int e = 0;
  for (; e + 4 <= d; e += 4) {
    s0 = fmaf(a_smem[e], to_f32<T>(row[e]), s0);
    s1 = fmaf(a_smem[e + 1], to_f32<T>(row[e + 1]), s1);
    s2 = fmaf(a_smem[e + 2], to_f32<T>(row[e + 2]), s2);
    s3 = fmaf(a_smem[e + 3], to_f32<T>(row[e + 3]), s3);
  }
  for (; e < d; ++e) s0 = fmaf(a_smem[e], to_f32<T>(row[e]), s0);
  return (s0 + s1) + (s2 + s3);
}

// local key row for list entry j of query tile t (hyper) / plain index (flash); -1 = not a key
__device__ __forceinline__ int fwd_key_row(const ha_attn_params& p, int seg, const Window& w, int n_blk, int j, int n_keys) {
  if (j >= n_keys) return -1;
  if (p.mode == HA_MODE_FLASH) return j;
  if (j < n_blk) {
    int pos = w.first + j;
    if (pos >= p.m_k) pos -= p.m_k;
    return p.k_idx[kseg_of(p, seg) * p.m_k + pos];
  }
  const int s = j - n_blk;
  return p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + s] : s;
}

// weighted sampling: is slot s dropped for sorted query tile t of this segment?
__device__ __forceinline__ bool slot_dropped(const ha_attn_params& p, int seg, int t, int s) {
  const long long base = ((long long)seg * (p.m_q / TILE) + t) * (p.sample_size / 32);
  return (p.sample_mask[base + (s >> 5)] >> (s & 31)) & 1u;
}

template <typename T>
__global__ void __launch_bounds__(SIMT_WARPS * 32) attn_simt_fwd_kernel(const ha_attn_params p, long long total_queries) {
  __shared__ int s_bail;
  if (cta_sees_failure(p.status, &s_bail)) return;   // a failed index check or an earlier timeout: touch nothing
  __shared__ float sq[SIMT_WARPS][MAXD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long wq = (long long)blockIdx.x * SIMT_WARPS + warp;
  if (wq >= total_queries) return;
  const int seg = (int)(wq / p.m_q);
  const int pos = (int)(wq - (long long)seg * p.m_q);
  const SegInfo si = seg_info(p, seg);
  const bool hyper = p.mode == HA_MODE_HYPER;
  const int qrow = hyper ? p.q_idx[(long long)seg * p.m_q + pos] : pos;
  const T* qp = (const T*)p.q + si.b * p.q_sb + si.h * p.q_sh + (si.q_row0 + qrow) * p.q_sn;
  for (int e = lane; e < p.d; e += 32) sq[warp][e] = to_f32<T>(qp[e]);
  __syncwarp();
  const T* kbase = (const T*)p.k + si.b * p.k_sb + si.hk * p.k_sh + si.k_row0 * p.k_sn;
  const T* vbase = (const T*)p.v + si.b * p.v_sb + si.hk * p.v_sh + si.k_row0 * p.v_sn;

  Window w{0, 0};
  int n_blk = 0, n_keys;
  const bool weighted = hyper && p.sample_logw != nullptr;
  float logw = 0.f;
  if (hyper) {
    const int bs = (p.block_size + TILE - 1) / TILE;
    w = block_window(pos / TILE, bs, p.m_k, p.flags & HA_FLAG_SMOOTH);
    n_blk = w.count;
    n_keys = n_blk + p.sample_size;
    if (weighted) logw = p.sample_logw[(long long)seg * (p.m_q / TILE) + pos / TILE];
  } else {
    n_keys = (p.flags & HA_FLAG_CAUSAL) ? min(pos + 1, p.m_k) : p.m_k;
  }

  constexpr int VR = MAXD / 32;
  float acc[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) acc[i] = 0.f;
  float mx = -INFINITY, l = 0.f;
  for (int j0 = 0; j0 < n_keys; j0 += 32) {
    int krow = fwd_key_row(p, seg, w, n_blk, j0 + lane, n_keys);
    const bool sampled = weighted && j0 + lane >= n_blk && krow >= 0;
    if (sampled && slot_dropped(p, seg, pos / TILE, j0 + lane - n_blk)) krow = -1;
    float s = -INFINITY;
    if (krow >= 0) s = dot_row<T>(sq[warp], kbase + (long long)krow * p.k_sn, p.d) * p.scale + (sampled ? logw : 0.f);
    float gm = s;
    for (int off = 16; off >= 1; off >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, off));
    const float mnew = fmaxf(mx, gm);
    const float alpha = mx == -INFINITY ? 0.f : expf(mx - mnew);
    const float pj = krow >= 0 ? expf(s - mnew) : 0.f;
    float ps = pj;
    for (int off = 16; off >= 1; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
    l = l * alpha + ps;
    mx = mnew;
#pragma unroll
    for (int i = 0; i < VR; ++i) acc[i] *= alpha;
    const int cnt = min(32, n_keys - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const int rb = __shfl_sync(0xffffffffu, krow, jj);
      if (rb < 0) continue;
      const T* vp = vbase + (long long)rb * p.v_sn;
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const int e = lane + 32 * i;
        if (e < p.dv) acc[i] = fmaf(pb, to_f32<T>(vp[e]), acc[i]);
      }
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  float lse = l > 0.f ? mx + logf(l) : -INFINITY;
  const long long orow = si.q_row0 + qrow;
  const long long lse_at = ((long long)(si.b * p.H + si.h)) * p.n + orow;
  T* op = (T*)p.o + si.b * p.o_sb + si.h * p.o_sh + orow * p.o_sn;
  if (p.part_o) {
    T* pp = (T*)p.part_o + si.b * p.o_sb + si.h * p.o_sh + orow * p.o_sn;
#pragma unroll
    for (int i = 0; i < VR; ++i) {
      const int e = lane + 32 * i;
      if (e < p.dv) pp[e] = from_f32<T>(acc[i] * inv);
    }
    if (lane == 0 && p.part_lse) p.part_lse[lse_at] = lse;
  }
  float w1 = 0.f, w2 = 1.f;
  if (p.flags & HA_FLAG_MERGE) {
    const float l1 = p.lse[lse_at], l2 = lse;
    if (p.flags & HA_FLAG_MERGE_EXACT) {
      const float m2 = fmaxf(l1, l2);
      const float e1 = expf(l1 - m2), e2 = expf(l2 - m2);
      w1 = e1 / (e1 + e2);
      w2 = e2 / (e1 + e2);
      lse = m2 + logf(e1 + e2);
    } else {
      const float c = round_to<T>(1.f / (1.f + expf(l2 - l1)));
      w1 = c;
      w2 = round_to<T>(1.f - c);
      lse = l1 - logf(c + 1.1920929e-07f);
    }
  }
#pragma unroll
  for (int i = 0; i < VR; ++i) {
    const int e = lane + 32 * i;
    if (e < p.dv) {
      float val = acc[i] * inv;
      if (p.flags & HA_FLAG_MERGE) val = w1 * to_f32<T>(op[e]) + w2 * round_to<T>(val);
      op[e] = from_f32<T>(val);
    }
  }
  __syncwarp();
  if (lane == 0) p.lse[lse_at] = lse;
}

// ---------------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------------
// phase 0: block part (hyper) / all keys (flash).  phase 1: sampled rows (hyper).
// The query list of a key and the mapping list entry -> local query row:
struct QList { int len; int kind; int a, b, c; };  // kind 0: contiguous positions (a + j) mod m through q_idx
                                                    // kind 1: natural rows a + j
                                                    // kind 2: up to `c` tiles counted down from tile a (exact smooth)
__device__ __forceinline__ int qlist_row(const ha_attn_params& p, int seg, const QList& ql, int j, int kappa, int bs) {
  if (ql.kind == 1) return ql.a + j;
  int pos;
  if (ql.kind == 0) {
    pos = ql.a + j;
    if (pos >= p.m_q) pos -= p.m_q;
  } else {
    // exact transpose of the smooth forward: candidate tile t = a - (j / 128); valid iff kappa lies in its window
    const int T_ = p.m_q / TILE;
    int t = ql.a - j / TILE;
    if (t < 0) t += T_;
    const Window w = block_window(t, bs, p.m_k, true);
    int off = kappa - w.first;
    if (off < 0) off += p.m_k;
    if (off >= w.count) return -1;
    pos = t * TILE + (j % TILE);
  }
  return p.q_idx[(long long)seg * p.m_q + pos];
}

template <typename T>
__global__ void __launch_bounds__(SIMT_WARPS * 32) attn_simt_bwd_kernel(const ha_attn_params p, int phase, int n_keys_per_seg,
                                                                        int chunks_per_key, long long total_items) {
  __shared__ int s_bail;
  if (cta_sees_failure(p.status, &s_bail)) return;   // a failed index check or an earlier timeout: touch nothing
  __shared__ float sk[SIMT_WARPS][MAXD];
  __shared__ float sv[SIMT_WARPS][MAXD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * SIMT_WARPS + warp;
  if (item >= total_items) return;
  const int chunk = (int)(item % chunks_per_key);
  const long long key_item = item / chunks_per_key;
  const int seg = (int)(key_item / n_keys_per_seg);
  const int kk = (int)(key_item - (long long)seg * n_keys_per_seg);  // sorted key position / sample slot / key row
  const SegInfo si = seg_info(p, seg);
  const bool hyper = p.mode == HA_MODE_HYPER;
  const int bs = (p.block_size + TILE - 1) / TILE;

  int krow;
  QList ql;
  if (!hyper) {
    krow = kk;
    const int first = (p.flags & HA_FLAG_CAUSAL) ? kk : 0;
    ql = {p.m_q - first, 1, first, 0, 0};
  } else if (phase == 1) {
    krow = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + kk] : kk;
    ql = {p.m_q, p.sample_logw ? 0 : 1, 0, 0, 0};   // weighted: by sorted position, so that j / 128 is the query tile
  } else {
    krow = p.k_idx[kseg_of(p, seg) * p.m_k + kk];
    const int t = kk / TILE;
    const bool smooth = p.flags & HA_FLAG_SMOOTH;
    if (!smooth || (p.flags & HA_FLAG_BWD_REF_SMOOTH)) {
      const Window w = block_window(t, bs, p.m_q, smooth);
      ql = {w.count, 0, w.first, 0, 0};
    } else {
      const int T_ = p.m_q / TILE;
      const int t_hi = ((kk + (TILE / 2) * (bs - 1)) / TILE) % T_;
      const int cand = min(bs, T_);   // with fewer tiles than a window spans, every tile pairs with the key once
      ql = {cand * TILE, 2, t_hi, 0, cand};
    }
  }
  const int j_begin = chunk * QCHUNK, j_end = min(ql.len, j_begin + QCHUNK);
  if (j_begin >= j_end) return;

  const T* kp = (const T*)p.k + si.b * p.k_sb + si.hk * p.k_sh + (si.k_row0 + krow) * p.k_sn;
  const T* vp = (const T*)p.v + si.b * p.v_sb + si.hk * p.v_sh + (si.k_row0 + krow) * p.v_sn;
  for (int e = lane; e < p.d; e += 32) sk[warp][e] = to_f32<T>(kp[e]);
  for (int e = lane; e < p.dv; e += 32) sv[warp][e] = to_f32<T>(vp[e]);
  __syncwarp();
  const T* qbase = (const T*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
  const T* gbase = (const T*)p.d_o + si.b * p.do_sb + si.h * p.do_sh + si.q_row0 * p.do_sn;
  const long long stat0 = ((long long)(si.b * p.H + si.h)) * p.n + si.q_row0;
  const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;

  constexpr int VR = MAXD / 32;
  float dk[VR], dvv[VR];
#pragma unroll
  for (int i = 0; i < VR; ++i) { dk[i] = 0.f; dvv[i] = 0.f; }

  for (int j0 = j_begin; j0 < j_end; j0 += 32) {
    const int j = j0 + lane;
    int qrow = -1;
    if (j < j_end) qrow = qlist_row(p, seg, ql, j, kk, bs);
    float logw = 0.f;
    if (hyper && phase == 1 && p.sample_logw && qrow >= 0) {
      if (slot_dropped(p, seg, j / TILE, kk)) qrow = -1;
      else logw = p.sample_logw[(long long)seg * (p.m_q / TILE) + j / TILE];
    }
    float pj = 0.f, ds = 0.f;
    if (qrow >= 0) {
      const float s = dot_row<T>(sk[warp], qbase + (long long)qrow * p.q_sn, p.d) * p.scale + logw;
      const float dp = dot_row<T>(sv[warp], gbase + (long long)qrow * p.do_sn, p.dv);
      pj = expf(s - p.lse[stat0 + qrow]);
      ds = pj * (dp - p.delta[stat0 + qrow]) * p.scale;
    }
    const int cnt = min(32, j_end - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const int rb = __shfl_sync(0xffffffffu, qrow, jj);
      if (rb < 0) continue;
      const float pb = __shfl_sync(0xffffffffu, pj, jj);
      const float db = __shfl_sync(0xffffffffu, ds, jj);
      const T* qp = qbase + (long long)rb * p.q_sn;
      const T* gp = gbase + (long long)rb * p.do_sn;
      float* dqp = p.dq_acc + (head0 + si.q_row0 + rb) * p.d;
#pragma unroll
      for (int i = 0; i < VR; ++i) {
        const int e = lane + 32 * i;
        if (e < p.d) {
          dk[i] = fmaf(db, to_f32<T>(qp[e]), dk[i]);
          atomicAdd(dqp + e, db * sk[warp][e]);
        }
        if (e < p.dv) dvv[i] = fmaf(pb, to_f32<T>(gp[e]), dvv[i]);
      }
    }
  }
  float* dkp = p.dk_acc + (si.khead0 + si.k_row0 + krow) * p.d;
  float* dvp = p.dv_acc + (si.khead0 + si.k_row0 + krow) * p.dv;
#pragma unroll
  for (int i = 0; i < VR; ++i) {
    const int e = lane + 32 * i;
    if (e < p.d) atomicAdd(dkp + e, dk[i]);
    if (e < p.dv) atomicAdd(dvp + e, dvv[i]);
  }
}

template <typename T>
int simt_fwd(const ha_attn_params& p, cudaStream_t st) {
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const long long total = segs * p.m_q;
  if (total == 0) return HA_OK;
  const long long grid = (total + SIMT_WARPS - 1) / SIMT_WARPS;
  if (grid > 0x7fffffffLL) return HA_ERR_INVALID;
  attn_simt_fwd_kernel<T><<<(unsigned)grid, SIMT_WARPS * 32, 0, st>>>(p, total);
  HA_LAUNCHED("ha_attn_fwd (cuda-core)");
  return HA_OK;
}

template <typename T>
int simt_bwd(const ha_attn_params& p, cudaStream_t st) {
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  if (segs == 0 || p.m_q == 0 || p.m_k == 0) return HA_OK;
  const int bs = (p.block_size + TILE - 1) / TILE;
  for (int phase = 0; phase < 2; ++phase) {
    int keys, chunks;
    if (p.mode == HA_MODE_FLASH) {
      if (phase == 1) break;
      keys = p.m_k;
      chunks = (p.m_q + QCHUNK - 1) / QCHUNK;
    } else if (phase == 0) {
      keys = p.m_k;
      chunks = (bs * TILE + QCHUNK - 1) / QCHUNK;
    } else {
      keys = p.sample_size;
      chunks = (p.m_q + QCHUNK - 1) / QCHUNK;
      if (keys == 0) break;
    }
    const long long items = segs * keys * chunks;
    const long long grid = (items + SIMT_WARPS - 1) / SIMT_WARPS;
    if (grid > 0x7fffffffLL) return HA_ERR_INVALID;
    attn_simt_bwd_kernel<T><<<(unsigned)grid, SIMT_WARPS * 32, 0, st>>>(p, phase, keys, chunks, items);
    HA_LAUNCHED("ha_attn_bwd (cuda-core)");
  }
  return HA_OK;
}

int simt_attn_fwd(const ha_attn_params& p, cudaStream_t st) {
  switch (p.dtype) {
    case HA_BF16: return simt_fwd<__nv_bfloat16>(p, st);
    case HA_FP16: return simt_fwd<__half>(p, st);
    case HA_FP32: return simt_fwd<float>(p, st);
  }
  return HA_ERR_DTYPE;
}
int simt_attn_bwd(const ha_attn_params& p, cudaStream_t st) {
  switch (p.dtype) {
    case HA_BF16: return simt_bwd<__nv_bfloat16>(p, st);
    case HA_FP16: return simt_bwd<__half>(p, st);
    case HA_FP32: return simt_bwd<float>(p, st);
  }
  return HA_ERR_DTYPE;
}

}  // namespace ha
