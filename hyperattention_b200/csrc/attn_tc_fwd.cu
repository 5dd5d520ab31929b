// Attention forward on 5th-generation tensor cores (tcgen05 + TMEM), bf16/fp16, head dims 64 and 128.
//
// One CTA of 128 threads owns one tile of 128 queries; thread i owns query row i = TMEM lane i.
//   * Operand rows are gathered straight from the caller's q/k/v by row index with 16-byte cp.async copies into
//     128-byte-swizzled shared-memory tiles (a 128-byte row is one full line, so a random row gather still moves
//     whole lines; 8 neighbouring lanes fetch one row).  K/V tiles are double buffered: tile j+1 is in flight while
//     tile j is computed.
//   * S = Q K^T: tcgen05.mma, both operands K-major in shared memory, fp32 accumulator in TMEM.
//   * softmax: each thread reads its row of S with tcgen05.ld (32x32b: one lane per thread, no shuffles), keeps the
//     running max / sum in base-2, rounds P to the input dtype and writes it back to TMEM with tcgen05.st.
//   * PV = P V: tcgen05.mma with P as the TMEM A operand and V as MN-major B in shared memory; the product of one
//     key tile lands in its own TMEM columns and is folded into the fp32 output registers with the rescale factor,
//     so TMEM is never read-modified-written.
//   * epilogue: normalise, optionally merge with the (o, lse) already stored for the row (the causal schedule's
//     in-place combine), round, stage through shared memory and store whole rows coalesced.
// The same kernel serves both patterns; only the list of key tiles of a query tile differs:
//   hyper: block-window tiles through k_idx, then the sampled rows;   flash: contiguous tiles, causal mask.
// TMEM budget per CTA: 128 (S) + 64 (P, packed pairs) + DV (PV) columns -> 256 for DV = 64, two CTAs per SM.
#include "attn_index.cuh"

#include <type_traits>

namespace ha {

template <int D, int DV> struct FwdCfg {
  static constexpr int Q_BYTES = TILE * D * 2;
  static constexpr int K_BYTES = TILE * D * 2;
  static constexpr int V_BYTES = TILE * DV * 2;
  static constexpr int O_BYTES = TILE * DV * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;            // two stages
  static constexpr int OFF_V = OFF_K + 2 * K_BYTES;        // two stages
  static constexpr int OFF_OLD = OFF_V + 2 * V_BYTES;      // previous o rows (merge) / output staging
  static constexpr int SMEM = OFF_OLD + O_BYTES + 1024;    // + alignment slack
  static constexpr int TMEM_COLS = (128 + 64 + DV) <= 256 ? 256 : 512;
  static constexpr int COL_S = 0, COL_P = 128, COL_PV = 192;
};

// 128 rows x COLS elements (2 bytes each) gathered by row index into swizzled slabs; 8 lanes per row.
// my_row = source row of smem row (warp*32 + lane), or -1 to zero-fill.
template <int COLS>
__device__ __forceinline__ void gather_tile(uint32_t smem_base, const uint16_t* __restrict__ base, int64_t row_stride, int my_row,
                                            int warp, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = 4 * i + (lane >> 3);
    const int src_row = __shfl_sync(0xffffffffu, my_row, rl);
    const int row = warp * 32 + rl;
    const int chunk = lane & 7;
    const uint32_t dst = smem_base + row * 128 + ((chunk ^ (row & 7)) << 4);
#pragma unroll
    for (int s = 0; s < COLS / 64; ++s) {
      const uint16_t* src = base + (int64_t)(src_row < 0 ? 0 : src_row) * row_stride + s * 64 + chunk * 8;
      cp_async16(dst + s * (TILE * 128), src, src_row >= 0 ? 16u : 0u);
    }
  }
}

// rows staged in swizzled slabs -> global rows by index, coalesced; my_row = destination row or -1 to skip
template <int COLS>
__device__ __forceinline__ void scatter_tile(const uint8_t* smem_base, uint16_t* __restrict__ base, int64_t row_stride, int my_row,
                                             int warp, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = 4 * i + (lane >> 3);
    const int dst_row = __shfl_sync(0xffffffffu, my_row, rl);
    const int row = warp * 32 + rl;
    const int chunk = lane & 7;
#pragma unroll
    for (int s = 0; s < COLS / 64; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(smem_base + s * (TILE * 128) + row * 128 + ((chunk ^ (row & 7)) << 4));
      if (dst_row >= 0) *reinterpret_cast<uint4*>(base + (int64_t)dst_row * row_stride + s * 64 + chunk * 8) = v;
    }
  }
}

struct TileList {
  int n_tiles;      // key tiles of this query tile
  int n_blk;        // hyper: how many of them are block-window tiles
  Window w;
};

template <typename T, int D, int DV>
__global__ void __launch_bounds__(128) attn_tc_fwd_kernel(const ha_attn_params p) {
  using Cfg = FwdCfg<D, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool hyper = p.mode == HA_MODE_HYPER;
  const bool causal = p.flags & HA_FLAG_CAUSAL;
  const int n_qt = (p.m_q + TILE - 1) / TILE;
  // heavy (late) causal tiles first
  const int qt = causal ? n_qt - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int seg = blockIdx.y;
  const SegInfo si = seg_info(p, seg);
  const uint32_t bar = smem_u32(&mma_bar);

  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), Cfg::TMEM_COLS);

  // ---- this thread's query row ----
  const int qpos = qt * TILE + tid;
  int qrow = -1;
  if (qpos < p.m_q) qrow = hyper ? p.q_idx[(long long)seg * p.m_q + qpos] : qpos;

  TileList tl;
  if (hyper) {
    const int bs = (p.block_size + TILE - 1) / TILE;
    tl.w = block_window(qt, bs, p.m_k, p.flags & HA_FLAG_SMOOTH);
    tl.n_blk = tl.w.count / TILE;
    tl.n_tiles = tl.n_blk + p.sample_size / TILE;
  } else {
    const int n_kt = (p.m_k + TILE - 1) / TILE;
    tl.n_blk = 0;
    tl.w = Window{0, 0};
    tl.n_tiles = causal ? min(qt + 1, n_kt) : n_kt;
  }
  // local key row that thread `tid` fetches for key tile j (-1: none)
  auto key_row = [&](int j) -> int {
    if (j >= tl.n_tiles) return -1;
    if (!hyper) {
      const int r = j * TILE + tid;
      return r < p.m_k ? r : -1;
    }
    if (j < tl.n_blk) {
      int pos = tl.w.first + j * TILE + tid;
      if (pos >= p.m_k) pos -= p.m_k;
      return p.k_idx[(long long)seg * p.m_k + pos];
    }
    const int s = (j - tl.n_blk) * TILE + tid;
    return p.sample_idx ? p.sample_idx[(long long)seg * p.sample_size + s] : s;
  };

  const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
  const uint16_t* kbase = (const uint16_t*)p.k + si.b * p.k_sb + si.h * p.k_sh + si.k_row0 * p.k_sn;
  const uint16_t* vbase = (const uint16_t*)p.v + si.b * p.v_sb + si.h * p.v_sh + si.k_row0 * p.v_sn;
  uint16_t* obase = (uint16_t*)p.o + si.b * p.o_sb + si.h * p.o_sh + si.q_row0 * p.o_sn;
  const bool merge = p.flags & HA_FLAG_MERGE;

  // ---- prologue: Q, previous o rows (merge), key tile 0 ----
  int krow_cur = key_row(0);
  gather_tile<D>(s_base + Cfg::OFF_Q, qbase, p.q_sn, qrow, warp, lane);
  if (merge) gather_tile<DV>(s_base + Cfg::OFF_OLD, obase, p.o_sn, qrow, warp, lane);
  gather_tile<D>(s_base + Cfg::OFF_K, kbase, p.k_sn, krow_cur, warp, lane);
  gather_tile<DV>(s_base + Cfg::OFF_V, vbase, p.v_sn, krow_cur, warp, lane);
  cp_async_commit();
  int krow_next = key_row(1);

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
  const uint32_t tS = tmem + Cfg::COL_S, tP = tmem + Cfg::COL_P, tPV = tmem + Cfg::COL_PV;
  constexpr int AB_FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const uint32_t idesc_s = mma_idesc(TILE, TILE, AB_FMT, 0, 0);
  const uint32_t idesc_pv = mma_idesc(TILE, DV, AB_FMT, 0, 1);

  float o_acc[DV];
#pragma unroll
  for (int i = 0; i < DV; ++i) o_acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float scale2 = p.scale * 1.4426950408889634f;
  uint32_t phase = 0;
  bool failed = false;

  for (int j = 0; j < tl.n_tiles; ++j) {
    const int st = j & 1;
    // prefetch tile j+1 into the other stage (its previous user, tile j-1, has completed both MMAs)
    if (j + 1 < tl.n_tiles) {
      gather_tile<D>(s_base + Cfg::OFF_K + (st ^ 1) * Cfg::K_BYTES, kbase, p.k_sn, krow_next, warp, lane);
      gather_tile<DV>(s_base + Cfg::OFF_V + (st ^ 1) * Cfg::V_BYTES, vbase, p.v_sn, krow_next, warp, lane);
    }
    cp_async_commit();
    const int krow_after = key_row(j + 2);   // index load for the tile after next, consumed next iteration
    cp_async_wait<1>();                       // tile j (and Q) have landed
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (tid == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t a_addr = s_base + Cfg::OFF_Q + (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        const uint32_t b_addr = s_base + Cfg::OFF_K + st * Cfg::K_BYTES + (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tS, smem_desc(a_addr, 16, 1024), smem_desc(b_addr, 16, 1024), idesc_s, kk > 0);
      }
      mma_commit(bar);
    }
    if (!mbar_wait(bar, phase)) { failed = true; }
    phase ^= 1;
    tc_fence_after();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- softmax over this tile's 128 columns ----
    // number of visible columns for this row: all, or clipped by the causal diagonal / end of keys
    int limit = TILE;
    if (!hyper) {
      limit = min(TILE, p.m_k - j * TILE);
      if (causal) limit = min(limit, qpos - j * TILE + 1);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + lane_sel + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float s = __uint_as_float(r[i]);
        if (c * 32 + i < limit) mx = fmaxf(mx, s);
      }
    }
    const float m_new = fmaxf(m_run, mx * scale2);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = fast_exp2(m_run - m_use);   // m_run = -inf -> 0
    float psum = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tS + lane_sel + c * 32, r);
      tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float p0 = fast_exp2(fmaf(__uint_as_float(r[i]), scale2, -m_use));
        float p1 = fast_exp2(fmaf(__uint_as_float(r[i + 1]), scale2, -m_use));
        if (c * 32 + i >= limit) p0 = 0.f;
        if (c * 32 + i + 1 >= limit) p1 = 0.f;
        psum += p0 + p1;
        pk[i >> 1] = pack2<T>(p0, p1);
      }
      tmem_st16(tP + lane_sel + c * 16, pk);
    }
    tmem_st_wait();
    l_run = l_run * alpha + psum;
    m_run = m_new;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (tid == 0) {
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        const uint32_t b_addr = s_base + Cfg::OFF_V + st * Cfg::V_BYTES + kk * 2048;
        mma_ts(tPV, tP + kk * 8, smem_desc(b_addr, TILE * 128, 1024), idesc_pv, kk > 0);
      }
      mma_commit(bar);
    }
    if (!mbar_wait(bar, phase)) { failed = true; }
    phase ^= 1;
    tc_fence_after();
    if (__syncthreads_or(failed)) { failed = true; break; }

#pragma unroll
    for (int c = 0; c < DV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(tPV + lane_sel + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o_acc[c * 32 + i] = fmaf(o_acc[c * 32 + i], alpha, __uint_as_float(r[i]));
    }
    krow_cur = krow_next;
    krow_next = krow_after;
  }
  cp_async_wait<0>();

  if (failed) {
    if (tid == 0 && p.status) atomicExch(p.status, HA_DEV_TIMEOUT);
  } else {
    // ---- epilogue ----
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    float lse = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    const long long lse_at = ((long long)(si.b * p.H + si.h)) * p.n + si.q_row0 + (qrow < 0 ? 0 : qrow);
    uint8_t* stage = smem + Cfg::OFF_OLD;
    float w1 = 0.f, w2 = 1.f;
    if (merge && qrow >= 0) {
      const float l1 = p.lse[lse_at], l2 = lse;
      if (p.flags & HA_FLAG_MERGE_EXACT) {
        const float m2 = fmaxf(l1, l2);
        const float e1 = __expf(l1 - m2), e2 = __expf(l2 - m2);
        w1 = e1 / (e1 + e2);
        w2 = e2 / (e1 + e2);
        lse = m2 + __logf(e1 + e2);
      } else {
        const float c = round_to<T>(1.f / (1.f + __expf(l2 - l1)));
        w1 = c;
        w2 = round_to<T>(1.f - c);
        lse = l1 - __logf(c + 1.1920929e-07f);
      }
    }
    if (p.part_o) {
      // un-merged result of this call, staged over the (now idle) Q tile
      uint8_t* st2 = smem + Cfg::OFF_Q;
      __syncthreads();   // all S MMAs reading Q have completed (waited above); make the reuse explicit
#pragma unroll
      for (int e = 0; e < DV; e += 2)
        *reinterpret_cast<uint32_t*>(st2 + swz_off(TILE, tid, e)) = pack2<T>(o_acc[e] * inv, o_acc[e + 1] * inv);
      __syncwarp();
      uint16_t* pbase = (uint16_t*)p.part_o + si.b * p.o_sb + si.h * p.o_sh + si.q_row0 * p.o_sn;
      scatter_tile<DV>(st2, pbase, p.o_sn, qrow, warp, lane);
      if (p.part_lse && qrow >= 0) p.part_lse[lse_at] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
#pragma unroll
    for (int e = 0; e < DV; e += 2) {
      float a = o_acc[e] * inv, b = o_acc[e + 1] * inv;
      uint32_t* slot = reinterpret_cast<uint32_t*>(stage + swz_off(TILE, tid, e));
      if (merge) {
        const float2 old = unpack2<T>(*slot);
        a = w1 * old.x + w2 * round_to<T>(a);
        b = w1 * old.y + w2 * round_to<T>(b);
      }
      *slot = pack2<T>(a, b);
    }
    __syncwarp();
    scatter_tile<DV>(stage, obase, p.o_sn, qrow, warp, lane);
    if (qrow >= 0) p.lse[lse_at] = lse;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

template <typename T, int D, int DV>
static int launch_fwd(const ha_attn_params& p, cudaStream_t st) {
  using Cfg = FwdCfg<D, DV>;
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const int n_qt = (p.m_q + TILE - 1) / TILE;
  if (segs == 0 || n_qt == 0) return HA_OK;
  if (segs > 65535) return HA_ERR_INVALID;
  // per device, so set on every launch (one process may drive several GPUs)
  HA_CUDA_OK(cudaFuncSetAttribute(attn_tc_fwd_kernel<T, D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM),
             "ha_attn_fwd smem attribute");
  attn_tc_fwd_kernel<T, D, DV><<<dim3(n_qt, (unsigned)segs), 128, Cfg::SMEM, st>>>(p);
  HA_LAUNCHED("ha_attn_fwd (tcgen05)");
  return HA_OK;
}

bool tc_supported(const ha_attn_params& p) {
  if (p.dtype != HA_BF16 && p.dtype != HA_FP16) return false;
  if (!(p.scale > 0.f)) return false;   // the running max is taken before scaling
  if (!((p.d == 64 || p.d == 128) && (p.dv == 64 || p.dv == 128))) return false;
  // 16-byte row alignment for the cp.async gathers and vector stores
  auto ok = [](const void* ptr, int64_t sb, int64_t sh, int64_t sn) {
    return ((uintptr_t)ptr % 16 == 0) && sb % 8 == 0 && sh % 8 == 0 && sn % 8 == 0;
  };
  if (!ok(p.q, p.q_sb, p.q_sh, p.q_sn) || !ok(p.k, p.k_sb, p.k_sh, p.k_sn) || !ok(p.v, p.v_sb, p.v_sh, p.v_sn) ||
      !ok(p.o, p.o_sb, p.o_sh, p.o_sn))
    return false;
  if (p.part_o && (uintptr_t)p.part_o % 16 != 0) return false;
  if ((long long)p.B * p.H * p.segs_per_head > 65535) return false;
  return true;
}

int tc_attn_fwd(const ha_attn_params& p, cudaStream_t st) {
#define HA_FWD_CASE(TT, DD, DDV) \
  if (p.d == DD && p.dv == DDV) return launch_fwd<TT, DD, DDV>(p, st);
  if (p.dtype == HA_BF16) {
    HA_FWD_CASE(__nv_bfloat16, 64, 64)
    HA_FWD_CASE(__nv_bfloat16, 128, 128)
    HA_FWD_CASE(__nv_bfloat16, 128, 64)
    HA_FWD_CASE(__nv_bfloat16, 64, 128)
  } else {
    HA_FWD_CASE(__half, 64, 64)
    HA_FWD_CASE(__half, 128, 128)
    HA_FWD_CASE(__half, 128, 64)
    HA_FWD_CASE(__half, 64, 128)
  }
#undef HA_FWD_CASE
  return HA_ERR_INVALID;
}

}  // namespace ha
