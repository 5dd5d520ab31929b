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
// TMEM budget per CTA: two regions of 128 columns (S; P in place; PV in the freed half) -> 256 for DV = 64, two CTAs
// per SM; the MMAs of one key tile and the S MMA of the next are issued as one batch (one commit per key tile).
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
  // TMEM: two regions (key tiles alternate).  A region holds S (128 fp32 columns); P is written in place over its first
  // 64 columns as S is consumed; the P.V product lands in the columns S no longer needs (DV = 64: the upper half of the
  // same 128 columns; DV = 128: 128 further columns).
  static constexpr int REGION = DV <= 64 ? 128 : 256;
  static constexpr int PV_OFF = DV <= 64 ? 64 : 128;
  static constexpr int TMEM_COLS = 2 * REGION;
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

// WT: weighted sampling (sample_logw / sample_mask given); a template flag so that the plain instantiation carries none of it
template <typename T, int D, int DV, bool WT>
__global__ void __launch_bounds__(128) attn_tc_fwd_kernel(const ha_attn_params p, const int pf_dist) {
  using Cfg = FwdCfg<D, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_bail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool hyper = p.mode == HA_MODE_HYPER;
  const bool causal = p.flags & HA_FLAG_CAUSAL;
  const int n_qt = (p.m_q + TILE - 1) / TILE;
  // heavy (late) causal tiles first
  const int qt = causal ? n_qt - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int seg = blockIdx.y;
  const SegInfo si = seg_info(p, seg);
  const uint32_t bar = smem_u32(&mma_bar);
  HA_T_DECL(8)

  if (cta_sees_failure(p.status, &s_bail)) return;   // an earlier CTA gave up: drain quickly (uniform over the CTA)
  if (tid == 0) {
    mbar_init(bar, 2);      // one arrival from each of the two MMA-issuing threads per batch
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
      return p.k_idx[kseg_of(p, seg) * p.m_k + pos];
    }
    const int s = (j - tl.n_blk) * TILE + tid;
    return p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + s] : s;
  };

  const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
  const uint16_t* kbase = (const uint16_t*)p.k + si.b * p.k_sb + si.hk * p.k_sh + si.k_row0 * p.k_sn;
  const uint16_t* vbase = (const uint16_t*)p.v + si.b * p.v_sb + si.hk * p.v_sh + si.k_row0 * p.v_sn;
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

  // ---- rows of the query tile that runs pf_dist CTAs later (one wave ahead): pulled into L2 while this CTA computes,
  //      so that tile's dependent index -> row gathers hit L2 instead of HBM.  Index loads are issued here, the prefetches
  //      after the first key tile, when the indices have arrived.
  constexpr int PF_TILES = 4;
  int pf_q = -1, pf_k[PF_TILES];
#pragma unroll
  for (int i = 0; i < PF_TILES; ++i) pf_k[i] = -1;
  SegInfo pf_si = si;
  {
    const long long lin = (long long)blockIdx.y * gridDim.x + blockIdx.x + pf_dist;
    if (hyper && pf_dist > 0 && lin < (long long)gridDim.x * gridDim.y) {
      const int pseg = (int)(lin / gridDim.x), pqt = (int)(lin - (long long)pseg * gridDim.x);
      pf_si = seg_info(p, pseg);
      const int bs = (p.block_size + TILE - 1) / TILE;
      const Window pw = block_window(pqt, bs, p.m_k, p.flags & HA_FLAG_SMOOTH);
      const int pn_blk = pw.count / TILE;
      pf_q = p.q_idx[(long long)pseg * p.m_q + pqt * TILE + tid];
#pragma unroll
      for (int i = 0; i < PF_TILES; ++i) {
        if (i < pn_blk) {
          int pos = pw.first + i * TILE + tid;
          if (pos >= p.m_k) pos -= p.m_k;
          pf_k[i] = p.k_idx[kseg_of(p, pseg) * p.m_k + pos];
        } else if (p.sample_idx && (i - pn_blk) * TILE < p.sample_size) {
          pf_k[i] = p.sample_idx[kseg_of(p, pseg) * p.sample_size + (i - pn_blk) * TILE + tid];
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
  constexpr int AB_FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const uint32_t idesc_s = mma_idesc(TILE, TILE, AB_FMT, 0, 0);
  const uint32_t idesc_pv = mma_idesc(TILE, DV, AB_FMT, 0, 1);

  __align__(8) float o_acc[DV];
#pragma unroll
  for (int i = 0; i < DV; ++i) o_acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const float scale2 = p.scale * 1.4426950408889634f;
  uint32_t phase = 0;
  bool failed = false;

  auto issue_s = [&](int stg, uint32_t t_s) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const uint32_t a_addr = s_base + Cfg::OFF_Q + (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
      const uint32_t b_addr = s_base + Cfg::OFF_K + stg * Cfg::K_BYTES + (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
      mma_ss(t_s, smem_desc(a_addr, 16, 1024), smem_desc(b_addr, 16, 1024), idesc_s, kk > 0);
    }
  };
  auto issue_pv = [&](int stg, uint32_t t_p, uint32_t t_pv) {
#pragma unroll
    for (int kk = 0; kk < TILE / 16; ++kk) {
      const uint32_t b_addr = s_base + Cfg::OFF_V + stg * Cfg::V_BYTES + kk * 2048;
      mma_ts(t_pv, t_p + kk * 8, smem_desc(b_addr, TILE * 128, 1024), idesc_pv, kk > 0);
    }
  };
  auto accumulate_pv = [&](uint32_t t_pv, float alpha) {
    const uint64_t al2 = pack_f2(alpha, alpha);
    uint64_t* o2 = reinterpret_cast<uint64_t*>(o_acc);
#pragma unroll
    for (int c = 0; c < DV / 32; ++c) {
      uint32_t r[32];
      tmem_ld32(t_pv + lane_sel + c * 32, r);
      tmem_ld_fence(r);
#pragma unroll
      for (int i = 0; i < 32; i += 2) o2[(c * 32 + i) >> 1] = ffma2(o2[(c * 32 + i) >> 1], al2, pack_u2(r[i], r[i + 1]));
    }
  };

  // Schedule: batch(j) = { P.V of key tile j ; S of key tile j+1 } is one commit; while it runs, the other CTA on the SM
  // has the pipes.  The product of tile j-1 is folded into the output registers at the top of iteration j.
  cp_async_wait<0>();
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Two threads issue the MMAs of a batch: thread 0 the P V product of key tile j, thread 32 S of key tile j + 1.  One thread
  // gets a tcgen05.mma accepted only about every 110-130 cycles whatever its shape (measured), so the 12 instructions of a
  // batch from one thread cost more than the tensor pipe needs for them; each thread arrives once per batch (a commit
  // after its instructions, or a plain arrival when it has none).
  if (tid == 0) mbar_arrive(bar);
  if (tid == 32) {
    issue_s(0, tmem);
    mma_commit(bar);
  }
  float alpha_prev = 0.f;
  HA_T_MARK(7)
  for (int j = 0; j < tl.n_tiles; ++j) {
    HA_T_MARK(0)
    const int st = j & 1;
    const uint32_t tS = tmem + st * Cfg::REGION, tP = tS, tPV = tS + Cfg::PV_OFF;
    if (!mbar_wait(bar, phase)) { failed = true; }     // batch(j-1): S of this tile (and P.V of the previous one) landed
    phase ^= 1;
    tc_fence_after();
    if (__syncthreads_or(failed)) { failed = true; break; }
    HA_T_MARK(1)
    // the other stage is free now: fetch key tile j+1
    if (j + 1 < tl.n_tiles) {
      gather_tile<D>(s_base + Cfg::OFF_K + (st ^ 1) * Cfg::K_BYTES, kbase, p.k_sn, krow_next, warp, lane);
      gather_tile<DV>(s_base + Cfg::OFF_V + (st ^ 1) * Cfg::V_BYTES, vbase, p.v_sn, krow_next, warp, lane);
    }
    cp_async_commit();
    const int krow_after = key_row(j + 2);   // index load for the tile after next, consumed next iteration
    if (j >= 1) accumulate_pv(tmem + (st ^ 1) * Cfg::REGION + Cfg::PV_OFF, alpha_prev);
    HA_T_MARK(2)
    // ---- softmax over this tile's 128 columns ----
    // visible columns of this row: all of them, except on a causal diagonal tile or a ragged last tile
    int limit = TILE;
    bool masked = false;   // uniform over the CTA
    // weighted sampling: a sampled tile's scores get the tile's log weight, and its dropped slots are masked
    uint32_t wm[4] = {0u, 0u, 0u, 0u};
    float bias2 = 0.f;
    if (WT && hyper && j >= tl.n_blk) {
      const long long qtile = (long long)seg * n_qt + qt;
      const uint32_t* mw = p.sample_mask + qtile * (p.sample_size / 32) + (j - tl.n_blk) * 4;
      wm[0] = mw[0]; wm[1] = mw[1]; wm[2] = mw[2]; wm[3] = mw[3];
      bias2 = p.sample_logw[qtile] * 1.4426950408889634f;
      masked = (wm[0] | wm[1] | wm[2] | wm[3]) != 0u;
    }
    if (!hyper) {
      limit = min(TILE, p.m_k - j * TILE);
      masked = limit < TILE;
      if (causal) {
        limit = min(limit, qpos - j * TILE + 1);
        masked = masked || (j == qt);
      }
    }
    float mx;
    {
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      uint32_t ra[32], rb[32];
      tmem_ld32(tS + lane_sel, ra);
      tmem_ld_fence(ra);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        if (c + 1 < 4) tmem_ld32(tS + lane_sel + (c + 1) * 32, nxt);
        if (!masked) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            m0 = fmax3(m0, __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
            m1 = fmax3(m1, __uint_as_float(cur[i + 2]), __uint_as_float(cur[i + 3]));
            m2 = fmax3(m2, __uint_as_float(cur[i + 4]), __uint_as_float(cur[i + 5]));
            m3 = fmax3(m3, __uint_as_float(cur[i + 6]), __uint_as_float(cur[i + 7]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < limit && !(WT && ((wm[c] >> i) & 1u))) m0 = fmaxf(m0, __uint_as_float(cur[i]));
        }
        if (c + 1 < 4) tmem_ld_fence(nxt);
      }
      mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
    }
    const float m_new = fmaxf(m_run, WT ? mx * scale2 + bias2 : mx * scale2);
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float alpha = fast_exp2(m_run - m_use);   // m_run = -inf -> 0
    float psum;
    {
      const uint64_t sc2 = pack_f2(scale2, scale2), negm = WT ? pack_f2(bias2 - m_use, bias2 - m_use) : pack_f2(-m_use, -m_use);
      uint64_t ps_a = pack_f2(0.f, 0.f), ps_b = ps_a;
      uint32_t ra[32], rb[32];
      tmem_ld32(tS + lane_sel, ra);
      tmem_ld_fence(ra);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t(&cur)[32] = (c & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (c & 1) ? ra : rb;
        // P chunk c below overwrites columns [16c, 16c+16), part of S chunk c/2, which is already in registers; the
        // chunk being loaded (c+1) lies in columns >= 32(c+1), disjoint from them
        if (c + 1 < 4) tmem_ld32(tS + lane_sel + (c + 1) * 32, nxt);
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float p0, p1, p2, p3;
          unpack_f2(ffma2(pack_u2(cur[i], cur[i + 1]), sc2, negm), p0, p1);
          unpack_f2(ffma2(pack_u2(cur[i + 2], cur[i + 3]), sc2, negm), p2, p3);
          p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
          if (masked) {
            if (c * 32 + i >= limit || (WT && ((wm[c] >> i) & 1u))) p0 = 0.f;
            if (c * 32 + i + 1 >= limit || (WT && ((wm[c] >> (i + 1)) & 1u))) p1 = 0.f;
            if (c * 32 + i + 2 >= limit || (WT && ((wm[c] >> (i + 2)) & 1u))) p2 = 0.f;
            if (c * 32 + i + 3 >= limit || (WT && ((wm[c] >> (i + 3)) & 1u))) p3 = 0.f;
          }
          ps_a = fadd2(ps_a, pack_f2(p0, p1));
          ps_b = fadd2(ps_b, pack_f2(p2, p3));
          pk[i >> 1] = pack2<T>(p0, p1);
          pk[(i >> 1) + 1] = pack2<T>(p2, p3);
        }
        tmem_st16(tP + lane_sel + c * 16, pk);
        if (c + 1 < 4) tmem_ld_fence(nxt);
      }
      float s0, s1;
      unpack_f2(fadd2(ps_a, ps_b), s0, s1);
      psum = s0 + s1;
    }
    tmem_st_wait();
    l_run = l_run * alpha + psum;
    m_run = m_new;
    alpha_prev = alpha;
    HA_T_MARK(3)
    cp_async_wait<0>();                        // key tile j+1 has landed
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (tid == 0) {
      issue_pv(st, tP, tPV);
      mma_commit(bar);
    }
    if (tid == 32) {
      if (j + 1 < tl.n_tiles) {
        issue_s(st ^ 1, tmem + (st ^ 1) * Cfg::REGION);
        mma_commit(bar);
      } else {
        mbar_arrive(bar);
      }
    }
    HA_T_MARK(4)
    krow_cur = krow_next;
    krow_next = krow_after;
    if (j == 0 && pf_q >= 0) {
      const uint16_t* pq = (const uint16_t*)p.q + pf_si.b * p.q_sb + pf_si.h * p.q_sh + (pf_si.q_row0 + pf_q) * p.q_sn;
      const uint16_t* pk = (const uint16_t*)p.k + pf_si.b * p.k_sb + pf_si.hk * p.k_sh + pf_si.k_row0 * p.k_sn;
      const uint16_t* pv = (const uint16_t*)p.v + pf_si.b * p.v_sb + pf_si.hk * p.v_sh + pf_si.k_row0 * p.v_sn;
      prefetch_l2(pq);
      if (D > 64) prefetch_l2(pq + 64);
      if (merge) {
        const uint16_t* po = (const uint16_t*)p.o + pf_si.b * p.o_sb + pf_si.h * p.o_sh + (pf_si.q_row0 + pf_q) * p.o_sn;
        prefetch_l2(po);
        if (DV > 64) prefetch_l2(po + 64);
      }
#pragma unroll
      for (int i = 0; i < PF_TILES; ++i) {
        if (pf_k[i] >= 0) {
          prefetch_l2(pk + (int64_t)pf_k[i] * p.k_sn);
          if (D > 64) prefetch_l2(pk + (int64_t)pf_k[i] * p.k_sn + 64);
          prefetch_l2(pv + (int64_t)pf_k[i] * p.v_sn);
          if (DV > 64) prefetch_l2(pv + (int64_t)pf_k[i] * p.v_sn + 64);
        }
      }
    }
    HA_T_MARK(5)
  }
  cp_async_wait<0>();
  if (!failed) {
    if (!mbar_wait(bar, phase)) failed = true;          // the last P.V
    phase ^= 1;
    tc_fence_after();
    failed = __syncthreads_or(failed);
    if (!failed) accumulate_pv(tmem + ((tl.n_tiles - 1) & 1) * Cfg::REGION + Cfg::PV_OFF, alpha_prev);
  }

  if (failed) {
    if (tid == 0) report_timeout(p.status, p.status_host);
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
    if (merge) {
      // merge (the causal schedule's rectangles): rows staged in shared memory and stored row-coalesced; measured faster
      // here than per-thread row stores (two output tensors per tile and the read of the previous rows)
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
        const float2 old = unpack2<T>(*slot);
        a = w1 * old.x + w2 * round_to<T>(a);
        b = w1 * old.y + w2 * round_to<T>(b);
        *slot = pack2<T>(a, b);
      }
      __syncwarp();
      scatter_tile<DV>(stage, obase, p.o_sn, qrow, warp, lane);
    } else {
      // each thread stores its own row: DV contiguous elements in 16-byte pieces straight from registers (whole 32-byte
      // sectors pair up in L2); much less code than staging, and this code runs once per tile
      if (p.part_o && qrow >= 0) {
        // un-merged result of this call
        uint4* prow = reinterpret_cast<uint4*>((uint16_t*)p.part_o + si.b * p.o_sb + si.h * p.o_sh + (si.q_row0 + qrow) * p.o_sn);
#pragma unroll
        for (int e = 0; e < DV; e += 8)
          prow[e >> 3] = make_uint4(pack2<T>(o_acc[e] * inv, o_acc[e + 1] * inv), pack2<T>(o_acc[e + 2] * inv, o_acc[e + 3] * inv),
                                    pack2<T>(o_acc[e + 4] * inv, o_acc[e + 5] * inv), pack2<T>(o_acc[e + 6] * inv, o_acc[e + 7] * inv));
        if (p.part_lse) p.part_lse[lse_at] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      }
      if (qrow >= 0) {
        uint4* orow = reinterpret_cast<uint4*>(obase + (int64_t)qrow * p.o_sn);
#pragma unroll
        for (int e = 0; e < DV; e += 8) {
          uint32_t w[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            w[h] = pack2<T>(o_acc[e + 2 * h] * inv, o_acc[e + 2 * h + 1] * inv);
          }
          orow[e >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
    if (qrow >= 0) p.lse[lse_at] = lse;
  }

  HA_T_MARK(6)
  HA_T_DUMP(8, (int)(blockIdx.y * gridDim.x + blockIdx.x), tid == 0)
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, Cfg::TMEM_COLS);
}

template <typename T, int D, int DV, bool WT>
static int launch_fwd(const ha_attn_params& p, cudaStream_t st) {
  using Cfg = FwdCfg<D, DV>;
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const int n_qt = (p.m_q + TILE - 1) / TILE;
  if (segs == 0 || n_qt == 0) return HA_OK;
  if (segs > 65535) return HA_ERR_INVALID;
  HA_SMEM_ATTR_ONCE((attn_tc_fwd_kernel<T, D, DV, WT>), Cfg::SMEM, "ha_attn_fwd smem attribute");
  // CTAs resident at once (shared memory and TMEM allow two per SM at head dim 64, one otherwise) = prefetch distance
  const int sms = sm_count();
  const int pf_dist = p.mode == HA_MODE_HYPER ? sms * (Cfg::TMEM_COLS == 256 ? 2 : 1) : 0;
  attn_tc_fwd_kernel<T, D, DV, WT><<<dim3(n_qt, (unsigned)segs), 128, Cfg::SMEM, st>>>(p, pf_dist);
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
  if (p.d == DD && p.dv == DDV) return p.sample_logw ? launch_fwd<TT, DD, DDV, true>(p, st) : launch_fwd<TT, DD, DDV, false>(p, st);
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

HA_T_SETTER(ha_debug_set_timing_buffer_fwd)
