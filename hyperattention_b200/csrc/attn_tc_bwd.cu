// Attention backward on tcgen05 tensor cores + TMEM, bf16/fp16, head dims 64 and 128.
//
// One CTA of 128 threads owns one tile of 128 keys and walks the query tiles that pair with it.  Per (key tile,
// query tile) pair, with thread i = TMEM lane i:
//   S  = Q K^T    (lanes = queries)      dP = dO V^T   (lanes = queries)            -> TMEM, fp32
//   p  = exp2(S*scale*log2e - lse*log2e),  ds = p * (dP - delta) * scale            per thread: its query row
//   P and dS are rounded to the input dtype and written to shared memory as [query][key] swizzled tiles, which serve
//   as MN-major A operands (P^T, dS^T: M = keys) and as a K-major A operand (dS: M = queries):
//   dV += P^T dO  (lanes = keys, accumulates in TMEM over the query tiles)
//   dK += dS^T Q  (lanes = keys, accumulates in TMEM)
//   dQ  = dS K    (lanes = queries) -> staged through shared memory -> coalesced fp32 vector reductions into dq_acc
// At the end the key tile's dK/dV rows are reduced into dk_acc/dv_acc (fp32, vector reductions).
//
// Work items of a segment: hyper = one item per sorted key tile (block window of query tiles through q_idx), plus
// (sampled key tile x chunk of query tiles in natural order) items; flash = (key tile x chunk of query tiles) with the
// causal mask applied on the diagonal pair.
// TMEM columns: S [0,128) (dQ reuses [0,D) once S is consumed), dP [128,256), dV [256,256+DV), dK [384,384+D).
#include "attn_index.cuh"

#include <type_traits>

namespace ha {

constexpr int BWD_CHUNK = 4;   // query tiles per sampled / flash work item

template <int D, int DV> struct BwdCfg {
  static constexpr int STAGES = (D == 64 && DV == 64) ? 2 : 1;
  static constexpr int K_BYTES = TILE * D * 2, V_BYTES = TILE * DV * 2;
  static constexpr int Q_BYTES = TILE * D * 2, DO_BYTES = TILE * DV * 2;
  static constexpr int P_BYTES = TILE * TILE * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_Q = OFF_V + V_BYTES;
  static constexpr int OFF_DO = OFF_Q + STAGES * Q_BYTES;
  static constexpr int OFF_P = OFF_DO + STAGES * DO_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  static constexpr int SMEM = OFF_DS + P_BYTES + 1024;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 384, COL_DQ = 0;
};

template <int COLS>
__device__ __forceinline__ void bwd_gather_tile(uint32_t smem_base, const uint16_t* __restrict__ base, int64_t row_stride, int my_row,
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

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// fp32 rows held one per thread (n_cols values in TMEM order) -> staged in shared memory -> reduced into global rows
// by index with 16-byte vector reductions, 16 lanes per 64-float slice so that a warp instruction covers two rows.
template <int NCOLS>
__device__ __forceinline__ void reduce_rows(uint8_t* stage, uint32_t tmem_addr, float* __restrict__ base, int64_t row_stride, int my_row,
                                            int tid, int warp, int lane) {
  // stage: row-major [128][NCOLS] floats, 16-byte chunk c of row r at chunk position c ^ (r & 7) within each 128-byte group
  float* srow = reinterpret_cast<float*>(stage) + tid * NCOLS;
#pragma unroll
  for (int c = 0; c < NCOLS / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tmem_addr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const int chunk = (c * 32 + i) >> 2;                          // 16-byte chunk index in the row
      const int sw = (chunk & ~7) | ((chunk ^ tid) & 7);
      *reinterpret_cast<uint4*>(srow + sw * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    }
  }
  __syncwarp();
  constexpr int CPR = NCOLS / 4;            // 16-byte chunks per row: 16 or 32
  constexpr int RPI = 32 / CPR;             // rows per warp instruction: 2 or 1
#pragma unroll
  for (int i = 0; i < 32 / RPI; ++i) {
    const int rl = i * RPI + lane / CPR;
    const int dst_row = __shfl_sync(0xffffffffu, my_row, rl);
    const int row = warp * 32 + rl;
    const int chunk = lane % CPR;
    const int sw = (chunk & ~7) | ((chunk ^ row) & 7);
    const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(stage) + row * NCOLS + sw * 4);
    if (dst_row >= 0) red_add_v4(base + (int64_t)dst_row * row_stride + chunk * 4, v.x, v.y, v.z, v.w);
  }
  __syncwarp();
}

template <typename T, int D, int DV>
__global__ void __launch_bounds__(128) attn_tc_bwd_kernel(const ha_attn_params p, int items_blk, int n_chunks) {
  using Cfg = BwdCfg<D, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_slot;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool hyper = p.mode == HA_MODE_HYPER;
  const bool causal = p.flags & HA_FLAG_CAUSAL;
  const int seg = blockIdx.y;
  const int item = blockIdx.x;
  const SegInfo si = seg_info(p, seg);
  const int n_qt = (p.m_q + TILE - 1) / TILE;

  // ---- decode the work item: key rows of this CTA and its list of query tiles ----
  int krow = -1;                 // local key row fetched / owned by this thread
  int qt_first = 0, qt_count = 0;
  bool q_sorted = false;         // query tiles addressed through q_idx (positions modulo m) or natural rows
  int q_pos0 = 0;                // sorted position of the first query of the list (hyper block part)
  int k_tile = 0;
  if (hyper && item < items_blk) {
    k_tile = item;
    krow = p.k_idx[(long long)seg * p.m_k + k_tile * TILE + tid];
    const int bs = (p.block_size + TILE - 1) / TILE;
    const Window w = block_window(k_tile, bs, p.m_q, p.flags & HA_FLAG_SMOOTH);
    q_sorted = true;
    q_pos0 = w.first;
    qt_count = w.count / TILE;
  } else {
    const int it = hyper ? item - items_blk : item;
    k_tile = it / n_chunks;
    const int z = it - k_tile * n_chunks;
    const int kr = k_tile * TILE + tid;
    if (hyper) krow = p.sample_idx ? p.sample_idx[(long long)seg * p.sample_size + kr] : kr;
    else krow = kr < p.m_k ? kr : -1;
    qt_first = z * BWD_CHUNK;
    if (!hyper && causal) qt_first = max(qt_first, k_tile);
    qt_count = min((z + 1) * BWD_CHUNK, n_qt) - qt_first;
  }
  if (qt_count <= 0) return;     // uniform over the CTA; nothing allocated yet

  const uint32_t bar = smem_u32(&mma_bar);
  if (tid == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 512);

  const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;
  const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
  const uint16_t* gbase = (const uint16_t*)p.d_o + si.b * p.do_sb + si.h * p.do_sh + si.q_row0 * p.do_sn;
  const uint16_t* kbase = (const uint16_t*)p.k + si.b * p.k_sb + si.h * p.k_sh + si.k_row0 * p.k_sn;
  const uint16_t* vbase = (const uint16_t*)p.v + si.b * p.v_sb + si.h * p.v_sh + si.k_row0 * p.v_sn;
  const float* lse_base = p.lse + head0 + si.q_row0;
  const float* delta_base = p.delta + head0 + si.q_row0;
  float* dq_base = p.dq_acc + (head0 + si.q_row0) * D;

  // local query row of thread `tid` in list entry jj (-1: none)
  auto q_row = [&](int jj) -> int {
    if (jj >= qt_count) return -1;
    if (q_sorted) {
      int pos = q_pos0 + jj * TILE + tid;
      if (pos >= p.m_q) pos -= p.m_q;
      return p.q_idx[(long long)seg * p.m_q + pos];
    }
    const int r = (qt_first + jj) * TILE + tid;
    return r < p.m_q ? r : -1;
  };

  constexpr float LOG2E = 1.4426950408889634f;
  const float scale2 = p.scale * LOG2E;

  // ---- prologue: K, V tiles and query tile 0 ----
  bwd_gather_tile<D>(s_base + Cfg::OFF_K, kbase, p.k_sn, krow, warp, lane);
  bwd_gather_tile<DV>(s_base + Cfg::OFF_V, vbase, p.v_sn, krow, warp, lane);
  int qrow_cur = q_row(0);
  bwd_gather_tile<D>(s_base + Cfg::OFF_Q, qbase, p.q_sn, qrow_cur, warp, lane);
  bwd_gather_tile<DV>(s_base + Cfg::OFF_DO, gbase, p.do_sn, qrow_cur, warp, lane);
  cp_async_commit();
  float lse_cur = qrow_cur >= 0 ? lse_base[qrow_cur] * LOG2E : INFINITY;
  float delta_cur = qrow_cur >= 0 ? delta_base[qrow_cur] : 0.f;
  int qrow_next = q_row(1);

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_sel = (uint32_t)(warp * 32) << 16;
  const uint32_t tS = tmem + Cfg::COL_S, tDP = tmem + Cfg::COL_DP, tDV = tmem + Cfg::COL_DV, tDK = tmem + Cfg::COL_DK,
                 tDQ = tmem + Cfg::COL_DQ;
  constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const uint32_t id_s = mma_idesc(TILE, TILE, AB, 0, 0);
  const uint32_t id_dv = mma_idesc(TILE, DV, AB, 1, 1);
  const uint32_t id_dk = mma_idesc(TILE, D, AB, 1, 1);
  const uint32_t id_dq = mma_idesc(TILE, D, AB, 0, 1);
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;

  uint32_t phase = 0;
  bool failed = false;

  for (int jj = 0; jj < qt_count; ++jj) {
    const int st = Cfg::STAGES == 2 ? (jj & 1) : 0;
    const uint32_t sQ = s_base + Cfg::OFF_Q + st * Cfg::Q_BYTES;
    const uint32_t sDO = s_base + Cfg::OFF_DO + st * Cfg::DO_BYTES;
    float lse_next = INFINITY, delta_next = 0.f;
    if (Cfg::STAGES == 2) {
      if (jj + 1 < qt_count) {
        bwd_gather_tile<D>(s_base + Cfg::OFF_Q + (st ^ 1) * Cfg::Q_BYTES, qbase, p.q_sn, qrow_next, warp, lane);
        bwd_gather_tile<DV>(s_base + Cfg::OFF_DO + (st ^ 1) * Cfg::DO_BYTES, gbase, p.do_sn, qrow_next, warp, lane);
        if (qrow_next >= 0) { lse_next = lse_base[qrow_next] * LOG2E; delta_next = delta_base[qrow_next]; }
      }
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    const int qrow_after = q_row(jj + 2);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- S = Q K^T and dP = dO V^T ----
    if (tid == 0) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tS, smem_desc(sQ + off, 16, 1024), smem_desc(s_base + Cfg::OFF_K + off, 16, 1024), id_s, kk > 0);
      }
#pragma unroll
      for (int kk = 0; kk < DV / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tDP, smem_desc(sDO + off, 16, 1024), smem_desc(s_base + Cfg::OFF_V + off, 16, 1024), id_s, kk > 0);
      }
      mma_commit(bar);
    }
    if (!mbar_wait(bar, phase)) failed = true;
    phase ^= 1;
    tc_fence_after();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- P and dS for this thread's query row ----
    int limit = TILE;   // visible key columns (causal diagonal pair only)
    if (!hyper && causal && qt_first + jj == k_tile) limit = tid + 1;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_sel + c * 32, rs);
      tmem_ld32(tDP + lane_sel + c * 32, rp);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint32_t pw[4], dw[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float p0 = fast_exp2(fmaf(__uint_as_float(rs[i + e]), scale2, -lse_cur));
          float p1 = fast_exp2(fmaf(__uint_as_float(rs[i + e + 1]), scale2, -lse_cur));
          if (c * 32 + i + e >= limit) p0 = 0.f;
          if (c * 32 + i + e + 1 >= limit) p1 = 0.f;
          const float d0 = p0 * (__uint_as_float(rp[i + e]) - delta_cur) * p.scale;
          const float d1 = p1 * (__uint_as_float(rp[i + e + 1]) - delta_cur) * p.scale;
          pw[e >> 1] = pack2<T>(p0, p1);
          dw[e >> 1] = pack2<T>(d0, d1);
        }
        const uint32_t off = swz_off(TILE, tid, c * 32 + i);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- dV += P^T dO, dK += dS^T Q, dQ = dS K ----
    if (tid == 0) {
      const uint32_t acc0 = jj > 0;
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        mma_ss(tDV, smem_desc(s_base + Cfg::OFF_P + kk * 2048, TILE * 128, 1024), smem_desc(sDO + kk * 2048, TILE * 128, 1024), id_dv,
               acc0 | (kk > 0));
      }
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        mma_ss(tDK, smem_desc(s_base + Cfg::OFF_DS + kk * 2048, TILE * 128, 1024), smem_desc(sQ + kk * 2048, TILE * 128, 1024), id_dk,
               acc0 | (kk > 0));
      }
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tDQ, smem_desc(s_base + Cfg::OFF_DS + off, 16, 1024), smem_desc(s_base + Cfg::OFF_K + kk * 2048, TILE * 128, 1024), id_dq,
               kk > 0);
      }
      mma_commit(bar);
    }
    if (!mbar_wait(bar, phase)) failed = true;
    phase ^= 1;
    tc_fence_after();
    if (__syncthreads_or(failed)) { failed = true; break; }

    // ---- dQ rows: TMEM -> staging (the P tile is idle now) -> fp32 reductions ----
    reduce_rows<D>(sP, tDQ + lane_sel, dq_base, D, qrow_cur, tid, warp, lane);
    if (Cfg::STAGES == 1 && jj + 1 < qt_count) {
      // single-stage variant: fetch the next query tile now that every MMA reading this one has completed
      __syncthreads();
      bwd_gather_tile<D>(s_base + Cfg::OFF_Q, qbase, p.q_sn, qrow_next, warp, lane);
      bwd_gather_tile<DV>(s_base + Cfg::OFF_DO, gbase, p.do_sn, qrow_next, warp, lane);
      cp_async_commit();
      if (qrow_next >= 0) { lse_next = lse_base[qrow_next] * LOG2E; delta_next = delta_base[qrow_next]; }
    }
    qrow_cur = qrow_next;
    qrow_next = qrow_after;
    lse_cur = lse_next;
    delta_cur = delta_next;
  }
  cp_async_wait<0>();

  if (failed) {
    if (tid == 0 && p.status) atomicExch(p.status, HA_DEV_TIMEOUT);
  } else {
    // dK / dV rows of this key tile (lanes = keys) -> reductions into the accumulators
    __syncthreads();
    float* dk_base = p.dk_acc + (head0 + si.k_row0) * D;
    float* dv_base = p.dv_acc + (head0 + si.k_row0) * DV;
    // the staging area (P and dS tiles, contiguous) is private per warp, so the two reductions can share it
    reduce_rows<DV>(sP, tDV + lane_sel, dv_base, DV, krow, tid, warp, lane);
    reduce_rows<D>(sP, tDK + lane_sel, dk_base, D, krow, tid, warp, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <typename T, int D, int DV>
static int launch_bwd(const ha_attn_params& p, cudaStream_t st) {
  using Cfg = BwdCfg<D, DV>;
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  if (segs == 0 || p.m_q == 0 || p.m_k == 0) return HA_OK;
  const int n_qt = (p.m_q + TILE - 1) / TILE, n_kt = (p.m_k + TILE - 1) / TILE;
  const int n_chunks = (n_qt + BWD_CHUNK - 1) / BWD_CHUNK;
  long long items;
  int items_blk = 0;
  if (p.mode == HA_MODE_HYPER) {
    items_blk = n_kt;
    items = (long long)n_kt + (long long)(p.sample_size / TILE) * n_chunks;
  } else {
    items = (long long)n_kt * n_chunks;
  }
  if (items > 0x7fffffffLL || segs > 65535) return HA_ERR_INVALID;
  HA_CUDA_OK(cudaFuncSetAttribute(attn_tc_bwd_kernel<T, D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM),
             "ha_attn_bwd smem attribute");
  attn_tc_bwd_kernel<T, D, DV><<<dim3((unsigned)items, (unsigned)segs), 128, Cfg::SMEM, st>>>(p, items_blk, n_chunks);
  HA_LAUNCHED("ha_attn_bwd (tcgen05)");
  return HA_OK;
}

bool tc_supported(const ha_attn_params& p);

bool tc_bwd_supported(const ha_attn_params& p) {
  if (!tc_supported(p)) return false;
  // the exact transpose of the smooth forward needs per-element masks; it runs on the CUDA-core kernel
  if ((p.flags & HA_FLAG_SMOOTH) && !(p.flags & HA_FLAG_BWD_REF_SMOOTH)) return false;
  if ((uintptr_t)p.d_o % 16 != 0 || p.do_sb % 8 != 0 || p.do_sh % 8 != 0 || p.do_sn % 8 != 0) return false;
  if ((uintptr_t)p.dq_acc % 16 != 0 || (uintptr_t)p.dk_acc % 16 != 0 || (uintptr_t)p.dv_acc % 16 != 0) return false;
  if (p.mode == HA_MODE_FLASH && p.m_q != p.m_k) return false;
  return true;
}

int tc_attn_bwd(const ha_attn_params& p, cudaStream_t st) {
#define HA_BWD_CASE(TT, DD, DDV) \
  if (p.d == DD && p.dv == DDV) return launch_bwd<TT, DD, DDV>(p, st);
  if (p.dtype == HA_BF16) {
    HA_BWD_CASE(__nv_bfloat16, 64, 64)
    HA_BWD_CASE(__nv_bfloat16, 128, 128)
    HA_BWD_CASE(__nv_bfloat16, 128, 64)
    HA_BWD_CASE(__nv_bfloat16, 64, 128)
  } else {
    HA_BWD_CASE(__half, 64, 64)
    HA_BWD_CASE(__half, 128, 128)
    HA_BWD_CASE(__half, 128, 64)
    HA_BWD_CASE(__half, 64, 128)
  }
#undef HA_BWD_CASE
  return HA_ERR_INVALID;
}

}  // namespace ha
