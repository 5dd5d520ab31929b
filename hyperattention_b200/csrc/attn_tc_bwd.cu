// Attention backward on tcgen05 tensor cores + TMEM, bf16/fp16, head dims 64 and 128.
//
// Persistent CTAs of 256 threads (two groups of 128; thread (g, i) = TMEM lane i, the groups split the columns of the
// elementwise phase and of the reductions), one per SM.  A CTA works through work items: it starts with item blockIdx.x
// and draws every further one from the launch's counter; a work item owns one tile of 128 keys (or the two key tiles of
// a 256-row block, or both sampled tiles) and walks the query tiles that pair with it.  As soon as an item's last MMAs
// have completed, the next item's K / V / Q / dO gathers are issued, so they travel while its gradient rows drain.
// Per (key tile, query tile) pair:
//   S  = Q K^T    (lanes = queries)      dP = dO V^T   (lanes = queries)            -> TMEM, fp32
//   p  = exp2(S*scale*log2e - lse*log2e),  ds = p * (dP - delta) * scale            per thread: its query row
//   P and dS are rounded to the input dtype and written to shared memory as [query][key] swizzled tiles, which serve
//   as MN-major A operands (P^T, dS^T: M = keys) and as a K-major A operand (dS: M = queries):
//   dV += P^T dO  (lanes = keys, accumulates in TMEM over the query tiles)
//   dK += dS^T Q  (lanes = keys, accumulates in TMEM)
//   dQ  = dS K    (lanes = queries) -> staged through shared memory -> coalesced fp32 vector reductions into dq_acc
//                 (or, where one work item holds a query tile's complete sum, the final typed rows: dq_out)
// At the end of a key tile its dK/dV rows are reduced into dk_acc/dv_acc the same way, or stored once in the tensors'
// dtype where one work item holds the complete sum (dk_out / dv_out; HA_FLAG_BWD_KV_INIT).
//
// Work items of a segment: hyper = one item per sorted key tile (block window of query tiles through q_idx) or per
// 256-row block, plus (sampled key tile x chunk of query tiles) items; flash = (key tile x chunk of query tiles) with
// the causal mask applied on the diagonal pair.
// TMEM columns (head dims 64): S [0,128), dP [128,256), dV [256,320), dK [320,384), dQ two buffers [384,512);
// (head dim 128): S [0,128) (dQ reuses [0,D) once S is consumed), dP [128,256), dV [256,256+DV), dK [384,384+D).
#include "attn_index.cuh"

#include <mutex>
#include <type_traits>

namespace ha {

constexpr int BWD_CHUNK = 16;  // query tiles per sampled / flash work item

// bytes of one column half of a reduction staging tile (128 rows x NC floats)
template <int NC> struct RedStage { static constexpr int BYTES = TILE * NC * 4; };

template <int D, int DV> struct BwdCfg {
  // PIPE (head dims 64): query tiles double buffered, dQ double buffered in its own TMEM columns and a separate staging
  // tile, so that the MMAs of pair j and the S/dP MMAs of pair j+1 run as one batch underneath the thread work.
  static constexpr bool PIPE = (D == 64 && DV == 64);
  static constexpr int STAGES = PIPE ? 2 : 1;
  static constexpr int K_BYTES = TILE * D * 2, V_BYTES = TILE * DV * 2;
  static constexpr int Q_BYTES = TILE * D * 2, DO_BYTES = TILE * DV * 2;
  static constexpr int P_BYTES = TILE * TILE * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_Q = OFF_V + V_BYTES;
  static constexpr int OFF_DO = OFF_Q + STAGES * Q_BYTES;
  static constexpr int OFF_P = OFF_DO + STAGES * DO_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  // staging rows of the reductions (two column halves): a tile of its own when pipelined, else over the idle
  // P / dS tiles (which it may outgrow by a few KB)
  static constexpr int MAXD = D > DV ? D : DV;
  static constexpr int STG_HALF = RedStage<MAXD / 2>::BYTES;
  static constexpr int OFF_STG = PIPE ? OFF_DS + P_BYTES : OFF_P;
  // second key tile of a paired block item (PIPE only): K, V of key tile 2b+1 next to those of 2b
  static constexpr int OFF_K2 = (OFF_STG + 2 * STG_HALF > OFF_DS + P_BYTES ? OFF_STG + 2 * STG_HALF : OFF_DS + P_BYTES);
  static constexpr int OFF_V2 = OFF_K2 + K_BYTES;
  static constexpr int SMEM = OFF_K2 + (PIPE ? K_BYTES + V_BYTES : 0) + 1024;
  // TMEM columns: S [0,128), dP [128,256), dV [256,256+DV), dK; dQ: two buffers of its own (PIPE) or over S
  static constexpr int COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = PIPE ? 320 : 384, COL_DQ = PIPE ? 384 : 0;
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

// NC fp32 values per thread (columns [0, NC) at tmem_addr of the thread's TMEM lane = row `row` of the tile) -> staged in
// shared memory -> reduced into global rows by index with 16-byte vector reductions; NC/4 neighbouring lanes cover one
// row, so a warp instruction adds whole 128-byte (NC = 32) or 256-byte (NC = 64) row slices.  `stage` holds 128 rows of
// NC floats (16-byte chunk c of row r at position c ^ (r & 7) of its 128-byte group); a warp only touches the 32 rows of
// its own lanes, so a warp-level sync suffices.  (A TMA bulk reduce-add per row was measured slower than this.)
// MODE 0: red.add into fp32 rows.  MODE 1: plain fp32 store (first contribution to rows nobody has written yet).
// MODE 2: the complete sum: stored in type T at `out` (same row / column layout); nothing is read.
// Every mode maps (row, 16-byte chunk) to the same lane, so a store and a later reduction of one address come from one
// thread, in program order.
template <int NC, int MODE = 0, typename T = float>
__device__ __forceinline__ void reduce_rows(uint8_t* stage, uint32_t tmem_addr, float* __restrict__ base, int64_t row_stride, int my_row,
                                            int row, T* __restrict__ out = nullptr) {
  const int lane = row & 31, qwarp = row >> 5;
  float* srow = reinterpret_cast<float*>(stage) + row * NC;
#pragma unroll
  for (int c = 0; c < NC / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tmem_addr + c * 32, r);
    tmem_ld_fence(r);
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const int chunk = (c * 32 + i) >> 2;
      const int sw = (chunk & ~7) | ((chunk ^ row) & 7);
      *reinterpret_cast<uint4*>(srow + sw * 4) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    }
  }
  __syncwarp();
  constexpr int CPR = NC / 4;               // 16-byte chunks per row: 8, 16 (or 32)
  constexpr int RPI = 32 / CPR;             // rows per warp instruction
  constexpr int NI = 32 / RPI;
  const int chunk = lane % CPR;
  if constexpr (MODE == 2) {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int rl = i * RPI + lane / CPR;
      const int dst_row = __shfl_sync(0xffffffffu, my_row, rl);
      const int rr = qwarp * 32 + rl;
      const int sw = (chunk & ~7) | ((chunk ^ rr) & 7);
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(stage) + rr * NC + sw * 4);
      if (dst_row >= 0)
        *reinterpret_cast<uint2*>(out + (int64_t)dst_row * row_stride + chunk * 4) = make_uint2(pack2<T>(v.x, v.y), pack2<T>(v.z, v.w));
    }
  } else {
#pragma unroll
    for (int i = 0; i < NI; ++i) {
      const int rl = i * RPI + lane / CPR;
      const int dst_row = __shfl_sync(0xffffffffu, my_row, rl);
      const int rr = qwarp * 32 + rl;
      const int sw = (chunk & ~7) | ((chunk ^ rr) & 7);
      const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(stage) + rr * NC + sw * 4);
      if (dst_row >= 0) {
        float* dst = base + (int64_t)dst_row * row_stride + chunk * 4;
        if (MODE == 0) red_add_v4(dst, v.x, v.y, v.z, v.w);
        else *reinterpret_cast<float4*>(dst) = v;
      }
    }
  }
  __syncwarp();
}

// NC fp32 values of the thread's TMEM lane -> NC values of type T stored at columns [0, NC) of global row my_row
// (16-byte stores; a thread writes NC*2 contiguous bytes, whole 32-byte sectors)
template <typename T, int NC>
__device__ __forceinline__ void store_rows(uint32_t tmem_addr, T* __restrict__ base, int64_t row_stride, int my_row) {
#pragma unroll
  for (int c = 0; c < NC / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(tmem_addr + c * 32, r);
    tmem_ld_fence(r);
    if (my_row >= 0) {
      uint4* dst = reinterpret_cast<uint4*>(base + (int64_t)my_row * row_stride + c * 32);
#pragma unroll
      for (int i = 0; i < 32; i += 8)
        dst[i >> 3] = make_uint4(pack2<T>(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                                 pack2<T>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                                 pack2<T>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                                 pack2<T>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
    }
  }
}

// One work item: the key rows of a CTA and its list of query tiles.
struct BwdItem {
  int krow;                  // local key row fetched / owned by thread tid (-1: none)
  int krow2;                 // paired block item: row of the second key tile
  bool paired;               // block item over BOTH key tiles of a 256-row block: pairs (A,Q0) (A,Q1) (B,Q0) (B,Q1)
  bool fused;                // paired item that also takes the two sampled key tiles: eight pairs (A, B, S0, S1) x (Q0, Q1)
  int srow0, srow1;          // fused item: this thread's rows of the two sampled key tiles
  int qt_first, qt_count;    // natural-order query tiles [qt_first, qt_first + qt_count) ...
  bool q_sorted;             // ... or, when set, qt_count tiles of sorted positions starting at q_pos0 (modulo m_q)
  int q_pos0;
  int k_tile;
};

__device__ __forceinline__ BwdItem bwd_decode(const ha_attn_params& p, int item, int seg, int items_blk, int n_chunks, int tid,
                                              bool weighted, bool paired, bool fused) {
  BwdItem it;
  it.fused = false;
  it.srow0 = it.srow1 = -1;
  it.krow2 = -1;
  it.paired = false;
  const bool hyper = p.mode == HA_MODE_HYPER;
  const int n_qt = (p.m_q + TILE - 1) / TILE;
  it.krow = -1;
  it.qt_first = 0;
  it.qt_count = 0;
  it.q_sorted = false;
  it.q_pos0 = 0;
  if (hyper && item < items_blk && paired) {
    // block size 256, plain windows: key tiles 2b, 2b+1 and query tiles 2b, 2b+1 form four pairs
    it.paired = true;
    it.k_tile = 2 * item;
    it.krow = p.k_idx[kseg_of(p, seg) * p.m_k + it.k_tile * TILE + tid];
    it.krow2 = p.k_idx[kseg_of(p, seg) * p.m_k + (it.k_tile + 1) * TILE + tid];
    it.q_sorted = true;
    it.q_pos0 = it.k_tile * TILE;
    it.qt_count = 4;
    if (fused) {
      // ... and the two sampled key tiles against the same two query tiles: pairs 4..7
      it.fused = true;
      it.qt_count = 8;
      it.srow0 = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + tid] : tid;
      it.srow1 = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + TILE + tid] : TILE + tid;
    }
  } else if (hyper && item < items_blk) {
    it.k_tile = item;
    it.krow = p.k_idx[kseg_of(p, seg) * p.m_k + it.k_tile * TILE + tid];
    const int bs = (p.block_size + TILE - 1) / TILE;
    const Window w = block_window(it.k_tile, bs, p.m_q, p.flags & HA_FLAG_SMOOTH);
    it.q_sorted = true;
    it.q_pos0 = w.first;
    it.qt_count = w.count / TILE;
  } else {
    const int i2 = hyper ? item - items_blk : item;
    int z;
    if (hyper) {
      // the items of the sampled key tiles that cover the same chunk of query tiles are neighbours in the grid: the
      // second one finds the query rows and the dQ rows of the chunk in L2
      const int ns = p.sample_size / TILE;
      z = i2 / ns;
      it.k_tile = i2 - z * ns;
    } else {
      it.k_tile = i2 / n_chunks;
      z = i2 - it.k_tile * n_chunks;
    }
    const int kr = it.k_tile * TILE + tid;
    if (hyper) it.krow = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + kr] : kr;
    else it.krow = kr < p.m_k ? kr : -1;
    it.qt_first = z * BWD_CHUNK;
    if (!hyper && (p.flags & HA_FLAG_CAUSAL)) it.qt_first = max(it.qt_first, it.k_tile);
    it.qt_count = min((z + 1) * BWD_CHUNK, n_qt) - it.qt_first;
    if (hyper && weighted) {
      // weighted sampling: the weight and the dropped slots belong to SORTED query tiles, so walk those
      it.q_sorted = true;
      it.q_pos0 = it.qt_first * TILE;
    }
  }
  return it;
}

// local query row of thread tid in list entry jj of an item (-1: none)
__device__ __forceinline__ int bwd_q_row(const ha_attn_params& p, const BwdItem& it, int seg, int jj, int tid) {
  if (jj >= it.qt_count) return -1;
  if (it.q_sorted) {
    int pos = it.q_pos0 + (it.paired ? (jj & 1) : jj) * TILE + tid;
    if (pos >= p.m_q) pos -= p.m_q;
    return p.q_idx[(long long)seg * p.m_q + pos];
  }
  const int r = (it.qt_first + jj) * TILE + tid;
  return r < p.m_q ? r : -1;
}

// One unit of a persistent CTA's work list: item `item` of segment `seg`, with the row indices its first loads need.
struct BwdWork {
  BwdItem me;
  SegInfo si;
  int seg, item;
  int qrow0, qrow1;          // local query rows of this thread for the first two list entries
  bool valid;
};

__device__ __forceinline__ BwdWork bwd_work(const ha_attn_params& p, long long w, long long n_work, int items_per_seg, int item_base,
                                            int items_blk, int n_chunks, int tid, bool weighted, bool paired, bool fused) {
  BwdWork wk;
  wk.valid = w < n_work;
  wk.seg = 0;
  wk.item = 0;
  wk.qrow0 = wk.qrow1 = -1;
  wk.me.qt_count = 0;
  if (wk.valid) {
    wk.seg = (int)(w / items_per_seg);
    wk.item = (int)(w - (long long)wk.seg * items_per_seg) + item_base;
    wk.si = seg_info(p, wk.seg);
    wk.me = bwd_decode(p, wk.item, wk.seg, items_blk, n_chunks, tid, weighted, paired, fused);
    wk.qrow0 = bwd_q_row(p, wk.me, wk.seg, 0, tid);
    wk.qrow1 = bwd_q_row(p, wk.me, wk.seg, 1, tid);
  }
  return wk;
}

// WT: weighted sampling (sample_logw / sample_mask given); a template flag so that the plain instantiation carries none of it
template <typename T, int D, int DV, bool WT>
__global__ void __launch_bounds__(256) attn_tc_bwd_kernel(const ha_attn_params p, int items_blk, int n_chunks, int items_per_seg,
                                                          long long n_work, int mode_bits, int item_base,
                                                          unsigned int* __restrict__ work_counter) {
  using Cfg = BwdCfg<D, DV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ long long s_next_w;     // the work item this CTA takes next (fetched by thread 0 from the launch's counter)
  __shared__ int s_bail;

  // 256 threads = two groups of 128.  Thread (wg, row): TMEM lane `row`; in the elementwise phase group wg handles key
  // columns [64 wg, 64 wg + 64) of that row, in the reductions the column half wg of its row.
  const int tid = threadIdx.x, lane = tid & 31;
  const int row = tid & 127, wg = tid >> 7, qwarp = (tid >> 5) & 3;
  const bool hyper = p.mode == HA_MODE_HYPER;
  const bool causal = p.flags & HA_FLAG_CAUSAL;
  // mode_bits: 1 = block items cover whole 256-row blocks (paired); 4 = fused: they also take the two sampled key tiles
  // (no sampled items); 2 = final dQ: a block item then holds a query tile's complete dQ sum and writes the dq_out rows
  const bool pair_blocks = Cfg::PIPE && (mode_bits & 1), final_dq = Cfg::PIPE && (mode_bits & 2), fuse_sampled = Cfg::PIPE && (mode_bits & 4);
  if (cta_sees_failure(p.status, &s_bail)) return;   // an earlier CTA gave up: drain quickly (uniform over the CTA)

  // ---- once per CTA: barrier, TMEM ----
  const uint32_t bar = smem_u32(&mma_bar);
  if (tid == 0) {
    mbar_init(bar, 5);      // one arrival per batch from each of the five MMA-issuing threads
    mbar_fence_init();
  }
  if (tid < 32) tmem_alloc(smem_u32(&tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t lane_sel = (uint32_t)(qwarp * 32) << 16;
  const uint32_t tS = tmem + Cfg::COL_S, tDP = tmem + Cfg::COL_DP, tDV = tmem + Cfg::COL_DV, tDK = tmem + Cfg::COL_DK,
                 tDQ = tmem + Cfg::COL_DQ;
  constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  const uint32_t id_s = mma_idesc(TILE, TILE, AB, 0, 0);
  const uint32_t id_dv = mma_idesc(TILE, DV, AB, 1, 1);
  const uint32_t id_dk = mma_idesc(TILE, D, AB, 1, 1);
  const uint32_t id_dq = mma_idesc(TILE, D, AB, 0, 1);
  uint8_t* sP = smem + Cfg::OFF_P;
  uint8_t* sDS = smem + Cfg::OFF_DS;
  constexpr float LOG2E = 1.4426950408889634f;
  const float scale2 = p.scale * LOG2E;

  uint32_t phase = 0;
  bool failed = false;
  HA_T_DECL(8)

  // The first loads of a work item: K, V tiles and query tile 0 (one copy group), then -- pipelined schedule -- query
  // tile 1 and a second key tile (another group).  Group 0 fetches the K / Q tiles, group 1 the V / dO tiles.  Both
  // groups are committed even when empty, so that the waits below always count the same groups.
  auto issue_loads = [&](const BwdWork& wk) {
    const bool go = wk.valid && wk.me.qt_count > 0;
    const uint16_t* qb = (const uint16_t*)p.q + wk.si.b * p.q_sb + wk.si.h * p.q_sh + wk.si.q_row0 * p.q_sn;
    const uint16_t* gb = (const uint16_t*)p.d_o + wk.si.b * p.do_sb + wk.si.h * p.do_sh + wk.si.q_row0 * p.do_sn;
    const uint16_t* kb = (const uint16_t*)p.k + wk.si.b * p.k_sb + wk.si.hk * p.k_sh + wk.si.k_row0 * p.k_sn;
    const uint16_t* vb = (const uint16_t*)p.v + wk.si.b * p.v_sb + wk.si.hk * p.v_sh + wk.si.k_row0 * p.v_sn;
    if (go) {
      if (wg == 0) {
        bwd_gather_tile<D>(s_base + Cfg::OFF_K, kb, p.k_sn, wk.me.krow, qwarp, lane);
        bwd_gather_tile<D>(s_base + Cfg::OFF_Q, qb, p.q_sn, wk.qrow0, qwarp, lane);
      } else {
        bwd_gather_tile<DV>(s_base + Cfg::OFF_V, vb, p.v_sn, wk.me.krow, qwarp, lane);
        bwd_gather_tile<DV>(s_base + Cfg::OFF_DO, gb, p.do_sn, wk.qrow0, qwarp, lane);
      }
    }
    cp_async_commit();
    if (Cfg::PIPE) {
      if (go && wk.me.qt_count > 1) {
        if (wg == 0) bwd_gather_tile<D>(s_base + Cfg::OFF_Q + Cfg::Q_BYTES, qb, p.q_sn, wk.qrow1, qwarp, lane);
        else bwd_gather_tile<DV>(s_base + Cfg::OFF_DO + Cfg::DO_BYTES, gb, p.do_sn, wk.qrow1, qwarp, lane);
      }
      if (go && wk.me.paired) {
        if (wg == 0) bwd_gather_tile<D>(s_base + Cfg::OFF_K2, kb, p.k_sn, wk.me.krow2, qwarp, lane);
        else bwd_gather_tile<DV>(s_base + Cfg::OFF_V2, vb, p.v_sn, wk.me.krow2, qwarp, lane);
      }
      cp_async_commit();
    }
  };
  auto next_work = [&](long long w) { return bwd_work(p, w, n_work, items_per_seg, item_base, items_blk, n_chunks, row, WT, pair_blocks, fuse_sampled); };

  // ---- persistent loop over work items.  A CTA starts with item blockIdx.x and draws every further one from the
  //      launch's counter (items differ in length: 1 to 16 pairs), early in the current item; the next item's first
  //      loads are issued as soon as the last MMAs of the current one have completed, i.e. underneath its drains ----
  auto draw_next = [&]() {
    if (tid == 0) s_next_w = (long long)gridDim.x + atomicAdd(work_counter, 1u);
  };
  BwdWork cur = next_work(blockIdx.x);
  issue_loads(cur);
  for (long long w = blockIdx.x; w < n_work && !failed;) {
  BwdWork nxt;
  nxt.valid = false;
  nxt.me.qt_count = 0;
  const BwdItem me = cur.me;
  const int seg = cur.seg, item = cur.item;
  const SegInfo si = cur.si;
  const bool paired = Cfg::PIPE && me.paired, fused = Cfg::PIPE && me.fused;
  const int krow = me.krow, qt_first = me.qt_first, qt_count = me.qt_count, k_tile = me.k_tile;
  if (qt_count <= 0) {           // nothing to do for this item (uniform over the CTA): its (empty) copy groups retire
    cp_async_wait<0>();
    draw_next();
    __syncthreads();
    w = s_next_w;
    __syncthreads();             // everybody has read the slot before it is written again
    nxt = next_work(w);
    issue_loads(nxt);
    cur = nxt;
    continue;
  }

  const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;
  const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
  const uint16_t* gbase = (const uint16_t*)p.d_o + si.b * p.do_sb + si.h * p.do_sh + si.q_row0 * p.do_sn;
  const float* lse_base = p.lse + head0 + si.q_row0;
  const float* delta_base = p.delta + head0 + si.q_row0;
  float* dq_base = p.dq_acc + (head0 + si.q_row0) * D;

  auto q_row = [&](int jj) -> int { return bwd_q_row(p, me, seg, jj, row); };
  auto fetch_q = [&](int stage, int qr) {
    if (wg == 0) bwd_gather_tile<D>(s_base + Cfg::OFF_Q + stage * Cfg::Q_BYTES, qbase, p.q_sn, qr, qwarp, lane);
    else bwd_gather_tile<DV>(s_base + Cfg::OFF_DO + stage * Cfg::DO_BYTES, gbase, p.do_sn, qr, qwarp, lane);
  };

  // ---- K, V and query tile 0 (and tile 1 / the second key tile) are in flight already ----
  int qrow_cur = cur.qrow0;
  float lse_cur = qrow_cur >= 0 ? lse_base[qrow_cur] * LOG2E : INFINITY;
  float delta_cur = qrow_cur >= 0 ? delta_base[qrow_cur] : 0.f;
  int qrow_next = cur.qrow1;

  // The MMAs of a batch are issued by five threads, one product each: one thread gets a tcgen05.mma accepted only about
  // every 110-130 cycles whatever its shape (measured), so the 32 instructions of a batch from one thread cost twice what
  // the tensor pipe needs for them.  Thread 0: dV, thread 32: dK, thread 64: dQ, thread 96: S, thread 160: dP.  Every one
  // of them arrives on the batch's barrier exactly once: a commit after its instructions, or a plain arrival when the
  // batch has none for it.
  const int issuer = tid == 0 ? 0 : tid == 32 ? 1 : tid == 64 ? 2 : tid == 96 ? 3 : tid == 160 ? 4 : -1;
  // S = Q K^T (issuer 3) and dP = dO V^T (issuer 4) of the query tile in stage `stg`; `on` = the batch has these products
  auto issue_mma1 = [&](bool on, int stg, bool second = false) {
    if (issuer != 3 && issuer != 4) return;
    if (!on) { mbar_arrive(bar); return; }
    const uint32_t sQ = s_base + Cfg::OFF_Q + stg * Cfg::Q_BYTES, sDO = s_base + Cfg::OFF_DO + stg * Cfg::DO_BYTES;
    const uint32_t sK = s_base + (second ? Cfg::OFF_K2 : Cfg::OFF_K), sV = s_base + (second ? Cfg::OFF_V2 : Cfg::OFF_V);
    if (issuer == 3) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tS, smem_desc(sQ + off, 16, 1024), smem_desc(sK + off, 16, 1024), id_s, kk > 0);
      }
    } else {
#pragma unroll
      for (int kk = 0; kk < DV / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(tDP, smem_desc(sDO + off, 16, 1024), smem_desc(sV + off, 16, 1024), id_s, kk > 0);
      }
    }
    mma_commit(bar);
  };
  // dV += P^T dO (issuer 0), dK += dS^T Q (issuer 1), dQ = dS K (issuer 2) for the query tile in stage `stg`
  // acc0: dV / dK accumulate onto what TMEM holds; dq_acc: so does dQ (paired block item, second key tile)
  auto issue_mma2 = [&](bool on, int stg, uint32_t acc0, uint32_t t_dq, bool second = false, uint32_t dq_acc = 0) {
    if (issuer < 0 || issuer > 2) return;
    if (!on) { mbar_arrive(bar); return; }
    const uint32_t sQ = s_base + Cfg::OFF_Q + stg * Cfg::Q_BYTES, sDO = s_base + Cfg::OFF_DO + stg * Cfg::DO_BYTES;
    const uint32_t sK = s_base + (second ? Cfg::OFF_K2 : Cfg::OFF_K);
    if (issuer == 0) {
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk)
        mma_ss(tDV, smem_desc(s_base + Cfg::OFF_P + kk * 2048, TILE * 128, 1024), smem_desc(sDO + kk * 2048, TILE * 128, 1024), id_dv,
               acc0 | (kk > 0));
    } else if (issuer == 1) {
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk)
        mma_ss(tDK, smem_desc(s_base + Cfg::OFF_DS + kk * 2048, TILE * 128, 1024), smem_desc(sQ + kk * 2048, TILE * 128, 1024), id_dk,
               acc0 | (kk > 0));
    } else {
#pragma unroll
      for (int kk = 0; kk < TILE / 16; ++kk) {
        const uint32_t off = (kk >> 2) * (TILE * 128) + (kk & 3) * 32;
        mma_ss(t_dq, smem_desc(s_base + Cfg::OFF_DS + off, 16, 1024), smem_desc(sK + kk * 2048, TILE * 128, 1024), id_dq,
               dq_acc | (kk > 0));
      }
    }
    mma_commit(bar);
  };
  // P and dS of this thread's query row, its group's 64 key columns -> shared memory
  // weighted sampling (sampled items only): pair jj meets sorted query tile qt_first + jj; its log weight is added to
  // the scores and the dropped slots among this group's 64 key columns give p = 0
  const bool weighted = WT && hyper && (item >= items_blk || fused);
  auto elementwise = [&](float lse2, float dlt, bool diag, int jj) {
    const int limit = diag ? row + 1 : TILE;
    uint32_t wm[2] = {0u, 0u};
    float bias2 = 0.f;
    if (WT && weighted && (!fused || jj >= 4)) {
      // sorted query tile and sampled tile of this pair (fused item: query tiles 2b, 2b+1 alternate; pairs 4,5 meet
      // sampled tile 0, pairs 6,7 sampled tile 1)
      const long long qtile = (long long)seg * (p.m_q / TILE) + (fused ? k_tile + (jj & 1) : qt_first + jj);
      const int stile = fused ? (jj >> 1) - 2 : k_tile;
      const uint32_t* mw = p.sample_mask + qtile * (p.sample_size / 32) + stile * 4 + wg * 2;
      wm[0] = mw[0];
      wm[1] = mw[1];
      bias2 = p.sample_logw[qtile] * LOG2E;
    }
    const bool masked = diag || (WT && (wm[0] | wm[1]) != 0u);
    const uint64_t sc2 = pack_f2(scale2, scale2), nlse = WT ? pack_f2(bias2 - lse2, bias2 - lse2) : pack_f2(-lse2, -lse2);
    const uint64_t scl = pack_f2(p.scale, p.scale), ndel = pack_f2(-dlt * p.scale, -dlt * p.scale);
    const int col0 = wg * 64;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t rs[32], rp[32];
      tmem_ld32(tS + lane_sel + col0 + c * 32, rs);
      tmem_ld32(tDP + lane_sel + col0 + c * 32, rp);
      tmem_ld_fence(rs);
      tmem_ld_fence(rp);
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint32_t pw[4], dw[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          float p0, p1, d0, d1;
          unpack_f2(ffma2(pack_u2(rs[i + e], rs[i + e + 1]), sc2, nlse), p0, p1);
          p0 = fast_exp2(p0);
          p1 = fast_exp2(p1);
          if (masked) {
            if (col0 + c * 32 + i + e >= limit || (WT && ((wm[c] >> (i + e)) & 1u))) p0 = 0.f;
            if (col0 + c * 32 + i + e + 1 >= limit || (WT && ((wm[c] >> (i + e + 1)) & 1u))) p1 = 0.f;
          }
          // ds = p * (dp - delta) * scale
          unpack_f2(fmul2(pack_f2(p0, p1), ffma2(pack_u2(rp[i + e], rp[i + e + 1]), scl, ndel)), d0, d1);
          pw[e >> 1] = pack2<T>(p0, p1);
          dw[e >> 1] = pack2<T>(d0, d1);
        }
        const uint32_t off = swz_off(TILE, row, col0 + c * 32 + i);
        *reinterpret_cast<uint4*>(sP + off) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        *reinterpret_cast<uint4*>(sDS + off) = make_uint4(dw[0], dw[1], dw[2], dw[3]);
      }
    }
  };
  const bool diag_possible = !hyper && causal;
  // dK / dV rows of a key tile (lanes = keys), one column half per thread group: fp32 reductions into the accumulators
  // (staging rows are private per warp), or -- direct mode -- stored once in the tensors' dtype (block items, which hold
  // the complete block part of their rows) / reduced into the slot-indexed fp32 buffers (sampled items)
  auto drain_kv = [&](int kr, int tile, bool sampled_tile) {
    uint8_t* stg = smem + Cfg::OFF_STG + wg * Cfg::STG_HALF;
    if (p.dk_out == nullptr) {
      float* dk_base = p.dk_acc + (si.khead0 + si.k_row0) * D;
      float* dv_base = p.dv_acc + (si.khead0 + si.k_row0) * DV;
      if (p.flags & HA_FLAG_BWD_KV_INIT) {   // (exact attention only) this item is the only writer of its key rows: store, nothing to add to
        reduce_rows<DV / 2, 1>(stg, tDV + lane_sel + wg * (DV / 2), dv_base + wg * (DV / 2), DV, kr, row);
        reduce_rows<D / 2, 1>(stg, tDK + lane_sel + wg * (D / 2), dk_base + wg * (D / 2), D, kr, row);
      } else {
        reduce_rows<DV / 2>(stg, tDV + lane_sel + wg * (DV / 2), dv_base + wg * (DV / 2), DV, kr, row);
        reduce_rows<D / 2>(stg, tDK + lane_sel + wg * (D / 2), dk_base + wg * (D / 2), D, kr, row);
      }
    } else if (!sampled_tile) {
      T* dk_base = (T*)p.dk_out + (head0 + si.k_row0) * D;
      T* dv_base = (T*)p.dv_out + (head0 + si.k_row0) * DV;
      store_rows<T, DV / 2>(tDV + lane_sel + wg * (DV / 2), dv_base + wg * (DV / 2), DV, kr);
      store_rows<T, D / 2>(tDK + lane_sel + wg * (D / 2), dk_base + wg * (D / 2), D, kr);
    } else {
      const int slot = tile * TILE + row;
      float* dk_base = p.dk_sacc + kseg_of(p, seg) * p.sample_size * D;
      float* dv_base = p.dv_sacc + kseg_of(p, seg) * p.sample_size * DV;
      reduce_rows<DV / 2>(stg, tDV + lane_sel + wg * (DV / 2), dv_base + wg * (DV / 2), DV, slot, row);
      reduce_rows<D / 2>(stg, tDK + lane_sel + wg * (D / 2), dk_base + wg * (D / 2), D, slot, row);
    }
  };

  if constexpr (Cfg::PIPE) {
    // ------------------------------------------------------------------------------------------------------------
    // Pipelined schedule.  batch(j) = { dV, dK, dQ of pair j ; S, dP of pair j+1 } is one commit.  While it runs, the
    // threads reduce dQ of pair j-1 (its own TMEM buffer, its own staging tile); the next pair's elementwise phase
    // starts as soon as the batch has landed.
    // ------------------------------------------------------------------------------------------------------------
    uint8_t* sSTG = smem + Cfg::OFF_STG;
    // dQ rows of pair jp (TMEM buffer jp & 1) -> global: fp32 reduction into dq_acc, or -- a paired item whose TMEM
    // buffer holds the query tile's complete sum (final_dq) -- the final rows of dq_out
    // under_batch: the drain runs while the batch issued just before executes.  A thread that issued eight of its
    // instructions is held by the tensor pipe for about a thousand cycles, so the share of the drain of warp 0 (the dV
    // issuer's) would come after everybody else's and delay the next pair: the warp of the other group that sits on the
    // same 32 TMEM lanes takes both column halves of those rows instead.
    auto drain_dq = [&](int jp, int qrow_of_pair, bool under_batch) {
      if (final_dq && paired) {
        reduce_rows<D / 2, 2, T>(sSTG + wg * Cfg::STG_HALF, tDQ + (jp & 1) * D + lane_sel + wg * (D / 2), dq_base + wg * (D / 2), D,
                                 qrow_of_pair, row, (T*)p.dq_out + (head0 + si.q_row0) * D + wg * (D / 2));
        return;
      }
      const int warp_id = tid >> 5;
      if (under_batch && warp_id == 0) return;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (half != wg && !(under_batch && warp_id == 4)) continue;
        reduce_rows<D / 2>(sSTG + half * Cfg::STG_HALF, tDQ + (jp & 1) * D + lane_sel + half * (D / 2), dq_base + half * (D / 2), D,
                           qrow_of_pair, row);
      }
    };
    float lse_next = INFINITY, delta_next = 0.f;
    if (qt_count > 1 && qrow_next >= 0) { lse_next = lse_base[qrow_next] * LOG2E; delta_next = delta_base[qrow_next]; }
    cp_async_wait<1>();                       // K, V, query tile 0
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    issue_mma2(false, 0, 0, tDQ);             // (first batch: S and dP of pair 0 only)
    issue_mma1(true, 0);
    draw_next();                              // read after the pair loop's barriers, below
    int qrow_prev = -1;
    for (int jj = 0; jj < qt_count; ++jj) {
      HA_T_MARK(0)
      const int st = jj & 1;
      if (!mbar_wait(bar, phase)) failed = true;     // batch(jj-1): S, dP of this pair are in TMEM
      phase ^= 1;
      tc_fence_after();
      if (__syncthreads_or(failed)) { failed = true; break; }
      HA_T_MARK(1)
      // stage st^1 is free now (its last reader was batch(jj-1)): fetch query tile jj+1 (tile 1 is already there)
      int qrow_after = -1;
      float lse_after = INFINITY, delta_after = 0.f;
      if (!paired && jj >= 1 && jj + 1 < qt_count) fetch_q(st ^ 1, qrow_next);   // (a paired item keeps both tiles)
      if (fused && (jj == 2 || jj == 4)) {
        // the key buffer whose tile is through (A at pair 2, B at pair 4) takes a sampled tile, needed two pairs later
        const int sr = jj == 2 ? me.srow0 : me.srow1;
        const uint16_t* kb = (const uint16_t*)p.k + si.b * p.k_sb + si.hk * p.k_sh + si.k_row0 * p.k_sn;
        const uint16_t* vb = (const uint16_t*)p.v + si.b * p.v_sb + si.hk * p.v_sh + si.k_row0 * p.v_sn;
        if (wg == 0) bwd_gather_tile<D>(s_base + (jj == 2 ? Cfg::OFF_K : Cfg::OFF_K2), kb, p.k_sn, sr, qwarp, lane);
        else bwd_gather_tile<DV>(s_base + (jj == 2 ? Cfg::OFF_V : Cfg::OFF_V2), vb, p.v_sn, sr, qwarp, lane);
      }
      cp_async_commit();
      if (jj + 2 < qt_count) {
        qrow_after = q_row(jj + 2);
      }
      HA_T_MARK(2)
      // paired block item: the first key tile's dV / dK are final once pair 1 is through; pair 2 starts them afresh
      if (paired && jj == 2) drain_kv(krow, k_tile, false);
      if (fused && jj == 4) drain_kv(me.krow2, k_tile + 1, false);
      if (fused && jj == 6) drain_kv(me.srow0, 0, true);
      elementwise(lse_cur, delta_cur, diag_possible && qt_first + jj == k_tile, jj);
      HA_T_MARK(3)
      cp_async_wait<0>();                     // query tile jj+1 has landed
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      tc_fence_after();
      if (paired) {
        // dV / dK restart with each key tile; dQ of a query tile sums over both key tiles in its own TMEM buffer
        // (key buffers alternate with the key tile jj / 2: A, B, and -- fused -- S0, S1)
        issue_mma2(true, st, jj & 1, tDQ + (jj & 1) * D, (jj >> 1) & 1, jj >= 2 ? 1u : 0u);
        issue_mma1(jj + 1 < qt_count, st ^ 1, ((jj + 1) >> 1) & 1);
      } else {
        issue_mma2(true, st, jj > 0, tDQ + (jj & 1) * D);
        issue_mma1(jj + 1 < qt_count, st ^ 1);
      }
      HA_T_MARK(4)
      // underneath the batch: dQ of the previous pair (paired item: of query tile 0, complete after pair 2)
      if (jj >= 1 && (!paired || jj == qt_count - 1)) drain_dq(jj - 1, qrow_prev, true);
      HA_T_MARK(5)
      // rotate the per-tile registers; lse/delta of tile jj+2 are loaded here so that they arrive during the next pair
      qrow_prev = qrow_cur;
      qrow_cur = qrow_next;
      lse_cur = lse_next;
      delta_cur = delta_next;
      qrow_next = qrow_after;
      if (qrow_after >= 0) { lse_after = lse_base[qrow_after] * LOG2E; delta_after = delta_base[qrow_after]; }
      lse_next = lse_after;
      delta_next = delta_after;
    }
    cp_async_wait<0>();
    if (!failed) {
      nxt = next_work(s_next_w);                     // its index loads travel while the last batch runs
      if (!mbar_wait(bar, phase)) failed = true;     // last batch
      phase ^= 1;
      tc_fence_after();
      failed = __syncthreads_or(failed);
    }
    HA_T_MARK(6)
    if (!failed) {
      issue_loads(nxt);                              // every operand tile is free now
      drain_dq(qt_count - 1, qrow_prev, false);
    }
  } else {
    // ------------------------------------------------------------------------------------------------------------
    // Serial schedule (head dim 128: TMEM has no room for a separate dQ buffer, shared memory none for a second stage)
    // ------------------------------------------------------------------------------------------------------------
    for (int jj = 0; jj < qt_count; ++jj) {
      HA_T_MARK(0)
      cp_async_wait<0>();
      const int qrow_after = q_row(jj + 2);
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      tc_fence_after();
      HA_T_MARK(1)
      issue_mma2(false, 0, 0, tDQ);
      issue_mma1(true, 0);
      if (jj == 0) draw_next();               // read after this loop (every iteration has barriers)
      if (!mbar_wait(bar, phase)) failed = true;
      phase ^= 1;
      tc_fence_after();
      if (__syncthreads_or(failed)) { failed = true; break; }
      HA_T_MARK(2)
      elementwise(lse_cur, delta_cur, diag_possible && qt_first + jj == k_tile, jj);
      fence_async_smem();
      tc_fence_before();
      __syncthreads();
      tc_fence_after();
      HA_T_MARK(3)
      issue_mma2(true, 0, jj > 0, tDQ);
      issue_mma1(false, 0);
      if (!mbar_wait(bar, phase)) failed = true;
      phase ^= 1;
      tc_fence_after();
      if (__syncthreads_or(failed)) { failed = true; break; }
      HA_T_MARK(4)
      // dQ rows: TMEM -> staging (the P / dS tiles are idle now) -> fp32 reductions; each group one column half
      reduce_rows<D / 2>(smem + Cfg::OFF_STG + wg * Cfg::STG_HALF, tDQ + lane_sel + wg * (D / 2), dq_base + wg * (D / 2), D, qrow_cur, row);
      HA_T_MARK(5)
      float lse_next = INFINITY, delta_next = 0.f;
      if (jj + 1 < qt_count) {
        // fetch the next query tile now that every MMA reading this one has completed
        __syncthreads();
        fetch_q(0, qrow_next);
        cp_async_commit();
        if (qrow_next >= 0) { lse_next = lse_base[qrow_next] * LOG2E; delta_next = delta_base[qrow_next]; }
      }
      qrow_cur = qrow_next;
      qrow_next = qrow_after;
      lse_cur = lse_next;
      delta_cur = delta_next;
    }
    cp_async_wait<0>();
    HA_T_MARK(6)
    if (!failed) {
      nxt = next_work(s_next_w);
      issue_loads(nxt);                              // every MMA of this item has completed: the operand tiles are free
    }
  }

  if (failed) {
    if (tid == 0) report_timeout(p.status, p.status_host);
  } else {
    __syncthreads();
    drain_kv(fused ? me.srow1 : paired ? me.krow2 : krow, fused ? 1 : paired ? k_tile + 1 : k_tile, fused || (hyper && item >= items_blk));
  }
  HA_T_MARK(7)
  w = failed ? n_work : s_next_w;    // (the slot is rewritten only after the next item's first barrier)
  cur = nxt;
  }   // work items
  cp_async_wait<0>();
  HA_T_DUMP(8, (int)blockIdx.x, tid == 0)
  tc_fence_before();
  __syncthreads();
  if (tid < 32) tmem_dealloc(tmem, 512);
}

// Work counters of the persistent launches: 256 words in the library image per device; a launch takes the next one in
// rotation (so launches in flight on different streams do not share a word) and zeroes it on its stream first.
static __device__ unsigned int g_work_counters[256];
static unsigned int* next_work_counter() {
  static std::mutex mu;
  static unsigned int* base[64] = {nullptr};
  static unsigned int turn[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_work_counters) != cudaSuccess) return nullptr;
    base[dev] = (unsigned int*)ptr;
  }
  return base[dev] + (turn[dev]++ % 256u);
}

template <typename T, int D, int DV, bool WT>
static int launch_bwd(const ha_attn_params& p, cudaStream_t st) {
  using Cfg = BwdCfg<D, DV>;
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  if (segs == 0 || p.m_q == 0 || p.m_k == 0) return HA_OK;
  const int n_qt = (p.m_q + TILE - 1) / TILE, n_kt = (p.m_k + TILE - 1) / TILE;
  const int n_chunks = (n_qt + BWD_CHUNK - 1) / BWD_CHUNK;
  long long items;
  int items_blk = 0;
  // block size 256 with plain windows on whole blocks: one item per block (both key tiles, both query tiles)
  const int pair_blocks = Cfg::PIPE && p.mode == HA_MODE_HYPER && !(p.flags & HA_FLAG_SMOOTH) && (p.block_size + TILE - 1) / TILE == 2 &&
                          p.m_k % (2 * TILE) == 0;
  // final dQ rows (dq_out given; tc_bwd_direct_level says when): every query tile's sum must be complete in one item
  const bool final_dq = p.dq_out != nullptr;
  if (final_dq && !(pair_blocks && (p.sample_size == 0 || p.sample_size == 2 * TILE))) return HA_ERR_INVALID;
  // Only with direct outputs: a fused item drains the sampled tiles' dK/dV sums once per block (eight times as often as
  // a sampled item over 16 query tiles); into the small slot buffers that is affordable, into the fp32 accumulators of
  // the causal rectangles it costs more than the fusing saves (measured: 31.7 ms against 31.2 ms on the causal step).
  const int fuse_sampled = pair_blocks && p.sample_size == 2 * TILE && p.dk_out != nullptr;
  if (p.mode == HA_MODE_HYPER) {
    items_blk = pair_blocks ? n_kt / 2 : n_kt;
    items = (long long)items_blk + (fuse_sampled ? 0 : (long long)(p.sample_size / TILE) * n_chunks);
  } else {
    items = (long long)n_kt * n_chunks;
  }
  if (items > 0x7fffffffLL) return HA_ERR_INVALID;
  HA_SMEM_ATTR_ONCE((attn_tc_bwd_kernel<T, D, DV, WT>), Cfg::SMEM, "ha_attn_bwd smem attribute");
  const int sms = sm_count();
  // persistent CTAs, one per SM (512 TMEM columns, > 190 KB shared memory each): CTA c starts with work item c and
  // draws the following ones from a counter, which is one of a small rotating set of device words zeroed in stream
  // order before the launch
  auto launch = [&](long long items_per_seg, int mode_bits, int item_base) -> int {
    const long long n_work = items_per_seg * segs;
    const unsigned grid = (unsigned)(n_work < sms ? n_work : sms);
    unsigned int* ctr = next_work_counter();
    if (!ctr) return HA_ERR_CUDA;
    HA_CUDA_OK(cudaMemsetAsync(ctr, 0, sizeof(unsigned int), st), "ha_attn_bwd work counter");
    attn_tc_bwd_kernel<T, D, DV, WT><<<grid, 256, Cfg::SMEM, st>>>(p, items_blk, n_chunks, (int)items_per_seg, n_work, mode_bits, item_base, ctr);
    return HA_OK;
  };
  int lrc;
  if (fuse_sampled) {
    if ((lrc = launch(items_blk, 1 | 4 | (final_dq ? 2 : 0), 0)) != HA_OK) return lrc;
  } else {
    if ((lrc = launch(items, (pair_blocks ? 1 : 0) | (final_dq ? 2 : 0), 0)) != HA_OK) return lrc;
  }
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
  if (p.d == DD && p.dv == DDV) return p.sample_logw ? launch_bwd<TT, DD, DDV, true>(p, st) : launch_bwd<TT, DD, DDV, false>(p, st);
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

HA_T_SETTER(ha_debug_set_timing_buffer_bwd)
