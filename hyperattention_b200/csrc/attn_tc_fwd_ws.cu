// Persistent, warp-specialised forward of the block-diagonal + sampled pattern (tcgen05 + TMEM), head dims 64,
// block size 129..256 on plain windows, bf16 / fp16.
//
// One CTA per SM walks work items; an item is one 256-row block of one segment: query tiles 2b and 2b+1, which pair
// with the same key tiles (the block's two window tiles, then the sampled tiles).  Roles (384 threads):
//   * group 0 / group 1 (128 threads each): softmax and output of query tile 2b / 2b+1; thread i owns query row i =
//     TMEM lane i, as in the one-tile kernel (attn_tc_fwd.cu), whose arithmetic this file repeats step for step.
//   * three loader warps (K tiles, V tiles, query side): gather rows by index with 16-byte cp.async into a ring of four
//     K/V stages (each key tile is fetched once for both query tiles), the two Q tiles (double buffered over the items)
//     and, for a merging call, the rows already stored for the two query tiles; they run ahead of the compute across
//     items, so index -> row latency and the next item's prologue are off the critical path.
//   * MMA warp (one thread): issues S = Q K^T for both groups one key tile ahead of their softmax, and P V as soon as
//     a group has written P; every completion is a tcgen05.commit onto an mbarrier.
// TMEM: group g, region r (key tiles alternate): columns 256 g + 128 r; S in 128 fp32 columns, P in place over the
// first 64, the P V product in the upper 64 once S is consumed.
// Hand-offs are mbarriers with bounded waits; a wait that gives up raises the CTA's abort flag and the status word, and
// every role leaves its loop at its next wait.
#include "attn_index.cuh"

#include <type_traits>

namespace ha {

namespace ws {
constexpr int D = 64, DV = 64;
constexpr int KV_STAGES = 4;
constexpr int TILE_B = TILE * 64 * 2;                          // one 128 x 64 tile of 2-byte elements
constexpr int OFF_KV = 0;                                      // stage s: K at s * 2 TILE_B, V after it
constexpr int OFF_Q = OFF_KV + KV_STAGES * 2 * TILE_B;         // two buffers (items alternate) of two Q tiles
constexpr int OFF_OLD = OFF_Q + 4 * TILE_B;                    // per group: the previously stored o rows of its tile (merge)
constexpr int SMEM = OFF_OLD + 2 * TILE_B + 1024;
constexpr int THREADS = 384;
// barrier slots
constexpr int B_KV_FULL = 0, B_KV_EMPTY = 4, B_Q_FULL = 8, B_Q_EMPTY = 10, B_S_READY = 12, B_P_READY = 16, B_PV_READY = 20,
              B_S_FREE = 24, B_OLD_FULL = 28, B_OLD_EMPTY = 30, N_BARS = 32;
}  // namespace ws

// 128 rows x 64 elements gathered by ONE warp: rows[q] = source row of tile row 32 q + lane (-1: zero fill)
__device__ __forceinline__ void ws_gather_tile(uint32_t smem_base, const uint16_t* __restrict__ base, int64_t row_stride, const int (&rows)[4],
                                               int lane) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int rl = 4 * i + (lane >> 3);
      const int src_row = __shfl_sync(0xffffffffu, rows[q], rl);
      const int row = q * 32 + rl;
      const int chunk = lane & 7;
      const uint32_t dst = smem_base + row * 128 + ((chunk ^ (row & 7)) << 4);
      const uint16_t* src = base + (int64_t)(src_row < 0 ? 0 : src_row) * row_stride + chunk * 8;
      cp_async16(dst, src, src_row >= 0 ? 16u : 0u);
    }
  }
}

// MG: merging call (HA_FLAG_MERGE; may also write the un-merged rows); a template flag so that the plain instantiation
// carries none of it
template <typename T, bool MG>
__global__ void __launch_bounds__(ws::THREADS, 1) attn_tc_fwd_ws_kernel(const ha_attn_params p, const int n_items, const int blocks_per_seg) {
  using namespace ws;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t bars[N_BARS];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ int s_bail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr bool merge = MG;
  const int n_blk = 2;                                   // window tiles of a block (block size rounded up to 256)
  const int n_tiles = n_blk + p.sample_size / TILE;      // key tiles per item

  if (cta_sees_failure(p.status, &s_bail)) return;   // an earlier CTA gave up: drain quickly (uniform over the CTA)
  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };
  if (tid == 0) {
    // arrivals per phase: 32 or 64 (every lane of the loaders of that buffer, when its copies have landed) on the "full"
    // barriers, 128 (a softmax group) on P-ready / S-free, 1 (a tcgen05.commit or one elected thread) elsewhere
    for (int i = 0; i < N_BARS; ++i) {
      const bool by_kv_loaders = i >= B_KV_FULL && i < B_KV_FULL + KV_STAGES;    // the K loader's and the V loader's lanes
      const bool by_loader = (i >= B_Q_FULL && i < B_Q_FULL + 2) || (i >= B_OLD_FULL && i < B_OLD_FULL + 2);
      const bool by_group = (i >= B_P_READY && i < B_PV_READY) || (i >= B_S_FREE && i < B_S_FREE + 4) || i >= B_OLD_EMPTY;
      mbar_init(bar(i), by_kv_loaders ? 64 : by_loader ? 32 : by_group ? 128 : 1);
    }
    s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 8) tmem_alloc(smem_u32(&tmem_slot), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  // a wait that fails (or finds the abort flag up) ends the role's loop
  auto wait = [&](int b, uint32_t parity) -> bool {
    if (*reinterpret_cast<volatile int*>(&s_abort)) return false;
    if (mbar_wait(bar(b), parity)) return true;
    *reinterpret_cast<volatile int*>(&s_abort) = 1;
    report_timeout(p.status, p.status_host);
    return false;
  };

  if (warp < 8) {
    // =====================================================================================================
    // softmax groups
    // =====================================================================================================
    // Register budget: 384 threads x 168 at launch.  The loader / MMA warpgroup gives registers back (56 each), the two
    // softmax groups take 224 each: 2 x 128 x 224 + 128 x 56 = 64512 of the SM's 65536, i.e. with slack -- a request that
    // the pool cannot satisfy would wait forever.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int g = warp >> 2, gw = warp & 3, row = tid & 127;
    const uint32_t lane_sel = (uint32_t)(gw * 32) << 16;
    const uint32_t t_group = tmem + g * 256;
    const float scale2 = p.scale * 1.4426950408889634f;
    uint32_t c = 0;          // key tiles this group has processed (region = c & 1, use count = c >> 1)
    bool ok = true;
    int it = 0;
    HA_T_DECL(8)
    auto item_qrow = [&](int item) -> int {
      if (item >= n_items) return 0;
      const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
      return p.q_idx[(long long)seg * p.m_q + (2 * blk + g) * TILE + row];
    };
    int qrow_next = item_qrow(blockIdx.x);
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      const int seg = item / blocks_per_seg;
      const SegInfo si = seg_info(p, seg);
      const int qrow = qrow_next;
      qrow_next = item_qrow(item + gridDim.x);     // the next item's row index arrives while this item computes
      const long long lse_at = ((long long)(si.b * p.H + si.h)) * p.n + si.q_row0 + qrow;
      const float lse_old = merge ? p.lse[lse_at] : 0.f;       // (merge) needed in the epilogue: requested now
      __align__(8) float o_acc[DV];
#pragma unroll
      for (int i = 0; i < DV; ++i) o_acc[i] = 0.f;
      float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
      auto fold_pv = [&](uint32_t t_pv, float alpha) {
        const uint64_t al2 = pack_f2(alpha, alpha);
        uint64_t* o2 = reinterpret_cast<uint64_t*>(o_acc);
#pragma unroll
        for (int cc = 0; cc < DV / 32; ++cc) {
          uint32_t r[32];
          tmem_ld32(t_pv + lane_sel + cc * 32, r);
          tmem_ld_fence(r);
#pragma unroll
          for (int i = 0; i < 32; i += 2) o2[(cc * 32 + i) >> 1] = ffma2(o2[(cc * 32 + i) >> 1], al2, pack_u2(r[i], r[i + 1]));
        }
      };
      for (int j = 0; j < n_tiles && ok; ++j, ++c) {
        const int r = c & 1;
        const uint32_t tS = t_group + r * 128, tP = tS;
        HA_T_MARK(0)
        if (!(ok = wait(B_S_READY + g * 2 + r, (c >> 1) & 1))) break;
        tc_fence_after();
        HA_T_MARK(1)
        HA_T_MARK(2)
        // ---- softmax over this tile's 128 columns (every column is visible in this pattern) ----
        float mx;
        {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
          uint32_t ra[32], rb[32];
          tmem_ld32(tS + lane_sel, ra);
          tmem_ld_fence(ra);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t(&cur)[32] = (cc & 1) ? rb : ra;
            uint32_t(&nxt)[32] = (cc & 1) ? ra : rb;
            if (cc + 1 < 4) tmem_ld32(tS + lane_sel + (cc + 1) * 32, nxt);
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              m0 = fmax3(m0, __uint_as_float(cur[i]), __uint_as_float(cur[i + 1]));
              m1 = fmax3(m1, __uint_as_float(cur[i + 2]), __uint_as_float(cur[i + 3]));
              m2 = fmax3(m2, __uint_as_float(cur[i + 4]), __uint_as_float(cur[i + 5]));
              m3 = fmax3(m3, __uint_as_float(cur[i + 6]), __uint_as_float(cur[i + 7]));
            }
            if (cc + 1 < 4) tmem_ld_fence(nxt);
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
        if (j >= 1) {
          // The product of the previous tile (other region), folded here rather than before the max pass: its MMAs were
          // issued when this group finished that tile's P and have had the max pass to complete.  Then the region goes
          // back for S of tile j+1.
          if (!(ok = wait(B_PV_READY + g * 2 + (r ^ 1), ((c - 1) >> 1) & 1))) break;
          tc_fence_after();
          fold_pv(t_group + (r ^ 1) * 128 + 64, alpha_prev);
          tc_fence_before();
          mbar_arrive(bar(B_S_FREE + g * 2 + (r ^ 1)));
        }
        const float m_new = fmaxf(m_run, mx * scale2);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = fast_exp2(m_run - m_use);   // m_run = -inf -> 0
        float psum;
        {
          const uint64_t sc2 = pack_f2(scale2, scale2), negm = pack_f2(-m_use, -m_use);
          uint64_t ps_a = pack_f2(0.f, 0.f), ps_b = ps_a;
          uint32_t ra[32], rb[32];
          tmem_ld32(tS + lane_sel, ra);
          tmem_ld_fence(ra);
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t(&cur)[32] = (cc & 1) ? rb : ra;
            uint32_t(&nxt)[32] = (cc & 1) ? ra : rb;
            // P chunk cc below overwrites columns [16cc, 16cc+16), part of S chunk cc/2, which is already in registers;
            // the chunk being loaded (cc+1) lies in columns >= 32(cc+1), disjoint from them
            if (cc + 1 < 4) tmem_ld32(tS + lane_sel + (cc + 1) * 32, nxt);
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float p0, p1, p2, p3;
              unpack_f2(ffma2(pack_u2(cur[i], cur[i + 1]), sc2, negm), p0, p1);
              unpack_f2(ffma2(pack_u2(cur[i + 2], cur[i + 3]), sc2, negm), p2, p3);
              p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
              ps_a = fadd2(ps_a, pack_f2(p0, p1));
              ps_b = fadd2(ps_b, pack_f2(p2, p3));
              pk[i >> 1] = pack2<T>(p0, p1);
              pk[(i >> 1) + 1] = pack2<T>(p2, p3);
            }
            tmem_st16(tP + lane_sel + cc * 16, pk);
            if (cc + 1 < 4) tmem_ld_fence(nxt);
          }
          float s0, s1;
          unpack_f2(fadd2(ps_a, ps_b), s0, s1);
          psum = s0 + s1;
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar(B_P_READY + g * 2 + r));       // P of this tile is in TMEM: its product may be issued
        l_run = l_run * alpha + psum;
        m_run = m_new;
        alpha_prev = alpha;
        HA_T_MARK(3)
      }
      if (!ok) break;
      {
        // the last product of the item
        const int r = (c - 1) & 1;
        if (!(ok = wait(B_PV_READY + g * 2 + r, ((c - 1) >> 1) & 1))) break;
        tc_fence_after();
        fold_pv(t_group + r * 128 + 64, alpha_prev);
        tc_fence_before();
        mbar_arrive(bar(B_S_FREE + g * 2 + r));
      }
      HA_T_MARK(4)
      // ---- epilogue: normalise, optionally merge with the stored (o, lse), store ----
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const float lse_own = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
      float lse = lse_own;
      uint16_t* obase = (uint16_t*)p.o + si.b * p.o_sb + si.h * p.o_sh + si.q_row0 * p.o_sn;
      float w1 = 0.f, w2 = 1.f;
      if (merge) {
        const float l1 = lse_old, l2 = lse_own;
        if (p.flags & HA_FLAG_MERGE_EXACT) {
          const float m2 = fmaxf(l1, l2);
          const float e1 = __expf(l1 - m2), e2 = __expf(l2 - m2);
          w1 = e1 / (e1 + e2);
          w2 = e2 / (e1 + e2);
          lse = m2 + __logf(e1 + e2);
        } else {
          const float cf = round_to<T>(1.f / (1.f + __expf(l2 - l1)));
          w1 = cf;
          w2 = round_to<T>(1.f - cf);
          lse = l1 - __logf(cf + 1.1920929e-07f);
        }
      }
      // Each thread stores its own row: 128 contiguous bytes in eight 16-byte pieces (whole 32-byte sectors pair up in
      // L2); far less code than staging the tile and storing it row-coalesced, and this code runs once per item.
      if (MG && p.part_o) {      // the un-merged result of this call
        uint4* prow = reinterpret_cast<uint4*>((uint16_t*)p.part_o + si.b * p.o_sb + si.h * p.o_sh + (si.q_row0 + qrow) * p.o_sn);
#pragma unroll
        for (int e = 0; e < DV; e += 8)
          prow[e >> 3] = make_uint4(pack2<T>(o_acc[e] * inv, o_acc[e + 1] * inv), pack2<T>(o_acc[e + 2] * inv, o_acc[e + 3] * inv),
                                    pack2<T>(o_acc[e + 4] * inv, o_acc[e + 5] * inv), pack2<T>(o_acc[e + 6] * inv, o_acc[e + 7] * inv));
        if (p.part_lse) p.part_lse[lse_at] = lse_own;
      }
      {
        uint4* orow = reinterpret_cast<uint4*>(obase + (int64_t)qrow * p.o_sn);
        if (merge) {
          // the rows stored before this call were fetched by the loader; chunk c of row r sits at chunk c ^ (r & 7)
          if (!(ok = wait(B_OLD_FULL + g, it & 1))) break;
          const uint8_t* old_row = smem + OFF_OLD + g * TILE_B + row * 128;
#pragma unroll
          for (int e = 0; e < DV; e += 8) {
            const uint4 ov = *reinterpret_cast<const uint4*>(old_row + ((((e >> 3) ^ (row & 7))) << 4));
            const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
            uint32_t w[4];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const float2 old = unpack2<T>(ow[h]);
              w[h] = pack2<T>(w1 * old.x + w2 * round_to<T>(o_acc[e + 2 * h] * inv), w1 * old.y + w2 * round_to<T>(o_acc[e + 2 * h + 1] * inv));
            }
            orow[e >> 3] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          mbar_arrive(bar(B_OLD_EMPTY + g));       // this thread has read its row: the loader may refill the tile
        } else {
#pragma unroll
          for (int e = 0; e < DV; e += 8)
            orow[e >> 3] = make_uint4(pack2<T>(o_acc[e] * inv, o_acc[e + 1] * inv), pack2<T>(o_acc[e + 2] * inv, o_acc[e + 3] * inv),
                                      pack2<T>(o_acc[e + 4] * inv, o_acc[e + 5] * inv), pack2<T>(o_acc[e + 6] * inv, o_acc[e + 7] * inv));
        }
      }
      HA_T_MARK(6)
      p.lse[lse_at] = lse;
      HA_T_MARK(5)
    }
    HA_T_DUMP(8, (int)blockIdx.x, tid == 0)
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 8 || warp == 10) {
      // ===================================================================================================
      // loaders of the key side: K tiles (warp 8) and V tiles (warp 10) of every key tile into the ring.  One warp issuing
      // every gather of the CTA was its bottleneck (the number of copies a warp has in flight is limited), so the three
      // operand streams have a warp each.  A stage is full when both warps' copies have landed (64 arrivals).
      // ===================================================================================================
      // The copies of a tile signal its barrier themselves when they land (every lane arrives once, through the copy
      // engine), so a loader never waits for its own copies: only for free buffers.
      auto push = [&](int b) {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(b)) : "memory");
      };
      const bool is_v = warp == 10;
      uint32_t kv_t = 0;      // key tiles fetched so far (ring stage = kv_t % KV_STAGES)
      bool ok = true;
      auto load_krows = [&](int seg, int blk, int j, int (&dst)[4]) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int rr = q * 32 + lane;
          if (j < n_blk) dst[q] = p.k_idx[kseg_of(p, seg) * p.m_k + (2 * blk + j) * TILE + rr];
          else {
            const int s = (j - n_blk) * TILE + rr;
            dst[q] = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + s] : s;
          }
        }
      };
      int krows[4] = {-1, -1, -1, -1};
      if ((int)blockIdx.x < n_items) load_krows(blockIdx.x / blocks_per_seg, blockIdx.x % blocks_per_seg, 0, krows);
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
        const SegInfo si = seg_info(p, seg);
        const uint16_t* base = is_v ? (const uint16_t*)p.v + si.b * p.v_sb + si.hk * p.v_sh + si.k_row0 * p.v_sn
                                    : (const uint16_t*)p.k + si.b * p.k_sb + si.hk * p.k_sh + si.k_row0 * p.k_sn;
        const int64_t sn = is_v ? p.v_sn : p.k_sn;
        for (int j = 0; j < n_tiles && ok; ++j, ++kv_t) {
          const int stage = kv_t % KV_STAGES;
          // the next tile's row indices (the next item's first tile after this item's last) travel during the wait
          int knext[4] = {-1, -1, -1, -1};
          if (j + 1 < n_tiles) load_krows(seg, blk, j + 1, knext);
          else if (item + (int)gridDim.x < n_items) load_krows((item + gridDim.x) / blocks_per_seg, (item + gridDim.x) % blocks_per_seg, 0, knext);
          if (kv_t >= KV_STAGES && !(ok = wait(B_KV_EMPTY + stage, ((kv_t / KV_STAGES) - 1) & 1))) break;
          ws_gather_tile(s_base + OFF_KV + stage * 2 * TILE_B + (is_v ? TILE_B : 0), base, sn, krows, lane);
          push(B_KV_FULL + stage);
#pragma unroll
          for (int q = 0; q < 4; ++q) krows[q] = knext[q];
        }
      }
      cp_async_commit();
      cp_async_wait<0>();      // nothing of this warp is in flight when the CTA retires
    } else if (warp == 11) {
      // ===================================================================================================
      // loader of the query side: per item the two Q tiles and, for a merging call, the rows already stored for them
      // ===================================================================================================
      auto push = [&](int b) {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(b)) : "memory");
      };
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
        const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
        const SegInfo si = seg_info(p, seg);
        const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
        int qrows[2][4];
#pragma unroll
        for (int x = 0; x < 2; ++x)
#pragma unroll
          for (int q = 0; q < 4; ++q) qrows[x][q] = p.q_idx[(long long)seg * p.m_q + (2 * blk + x) * TILE + q * 32 + lane];
        const int qb = it & 1;                                                // Q buffer of this item
        if (it >= 2 && !(ok = wait(B_Q_EMPTY + qb, ((it >> 1) - 1) & 1))) break;   // its previous user's S MMAs are through
        ws_gather_tile(s_base + OFF_Q + qb * 2 * TILE_B, qbase, p.q_sn, qrows[0], lane);
        ws_gather_tile(s_base + OFF_Q + qb * 2 * TILE_B + TILE_B, qbase, p.q_sn, qrows[1], lane);
        push(B_Q_FULL + qb);
        // (merge) the rows stored before this call, needed in the item's epilogue only
        if (merge) {
          const uint16_t* obase = (const uint16_t*)p.o + si.b * p.o_sb + si.h * p.o_sh + si.q_row0 * p.o_sn;
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            if (it > 0 && !(ok = wait(B_OLD_EMPTY + x, (it - 1) & 1))) break;
            ws_gather_tile(s_base + OFF_OLD + x * TILE_B, obase, p.o_sn, qrows[x], lane);
            push(B_OLD_FULL + x);
          }
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
    } else if (warp == 9 && lane == 0) {
      // ===================================================================================================
      // MMA issue
      // ===================================================================================================
      constexpr int AB_FMT = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const uint32_t idesc_s = mma_idesc(TILE, TILE, AB_FMT, 0, 0);
      const uint32_t idesc_pv = mma_idesc(TILE, DV, AB_FMT, 0, 1);
      auto issue_pv = [&](int stage, uint32_t t_p, uint32_t t_pv) {
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk) {
          const uint32_t b_addr = s_base + OFF_KV + stage * 2 * TILE_B + TILE_B + kk * 2048;
          mma_ts(t_pv, t_p + kk * 8, smem_desc(b_addr, TILE * 128, 1024), idesc_pv, kk > 0);
        }
      };
      // Both groups advance independently.  Per group: cs = key tiles whose S has been issued, cp = whose P V has been
      // issued (global counts over the items: region = count & 1, K/V stage = count % KV_STAGES).  S may run one tile
      // ahead of P V.  The thread polls the barriers of whatever either group could do next and issues what is ready, so
      // a group that is late never holds up the other.
      auto ready = [&](int b, uint32_t parity) -> bool {
        uint32_t okk;
        asm volatile("{\n .reg .pred pp;\n mbarrier.test_wait.parity.shared::cta.b64 pp, [%1], %2;\n selp.u32 %0, 1, 0, pp;\n}\n"
                     : "=r"(okk) : "r"(bar(b)), "r"(parity) : "memory");
        return okk != 0;
      };
      const int my_items = n_items > (int)blockIdx.x ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      const uint32_t total = (uint32_t)my_items * (uint32_t)n_tiles;
      uint32_t cs[2] = {0, 0}, cp[2] = {0, 0};
      uint32_t kv_released = 0;      // key tiles whose stage has been handed back (both products issued)
      long long idle = 0;
      const long long idle_limit = (long long)SPIN_LIMIT * 16;
      bool ok = true;
      while (ok && (cp[0] < total || cp[1] < total)) {
        bool progressed = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          // ---- S of tile cs[g]: needs the item's Q, the tile's K/V stage, a free region ----
          if (cs[g] < total && cs[g] <= cp[g] + 1) {
            const uint32_t cc = cs[g];
            const int it = cc / n_tiles, j = cc - it * n_tiles, qb = it & 1;
            const int stage = cc % KV_STAGES, r = cc & 1;
            if ((j > 0 || ready(B_Q_FULL + qb, (it >> 1) & 1)) && ready(B_KV_FULL + stage, (cc / KV_STAGES) & 1) &&
                (cc < 2 || ready(B_S_FREE + g * 2 + r, ((cc >> 1) - 1) & 1))) {
              fence_async_smem();          // the copies that filled Q / K / V are ordered before the operand reads
              tc_fence_after();
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t a_addr = s_base + OFF_Q + qb * 2 * TILE_B + g * TILE_B + kk * 32;
                const uint32_t b_addr = s_base + OFF_KV + stage * 2 * TILE_B + kk * 32;
                mma_ss(tmem + g * 256 + r * 128, smem_desc(a_addr, 16, 1024), smem_desc(b_addr, 16, 1024), idesc_s, kk > 0);
              }
              mma_commit(bar(B_S_READY + g * 2 + r));
              ++cs[g];
              progressed = true;
              // the item's last S of both groups is issued: its Q buffer is free once they complete
              if (j == n_tiles - 1 && cs[g ^ 1] >= cc + 1) mma_commit(bar(B_Q_EMPTY + qb));
            }
          }
          // ---- P V of tile cp[g]: needs the group's P ----
          if (cp[g] < cs[g]) {
            const uint32_t cc = cp[g];
            const int stage = cc % KV_STAGES, r = cc & 1;
            if (ready(B_P_READY + g * 2 + r, (cc >> 1) & 1)) {
              fence_async_smem();
              tc_fence_after();
              const uint32_t tS = tmem + g * 256 + r * 128;
              issue_pv(stage, tS, tS + 64);
              mma_commit(bar(B_PV_READY + g * 2 + r));
              ++cp[g];
              progressed = true;
              // both products of a key tile issued: hand its stage back
              while (kv_released < cp[0] && kv_released < cp[1]) {
                mma_commit(bar(B_KV_EMPTY + kv_released % KV_STAGES));
                ++kv_released;
              }
            }
          }
        }
        if (progressed) idle = 0;
        else if (++idle > idle_limit || *reinterpret_cast<volatile int*>(&s_abort)) {
          *reinterpret_cast<volatile int*>(&s_abort) = 1;
          report_timeout(p.status, p.status_host);
          ok = false;
        }
      }
    }
  }
  // every role is done (or has given up); TMEM goes back
  tc_fence_before();
  __syncthreads();
  if (warp == 8) tmem_dealloc(tmem, 512);
}

bool tc_supported(const ha_attn_params& p);

// Conditions of the warp-specialised kernel on top of those of the one-tile kernel.
bool ws_fwd_supported(const ha_attn_params& p) {
  if (!tc_supported(p)) return false;
  if (p.mode != HA_MODE_HYPER || p.d != 64 || p.dv != 64) return false;
  if (p.flags & (HA_FLAG_SMOOTH | HA_FLAG_NO_WS)) return false;
  if (p.sample_logw) return false;                                   // weighted sampling stays on the one-tile kernel
  if (p.part_o && (!(p.flags & HA_FLAG_MERGE) || (uintptr_t)p.part_o % 16 != 0)) return false;
  if ((p.block_size + TILE - 1) / TILE != 2 || p.m_q % (2 * TILE) != 0 || p.m_q != p.m_k) return false;
  return true;
}

int ws_attn_fwd(const ha_attn_params& p, cudaStream_t st) {
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const int blocks_per_seg = p.m_q / (2 * TILE);
  const long long items = segs * blocks_per_seg;
  if (items == 0) return HA_OK;
  if (items > 0x7fffffffLL) return HA_ERR_TOO_LARGE;
  const int sms = sm_count();
  const int grid = (int)(items < sms ? items : sms);
  const bool mg = p.flags & HA_FLAG_MERGE;
#define HA_WS_LAUNCH(TT, MM)                                                                                                     \
  do {                                                                                                                           \
    HA_SMEM_ATTR_ONCE((attn_tc_fwd_ws_kernel<TT, MM>), ws::SMEM, "ha_attn_fwd smem attribute");                                  \
    attn_tc_fwd_ws_kernel<TT, MM><<<grid, ws::THREADS, ws::SMEM, st>>>(p, (int)items, blocks_per_seg);                           \
  } while (0)
  if (p.dtype == HA_BF16) {
    if (mg) HA_WS_LAUNCH(__nv_bfloat16, true);
    else HA_WS_LAUNCH(__nv_bfloat16, false);
  } else {
    if (mg) HA_WS_LAUNCH(__half, true);
    else HA_WS_LAUNCH(__half, false);
  }
#undef HA_WS_LAUNCH
  HA_LAUNCHED("ha_attn_fwd (tcgen05, warp-specialised)");
  return HA_OK;
}

}  // namespace ha

HA_T_SETTER(ha_debug_set_timing_buffer_fwd_ws)
