// Persistent, warp-specialised backward of the block-diagonal + sampled pattern (tcgen05 + TMEM), head dims 64,
// block size 129..256 on plain windows, bf16 / fp16.  Replaces _bwd_permuted_block_diagonal_kernel and
// _bwd_sampled_col_kernel (src/hyper_attn_triton.py:399-506, :517-665) for that case in one launch.
//
// One CTA per SM walks work items; an item is one 256-row block of one segment: its two window key tiles and the
// sampled key tiles (nX key tiles in all) against its two query tiles -- 2 nX (key tile, query tile) pairs.  Every
// gradient row of the item is complete inside it: dQ of a query tile is summed over all its key tiles in TMEM, dK / dV
// of a window key tile over both query tiles; only the sampled rows collect terms from every block of the segment.
//
// Scores are computed TRANSPOSED, lanes = keys:  S^T = K Q^T,  dP^T = V dO^T.  Then P^T and dS^T, rounded to the input
// dtype, are written back to TMEM in place and feed  dV += P^T dO  and  dK += dS^T Q  as TMEM A operands; only dS also
// goes to shared memory ([key][query] rows, an MN-major A operand) for  dQ += dS K.  A pair is processed as two halves
// of 64 query columns, so that two TMEM stages of (S^T, dP^T) fit beside the accumulators and the elementwise phase of
// one half runs underneath the tensor work of the other.
//
// Roles (512 threads):
//   * elementwise group g (g = 0, 1; 128 threads, thread = key row = TMEM lane): the halves with query columns
//     [64 g, 64 g + 64) of every pair, on TMEM stage g.
//   * drain group (128 threads, thread = TMEM lane): dK / dV rows of a finished key tile, dQ rows of a finished query
//     tile -> global memory (typed rows, or fp32 reductions into accumulators / slot buffers).
//   * loader warp: gathers rows by index with cp.async into two K/V stages and two (Q, dO, lse, delta) stages; the
//     copies signal the "full" barriers themselves, the warp only waits for free buffers and runs ahead.
//   * three MMA-issuing threads (one per warp): S^T / dP^T of every half; dV / dK of every half as soon as its P^T / dS^T
//     are written; dQ of every pair.  Every completion is a tcgen05.commit onto an mbarrier.
// TMEM columns: stage g at 128 g (S^T 64 columns, dP^T 64 columns; P^T / dS^T in place over the first 32 of each),
// dV 256, dK 320, dQ of query tile 0 / 1 at 384 / 448.
// Hand-offs are mbarriers with bounded waits; a wait that gives up raises the CTA's abort flag and the status words,
// and every role leaves its loop at its next wait.
#include "attn_index.cuh"

#include <mutex>
#include <type_traits>

namespace ha {

namespace bws {
constexpr int D = 64, DV = 64;
constexpr int TILE_B = TILE * 64 * 2;                          // one 128 x 64 tile of 2-byte elements
constexpr int OFF_KV = 0;                                      // stage s: K at s * 2 TILE_B, V after it
constexpr int OFF_QD = OFF_KV + 2 * 2 * TILE_B;                // stage y (query tile y of the item): Q, then dO
constexpr int OFF_DS = OFF_QD + 2 * 2 * TILE_B;                // two buffers (pairs alternate) of two slabs (column halves)
constexpr int OFF_LD = OFF_DS + 2 * 2 * TILE_B;                // per query-tile stage: lse[128], delta[128] (fp32)
constexpr int SMEM = OFF_LD + 2 * 1024 + 1024;                 // + alignment slack
constexpr int THREADS = 512;
constexpr int COL_DV = 256, COL_DK = 320, COL_DQ = 384;
// barrier slots
constexpr int B_KV_FULL = 0, B_KV_EMPTY = 2, B_QD_FULL = 4, B_QD_EMPTY = 6, B_S_READY = 8, B_P_READY = 10, B_ST_FREE = 12,
              B_DS_FREE = 14, B_DQ_FULL = 16, B_DQ_FREE = 18, B_ACC_FULL = 20, B_ACC_FREE = 21, N_BARS = 22;
}  // namespace bws

// 128 rows x 64 elements gathered by ONE warp: rows[q] = source row of tile row 32 q + lane (-1: zero fill)
__device__ __forceinline__ void bws_gather_tile(uint32_t smem_base, const uint16_t* __restrict__ base, int64_t row_stride, const int (&rows)[4],
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
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bws_red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(bws::THREADS, 1) attn_tc_bwd_ws_kernel(const ha_attn_params p, const int n_items, const int blocks_per_seg) {
  using namespace bws;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t s_base = smem_u32(smem);
  __shared__ uint64_t bars[N_BARS];
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;
  __shared__ int s_bail;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_samp = p.sample_size / TILE;
  const int nX = 2 + n_samp;                             // key tiles per item: two window tiles, then the sampled tiles
  const bool dq_direct = p.dq_out != nullptr, kv_direct = p.dk_out != nullptr;

  if (cta_sees_failure(p.status, &s_bail)) return;   // an earlier CTA gave up: drain quickly (uniform over the CTA)
  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };
  if (tid == 0) {
    // arrivals per phase: 32 (every loader lane, through its copies) on the "full" barriers of the operand stages, 128 (a
    // thread group) on P-ready / dQ-free / accumulator-free, 1 or 2 (tcgen05.commit) elsewhere
    for (int i = 0; i < N_BARS; ++i) {
      const bool by_loader = (i >= B_KV_FULL && i < B_KV_FULL + 2) || (i >= B_QD_FULL && i < B_QD_FULL + 2);
      const bool by_group = (i >= B_P_READY && i < B_P_READY + 2) || (i >= B_DQ_FREE && i < B_DQ_FREE + 2) || i == B_ACC_FREE;
      // the "empty" barriers of the operand stages: one commit from each of the two MMA-issuing threads that read the stage
      const bool by_two = (i >= B_KV_EMPTY && i < B_KV_EMPTY + 2) || (i >= B_QD_EMPTY && i < B_QD_EMPTY + 2);
      mbar_init(bar(i), by_loader ? 32 : by_group ? 128 : by_two ? 2 : 1);
    }
    s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 12) tmem_alloc(smem_u32(&tmem_slot), 512);
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
  constexpr float LOG2E = 1.4426950408889634f;

  if (warp < 8) {
    // =====================================================================================================
    // elementwise groups: P^T = exp2(S^T scale log2e - lse log2e), dS^T = P^T (dP^T - delta) scale
    // =====================================================================================================
    // Register budget: 512 threads x 128 at launch = the whole register file.  The drain group goes down to 96 and the
    // loader / MMA warpgroup to 72, the two elementwise groups take 168: 2 x 128 x 168 + 128 x 96 + 128 x 72 = 64512 of
    // 65536, i.e. with slack -- a request that the pool cannot satisfy would wait forever.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
    const int g = warp >> 2, gw = warp & 3, row = tid & 127;
    const uint32_t lane_sel = (uint32_t)(gw * 32) << 16;
    const uint32_t tST = tmem + 128 * g + lane_sel, tDPT = tST + 64;
    const uint64_t sc2 = pack_f2(p.scale * LOG2E, p.scale * LOG2E), nl2e = pack_f2(-LOG2E, -LOG2E);
    const uint64_t scl = pack_f2(p.scale, p.scale), nscl = pack_f2(-p.scale, -p.scale);
    uint32_t pairs = 0;      // pairs this group has processed (stage g is used once per pair)
    bool ok = true;
    int it = 0;
    HA_T_DECL(8)
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      for (int x = 0; x < nX && ok; ++x) {
        for (int y = 0; y < 2 && ok; ++y, ++pairs) {
          HA_T_MARK(4)
          if (!(ok = wait(B_S_READY + g, pairs & 1))) break;
          HA_T_MARK(0)
          if (x == 0 && !(ok = wait(B_QD_FULL + y, it & 1))) break;                    // lse / delta of the tile have landed
          HA_T_MARK(1)
          if (pairs >= 2 && !(ok = wait(B_DS_FREE + (pairs & 1), ((pairs >> 1) - 1) & 1))) break;   // dQ of pair - 2 has read the buffer
          HA_T_MARK(2)
          tc_fence_after();
          const float* ld = reinterpret_cast<const float*>(smem + OFF_LD + y * 1024) + 64 * g;
          uint8_t* ds_row = smem + OFF_DS + (pairs & 1) * 2 * TILE_B + g * TILE_B + row * 128;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t rs[32], rp[32];
            tmem_ld32(tST + c * 32, rs);
            tmem_ld32(tDPT + c * 32, rp);
            tmem_ld_fence(rs);
            tmem_ld_fence(rp);
            uint32_t pk[16], dk[16];
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              // four query columns: their lse and delta (the same for every thread: broadcast reads)
              const ulonglong2 L = *reinterpret_cast<const ulonglong2*>(ld + c * 32 + i);
              const ulonglong2 Dl = *reinterpret_cast<const ulonglong2*>(ld + 128 + c * 32 + i);
              float p0, p1, p2, p3, d0, d1, d2, d3;
              unpack_f2(ffma2(pack_u2(rs[i], rs[i + 1]), sc2, fmul2(L.x, nl2e)), p0, p1);
              unpack_f2(ffma2(pack_u2(rs[i + 2], rs[i + 3]), sc2, fmul2(L.y, nl2e)), p2, p3);
              p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
              // ds = p * (dp - delta) * scale
              unpack_f2(fmul2(pack_f2(p0, p1), ffma2(pack_u2(rp[i], rp[i + 1]), scl, fmul2(Dl.x, nscl))), d0, d1);
              unpack_f2(fmul2(pack_f2(p2, p3), ffma2(pack_u2(rp[i + 2], rp[i + 3]), scl, fmul2(Dl.y, nscl))), d2, d3);
              pk[i >> 1] = pack2<T>(p0, p1);
              pk[(i >> 1) + 1] = pack2<T>(p2, p3);
              dk[i >> 1] = pack2<T>(d0, d1);
              dk[(i >> 1) + 1] = pack2<T>(d2, d3);
            }
            // P^T / dS^T chunk c overwrite columns [16 c, 16 c + 16) of S^T / dP^T: part of chunk 0, which is in registers
            tmem_st16(tST + c * 16, pk);
            tmem_st16(tDPT + c * 16, dk);
            // dS^T rows to shared memory: this key row, query columns 64 g + 32 c + [0, 32) = 16-byte chunks 4 c .. 4 c + 3
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(ds_row + ((((c * 4 + j) ^ row) & 7) << 4)) = make_uint4(dk[4 * j], dk[4 * j + 1], dk[4 * j + 2], dk[4 * j + 3]);
          }
          HA_T_MARK(3)
          tmem_st_wait();
          fence_async_smem();       // the dS rows are read by the tensor core (async proxy)
          tc_fence_before();
          mbar_arrive(bar(B_P_READY + g));
        }
      }
    }
    HA_T_DUMP(8, (int)blockIdx.x * 4 + g, row == 0)
  } else if (warp < 12) {
    // =====================================================================================================
    // drain group: finished accumulators -> global memory
    // =====================================================================================================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    const int gw = warp & 3, row = tid & 127;
    const uint32_t lane_sel = (uint32_t)(gw * 32) << 16;
    bool ok = true;
    int it = 0;
    uint32_t xg = 0;         // key tiles drained so far
    HA_T_DECL(8)
    // 32 fp32 columns of this lane -> 32 typed elements at dst (64 contiguous bytes), or fp32 reductions at acc
    auto out_chunk = [&](uint32_t taddr, T* dst, float* acc, bool typed, bool valid, bool last, int free_bar) {
      uint32_t r[32];
      tmem_ld32(taddr, r);
      tmem_ld_fence(r);
      if (last) {            // everything this thread reads from the accumulator is in registers: hand it back
        tc_fence_before();
        mbar_arrive(bar(free_bar));
      }
      if (!valid) return;
      if (typed) {
        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          d4[i >> 3] = make_uint4(pack2<T>(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), pack2<T>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                                  pack2<T>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])), pack2<T>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
      } else {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          bws_red_add_v4(acc + i, __uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
      }
    };
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
      const SegInfo si = seg_info(p, seg);
      const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;
      // this lane's rows: query rows of both tiles, key row of the first key tile (loaded ahead of the waits)
      const int qrow0 = p.q_idx[(long long)seg * p.m_q + (2 * blk) * TILE + row];
      const int qrow1 = p.q_idx[(long long)seg * p.m_q + (2 * blk + 1) * TILE + row];
      auto key_row = [&](int x) -> int {
        if (x < 2) return p.k_idx[(long long)seg * p.m_k + (2 * blk + x) * TILE + row];
        const int s = (x - 2) * TILE + row;
        return p.sample_idx ? p.sample_idx[(long long)seg * p.sample_size + s] : s;
      };
      auto drain_dq = [&](int y) -> bool {
        HA_T_MARK(1)
        if (!wait(B_DQ_FULL + y, it & 1)) return false;
        HA_T_MARK(2)
        tc_fence_after();
        const long long r = head0 + si.q_row0 + (y ? qrow1 : qrow0);
        const uint32_t t = tmem + COL_DQ + y * D + lane_sel;
        out_chunk(t, (T*)p.dq_out + r * D, p.dq_acc + r * D, dq_direct, true, false, 0);
        out_chunk(t + 32, (T*)p.dq_out + r * D + 32, p.dq_acc + r * D + 32, dq_direct, true, true, B_DQ_FREE + y);
        HA_T_MARK(3)
        return true;
      };
      int krow = key_row(0);
      for (int x = 0; x < nX && ok; ++x, ++xg) {
        const int krow_next = x + 1 < nX ? key_row(x + 1) : 0;
        if (x == nX - 1 && !(ok = drain_dq(0))) break;     // complete one pair before the last key tile is
        HA_T_MARK(1)
        if (!(ok = wait(B_ACC_FULL, xg & 1))) break;
        HA_T_MARK(0)
        tc_fence_after();
        const bool sampled = x >= 2;
        // window tiles: the row's complete block part, stored once (typed) / added (accumulators); sampled tiles: this
        // block's share of the row's sum, reduced into the slot buffers (typed outputs) / the accumulators
        const bool typed = kv_direct && !sampled;
        const long long r = head0 + si.k_row0 + krow;
        float* acc_k = nullptr;
        float* acc_v = nullptr;
        if (kv_direct && sampled) {
          const long long slot = (long long)seg * p.sample_size + (x - 2) * TILE + row;
          acc_k = p.dk_sacc + slot * D;
          acc_v = p.dv_sacc + slot * DV;
        } else if (!kv_direct) {
          acc_k = p.dk_acc + r * D;
          acc_v = p.dv_acc + r * DV;
        }
        const uint32_t tv = tmem + COL_DV + lane_sel, tk = tmem + COL_DK + lane_sel;
        out_chunk(tv, (T*)p.dv_out + r * DV, acc_v, typed, true, false, 0);
        out_chunk(tv + 32, (T*)p.dv_out + r * DV + 32, acc_v + 32, typed, true, false, 0);
        out_chunk(tk, (T*)p.dk_out + r * D, acc_k, typed, true, false, 0);
        out_chunk(tk + 32, (T*)p.dk_out + r * D + 32, acc_k + 32, typed, true, true, B_ACC_FREE);
        krow = krow_next;
      }
      if (ok) ok = drain_dq(1);
    }
    HA_T_DUMP(8, (int)blockIdx.x * 4 + 2, row == 0)
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    if (warp == 12) {
      // ===================================================================================================
      // loader: per item K/V of the first key tile, (Q, dO, lse, delta) of both query tiles, then the other key tiles
      // ===================================================================================================
      // The copies of a tile signal its barrier themselves when they land (every lane arrives once, through the copy
      // engine), so this warp never waits for its own copies: only for free buffers.
      auto push = [&](int b) {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(b)) : "memory");
      };
      uint32_t xg = 0;        // key tiles fetched so far (stage = xg & 1)
      bool ok = true;
      int it = 0;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
        const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
        const SegInfo si = seg_info(p, seg);
        const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;
        const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
        const uint16_t* gbase = (const uint16_t*)p.d_o + si.b * p.do_sb + si.h * p.do_sh + si.q_row0 * p.do_sn;
        const uint16_t* kbase = (const uint16_t*)p.k + si.b * p.k_sb + si.h * p.k_sh + si.k_row0 * p.k_sn;
        const uint16_t* vbase = (const uint16_t*)p.v + si.b * p.v_sb + si.h * p.v_sh + si.k_row0 * p.v_sn;
        const float* lse_base = p.lse + head0 + si.q_row0;
        const float* delta_base = p.delta + head0 + si.q_row0;
        auto load_krows = [&](int x, int (&dst)[4]) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int rr = q * 32 + lane;
            if (x < 2) dst[q] = p.k_idx[(long long)seg * p.m_k + (2 * blk + x) * TILE + rr];
            else {
              const int s = (x - 2) * TILE + rr;
              dst[q] = p.sample_idx ? p.sample_idx[(long long)seg * p.sample_size + s] : s;
            }
          }
        };
        int krows[4];
        load_krows(0, krows);
        for (int x = 0; x < nX && ok; ++x, ++xg) {
          const int stage = xg & 1;
          int knext[4] = {-1, -1, -1, -1};
          if (x + 1 < nX) load_krows(x + 1, knext);
          int qrows[2][4];
          if (x == 0) {
#pragma unroll
            for (int y = 0; y < 2; ++y)
#pragma unroll
              for (int q = 0; q < 4; ++q) qrows[y][q] = p.q_idx[(long long)seg * p.m_q + (2 * blk + y) * TILE + q * 32 + lane];
          }
          if (xg >= 2 && !(ok = wait(B_KV_EMPTY + stage, ((xg >> 1) - 1) & 1))) break;
          bws_gather_tile(s_base + OFF_KV + stage * 2 * TILE_B, kbase, p.k_sn, krows, lane);
          bws_gather_tile(s_base + OFF_KV + stage * 2 * TILE_B + TILE_B, vbase, p.v_sn, krows, lane);
          push(B_KV_FULL + stage);
          if (x == 0) {
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              if (it >= 1 && !(ok = wait(B_QD_EMPTY + y, (it - 1) & 1))) break;
              bws_gather_tile(s_base + OFF_QD + y * 2 * TILE_B, qbase, p.q_sn, qrows[y], lane);
              bws_gather_tile(s_base + OFF_QD + y * 2 * TILE_B + TILE_B, gbase, p.do_sn, qrows[y], lane);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint32_t dst = s_base + OFF_LD + y * 1024 + (q * 32 + lane) * 4;
                cp_async4(dst, lse_base + qrows[y][q]);
                cp_async4(dst + 512, delta_base + qrows[y][q]);
              }
              push(B_QD_FULL + y);
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) krows[q] = knext[q];
        }
      }
      cp_async_commit();
      cp_async_wait<0>();      // nothing of this warp is in flight when the CTA retires
    } else if (lane == 0) {
      // ===================================================================================================
      // MMA issue, three threads.  A single thread gets one tcgen05.mma accepted about every 100 cycles whatever its
      // shape (measured: 107 cycles per instruction for N <= 128, issue time = completion time), while the tensor pipe
      // itself finishes an M 128 x N 64 x K 16 step in under 60: so the 40 instructions of a pair are issued from three
      // threads, each with a product of its own (no accumulator is shared between them):
      //   warp 13: S^T, dP^T of every half        -> S-ready;   frees (with the others) the K/V and Q/dO stages
      //   warp 14: dV, dK of every half           -> stage-free, accumulators-full
      //   warp 15: dQ of every pair               -> dS-buffer-free, dQ-full
      // Every thread walks the halves / pairs in order and blocks (bounded) on what its next instruction needs.
      // ===================================================================================================
      constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const int my_items = n_items > (int)blockIdx.x ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      const uint32_t NH = 4u * (uint32_t)nX;                 // halves per item
      const uint32_t total = (uint32_t)my_items * NH;
      // Half hh (a count over this CTA's items): item hh / NH, key tile x = (hh % NH) / 4, query tile y = bit 1, column half
      // g = bit 0.  Pair = hh / 2, key tile count = hh / 4.
      bool ok = true;
      HA_T_DECL(8)
      if (warp == 13) {
        const uint32_t id_st = mma_idesc(TILE, 64, AB, 0, 0);      // M = 128 keys, N = 64 queries, both operands K-major
        for (uint32_t hh = 0; hh < total && ok; ++hh) {
          const uint32_t r = hh % NH, itc = hh / NH, x = r >> 2, y = (r >> 1) & 1, g = r & 1;
          const uint32_t pair = hh >> 1, xg = hh >> 2;
          HA_T_MARK(0)
          if (pair >= 1 && !(ok = wait(B_ST_FREE + g, (pair - 1) & 1))) break;        // dV / dK of the stage's previous half completed
          HA_T_MARK(1)
          if ((r & 3) == 0 && !(ok = wait(B_KV_FULL + (xg & 1), (xg >> 1) & 1))) break;
          if (x == 0 && g == 0 && !(ok = wait(B_QD_FULL + y, itc & 1))) break;
          HA_T_MARK(2)
          fence_async_smem();          // the copies that filled the operand tiles are ordered before the operand reads
          tc_fence_after();
          const uint32_t sQ = s_base + OFF_QD + y * 2 * TILE_B + g * (TILE_B / 2), sDO = sQ + TILE_B;
          const uint32_t sK = s_base + OFF_KV + (xg & 1) * 2 * TILE_B, sV = sK + TILE_B;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ss(tmem + 128 * g, smem_desc(sK + kk * 32, 16, 1024), smem_desc(sQ + kk * 32, 16, 1024), id_st, kk > 0);
#pragma unroll
          for (int kk = 0; kk < DV / 16; ++kk)
            mma_ss(tmem + 128 * g + 64, smem_desc(sV + kk * 32, 16, 1024), smem_desc(sDO + kk * 32, 16, 1024), id_st, kk > 0);
          mma_commit(bar(B_S_READY + g));
          if ((r & 3) == 3) mma_commit(bar(B_KV_EMPTY + (xg & 1)));               // this thread's last read of the K/V stage
          if (x == (uint32_t)nX - 1 && g == 1) mma_commit(bar(B_QD_EMPTY + y));      // ... and of the Q / dO stage
          HA_T_MARK(3)
        }
        HA_T_DUMP(8, (int)blockIdx.x * 4 + 3, true)
      } else if (warp == 14) {
        const uint32_t id_kv = mma_idesc(TILE, 64, AB, 0, 1);      // A = P^T / dS^T in TMEM, B = dO / Q rows as MN-major
        for (uint32_t hh = 0; hh < total && ok; ++hh) {
          const uint32_t r = hh % NH, x = r >> 2, y = (r >> 1) & 1, g = r & 1;
          const uint32_t pair = hh >> 1, xg = hh >> 2;
          if (!(ok = wait(B_P_READY + g, pair & 1))) break;
          if ((r & 3) == 0 && xg >= 1 && !(ok = wait(B_ACC_FREE, (xg - 1) & 1))) break;    // dV / dK restart with the key tile
          fence_async_smem();
          tc_fence_after();
          const uint32_t sQ = s_base + OFF_QD + y * 2 * TILE_B + g * (TILE_B / 2), sDO = sQ + TILE_B;
          const uint32_t tP = tmem + 128 * g, tDS = tP + 64;
          const uint32_t acc0 = (r & 3) != 0;
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // dV += P^T dO over this half's 64 query rows
            mma_ts(tmem + COL_DV, tP + kk * 8, smem_desc(sDO + kk * 2048, TILE * 128, 1024), id_kv, acc0 | (kk > 0));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)     // dK += dS^T Q
            mma_ts(tmem + COL_DK, tDS + kk * 8, smem_desc(sQ + kk * 2048, TILE * 128, 1024), id_kv, acc0 | (kk > 0));
          mma_commit(bar(B_ST_FREE + g));
          if ((r & 3) == 3) mma_commit(bar(B_ACC_FULL));                            // dV / dK of the key tile are complete
          if (x == (uint32_t)nX - 1 && g == 1) mma_commit(bar(B_QD_EMPTY + y));
        }
      } else if (warp == 15) {
        const uint32_t id_dq = mma_idesc(TILE, 64, AB, 1, 1);      // A = dS ([key][query] rows: MN-major), B = K rows as MN-major
        const uint32_t total_pairs = total >> 1;
        for (uint32_t pair = 0; pair < total_pairs && ok; ++pair) {
          const uint32_t r = (2 * pair) % NH, itc = (2 * pair) / NH, x = r >> 2, y = (r >> 1) & 1, xg = pair >> 1;
          // both halves of the pair have written their dS slabs
          if (!(ok = wait(B_P_READY + 0, pair & 1))) break;
          if (!(ok = wait(B_P_READY + 1, pair & 1))) break;
          if (x == 0 && itc >= 1 && !(ok = wait(B_DQ_FREE + y, (itc - 1) & 1))) break;      // dQ restarts with the item
          fence_async_smem();
          tc_fence_after();
          const uint32_t sK = s_base + OFF_KV + (xg & 1) * 2 * TILE_B;
          const uint32_t sDS = s_base + OFF_DS + (pair & 1) * 2 * TILE_B;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)     // dQ_y += dS K over the 128 keys
            mma_ss(tmem + COL_DQ + y * D, smem_desc(sDS + kk * 2048, TILE_B, 1024), smem_desc(sK + kk * 2048, TILE_B, 1024), id_dq,
                   (x > 0) | (kk > 0));
          mma_commit(bar(B_DS_FREE + (pair & 1)));
          if (x == (uint32_t)nX - 1) mma_commit(bar(B_DQ_FULL + y));                  // the query tile's dQ is complete
          if (y == 1) mma_commit(bar(B_KV_EMPTY + (xg & 1)));                         // this thread's last read of the K tile
        }
      }
    }
  }
  // every role is done (or has given up); TMEM goes back
  tc_fence_before();
  __syncthreads();
  if (warp == 12) tmem_dealloc(tmem, 512);
}

bool tc_bwd_supported(const ha_attn_params& p);

// Conditions of the warp-specialised backward on top of those of the tensor-core backward: the shape ...
bool ws_bwd_shape_ok(const ha_attn_params& p) {
  if (!tc_bwd_supported(p)) return false;
  if (p.mode != HA_MODE_HYPER || p.d != 64 || p.dv != 64) return false;
  if (p.flags & (HA_FLAG_SMOOTH | HA_FLAG_NO_WS)) return false;
  if (p.sample_logw) return false;                                   // weighted sampling stays on the other kernel
  if ((p.block_size + TILE - 1) / TILE != 2 || p.m_q % (2 * TILE) != 0 || p.m_q != p.m_k) return false;
  return true;
}
// ... and the outputs
bool ws_bwd_supported(const ha_attn_params& p) {
  if (!ws_bwd_shape_ok(p)) return false;
  // outputs: typed rows or fp32 accumulators, for dQ and for dK / dV independently
  if (!p.dq_out && !p.dq_acc) return false;
  if (p.dk_out) {
    if (!p.dv_out || (p.sample_size > 0 && (!p.dk_sacc || !p.dv_sacc))) return false;
  } else if (!p.dk_acc || !p.dv_acc) {
    return false;
  }
  return true;
}

int ws_attn_bwd(const ha_attn_params& p, cudaStream_t st) {
  const long long segs = (long long)p.B * p.H * p.segs_per_head;
  const int blocks_per_seg = p.m_q / (2 * TILE);
  const long long items = segs * blocks_per_seg;
  if (items == 0) return HA_OK;
  if (items * 4 * (2 + p.sample_size / TILE) > 0x7fffffffLL) return HA_ERR_TOO_LARGE;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)(items < sms ? items : sms);
#define HA_BWS_LAUNCH(TT)                                                                                                        \
  do {                                                                                                                           \
    HA_CUDA_OK(cudaFuncSetAttribute(attn_tc_bwd_ws_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, bws::SMEM),           \
               "ha_attn_bwd smem attribute");                                                                                    \
    attn_tc_bwd_ws_kernel<TT><<<grid, bws::THREADS, bws::SMEM, st>>>(p, (int)items, blocks_per_seg);                             \
  } while (0)
  if (p.dtype == HA_BF16) HA_BWS_LAUNCH(__nv_bfloat16);
  else HA_BWS_LAUNCH(__half);
#undef HA_BWS_LAUNCH
  HA_LAUNCHED("ha_attn_bwd (tcgen05, warp-specialised)");
  return HA_OK;
}

}  // namespace ha

HA_T_SETTER(ha_debug_set_timing_buffer_bwd_ws)
