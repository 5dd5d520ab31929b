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
// Roles (640 threads):
//   * elementwise groups g = 0, 1 (128 threads each, thread = key row = TMEM lane): query columns [32 g, 32 g + 32) of
//     every half.  Both groups work on the same half, so a half's elementwise phase is short and the other TMEM stage
//     is in its tensor phases meanwhile.
//   * drain group (128 threads, thread = TMEM lane): dK / dV rows of a finished key tile, dQ rows of a finished query
//     tile -> global memory.  Rows are transposed through a staging tile and leave coalesced (typed rows, fp32
//     reductions into accumulators); the sampled rows' slot sums leave as whole-tile bulk additions of the copy engine.
//   * three loader warps, one per operand stream (K tiles: ring of two; V tiles: ring of two; (Q, dO, lse, delta): one
//     stage per query tile of the item): rows gathered by index with cp.async; the copies signal the "full" barriers
//     themselves, a loader only waits for free buffers and runs ahead.  The rows of the next tile are pulled into L2 first.
//   * five MMA-issuing threads (one per warp), one product each: S^T, dP^T, dV, dK of every half, dQ of every pair.
//     One thread gets a tcgen05.mma accepted only about every 100 cycles, whatever its shape, while the tensor pipe
//     finishes an M 128 x N 64 x K 16 step in under 60 (measured); five issuers keep the pipe fed and keep the 4-instruction
//     products on the stage's critical path short.  Every completion is a tcgen05.commit onto an mbarrier.
// TMEM columns: stage s at 128 s: S^T in [0, 64), dP^T in [64, 128); group g writes P^T / dS^T (16 packed columns) in place
// over the first half of the 32 columns it has read.  dV 256, dK 320, dQ of query tile 0 / 1 at 384 / 448.
// Hand-offs are mbarriers with bounded waits; a wait that gives up raises the CTA's abort flag and the status words,
// and every role leaves its loop at its next wait.
#include "attn_index.cuh"

#include <mutex>
#include <type_traits>

namespace ha {

namespace bws {
constexpr int D = 64;
constexpr int TILE_B = TILE * 64 * 2;                          // one 128 x 64 tile of 2-byte elements
constexpr int K_STAGES = 2, V_STAGES = 2;
constexpr int OFF_K = 0;                                       // K ring
constexpr int OFF_V = OFF_K + K_STAGES * TILE_B;               // V ring
constexpr int OFF_QD = OFF_V + V_STAGES * TILE_B;              // stage y (query tile y of the item): Q, then dO
constexpr int OFF_DS = OFF_QD + 2 * 2 * TILE_B;                // two buffers (pairs alternate) of two slabs (column halves)
constexpr int OFF_LD = OFF_DS + 2 * 2 * TILE_B;                // per query-tile stage: lse[128], delta[128] (fp32)
constexpr int OFF_ST = OFF_LD + 2 * 1024;                      // two staging tiles of the drain group: 128 rows x 128 bytes
constexpr int SMEM_USED = OFF_ST + 2 * TILE * 128;             // from the 1024-byte aligned base
constexpr int SMEM_LIMIT = 227 * 1024;                         // per CTA, static + dynamic
constexpr int THREADS = 640;
constexpr int COL_DV = 256, COL_DK = 320, COL_DQ = 384;
// barrier slots (index + stage / buffer / query tile) and their arrivals per phase
enum {
  B_K_FULL = 0,      // 3 x 32: every loader lane, through its copies
  B_K_EMPTY = 3,     // 3 x 2: the S^T and dQ issuers
  B_V_FULL = 6,      // 2 x 32
  B_V_EMPTY = 8,     // 2 x 1: the dP^T issuer
  B_QD_FULL = 10,    // 2 x 32
  B_QD_EMPTY = 12,   // 2 x 4: the S^T, dP^T, dV and dK issuers
  B_S_READY = 14,    // 2 x 2: S^T and dP^T of a half are in TMEM
  B_P_READY = 16,    // 2 x 256: both elementwise groups have written P^T / dS^T of the half
  B_SF_S = 18,       // 2 x 1: dV of the stage's half completed: its S^T columns may be overwritten
  B_SF_P = 20,       // 2 x 1: dK ...: its dP^T columns
  B_DS_FREE = 22,    // 2 x 1: dQ of the pair has read the dS buffer
  B_DQ_FULL = 24,    // 2 x 1: dQ of a query tile complete
  B_DQ_FREE = 26,    // 2 x 128: ... drained
  B_LDT = 28,        // (2 query tiles x 2 groups) x 128: an elementwise group has pre-scaled the lse / delta of its own columns
  B_DS_FULL = 32,    // 2 x 512: both halves' dS slabs of a pair are in the buffer (every elementwise thread, twice)
  B_ACC_FULL = 34,   // 2: dV and dK of a key tile complete
  B_ACC_FREE = 35,   // 128: ... drained
  B_ST_FULL = 36,    // 128: every drain thread has written its row of staging tile B (whole-tile additions)
  B_ST_FREE = 37,    // 1: the copy engine has read the tile
  N_BARS = 38
};
__device__ __forceinline__ int bar_count(int i) {
  if (i < B_K_EMPTY) return 32;
  if (i < B_V_FULL) return 2;
  if (i < B_V_EMPTY) return 32;
  if (i < B_QD_FULL) return 1;
  if (i < B_QD_EMPTY) return 32;
  if (i < B_S_READY) return 4;
  if (i < B_P_READY) return 2;
  if (i < B_SF_S) return 256;
  if (i < B_DQ_FREE) return 1;          // stage-free (S, P), dS-free, dQ-full
  if (i < B_DS_FULL) return 128;        // dQ-free, pre-scaled lse / delta
  if (i < B_ACC_FULL) return 512;
  if (i == B_ACC_FULL) return 2;
  return i >= B_ST_FREE ? 1 : 128;
}
}  // namespace bws

// Bulk fp32 addition shared -> global by the copy engine (a whole staging tile).
__device__ __forceinline__ void bws_bulk_add_f32(float* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bws_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// this thread's earlier bulk copies have read their source (the staging row may be rewritten) / have completed
__device__ __forceinline__ void bws_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bws_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

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
  {
    // The layout fills the CTA's shared memory to the last kilobyte; the launch sizes the dynamic window from the kernel's
    // static size.  Should the window nevertheless start somewhere else than assumed, do nothing rather than run over it.
    uint32_t dyn;
    asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
    if ((uint32_t)(smem - smem_raw) + (uint32_t)SMEM_USED > dyn) {      // uniform over the grid
      if (tid == 0) {
        if (p.status) atomicExch(p.status, HA_DEV_BAD_LAUNCH);
        if (p.status_host) {
          *reinterpret_cast<volatile int32_t*>(p.status_host) = HA_DEV_BAD_LAUNCH;
          __threadfence_system();
        }
      }
      return;
    }
  }
  auto bar = [&](int i) -> uint32_t { return smem_u32(&bars[i]); };
  if (tid == 0) {
    for (int i = 0; i < N_BARS; ++i) mbar_init(bar(i), bar_count(i));
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
    // Register budget.  What setmaxnreg redistributes is the CTA's own allocation at launch: 640 threads x 96 registers =
    // 61440 (not the SM's whole file); a request beyond it waits forever.  The two elementwise groups go up to 104, the
    // drain group to 144 (it holds two packed accumulator rows while it writes them out), the two warpgroups of the
    // loaders and the MMA issuers go down to 64: 2 x 128 x 104 + 128 x 144 + 2 x 128 x 64 = 61440.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int g = warp >> 2, gw = warp & 3, row = tid & 127;
    const uint32_t lane_sel = (uint32_t)(gw * 32) << 16;
    const uint64_t sc2 = pack_f2(p.scale * LOG2E, p.scale * LOG2E), scl = pack_f2(p.scale, p.scale);
    uint32_t hh = 0;         // halves processed (pair = hh / 2, TMEM stage = dS slab = hh & 1)
    bool ok = true;
    int it = 0;
    HA_T_DECL(8)
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
      for (int xy = 0; xy < 2 * nX && ok; ++xy) {
        const int x = xy >> 1, y = xy & 1;
        for (int s = 0; s < 2 && ok; ++s, ++hh) {
          const uint32_t pair = hh >> 1;
          HA_T_MARK(4)
          if (!(ok = wait(B_S_READY + s, pair & 1))) break;
          HA_T_MARK(0)
          float* ldt = reinterpret_cast<float*>(smem + OFF_LD + y * 1024);
          if (x == 0 && s == 0) {
            // lse / delta of the query tile have landed: scale them once for all of the item's pairs.  Each group scales
            // what it reads itself (its 32 columns of either half: 64 lse and 64 delta values, one per thread) and meets on
            // a barrier of its own, so that neither group waits for the other here.
            if (!(ok = wait(B_QD_FULL + y, it & 1))) break;
            const int j = row & 63;
            ldt[(row >> 6) * TILE + 64 * (j >> 5) + 32 * g + (j & 31)] *= row < 64 ? -LOG2E : -p.scale;
            mbar_arrive(bar(B_LDT + 2 * y + g));
            if (!(ok = wait(B_LDT + 2 * y + g, it & 1))) break;
          }
          HA_T_MARK(1)
          if (pair >= 2 && !(ok = wait(B_DS_FREE + (pair & 1), ((pair >> 1) - 1) & 1))) break;   // dQ of pair - 2 has read the buffer
          HA_T_MARK(2)
          tc_fence_after();
          // this thread: key row `row`, query columns 64 s + 32 g + [0, 32) of the pair
          const uint32_t tS = tmem + 128 * s + 32 * g + lane_sel, tDP = tS + 64;
          const float* ld = ldt + 64 * s + 32 * g;
          uint8_t* ds_row = smem + OFF_DS + (pair & 1) * 2 * TILE_B + s * TILE_B + row * 128;
          // 32 columns in two chunks of 16: few enough live registers that the compiler can keep several columns' chains
          // in flight (with 32 at a time the loop was bound by the latency of one chain after the other); the second
          // chunk's TMEM loads travel while the first is computed
          uint32_t rs[2][16], rp[2][16];
          tmem_ld16(tS, rs[0]);
          tmem_ld16(tDP, rp[0]);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tmem_ld_fence16(rs[c]);
            tmem_ld_fence16(rp[c]);
            if (c == 0) {
              tmem_ld16(tS + 16, rs[1]);
              tmem_ld16(tDP + 16, rp[1]);
            }
            uint32_t pk[8], dk[8];
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              // four query columns: their (scaled) lse and delta, the same for every thread: broadcast reads
              const ulonglong2 L = *reinterpret_cast<const ulonglong2*>(ld + c * 16 + i);
              const ulonglong2 Dl = *reinterpret_cast<const ulonglong2*>(ld + TILE + c * 16 + i);
              float p0, p1, p2, p3, d0, d1, d2, d3;
              unpack_f2(ffma2(pack_u2(rs[c][i], rs[c][i + 1]), sc2, L.x), p0, p1);
              unpack_f2(ffma2(pack_u2(rs[c][i + 2], rs[c][i + 3]), sc2, L.y), p2, p3);
              p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
              // ds = p * (dp - delta) * scale
              unpack_f2(fmul2(pack_f2(p0, p1), ffma2(pack_u2(rp[c][i], rp[c][i + 1]), scl, Dl.x)), d0, d1);
              unpack_f2(fmul2(pack_f2(p2, p3), ffma2(pack_u2(rp[c][i + 2], rp[c][i + 3]), scl, Dl.y)), d2, d3);
              pk[i >> 1] = pack2<T>(p0, p1);
              pk[(i >> 1) + 1] = pack2<T>(p2, p3);
              dk[i >> 1] = pack2<T>(d0, d1);
              dk[(i >> 1) + 1] = pack2<T>(d2, d3);
            }
            // P^T / dS^T of the chunk (8 packed columns) over columns this thread has already consumed
            tmem_st8(tS + c * 8, pk);
            tmem_st8(tDP + c * 8, dk);
            // dS^T row to shared memory: slab s, this key row, 16-byte chunks 4 g + 2 c, 4 g + 2 c + 1
#pragma unroll
            for (int j = 0; j < 2; ++j)
              *reinterpret_cast<uint4*>(ds_row + ((((g * 4 + c * 2 + j) ^ row) & 7) << 4)) = make_uint4(dk[4 * j], dk[4 * j + 1], dk[4 * j + 2], dk[4 * j + 3]);
          }
          HA_T_MARK(3)
          tmem_st_wait();
          fence_async_smem();       // the dS rows are read by the tensor core (async proxy)
          tc_fence_before();
          mbar_arrive(bar(B_P_READY + s));
          // The dQ issuer follows the dS buffers, not the TMEM stages: it may run up to two pairs behind this thread, and a
          // parity wait must never fall two phases behind its barrier; the buffer's own barrier cannot run ahead of it,
          // because the buffer is not rewritten before its dQ has completed.
          mbar_arrive(bar(B_DS_FULL + (pair & 1)));
        }
      }
    }
    HA_T_DUMP(8, (int)blockIdx.x * 8 + g, row == 0)
  } else if (warp < 12) {
    // =====================================================================================================
    // drain group: finished accumulators -> global memory
    // =====================================================================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 144;");
    const int gw = warp & 3, row = tid & 127;
    const uint32_t lane_sel = (uint32_t)(gw * 32) << 16;
    bool ok = true;
    int it = 0;
    uint32_t xg = 0;         // key tiles drained so far
    HA_T_DECL(8)
    // An accumulator is handed back as early as possible: its 64 fp32 columns of this lane are read and rounded to the
    // tensors' dtype in registers (32 packed words), the "free" barrier is signalled, and only then do the words go out --
    // as one typed row (128 contiguous bytes), or, unpacked again, as fp32 reductions.  (What is added into an fp32
    // accumulator or slot buffer is therefore rounded per work item, as the typed rows are.)
    // (both halves of the row are requested before the one wait: the issuers are blocked for as long as this takes)
    auto grab = [&](uint32_t taddr, uint32_t (&w)[32]) {
      uint32_t r0[32], r1[32];
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32, r1);
      tmem_ld_fence(r0);
      tmem_ld_fence(r1);
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        w[i >> 1] = pack2<T>(__uint_as_float(r0[i]), __uint_as_float(r0[i + 1]));
        w[16 + (i >> 1)] = pack2<T>(__uint_as_float(r1[i]), __uint_as_float(r1[i + 1]));
      }
    };
    // How rows leave.  A lane owns a row, and stores or reductions issued row by row touch 32 different lines per
    // instruction: they kept the load / store unit -- which also serves the shared-memory traffic of every other role --
    // busy enough to slow the whole CTA by a third.  So:
    //  * rows with a destination of their own (typed dK / dV / dQ rows, fp32 accumulator rows) are transposed through the
    //    warp's 4 KB of staging tile A (rows written with their 16-byte chunks XOR-swizzled, read back four whole rows per
    //    instruction) and leave as coalesced stores / reductions: eight lanes cover the 128 contiguous bytes of a row;
    //  * the sampled rows' slot buffers are laid out as staging tile B is ([key tile][half][row][32 floats], chunks
    //    swizzled the same way), so half an accumulator of all 128 rows is ONE bulk fp32 addition of 16 KB by one thread.
    //    (Bulk copies of single rows were tried for everything: the copy engine accepts one every ~15 cycles, and 1800
    //    of them per work item made the drain group the bottleneck of the CTA.)
    const int rot = row & 7;
    uint8_t* my_row_a = smem + OFF_ST + row * 128;
    const uint8_t* warp_rows = smem + OFF_ST + (row & ~31) * 128;
    uint8_t* my_row_b = smem + OFF_ST + TILE * 128 + row * 128;
    uint32_t tile_ops = 0;       // whole-tile additions issued so far
    bool tile_pending = false;   // ... and the last one may still be reading tile B
    auto put_tile = [&](const uint32_t (&w)[32], float* acc_tile) -> bool {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        HA_T_MARK(1)
        if (tile_pending && !wait(B_ST_FREE, (tile_ops - 1) & 1)) return false;
        HA_T_MARK(5)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 lo = unpack2<T>(w[16 * h + 2 * i]), hi = unpack2<T>(w[16 * h + 2 * i + 1]);
          *reinterpret_cast<float4*>(my_row_b + ((i ^ rot) << 4)) = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
        HA_T_MARK(1)
        fence_async_smem();
        HA_T_MARK(6)
        mbar_arrive(bar(B_ST_FULL));
        if (row == 0) {
          if (!wait(B_ST_FULL, tile_ops & 1)) return false;
          bws_bulk_add_f32(acc_tile + h * (TILE * 32), smem_u32(smem + OFF_ST + TILE * 128), TILE * 128);
          bws_bulk_commit();
          bws_bulk_wait_read();
          mbar_arrive(bar(B_ST_FREE));
        }
        ++tile_ops;
        tile_pending = true;
        HA_T_MARK(7)
      }
      return true;
    };
    // `rid`: this lane's destination row in dst (typed rows of 64 elements) or acc (fp32 rows of 64)
    auto put = [&](const uint32_t (&w)[32], T* dst, float* acc, uint32_t rid, bool typed) {
      if (typed) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(my_row_a + ((i ^ rot) << 4)) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int rl = 4 * j + (lane >> 3), c = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(warp_rows + rl * 128 + ((c ^ (rl & 7)) << 4));
          const size_t rr = __shfl_sync(0xffffffffu, rid, rl);
          *reinterpret_cast<uint4*>(dst + rr * 64 + c * 8) = v;
        }
        __syncwarp();
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float2 lo = unpack2<T>(w[16 * h + 2 * i]), hi = unpack2<T>(w[16 * h + 2 * i + 1]);
            *reinterpret_cast<float4*>(my_row_a + ((i ^ rot) << 4)) = make_float4(lo.x, lo.y, hi.x, hi.y);
          }
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rl = 4 * j + (lane >> 3), c = lane & 7;
            const float4 v = *reinterpret_cast<const float4*>(warp_rows + rl * 128 + ((c ^ (rl & 7)) << 4));
            const size_t rr = __shfl_sync(0xffffffffu, rid, rl);
            bws_red_add_v4(acc + rr * 64 + 32 * h + c * 4, v.x, v.y, v.z, v.w);
          }
          __syncwarp();
        }
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
        if (x < 2) return p.k_idx[kseg_of(p, seg) * p.m_k + (2 * blk + x) * TILE + row];
        const int s = (x - 2) * TILE + row;
        return p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + s] : s;
      };
      auto drain_dq = [&](int y) -> bool {
        HA_T_MARK(1)
        if (!wait(B_DQ_FULL + y, it & 1)) return false;
        HA_T_MARK(2)
        tc_fence_after();
        const long long r = head0 + si.q_row0 + (y ? qrow1 : qrow0);
        uint32_t w[32];
        grab(tmem + COL_DQ + y * D + lane_sel, w);
        tc_fence_before();
        mbar_arrive(bar(B_DQ_FREE + y));
        put(w, (T*)p.dq_out, p.dq_acc, (uint32_t)r, dq_direct);
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
        const long long r = si.khead0 + si.k_row0 + krow;
        float* acc_k = p.dk_acc;
        float* acc_v = p.dv_acc;
        if (kv_direct && sampled) {
          // the sampled tile's 128 x 64 block of the slot buffer
          const long long tile_at = (kseg_of(p, seg) * p.sample_size + (x - 2) * TILE) * D;
          acc_k = p.dk_sacc + tile_at;
          acc_v = p.dv_sacc + tile_at;
        }
        {
          uint32_t wv[32], wk[32];
          grab(tmem + COL_DV + lane_sel, wv);
          grab(tmem + COL_DK + lane_sel, wk);
          tc_fence_before();
          mbar_arrive(bar(B_ACC_FREE));
          HA_T_MARK(4)
          if (kv_direct && sampled) {
            ok = put_tile(wv, acc_v) && put_tile(wk, acc_k);
          } else {
            put(wv, (T*)p.dv_out, acc_v, (uint32_t)r, typed);
            put(wk, (T*)p.dk_out, acc_k, (uint32_t)r, typed);
          }
        }
        krow = krow_next;
      }
      if (ok) ok = drain_dq(1);
    }
    bws_bulk_wait_all();       // nothing of this thread is in flight when the CTA retires
    HA_T_DUMP(8, (int)blockIdx.x * 8 + 2, row == 0)
  } else {
    // warps 12 .. 19: three loader warps and five MMA-issuing threads (two warpgroups of 64 registers)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp <= 14) {
      // ===================================================================================================
      // loaders, one warp per operand stream: K tiles (warp 12), V tiles (warp 13), (Q, dO, lse, delta) tiles (warp 14).
      // One warp issuing every gather was the bottleneck of the whole CTA (measured: about 3500 cycles to issue one
      // tile's copies); the streams are independent -- each has its own ring and its own barriers.
      // ===================================================================================================
      // The copies of a tile signal its barrier themselves when they land (every lane arrives once, through the copy
      // engine), so a loader never waits for its own copies: only for free buffers.
      auto push = [&](int b) {
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar(b)) : "memory");
      };
      bool ok = true;
      int it = 0;
      HA_T_DECL(8)
      if (warp <= 13) {
        const bool is_v = warp == 13;
        const int n_st = is_v ? V_STAGES : K_STAGES;
        uint32_t xg = 0;        // key tiles fetched so far
        auto load_krows = [&](int seg, int blk, int x, int (&dst)[4]) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int rr = q * 32 + lane;
            if (x < 2) dst[q] = p.k_idx[kseg_of(p, seg) * p.m_k + (2 * blk + x) * TILE + rr];
            else {
              const int s = (x - 2) * TILE + rr;
              dst[q] = p.sample_idx ? p.sample_idx[kseg_of(p, seg) * p.sample_size + s] : s;
            }
          }
        };
        int krows[4] = {-1, -1, -1, -1};
        if ((int)blockIdx.x < n_items) load_krows(blockIdx.x / blocks_per_seg, blockIdx.x % blocks_per_seg, 0, krows);
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
          const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
          const SegInfo si = seg_info(p, seg);
          const uint16_t* base = is_v ? (const uint16_t*)p.v + si.b * p.v_sb + si.hk * p.v_sh + si.k_row0 * p.v_sn
                                      : (const uint16_t*)p.k + si.b * p.k_sb + si.hk * p.k_sh + si.k_row0 * p.k_sn;
          const int64_t sn = is_v ? p.v_sn : p.k_sn;
          for (int x = 0; x < nX && ok; ++x, ++xg) {
            // the next tile's row indices (the next item's first tile after this item's last) travel during the wait
            int knext[4] = {-1, -1, -1, -1};
            if (x + 1 < nX) load_krows(seg, blk, x + 1, knext);
            else if (item + (int)gridDim.x < n_items) load_krows((item + gridDim.x) / blocks_per_seg, (item + gridDim.x) % blocks_per_seg, 0, knext);
            // ... and its rows are pulled into L2 (one 128-byte line each), so that the copies below, whose number in flight
            // is limited, meet L2 latency rather than DRAM latency
            if (x + 1 < 2 || x + 1 == nX) {       // window tiles only: the sampled rows are shared by the whole segment
              const SegInfo nsi = x + 1 < nX ? si : seg_info(p, (item + (int)gridDim.x) / blocks_per_seg);
              const uint16_t* nbase = is_v ? (const uint16_t*)p.v + nsi.b * p.v_sb + nsi.hk * p.v_sh + nsi.k_row0 * p.v_sn
                                           : (const uint16_t*)p.k + nsi.b * p.k_sb + nsi.hk * p.k_sh + nsi.k_row0 * p.k_sn;
#pragma unroll
              for (int q = 0; q < 4; ++q)
                if (knext[q] >= 0) prefetch_l2(nbase + (int64_t)knext[q] * sn);
            }
            const int st = xg % n_st;
            HA_T_MARK(0)
            if (xg >= (uint32_t)n_st && !(ok = wait((is_v ? B_V_EMPTY : B_K_EMPTY) + st, (xg / n_st - 1) & 1))) break;
            HA_T_MARK(1)
            bws_gather_tile(s_base + (is_v ? OFF_V : OFF_K) + st * TILE_B, base, sn, krows, lane);
            push((is_v ? B_V_FULL : B_K_FULL) + st);
            HA_T_MARK(2)
#pragma unroll
            for (int q = 0; q < 4; ++q) krows[q] = knext[q];
          }
        }
        HA_T_DUMP(8, (int)blockIdx.x * 8 + 3, lane == 0 && warp == 12)
      } else {
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++it) {
          const int seg = item / blocks_per_seg, blk = item - seg * blocks_per_seg;
          const SegInfo si = seg_info(p, seg);
          const long long head0 = ((long long)(si.b * p.H + si.h)) * p.n;
          const uint16_t* qbase = (const uint16_t*)p.q + si.b * p.q_sb + si.h * p.q_sh + si.q_row0 * p.q_sn;
          const uint16_t* gbase = (const uint16_t*)p.d_o + si.b * p.do_sb + si.h * p.do_sh + si.q_row0 * p.do_sn;
          const float* lse_base = p.lse + head0 + si.q_row0;
          const float* delta_base = p.delta + head0 + si.q_row0;
#pragma unroll
          for (int y = 0; y < 2; ++y) {
            int qrows[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) qrows[q] = p.q_idx[(long long)seg * p.m_q + (2 * blk + y) * TILE + q * 32 + lane];
            HA_T_MARK(0)
            if (it >= 1 && !(ok = wait(B_QD_EMPTY + y, (it - 1) & 1))) break;
            HA_T_MARK(1)
            bws_gather_tile(s_base + OFF_QD + y * 2 * TILE_B, qbase, p.q_sn, qrows, lane);
            bws_gather_tile(s_base + OFF_QD + y * 2 * TILE_B + TILE_B, gbase, p.do_sn, qrows, lane);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t dst = s_base + OFF_LD + y * 1024 + (q * 32 + lane) * 4;
              cp_async4(dst, lse_base + qrows[q]);
              cp_async4(dst + 512, delta_base + qrows[q]);
            }
            push(B_QD_FULL + y);
            HA_T_MARK(2)
          }
          // The next item's query-side rows: pulled into L2 now, so that the copies issued when their stages come free
          // (at the very end of this item) find them there instead of in DRAM.
          const int nitem = item + gridDim.x;
          if (ok && nitem < n_items) {
            const int nseg = nitem / blocks_per_seg, nblk = nitem - nseg * blocks_per_seg;
            const SegInfo ns = seg_info(p, nseg);
            const uint16_t* nq = (const uint16_t*)p.q + ns.b * p.q_sb + ns.h * p.q_sh + ns.q_row0 * p.q_sn;
            const uint16_t* ng = (const uint16_t*)p.d_o + ns.b * p.do_sb + ns.h * p.do_sh + ns.q_row0 * p.do_sn;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int qr = p.q_idx[(long long)nseg * p.m_q + 2 * nblk * TILE + j * 32 + lane];
              prefetch_l2(nq + (int64_t)qr * p.q_sn);
              prefetch_l2(ng + (int64_t)qr * p.do_sn);
            }
          }
        }
        HA_T_DUMP(8, (int)blockIdx.x * 8 + 7, lane == 0)
      }
      cp_async_commit();
      cp_async_wait<0>();      // nothing of this warp is in flight when the CTA retires
    } else if (lane == 0) {
      // ===================================================================================================
      // MMA issue: five threads, one product each (no accumulator is shared between them).  Each walks the halves /
      // pairs in order and blocks (bounded) on what its next instructions need.
      //   warp 15: S^T of every half    warp 16: dP^T of every half    -> S-ready (two commits)
      //   warp 17: dV of every half     warp 18: dK of every half      -> the stage's S^T / dP^T columns free, accumulators full
      //   warp 19: dQ of every pair                                    -> dS buffer free, dQ full
      // The "empty" barriers of the operand stages collect one commit from every issuer that reads the stage.
      // ===================================================================================================
      constexpr int AB = std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
      const int my_items = n_items > (int)blockIdx.x ? (n_items - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
      const uint32_t NH = 4u * (uint32_t)nX;                 // halves per item
      const uint32_t total = (uint32_t)my_items * NH;
      // Half hh (a count over this CTA's items): item hh / NH, key tile x = (hh % NH) / 4, query tile y = bit 1, stage s = bit 0.
      // Pair = hh / 2, key tile count = hh / 4.
      bool ok = true;
      if (warp == 15 || warp == 16) {
        // S^T = K Q^T (warp 15) / dP^T = V dO^T (warp 16) of the half: M = 128 keys, N = 64 query rows, both operands K-major
        const bool second = warp == 16;
        const uint32_t id_st = mma_idesc(TILE, 64, AB, 0, 0);
        HA_T_DECL(8)
        for (uint32_t hh = 0; hh < total && ok; ++hh) {
          const uint32_t r = hh % NH, itc = hh / NH, x = r >> 2, y = (r >> 1) & 1, s = r & 1;
          const uint32_t pair = hh >> 1, xg = hh >> 2;
          HA_T_MARK(0)
          // the product that read P^T (dS^T) out of these columns for the stage's previous half has completed
          if (pair >= 1 && !(ok = wait((second ? B_SF_P : B_SF_S) + s, (pair - 1) & 1))) break;
          HA_T_MARK(1)
          const uint32_t ks = xg % K_STAGES, vs = xg & 1;
          if ((r & 3) == 0 && !(ok = second ? wait(B_V_FULL + vs, (xg >> 1) & 1) : wait(B_K_FULL + ks, (xg / K_STAGES) & 1))) break;
          if (x == 0 && s == 0 && !(ok = wait(B_QD_FULL + y, itc & 1))) break;
          HA_T_MARK(2)
          fence_async_smem();          // the copies that filled the operand tiles are ordered before the operand reads
          tc_fence_after();
          const uint32_t sB = s_base + OFF_QD + y * 2 * TILE_B + s * (TILE_B / 2) + (second ? TILE_B : 0);
          const uint32_t sA = s_base + (second ? OFF_V + vs * TILE_B : OFF_K + ks * TILE_B);
          const uint32_t tD = tmem + 128 * s + (second ? 64 : 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) mma_ss(tD, smem_desc(sA + kk * 32, 16, 1024), smem_desc(sB + kk * 32, 16, 1024), id_st, kk > 0);
          mma_commit(bar(B_S_READY + s));
          if ((r & 3) == 3) mma_commit(bar(second ? B_V_EMPTY + vs : B_K_EMPTY + ks));   // this thread's last read of the K (V) stage
          if (x == (uint32_t)nX - 1 && s == 1) mma_commit(bar(B_QD_EMPTY + y));      // ... and of the Q / dO stage
          HA_T_MARK(3)
        }
        HA_T_DUMP(8, (int)blockIdx.x * 8 + 4, warp == 15)
      } else if (warp == 17 || warp == 18) {
        // dV += P^T dO (warp 17) / dK += dS^T Q (warp 18) over the half's 64 query rows: A in TMEM, B rows as MN-major
        const bool second = warp == 18;
        const uint32_t id_kv = mma_idesc(TILE, 64, AB, 0, 1);
        HA_T_DECL(8)
        for (uint32_t hh = 0; hh < total && ok; ++hh) {
          const uint32_t r = hh % NH, x = r >> 2, y = (r >> 1) & 1, s = r & 1;
          const uint32_t pair = hh >> 1, xg = hh >> 2;
          HA_T_MARK(0)
          if (!(ok = wait(B_P_READY + s, pair & 1))) break;
          HA_T_MARK(1)
          if ((r & 3) == 0 && xg >= 1 && !(ok = wait(B_ACC_FREE, (xg - 1) & 1))) break;    // the accumulator restarts with the key tile
          HA_T_MARK(2)
          fence_async_smem();
          tc_fence_after();
          const uint32_t sB = s_base + OFF_QD + y * 2 * TILE_B + s * (TILE_B / 2) + (second ? 0 : TILE_B);   // Q rows (dK) / dO rows (dV)
          const uint32_t tA = tmem + 128 * s + (second ? 64 : 0);
          const uint32_t tD = tmem + (second ? COL_DK : COL_DV);
          const uint32_t acc0 = (r & 3) != 0;
          // group 0 packed its 32 query columns into TMEM columns [0, 16), group 1 into [32, 48): K steps 0, 1 and 2, 3
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_ts(tD, tA + (kk >> 1) * 32 + (kk & 1) * 8, smem_desc(sB + kk * 2048, TILE * 128, 1024), id_kv, acc0 | (kk > 0));
          mma_commit(bar((second ? B_SF_P : B_SF_S) + s));
          if ((r & 3) == 3) mma_commit(bar(B_ACC_FULL));                            // the key tile's accumulator is complete
          if (x == (uint32_t)nX - 1 && s == 1) mma_commit(bar(B_QD_EMPTY + y));
          HA_T_MARK(3)
        }
        HA_T_DUMP(8, (int)blockIdx.x * 8 + 5, warp == 17)
      } else {
        // dQ_y += dS K over the pair's 128 keys: A = dS ([key][query] rows: MN-major), B = K rows as MN-major
        const uint32_t id_dq = mma_idesc(TILE, 64, AB, 1, 1);
        const uint32_t total_pairs = total >> 1;
        HA_T_DECL(8)
        for (uint32_t pair = 0; pair < total_pairs && ok; ++pair) {
          const uint32_t r = (2 * pair) % NH, itc = (2 * pair) / NH, x = r >> 2, y = (r >> 1) & 1, xg = pair >> 1;
          HA_T_MARK(0)
          // both halves of the pair have written their dS slabs
          if (!(ok = wait(B_DS_FULL + (pair & 1), (pair >> 1) & 1))) break;
          HA_T_MARK(1)
          if (x == 0 && itc >= 1 && !(ok = wait(B_DQ_FREE + y, (itc - 1) & 1))) break;      // dQ restarts with the item
          HA_T_MARK(2)
          fence_async_smem();
          tc_fence_after();
          const uint32_t sK = s_base + OFF_K + (xg % K_STAGES) * TILE_B;
          const uint32_t sDS = s_base + OFF_DS + (pair & 1) * 2 * TILE_B;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ss(tmem + COL_DQ + y * D, smem_desc(sDS + kk * 2048, TILE_B, 1024), smem_desc(sK + kk * 2048, TILE_B, 1024), id_dq,
                   (x > 0) | (kk > 0));
          mma_commit(bar(B_DS_FREE + (pair & 1)));
          if (x == (uint32_t)nX - 1) mma_commit(bar(B_DQ_FULL + y));                  // the query tile's dQ is complete
          if (y == 1) mma_commit(bar(B_K_EMPTY + xg % K_STAGES));                     // this thread's last read of the K tile
          HA_T_MARK(3)
        }
        HA_T_DUMP(8, (int)blockIdx.x * 8 + 6, true)
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
  const int sms = sm_count();
  const int grid = (int)(items < sms ? items : sms);
  // The dynamic window is everything the CTA may have beyond the kernel's static variables; the tiles start at its first
  // 1 KB boundary.
#define HA_BWS_LAUNCH(TT)                                                                                                        \
  do {                                                                                                                           \
    static int dyn_bytes = 0;                                                                                                    \
    if (dyn_bytes == 0) {                                                                                                        \
      cudaFuncAttributes fa;                                                                                                     \
      HA_CUDA_OK(cudaFuncGetAttributes(&fa, attn_tc_bwd_ws_kernel<TT>), "ha_attn_bwd kernel attributes");                        \
      const int stat = ((int)fa.sharedSizeBytes + 15) / 16 * 16;                                                                 \
      const int pad = (1024 - stat % 1024) % 1024;                                                                               \
      if (stat + pad + bws::SMEM_USED > bws::SMEM_LIMIT) return HA_ERR_CUDA;                                                     \
      dyn_bytes = bws::SMEM_LIMIT - stat;                                                                                        \
    }                                                                                                                            \
    HA_SMEM_ATTR_ONCE(attn_tc_bwd_ws_kernel<TT>, dyn_bytes, "ha_attn_bwd smem attribute");                                      \
    attn_tc_bwd_ws_kernel<TT><<<grid, bws::THREADS, dyn_bytes, st>>>(p, (int)items, blocks_per_seg);                             \
  } while (0)
  if (p.dtype == HA_BF16) HA_BWS_LAUNCH(__nv_bfloat16);
  else HA_BWS_LAUNCH(__half);
#undef HA_BWS_LAUNCH
  HA_LAUNCHED("ha_attn_bwd (tcgen05, warp-specialised)");
  return HA_OK;
}

}  // namespace ha

HA_T_SETTER(ha_debug_set_timing_buffer_bwd_ws)
