// Causal HyperAttention as one host-side schedule over the segment kernels.
//
// The reference recurses on the host: split the sequence in two, fold the halves into extra heads, recurse on the
// diagonal blocks, run the un-masked kernel on the lower-left rectangle, merge, concatenate
// (hyper_attention.py:51-96).  Unrolled, depth l (0 = top) holds 2^l spans of n/2^l rows per head; its rectangles
// pair the second half of every span (queries) with the first half (keys), and the leaves at depth `levels` are
// exact causal attention on spans of n/2^levels rows.  Here the whole tree is a flat list of launches on the
// caller's [B,H,n,*] buffers: hash q and k once (a token's bucket does not depend on the depth), the leaves write
// (o, lse), then the rectangles run deepest first and merge into the same rows in their epilogue -- the order in
// which the reference's merges nest (stored value = attn1, rectangle = attn2).  No concatenation, no per-depth
// copies.
#include "attn_index.cuh"

#include <mutex>

namespace ha {

bool tc_bwd_supported(const ha_attn_params& p);   // attn_tc_bwd.cu

// One helper stream and two events per device, created on first use and kept for the life of the process.
// `mu` serialises the callers of one device over the fork .. join section (the two events are shared).
struct SideStream { cudaStream_t stream; cudaEvent_t fork, join; std::mutex* mu; };
static SideStream* side_stream() {
  static std::mutex mu;
  static SideStream per_dev[64];
  static bool ready[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[dev]) {
    SideStream s;
    // highest priority: its short kernels take the next free CTA slots instead of queueing behind a large grid
    int prio_lo = 0, prio_hi = 0;
    cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    if (cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, prio_hi) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    s.mu = new std::mutex();
    per_dev[dev] = s;
    ready[dev] = true;
  }
  return &per_dev[dev];
}

struct CausalPlan {
  long long rows;          // B*H*n
  long long rows_k;        // B*(H / kv_group)*n: rows of k, v, dk, dv
  int Hk;                  // K/V heads
  long long idx_bytes;     // one depth's q_idx or k_idx
  long long part_o_bytes, part_lse_bytes;
  long long sort_ws;       // largest sort workspace over the depths
  int leaf;
};

static int make_plan(const ha_causal_params& p, CausalPlan& pl) {
  if (p.dtype != HA_BF16 && p.dtype != HA_FP16 && p.dtype != HA_FP32) return HA_ERR_DTYPE;
  if (p.B <= 0 || p.H <= 0 || p.n <= 0 || p.d <= 0 || p.dv <= 0 || p.d > 256 || p.dv > 256) return HA_ERR_INVALID;
  if (p.levels < 1 || p.levels > 24 || p.lsh_bits < 1 || p.lsh_bits > 16) return HA_ERR_INVALID;
  if (p.n % (1 << p.levels) != 0) return HA_ERR_INVALID;
  if (p.sample_size < 0 || p.sample_size % TILE != 0 || p.block_size < 1) return HA_ERR_INVALID;
  pl.leaf = p.n >> p.levels;
  // every rectangle must be a whole number of 128-row tiles, and those on the hyper pattern must hold the sampled rows
  // (the deepest ones are exact where they are shorter than min_seq_len)
  if (pl.leaf % TILE != 0) return HA_ERR_INVALID;
  const bool deepest_is_exact = p.min_seq_len > pl.leaf;
  if (!(deepest_is_exact && p.levels == 1) && p.sample_size > (deepest_is_exact ? 2 * pl.leaf : pl.leaf)) return HA_ERR_INVALID;
  if (p.kv_group < 0 || (p.kv_group > 1 && p.H % p.kv_group != 0)) return HA_ERR_INVALID;
  pl.Hk = p.kv_group > 1 ? p.H / p.kv_group : p.H;
  pl.rows = (long long)p.B * p.H * p.n;
  pl.rows_k = (long long)p.B * pl.Hk * p.n;
  pl.idx_bytes = pl.rows / 2 * 4;
  pl.part_o_bytes = pl.rows * p.dv * dtype_size(p.dtype);
  pl.part_lse_bytes = pl.rows * 4;
  pl.sort_ws = 0;
  for (int l = 0; l < p.levels; ++l) {
    const int span = p.n >> l;
    const long long ws = ha_seg_sort_workspace_bytes(p.B * p.H, p.n, span, span / 2, p.lsh_bits);
    if (ws > pl.sort_ws) pl.sort_ws = ws;
  }
  return HA_OK;
}


// delta of every part in one pass: dO is read once per row; the leaf part is needed by every row, the rectangle of
// depth l only by rows in the second half of their span.  Output delta[part][B*H*n], part = depth, leaves last.
// Both multi-part passes below are bound by instruction issue, not by DRAM (ncu: issue slots 67-71% busy at 28-35% of the
// DRAM rate), so the index arithmetic is kept off the loop: a row's position inside its head advances by a constant
// from one iteration to the next (one conditional subtraction instead of a 64-bit modulo), and with n a power of two
// (log2n >= 0) the half-span test of a depth is a shift instead of a division.
__device__ __forceinline__ int half_bit(int i, int n, int depth, int log2n) {
  return (log2n >= 0 ? i >> (log2n - depth - 1) : i / (n >> (depth + 1))) & 1;
}
static int log2_if_pow2(int n) {
  if (n <= 0 || (n & (n - 1))) return -1;
  int l = 0;
  while ((1 << l) < n) ++l;
  return l;
}

template <typename T, int EPC>
__global__ void __launch_bounds__(256) delta_parts_kernel(const T* __restrict__ d_o, const uint8_t* __restrict__ parts0, long long part_stride_bytes,
                                                          int levels, int n, int lpr, float* __restrict__ delta, long long total_rows,
                                                          int log2n) {
  const int lane = threadIdx.x & 31;
  const int rpw = 32 / lpr, chunk = lane % lpr, sub = lane / lpr;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int dv = lpr * EPC;
  constexpr int UN = 2;   // row groups per iteration
  constexpr int PG = 4;   // parts whose rows are requested together: UN * (PG + 1) independent 16-byte loads in flight per lane
  const int step = (int)((n_warps * rpw * UN) % n);
  int i[UN];
#pragma unroll
  for (int u = 0; u < UN; ++u) i[u] = (int)((warp_id * rpw * UN + u * rpw + sub) % n);
  for (long long base = warp_id * rpw * UN; base < total_rows; base += n_warps * rpw * UN) {
    long long row[UN];
    bool ok[UN];
    uint4 g[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      row[u] = base + u * rpw + sub;
      ok[u] = row[u] < total_rows;
      g[u] = make_uint4(0, 0, 0, 0);
      if (ok[u]) g[u] = __ldg(reinterpret_cast<const uint4*>(d_o + row[u] * dv + chunk * EPC));
    }
    float gf[UN][8];      // this lane's dO elements, unpacked once for all parts
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const uint32_t gw[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if constexpr (EPC == 8) {
          const float2 fg = unpack2<T>(gw[w]);
          gf[u][2 * w] = fg.x;
          gf[u][2 * w + 1] = fg.y;
        } else {
          gf[u][w] = __uint_as_float(gw[w]);
        }
      }
    }
    for (int part0 = 0; part0 <= levels; part0 += PG) {
      bool need[PG][UN];
      uint4 a[PG][UN];
#pragma unroll
      for (int pp = 0; pp < PG; ++pp) {
        const int part = part0 + pp;
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          need[pp][u] = part <= levels && ok[u] && (part == levels || half_bit(i[u], n, part, log2n));
          a[pp][u] = make_uint4(0, 0, 0, 0);
          if (need[pp][u])
            a[pp][u] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(parts0 + part * part_stride_bytes) + row[u] * dv + chunk * EPC));
        }
      }
#pragma unroll
      for (int pp = 0; pp < PG; ++pp) {
        const int part = part0 + pp;
#pragma unroll
        for (int u = 0; u < UN; ++u) {
          // a warp's rows are consecutive: they nearly always need the same parts, and a part nobody needs is skipped whole
          if (!__any_sync(0xffffffffu, need[pp][u])) continue;
          float s = 0.f;
          const uint32_t aw[4] = {a[pp][u].x, a[pp][u].y, a[pp][u].z, a[pp][u].w};
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            if constexpr (EPC == 8) {
              const float2 fa = unpack2<T>(aw[w]);
              s = fmaf(fa.x, gf[u][2 * w], s);
              s = fmaf(fa.y, gf[u][2 * w + 1], s);
            } else {
              s = fmaf(__uint_as_float(aw[w]), gf[u][w], s);
            }
          }
          for (int off = lpr >> 1; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
          if (need[pp][u] && chunk == 0) delta[(long long)part * total_rows + row[u]] = s;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      i[u] += step;
      if (i[u] >= n) i[u] -= n;
    }
  }
}

static inline long long align256(long long x) { return (x + 255) / 256 * 256; }

struct SavedLayout {
  uint8_t* base;
  CausalPlan pl;
  int levels, keep_parts;
  int32_t* q_idx(int l) const { return (int32_t*)(base + (long long)l * 2 * align256(pl.idx_bytes)); }
  int32_t* k_idx(int l) const { return (int32_t*)(base + ((long long)l * 2 + 1) * align256(pl.idx_bytes)); }
  long long parts_off() const { return (long long)levels * 2 * align256(pl.idx_bytes); }
  // part index: 0..levels-1 = rectangles of that depth, levels = leaves
  void* part_o(int part) const { return base + parts_off() + (long long)part * (align256(pl.part_o_bytes) + align256(pl.part_lse_bytes)); }
  float* part_lse(int part) const { return (float*)((uint8_t*)part_o(part) + align256(pl.part_o_bytes)); }
  long long total() const {
    return parts_off() + (keep_parts ? (long long)(levels + 1) * (align256(pl.part_o_bytes) + align256(pl.part_lse_bytes)) : 0);
  }
};

// The merges of the causal schedule as one pass over the stored parts (training calls keep every part's (o, lse) for the
// backward anyway): a row starts from its leaf part and takes in, from the deepest rectangle up, every rectangle part
// whose query half it lies in -- the arithmetic of the attention kernels' merging epilogue (add_self_attentions,
// utils.py:82-88 of the reference: weights rounded to the tensors' dtype, the merged row rounded after every step), in
// the same order.  The rectangle launches then run as plain calls that write their part and read nothing back, which
// costs them a third less time than merging in their epilogue (old rows gathered, two outputs stored).
// One lane per 16-byte chunk of a row; part = depth, leaves last, as in the saved layout.
template <typename T>
__global__ void __launch_bounds__(256) merge_parts_kernel(const uint8_t* __restrict__ parts0, long long part_stride_bytes, long long lse_off_bytes,
                                                          int levels, int n, int lpr, T* __restrict__ o, float* __restrict__ lse,
                                                          long long total_rows, int exact, int log2n) {
  const int lane = threadIdx.x & 31;
  const int rpw = 32 / lpr, chunk = lane % lpr, sub = lane / lpr;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int dv = lpr * 8;
  const int step = (int)((n_warps * rpw) % n);
  int i = (int)((warp_id * rpw + sub) % n) - step;
  for (long long base = warp_id * rpw; base < total_rows; base += n_warps * rpw) {
    i += step;
    if (i >= n) i -= n;
    const long long row = base + sub;
    if (row >= total_rows) continue;
    auto part_row = [&](int part) { return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(parts0 + part * part_stride_bytes) + row * dv + chunk * 8)); };
    auto part_lse = [&](int part) { return __ldg(reinterpret_cast<const float*>(parts0 + part * part_stride_bytes + lse_off_bytes) + row); };
    // every part this row needs is requested before the first merge
    uint4 cur = part_row(levels);
    float l1 = part_lse(levels);
    for (int l0 = levels - 1; l0 >= 0; l0 -= 4) {
      uint4 nw[4];
      float l2[4];
      bool need[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int l = l0 - j;
        need[j] = l >= 0 && half_bit(i, n, l, log2n);
        nw[j] = make_uint4(0, 0, 0, 0);
        l2[j] = 0.f;
        if (need[j]) {
          nw[j] = part_row(l);
          l2[j] = part_lse(l);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!need[j]) continue;
        float w1, w2, lm;
        if (exact) {
          const float m2 = fmaxf(l1, l2[j]);
          const float e1 = __expf(l1 - m2), e2 = __expf(l2[j] - m2);
          w1 = e1 / (e1 + e2);
          w2 = e2 / (e1 + e2);
          lm = m2 + __logf(e1 + e2);
        } else {
          const float cf = round_to<T>(1.f / (1.f + __expf(l2[j] - l1)));
          w1 = cf;
          w2 = round_to<T>(1.f - cf);
          lm = l1 - __logf(cf + 1.1920929e-07f);
        }
        const uint32_t ow[4] = {cur.x, cur.y, cur.z, cur.w}, pw[4] = {nw[j].x, nw[j].y, nw[j].z, nw[j].w};
        uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 old = unpack2<T>(ow[h]), mine = unpack2<T>(pw[h]);
          w[h] = pack2<T>(w1 * old.x + w2 * mine.x, w1 * old.y + w2 * mine.y);
        }
        cur = make_uint4(w[0], w[1], w[2], w[3]);
        l1 = lm;
      }
    }
    *reinterpret_cast<uint4*>(o + row * dv + chunk * 8) = cur;
    if (chunk == 0) lse[row] = l1;
  }
}

static void fill_attn(const ha_causal_params& p, ha_attn_params& a) {
  a = ha_attn_params{};
  a.dtype = p.dtype;
  a.B = p.B; a.H = p.H; a.n = p.n; a.d = p.d; a.dv = p.dv;
  a.block_size = p.block_size; a.sample_size = p.sample_size; a.scale = p.scale;
  a.q = p.q; a.k = p.k; a.v = p.v;
  a.q_sn = p.d; a.q_sh = (int64_t)p.n * p.d; a.q_sb = a.q_sh * p.H;
  const int Hk = p.kv_group > 1 ? p.H / p.kv_group : p.H;
  a.kv_group = p.kv_group;
  a.k_sn = p.d; a.k_sh = a.q_sh; a.k_sb = a.k_sh * Hk;
  a.v_sn = p.dv; a.v_sh = (int64_t)p.n * p.dv; a.v_sb = a.v_sh * Hk;
  a.o = p.o; a.o_sn = p.dv; a.o_sh = a.v_sh; a.o_sb = a.o_sh * p.H;
  a.lse = p.lse;
  a.d_o = p.d_o; a.do_sn = p.dv; a.do_sh = a.v_sh; a.do_sb = a.o_sb;
  a.status = p.status;
  a.status_host = p.status_host;
}

// The deepest rectangles (n / 2^levels rows a side) are exact where they are shorter than min_seq_len, as in the
// reference's forward_no_causal_mask (hyper_attention.py:109-113).
static bool deepest_exact(const ha_causal_params& p, const CausalPlan& pl) { return p.min_seq_len > pl.leaf; }

}  // namespace ha

using namespace ha;

extern "C" {

int64_t ha_causal_saved_bytes(const ha_causal_params* p) {
  CausalPlan pl;
  if (!p || make_plan(*p, pl) != HA_OK) return -1;
  SavedLayout s{nullptr, pl, p->levels, p->keep_parts};
  return s.total();
}

// Can the merges of this call run as one pass over the parts (merge_parts_kernel)?
static bool merges_deferrable(const ha_causal_params& p) {
  return p.levels > 0 && p.dtype != HA_FP32 && !(p.flags & HA_FLAG_FORCE_SIMT) && p.dv % 8 == 0 && 256 % p.dv == 0;
}
// A forward that keeps no parts for a backward still runs that way when the parts fit a scratch budget: a merging
// rectangle launch costs a third more than a plain one (config 2 forward: 8.6 -> 7.7 ms).
static long long scratch_part_bytes(const ha_causal_params& p, const CausalPlan& pl) {
  if (p.keep_parts || !merges_deferrable(p)) return 0;
  const long long bytes = (long long)(p.levels + 1) * (align256(pl.part_o_bytes) + align256(pl.part_lse_bytes));
  return bytes <= (16LL << 30) ? bytes : 0;
}

int64_t ha_causal_scratch_bytes(const ha_causal_params* p, int32_t backward) {
  CausalPlan pl;
  if (!p || make_plan(*p, pl) != HA_OK) return -1;
  if (!backward) return 2 * align256(pl.rows * 4) + align256(pl.sort_ws) + scratch_part_bytes(*p, pl);
  return align256(pl.rows * p->d * 4) + align256(pl.rows_k * p->d * 4) + align256(pl.rows_k * p->dv * 4) + align256(pl.rows * 4 * (p->levels + 1));
}

int ha_causal_fwd(const ha_causal_params* pp, void* stream) {
  if (!pp) return HA_ERR_INVALID;
  const ha_causal_params& p = *pp;
  CausalPlan pl;
  int rc = make_plan(p, pl);
  if (rc != HA_OK) return rc;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse || !p.proj) return HA_ERR_INVALID;
  SavedLayout sv{(uint8_t*)p.saved, pl, p.levels, p.keep_parts};
  if (!p.saved || p.saved_bytes < sv.total()) return HA_ERR_WORKSPACE;
  if (!p.scratch || p.scratch_bytes < ha_causal_scratch_bytes(pp, 0)) return HA_ERR_WORKSPACE;
  int32_t* codes_q = (int32_t*)p.scratch;
  int32_t* codes_k = (int32_t*)((uint8_t*)p.scratch + align256(pl.rows * 4));
  void* sort_ws = (uint8_t*)p.scratch + 2 * align256(pl.rows * 4);

  const int64_t sn = p.d, sh = (int64_t)p.n * p.d, sb = sh * p.H;
  rc = ha_lsh_hash(p.q, sb, sh, sn, p.B, p.H, p.n, p.d, p.dtype, p.proj, p.lsh_bits, codes_q, stream);
  if (rc != HA_OK) return rc;
  rc = ha_lsh_hash(p.k, sh * pl.Hk, sh, sn, p.B, pl.Hk, p.n, p.d, p.dtype, p.proj, p.lsh_bits, codes_k, stream);
  if (rc != HA_OK) return rc;

  // The sorts of every depth depend on the codes only: they run on a side stream (forked here, joined before the first
  // rectangle) underneath the leaves' kernel, which does not need them.  36 short launches leave the critical path.
  SideStream* side = side_stream();
  cudaStream_t main_st = (cudaStream_t)stream;
  const bool exact_deepest = deepest_exact(p, pl);
  // two host threads driving one device share the side stream and its events: one caller at a time from fork to join
  std::unique_lock<std::mutex> side_lock;
  if (side) side_lock = std::unique_lock<std::mutex>(*side->mu);
  if (side) {
    HA_CUDA_OK(cudaEventRecord(side->fork, main_st), "ha_causal_fwd fork");
    HA_CUDA_OK(cudaStreamWaitEvent(side->stream, side->fork, 0), "ha_causal_fwd fork");
  }
  void* sort_stream = side ? (void*)side->stream : stream;
  int sort_rc = HA_OK;
  for (int l = p.levels - 1 - (exact_deepest ? 1 : 0); l >= 0 && sort_rc == HA_OK; --l) {
    const int span = p.n >> l, m = span / 2;
    sort_rc = ha_seg_sort(codes_q, p.B * p.H, p.n, span, m, m, p.lsh_bits, sv.q_idx(l), sort_ws, pl.sort_ws, sort_stream);
    if (sort_rc == HA_OK)
      sort_rc = ha_seg_sort(codes_k, p.B * pl.Hk, p.n, span, 0, m, p.lsh_bits, sv.k_idx(l), sort_ws, pl.sort_ws, sort_stream);
  }
  if (side) {   // joined in every case, so that the caller's stream also orders after whatever the side stream holds
    HA_CUDA_OK(cudaEventRecord(side->join, side->stream), "ha_causal_fwd join");
  }
  if (sort_rc != HA_OK) {
    if (side) cudaStreamWaitEvent(main_st, side->join, 0);
    return sort_rc;
  }

  ha_attn_params a;
  fill_attn(p, a);
  // leaves: exact causal attention on 2^levels spans per head
  a.mode = HA_MODE_FLASH;
  a.flags = HA_FLAG_CAUSAL | (p.flags & HA_FLAG_FORCE_SIMT);
  a.segs_per_head = 1 << p.levels;
  a.span = pl.leaf; a.q_off = 0; a.k_off = 0; a.m_q = pl.leaf; a.m_k = pl.leaf;
  // A call that keeps the parts (16-bit tensors, tensor-core kernels) writes every part straight into its slot and merges
  // them in one pass at the end; otherwise every rectangle merges into (o, lse) in its epilogue.
  const long long in_scratch = scratch_part_bytes(p, pl);
  const bool deferred = merges_deferrable(p) && (p.keep_parts || in_scratch > 0);
  // the parts' slots: in the saved buffer (kept for the backward) or, for a call that keeps nothing, in the scratch
  uint8_t* const slots = !deferred ? nullptr : p.keep_parts ? (uint8_t*)sv.part_o(0) : (uint8_t*)p.scratch + 2 * align256(pl.rows * 4) + align256(pl.sort_ws);
  const long long slot_stride = align256(pl.part_o_bytes) + align256(pl.part_lse_bytes), slot_lse = align256(pl.part_o_bytes);
  auto slot_o = [&](int part) -> void* { return slots + part * slot_stride; };
  auto slot_lse_of = [&](int part) -> float* { return (float*)(slots + part * slot_stride + slot_lse); };
  if (deferred) { a.o = slot_o(p.levels); a.lse = slot_lse_of(p.levels); }
  else if (p.keep_parts) { a.part_o = sv.part_o(p.levels); a.part_lse = sv.part_lse(p.levels); }
  rc = ha_attn_fwd(&a, stream);
  if (side) HA_CUDA_OK(cudaStreamWaitEvent(main_st, side->join, 0), "ha_causal_fwd join");
  if (side) side_lock.unlock();
  if (rc != HA_OK) return rc;

  for (int l = p.levels - 1; l >= 0; --l) {
    const int span = p.n >> l, m = span / 2;
    const bool exact = exact_deepest && l == p.levels - 1;
    a.mode = exact ? HA_MODE_FLASH : HA_MODE_HYPER;
    a.flags = (deferred ? 0 : HA_FLAG_MERGE | (p.flags & HA_FLAG_MERGE_EXACT)) | (p.flags & HA_FLAG_FORCE_SIMT) |
              (exact ? 0 : (p.flags & (HA_FLAG_SMOOTH | HA_FLAG_NO_WS)));
    a.segs_per_head = 1 << l;
    a.span = span; a.q_off = m; a.k_off = 0; a.m_q = m; a.m_k = m;
    a.q_idx = exact ? nullptr : sv.q_idx(l); a.k_idx = exact ? nullptr : sv.k_idx(l); a.sample_idx = nullptr;
    if (deferred) { a.o = slot_o(l); a.lse = slot_lse_of(l); }
    else if (p.keep_parts) { a.part_o = sv.part_o(l); a.part_lse = sv.part_lse(l); }
    rc = ha_attn_fwd(&a, stream);
    if (rc != HA_OK) return rc;
  }
  if (deferred) {
    const int lpr = p.dv / 8;
    const long long per_cta = 8LL * (32 / lpr) * 8;
    const long long want = (pl.rows + per_cta - 1) / per_cta;
    const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
    const long long part_stride = slot_stride, lse_off = slot_lse;
    const int exact_merge = (p.flags & HA_FLAG_MERGE_EXACT) ? 1 : 0;
    if (p.dtype == HA_BF16)
      merge_parts_kernel<__nv_bfloat16><<<grid, 256, 0, main_st>>>((const uint8_t*)slots, part_stride, lse_off, p.levels, p.n, lpr,
                                                                  (__nv_bfloat16*)p.o, p.lse, pl.rows, exact_merge, log2_if_pow2(p.n));
    else
      merge_parts_kernel<__half><<<grid, 256, 0, main_st>>>((const uint8_t*)slots, part_stride, lse_off, p.levels, p.n, lpr, (__half*)p.o,
                                                           p.lse, pl.rows, exact_merge, log2_if_pow2(p.n));
    HA_LAUNCHED("ha_causal_fwd merge");
  }
  return HA_OK;
}

int ha_causal_bwd(const ha_causal_params* pp, void* stream) {
  if (!pp) return HA_ERR_INVALID;
  const ha_causal_params& p = *pp;
  CausalPlan pl;
  int rc = make_plan(p, pl);
  if (rc != HA_OK) return rc;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse || !p.d_o || !p.dq || !p.dk || !p.dv_out) return HA_ERR_INVALID;
  SavedLayout sv{(uint8_t*)p.saved, pl, p.levels, p.keep_parts};
  if (!p.saved || p.saved_bytes < sv.total()) return HA_ERR_WORKSPACE;
  if (!p.scratch || p.scratch_bytes < ha_causal_scratch_bytes(pp, 1)) return HA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* s = (uint8_t*)p.scratch;
  float* dq_acc = (float*)s;                 s += align256(pl.rows * p.d * 4);
  float* dk_acc = (float*)s;                 s += align256(pl.rows_k * p.d * 4);
  float* dv_acc = (float*)s;                 s += align256(pl.rows_k * p.dv * 4);
  float* delta = (float*)s;
  ha_attn_params a;
  fill_attn(p, a);
  a.delta = delta; a.dq_acc = dq_acc; a.dk_acc = dk_acc; a.dv_acc = dv_acc;
  // The leaves run first and cover every key row; on the tensor-core kernel one work item owns a key tile's whole
  // dK/dV there (leaves of up to 2048 rows), so it stores them and the two accumulators need no zero-fill.
  bool kv_init = false;
  {
    ha_attn_params probe = a;
    probe.mode = HA_MODE_FLASH;
    probe.flags = HA_FLAG_CAUSAL | (p.flags & HA_FLAG_FORCE_SIMT);
    probe.segs_per_head = 1 << p.levels;
    probe.span = pl.leaf; probe.m_q = pl.leaf; probe.m_k = pl.leaf;
    kv_init = pl.leaf <= 16 * TILE && !(p.flags & HA_FLAG_FORCE_SIMT) && p.kv_group <= 1 && tc_bwd_supported(probe);
  }
  HA_CUDA_OK(cudaMemsetAsync(dq_acc, 0, pl.rows * p.d * 4, st), "ha_causal_bwd memset");
  if (!kv_init) {
    HA_CUDA_OK(cudaMemsetAsync(dk_acc, 0, pl.rows_k * p.d * 4, st), "ha_causal_bwd memset");
    HA_CUDA_OK(cudaMemsetAsync(dv_acc, 0, pl.rows_k * p.dv * 4, st), "ha_causal_bwd memset");
  }
  // reference gradient convention: every part uses sum(o_part * dO) of its own output (its d(lse) is dropped);
  // exact convention: sum(o * dO) of the merged output, computed once
  bool fused_parts = false;
  if (p.keep_parts) {
    const int es = dtype_size(p.dtype), epc = 16 / es, lpr = p.dv / epc;
    if (p.dv % epc == 0 && (lpr == 2 || lpr == 4 || lpr == 8 || lpr == 16 || lpr == 32) && (uintptr_t)p.d_o % 16 == 0) {
      const long long part_stride = (uint8_t*)sv.part_o(1) - (uint8_t*)sv.part_o(0);
      const long long per_cta = 8LL * (32 / lpr) * 2;
      long long want = (pl.rows + per_cta - 1) / per_cta;
      const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
      if (p.dtype == HA_BF16)
        delta_parts_kernel<__nv_bfloat16, 8><<<grid, 256, 0, st>>>((const __nv_bfloat16*)p.d_o, (const uint8_t*)sv.part_o(0), part_stride, p.levels, p.n, lpr, delta, pl.rows, log2_if_pow2(p.n));
      else if (p.dtype == HA_FP16)
        delta_parts_kernel<__half, 8><<<grid, 256, 0, st>>>((const __half*)p.d_o, (const uint8_t*)sv.part_o(0), part_stride, p.levels, p.n, lpr, delta, pl.rows, log2_if_pow2(p.n));
      else
        delta_parts_kernel<float, 4><<<grid, 256, 0, st>>>((const float*)p.d_o, (const uint8_t*)sv.part_o(0), part_stride, p.levels, p.n, lpr, delta, pl.rows, log2_if_pow2(p.n));
      HA_LAUNCHED("ha_causal_bwd delta");
      fused_parts = true;
    }
  }
  auto part_delta = [&](int part) -> int {
    if (fused_parts) { a.delta = delta + (long long)part * pl.rows; return HA_OK; }
    if (!p.keep_parts && part != p.levels) return HA_OK;   // one delta from the merged output serves every part
    const void* o_src = p.keep_parts ? sv.part_o(part) : p.o;
    a.delta = delta;
    return ha_delta(o_src, a.o_sb, a.o_sh, a.o_sn, p.d_o, a.do_sb, a.do_sh, a.do_sn, p.B, p.H, p.n, p.dv, p.dtype, delta, stream);
  };
  rc = part_delta(p.levels);
  if (rc != HA_OK) return rc;
  a.mode = HA_MODE_FLASH;
  a.flags = HA_FLAG_CAUSAL | (p.flags & HA_FLAG_FORCE_SIMT) | (kv_init ? HA_FLAG_BWD_KV_INIT : 0);
  a.segs_per_head = 1 << p.levels;
  a.span = pl.leaf; a.q_off = 0; a.k_off = 0; a.m_q = pl.leaf; a.m_k = pl.leaf;
  rc = ha_attn_bwd(&a, stream);
  if (rc != HA_OK) return rc;
  for (int l = p.levels - 1; l >= 0; --l) {
    const int span = p.n >> l, m = span / 2;
    rc = part_delta(l);
    if (rc != HA_OK) return rc;
    const bool exact = deepest_exact(p, pl) && l == p.levels - 1;
    a.mode = exact ? HA_MODE_FLASH : HA_MODE_HYPER;
    a.flags = exact ? (p.flags & HA_FLAG_FORCE_SIMT) : (p.flags & (HA_FLAG_SMOOTH | HA_FLAG_BWD_REF_SMOOTH | HA_FLAG_FORCE_SIMT | HA_FLAG_NO_WS));
    a.segs_per_head = 1 << l;
    a.span = span; a.q_off = m; a.k_off = 0; a.m_q = m; a.m_k = m;
    a.q_idx = exact ? nullptr : sv.q_idx(l); a.k_idx = exact ? nullptr : sv.k_idx(l); a.sample_idx = nullptr;
    rc = ha_attn_bwd(&a, stream);
    if (rc != HA_OK) return rc;
  }
  rc = ha_cast_from_f32(dq_acc, p.dq, pl.rows * p.d, p.dtype, stream);
  if (rc != HA_OK) return rc;
  rc = ha_cast_from_f32(dk_acc, p.dk, pl.rows_k * p.d, p.dtype, stream);
  if (rc != HA_OK) return rc;
  return ha_cast_from_f32(dv_acc, p.dv_out, pl.rows_k * p.dv, p.dtype, stream);
}


/* ---------------------------------------------------------------------------------------------------------------
 * The non-causal module call (forward_no_causal_mask, hyper_attention.py:103-132, on sequences of at least min_seq_len)
 * as one call: hash q and k, sort both (one segmented sort over 2 B H rows), attention; and its backward: delta, the
 * backward kernel with whatever direct outputs it supports, the finishing pass.  Same parameter struct as the causal
 * schedule (levels, keep_parts, min_seq_len unused).
 * saved: q_idx | k_idx.  scratch: forward = codes of q and k + sort workspace; backward = delta + slot buffers / fp32
 * accumulators as the backward kernel needs them.
 * --------------------------------------------------------------------------------------------------------------- */
static int noncausal_check(const ha_causal_params& p, long long& rows, long long& rows_k) {
  if (p.dtype != HA_BF16 && p.dtype != HA_FP16 && p.dtype != HA_FP32) return HA_ERR_DTYPE;
  if (p.B <= 0 || p.H <= 0 || p.n <= 0 || p.d <= 0 || p.dv <= 0 || p.d > 256 || p.dv > 256) return HA_ERR_INVALID;
  if (p.lsh_bits < 1 || p.lsh_bits > 16 || p.n % TILE != 0) return HA_ERR_INVALID;
  if (p.sample_size < 0 || p.sample_size % TILE != 0 || p.sample_size > p.n || p.block_size < 1) return HA_ERR_INVALID;
  if (p.kv_group < 0 || (p.kv_group > 1 && p.H % p.kv_group != 0)) return HA_ERR_INVALID;
  rows = (long long)p.B * p.H * p.n;
  rows_k = p.kv_group > 1 ? rows / p.kv_group : rows;
  return HA_OK;
}

static void noncausal_attn(const ha_causal_params& p, ha_attn_params& a, long long rows) {
  fill_attn(p, a);
  a.mode = HA_MODE_HYPER;
  a.flags = p.flags & (HA_FLAG_SMOOTH | HA_FLAG_BWD_REF_SMOOTH | HA_FLAG_FORCE_SIMT | HA_FLAG_NO_WS);
  a.segs_per_head = 1;
  a.span = p.n; a.q_off = 0; a.k_off = 0; a.m_q = p.n; a.m_k = p.n;
  a.q_idx = (const int32_t*)p.saved;
  a.k_idx = (const int32_t*)((const uint8_t*)p.saved + align256(rows * 4));
}

// what the backward needs beyond delta: 2 = slot buffers only, 1 = slot buffers + fp32 dQ, 0 = three fp32 accumulators
static int noncausal_bwd_level(const ha_causal_params& p, long long rows) {
  ha_attn_params a;
  noncausal_attn(p, a, rows);
  float dummy = 0.f;
  a.delta = &dummy;                               // (only looked at for being there)
  a.dq_acc = a.dk_acc = a.dv_acc = nullptr;
  return p.dtype == HA_FP32 ? 0 : ha_attn_bwd_direct_level(&a);
}

int64_t ha_noncausal_saved_bytes(const ha_causal_params* p) {
  long long rows, rows_k;
  if (!p || noncausal_check(*p, rows, rows_k) != HA_OK) return -1;
  return 2 * align256(rows * 4);
}

int64_t ha_noncausal_scratch_bytes(const ha_causal_params* p, int32_t backward) {
  long long rows, rows_k;
  if (!p || noncausal_check(*p, rows, rows_k) != HA_OK) return -1;
  if (!backward) return 2 * align256(rows * 4) + align256(ha_seg_sort_workspace_bytes(2 * p->B * p->H, p->n, p->n, p->n, p->lsh_bits));
  const int level = noncausal_bwd_level(*p, rows);
  const long long sacc = align256((long long)p->B * p->H * p->sample_size * (p->d + p->dv) * 4);
  long long bytes = align256(rows * 4);
  if (level == 2) bytes += sacc;
  else if (level == 1) bytes += sacc + align256(rows * p->d * 4);
  else bytes += align256(rows * p->d * 4) + align256(rows_k * p->d * 4) + align256(rows_k * p->dv * 4);
  return bytes;
}

int ha_noncausal_fwd(const ha_causal_params* pp, void* stream) {
  if (!pp) return HA_ERR_INVALID;
  const ha_causal_params& p = *pp;
  long long rows, rows_k;
  int rc = noncausal_check(p, rows, rows_k);
  if (rc != HA_OK) return rc;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse || !p.proj) return HA_ERR_INVALID;
  if (!p.saved || p.saved_bytes < ha_noncausal_saved_bytes(pp)) return HA_ERR_WORKSPACE;
  if (!p.scratch || p.scratch_bytes < ha_noncausal_scratch_bytes(pp, 0)) return HA_ERR_WORKSPACE;
  // codes of q and k side by side: one segmented sort call covers both, and its output is q_idx | k_idx -- if the two
  // halves of `saved` are contiguous, which they are when rows * 4 is a multiple of 256 (n is a multiple of 128)
  int32_t* codes = (int32_t*)p.scratch;
  void* sort_ws = (uint8_t*)p.scratch + 2 * align256(rows * 4);
  const long long sort_ws_bytes = p.scratch_bytes - 2 * align256(rows * 4);
  const int64_t sn = p.d, sh = (int64_t)p.n * p.d, sb = sh * p.H;
  rc = ha_lsh_hash(p.q, sb, sh, sn, p.B, p.H, p.n, p.d, p.dtype, p.proj, p.lsh_bits, codes, stream);
  if (rc != HA_OK) return rc;
  const int Hk = p.kv_group > 1 ? p.H / p.kv_group : p.H;
  rc = ha_lsh_hash(p.k, sh * Hk, sh, sn, p.B, Hk, p.n, p.d, p.dtype, p.proj, p.lsh_bits, codes + rows, stream);
  if (rc != HA_OK) return rc;
  if (align256(rows * 4) == rows * 4 && Hk == p.H) {
    rc = ha_seg_sort(codes, 2 * p.B * p.H, p.n, p.n, 0, p.n, p.lsh_bits, (int32_t*)p.saved, sort_ws, sort_ws_bytes, stream);
  } else {
    rc = ha_seg_sort(codes, p.B * p.H, p.n, p.n, 0, p.n, p.lsh_bits, (int32_t*)p.saved, sort_ws, sort_ws_bytes, stream);
    if (rc == HA_OK)
      rc = ha_seg_sort(codes + rows, p.B * Hk, p.n, p.n, 0, p.n, p.lsh_bits, (int32_t*)((uint8_t*)p.saved + align256(rows * 4)), sort_ws,
                       sort_ws_bytes, stream);
  }
  if (rc != HA_OK) return rc;
  ha_attn_params a;
  noncausal_attn(p, a, rows);
  return ha_attn_fwd(&a, stream);
}

int ha_noncausal_bwd(const ha_causal_params* pp, void* stream) {
  if (!pp) return HA_ERR_INVALID;
  const ha_causal_params& p = *pp;
  long long rows, rows_k;
  int rc = noncausal_check(p, rows, rows_k);
  if (rc != HA_OK) return rc;
  if (!p.q || !p.k || !p.v || !p.o || !p.lse || !p.d_o || !p.dq || !p.dk || !p.dv_out) return HA_ERR_INVALID;
  if (!p.saved || p.saved_bytes < ha_noncausal_saved_bytes(pp)) return HA_ERR_WORKSPACE;
  if (!p.scratch || p.scratch_bytes < ha_noncausal_scratch_bytes(pp, 1)) return HA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* s = (uint8_t*)p.scratch;
  float* delta = (float*)s;                  s += align256(rows * 4);
  ha_attn_params a;
  noncausal_attn(p, a, rows);
  a.delta = delta;
  rc = ha_delta(p.o, a.o_sb, a.o_sh, a.o_sn, p.d_o, a.do_sb, a.do_sh, a.do_sn, p.B, p.H, p.n, p.dv, p.dtype, delta, stream);
  if (rc != HA_OK) return rc;
  const int level = noncausal_bwd_level(p, rows);
  if (level >= 1) {
    const long long segs = (long long)p.B * p.H;
    const long long sacc_bytes = segs * p.sample_size * (p.d + p.dv) * 4;
    a.dk_sacc = (float*)s;
    a.dv_sacc = a.dk_sacc + segs * p.sample_size * p.d;
    s += align256(sacc_bytes);
    if (sacc_bytes > 0) HA_CUDA_OK(cudaMemsetAsync(a.dk_sacc, 0, sacc_bytes, st), "ha_noncausal_bwd memset");
    a.dk_out = p.dk;
    a.dv_out = p.dv_out;
    if (level == 2) {
      a.dq_out = p.dq;
    } else {
      a.dq_acc = (float*)s;
      HA_CUDA_OK(cudaMemsetAsync(a.dq_acc, 0, rows * p.d * 4, st), "ha_noncausal_bwd memset");
    }
    rc = ha_attn_bwd(&a, stream);
    if (rc != HA_OK) return rc;
    rc = ha_attn_bwd_finish(&a, stream);
    if (rc != HA_OK) return rc;
    if (level == 1) rc = ha_cast_from_f32(a.dq_acc, p.dq, rows * p.d, p.dtype, stream);
    return rc;
  }
  a.dq_acc = (float*)s;                      s += align256(rows * p.d * 4);
  a.dk_acc = (float*)s;                      s += align256(rows_k * p.d * 4);
  a.dv_acc = (float*)s;
  HA_CUDA_OK(cudaMemsetAsync(a.dq_acc, 0, rows * p.d * 4, st), "ha_noncausal_bwd memset");
  HA_CUDA_OK(cudaMemsetAsync(a.dk_acc, 0, rows_k * p.d * 4, st), "ha_noncausal_bwd memset");
  HA_CUDA_OK(cudaMemsetAsync(a.dv_acc, 0, rows_k * p.dv * 4, st), "ha_noncausal_bwd memset");
  rc = ha_attn_bwd(&a, stream);
  if (rc != HA_OK) return rc;
  if (p.dtype == HA_FP32) {
    HA_CUDA_OK(cudaMemcpyAsync(p.dq, a.dq_acc, rows * p.d * 4, cudaMemcpyDeviceToDevice, st), "ha_noncausal_bwd copy");
    HA_CUDA_OK(cudaMemcpyAsync(p.dk, a.dk_acc, rows_k * p.d * 4, cudaMemcpyDeviceToDevice, st), "ha_noncausal_bwd copy");
    HA_CUDA_OK(cudaMemcpyAsync(p.dv_out, a.dv_acc, rows_k * p.dv * 4, cudaMemcpyDeviceToDevice, st), "ha_noncausal_bwd copy");
    return HA_OK;
  }
  rc = ha_cast_from_f32(a.dq_acc, p.dq, rows * p.d, p.dtype, stream);
  if (rc != HA_OK) return rc;
  rc = ha_cast_from_f32(a.dk_acc, p.dk, rows_k * p.d, p.dtype, stream);
  if (rc != HA_OK) return rc;
  return ha_cast_from_f32(a.dv_acc, p.dv_out, rows_k * p.dv, p.dtype, stream);
}

}  // extern "C"
