// Index arithmetic shared by every attention kernel (CUDA-core and tensor-core): which rows a segment owns and
// which sorted key positions a query tile pairs with.
#pragma once
#include "common.cuh"

namespace ha {

struct SegInfo {
  long long q_row0, k_row0;   // first query / key row of the segment inside its head (in rows)
  long long khead0;           // first row of the segment's K/V head in a contiguous [B, H_kv, n, *] tensor (dK/dV accumulators)
  int b, h;
  int hk;                     // K/V head: h, or h / kv_group with grouped-query attention
};

__device__ __forceinline__ SegInfo seg_info(const ha_attn_params& p, int seg) {
  SegInfo s;
  const int bh = seg / p.segs_per_head, part = seg - bh * p.segs_per_head;
  s.b = bh / p.H;
  s.h = bh - s.b * p.H;
  s.q_row0 = (long long)part * p.span + p.q_off;
  s.k_row0 = (long long)part * p.span + p.k_off;
  const int g = p.kv_group > 1 ? p.kv_group : 1;
  s.hk = s.h / g;
  s.khead0 = ((long long)s.b * (p.H / g) + s.hk) * p.n;
  return s;
}

// Index of segment `seg` on the key side (rows of k_idx / sample_idx): the same segment of the K/V head.
__device__ __forceinline__ long long kseg_of(const ha_attn_params& p, long long seg) {
  if (p.kv_group <= 1) return seg;
  const long long bh = seg / p.segs_per_head, part = seg - bh * p.segs_per_head;
  const long long b = bh / p.H, h = bh - b * p.H;
  return (b * (p.H / p.kv_group) + h / p.kv_group) * p.segs_per_head + part;
}

// Block window of a 128-row tile t of one side (hyper mode, m rows per side, W = block size rounded up to tiles):
// the other side's sorted positions are (first + j) mod m for j in [0, count).
//   plain:  first = beta*W                       (src/hyper_attn_triton.py:104-108)
//   smooth: first = 128*t - 64*(bs-1) (mod m)    (:102, :106)
// count = min(W, m - beta*W): the reference's loop stops at the end of the sequence (:103-104).
struct Window { int first, count; };
__device__ __forceinline__ Window block_window(int t, int bs, int m, bool smooth) {
  const int W = bs * TILE;
  const int beta = t / bs;
  Window w;
  w.count = min(W, m - beta * W);
  if (smooth) {
    int f = (TILE * t - (TILE / 2) * (bs - 1)) % m;
    w.first = f < 0 ? f + m : f;
  } else {
    w.first = beta * W;
  }
  return w;
}

}  // namespace ha
