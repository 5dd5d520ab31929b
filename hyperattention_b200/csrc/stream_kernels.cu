// HBM-bound streaming kernels: angular LSH hash, row gather, delta (rowwise o.do), fp32->dtype cast, LSE merge.
#include "common.cuh"
#include "attn_index.cuh"

#include <mutex>
#include <string>
#include <type_traits>

namespace ha {

std::atomic<long long> g_launches{0};
static std::mutex g_err_mu;
static std::string g_err = "";
void set_cuda_error(cudaError_t e, const char* where) {
  std::lock_guard<std::mutex> lk(g_err_mu);
  g_err = std::string(where) + ": " + cudaGetErrorString(e);
}

// ---------------------------------------------------------------------------------------------------
// Angular LSH, vectorised path.  A row of d elements is read as LPR = d*sizeof(T)/16 chunks of 16 bytes by LPR
// neighbouring lanes; a lane keeps the projection rows of its chunk in registers (EPC x RP floats) for the whole
// kernel, accumulates EPC x RP fp32 FMAs per row in a fixed order, and the LPR partial sums are combined by a
// shuffle tree that leaves projection j's total on lane (j & 7) of the row's lane group.  A ballot then yields the
// binary code, c ^ (c >> 1) the Gray code.  Traffic: d*sizeof(T) + 4 bytes per row.
// ---------------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec16<__half> { static constexpr int N = 8; };

template <typename T> __device__ __forceinline__ void unpack16(const uint4& v, float (&f)[Vec16<T>::N]);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& v, float (&f)[4]) {
  f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& v, float (&f)[8]) {
  float2 a = unpack2<__nv_bfloat16>(v.x), b = unpack2<__nv_bfloat16>(v.y), c = unpack2<__nv_bfloat16>(v.z), d = unpack2<__nv_bfloat16>(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& v, float (&f)[8]) {
  float2 a = unpack2<__half>(v.x), b = unpack2<__half>(v.y), c = unpack2<__half>(v.z), d = unpack2<__half>(v.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// 8 partial sums on each of 8 neighbouring lanes -> lane (l & 7) holds the total of value (l & 7)
__device__ __forceinline__ float tree8(float (&a)[8], int lane) {
  const bool hi4 = lane & 4, hi2 = lane & 2, hi1 = lane & 1;
  float b[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float send = hi4 ? a[i] : a[i + 4];
    float recv = __shfl_xor_sync(0xffffffffu, send, 4);
    b[i] = (hi4 ? a[i + 4] : a[i]) + recv;
  }
  float c[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    float send = hi2 ? b[i] : b[i + 2];
    float recv = __shfl_xor_sync(0xffffffffu, send, 2);
    c[i] = (hi2 ? b[i + 2] : b[i]) + recv;
  }
  float send = hi1 ? c[0] : c[1];
  float recv = __shfl_xor_sync(0xffffffffu, send, 1);
  return (hi1 ? c[1] : c[0]) + recv;
}

template <typename T, int RP, int UNROLL>
__global__ void __launch_bounds__(256) lsh_hash_vec_kernel(const T* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int n,
                                                           int d, const float* __restrict__ proj, int r, int32_t* __restrict__ codes,
                                                           long long total_rows) {
  constexpr int EPC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int lpr = d / EPC;            // lanes per row: 8, 16 or 32
  const int rpw = 32 / lpr;           // rows per warp step
  const int chunk = lane % lpr;
  const int sub = lane / lpr;
  float pr[EPC][RP];
#pragma unroll
  for (int e = 0; e < EPC; ++e)
#pragma unroll
    for (int j = 0; j < RP; ++j) pr[e][j] = j < r ? proj[(chunk * EPC + e) * r + j] : 0.f;

  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long step = (long long)rpw * UNROLL;
  for (long long base = warp_id * step; base < total_rows; base += n_warps * step) {
    uint4 v[UNROLL];
    long long row[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      row[u] = base + u * rpw + sub;
      v[u] = make_uint4(0, 0, 0, 0);
      if (row[u] < total_rows) {
        long long bh = row[u] / n;
        int i = (int)(row[u] - bh * n);
        const T* p = x + (bh / H) * sb + (bh % H) * sh + (long long)i * sn + chunk * EPC;
        v[u] = __ldg(reinterpret_cast<const uint4*>(p));
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float f[EPC];
      unpack16<T>(v[u], f);
      uint32_t code = 0;
#pragma unroll
      for (int half = 0; half < RP / 8; ++half) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int e = 0; e < EPC; ++e)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = fmaf(f[e], pr[e][half * 8 + j], acc[j]);
        for (int off = lpr >> 1; off >= 8; off >>= 1)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
        float tot = tree8(acc, lane);
        uint32_t ball = __ballot_sync(0xffffffffu, tot > 0.f);
        code |= ((ball >> (sub * lpr)) & 0xFFu) << (8 * half);
      }
      if (chunk == 0 && row[u] < total_rows) codes[row[u]] = (int32_t)(code ^ (code >> 1));
    }
  }
}


// ---------------------------------------------------------------------------------------------------
// Angular LSH for 16-bit inputs on the tensor cores (mma.sync m16n8k16, fp32 accumulate; products of two bf16/fp16
// values are exact in fp32, so the result equals an fp32 dot product up to summation order).  A warp takes 16 rows at
// a time; thread (g = lane/4, t = lane%4) reads 16 bytes of rows g and g+8 per 32-column chunk and feeds them to two
// MMAs as the A fragment.  The MMA's k index is only a summation label, so instead of shuffling the 16 bytes into
// the canonical fragment order, the projection rows are permuted once, at kernel start, into the matching order of
// the B fragment (8 registers per 64 columns, resident for the whole kernel).  N = 8 projections per MMA; a second
// set of B fragments covers projections 8..15.  Sign bits come out of four ballots per 16 rows.
// Per 16 rows and 64 columns: 4 x LDG.128 per thread, 4 MMAs, 4 ballots -> HBM-bound.
// ---------------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t spread4(uint32_t x) {   // bit i -> bit 2i, i < 4
  return (x & 1u) | ((x & 2u) << 1) | ((x & 4u) << 2) | ((x & 8u) << 3);
}

// CH = d / 32 column chunks; NSET = 1 (r <= 8) or 2 (r <= 16)
template <typename T, int CH, int NSET, int UNROLL>
__global__ void __launch_bounds__(256, 4) lsh_hash_mma_kernel(const T* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int n,
                                                           const float* __restrict__ proj, int r, int32_t* __restrict__ codes,
                                                           long long total_rows) {
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // B fragments: for chunk c, MMA m (0/1), register j (0/1): projection column (set*8 + g), rows c*32 + 8t + 4m + 2j + {0,1}
  uint32_t bf[NSET][CH][2][2];
#pragma unroll
  for (int set = 0; set < NSET; ++set)
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int col = set * 8 + g;
          const int row = c * 32 + 8 * t + 4 * m + 2 * j;
          const float lo = col < r ? proj[row * r + col] : 0.f;
          const float hi = col < r ? proj[(row + 1) * r + col] : 0.f;
          bf[set][c][m][j] = pack2<T>(lo, hi);
        }
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long step = 16LL * UNROLL;
  for (long long base = warp_id * step; base < total_rows; base += n_warps * step) {
    uint4 v[UNROLL][2][CH];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        const long long row = base + u * 16 + g + 8 * hrow;
        const bool ok = row < total_rows;
        const long long bh = ok ? row / n : 0;
        const int i = ok ? (int)(row - bh * n) : 0;
        const T* p = x + (bh / H) * sb + (bh % H) * sh + (long long)i * sn + 8 * t;
#pragma unroll
        for (int c = 0; c < CH; ++c) v[u][hrow][c] = ok ? __ldg(reinterpret_cast<const uint4*>(p + 32 * c)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      uint32_t code_lo = 0, code_hi = 0;   // codes of rows g and g+8
#pragma unroll
      for (int set = 0; set < NSET; ++set) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const uint4 lo = v[u][0][c], hi = v[u][1][c];
          const uint32_t a0[4] = {lo.x, hi.x, lo.y, hi.y};   // k-slots {2t,2t+1} and {2t+8,2t+9} of rows g / g+8
          const uint32_t a1[4] = {lo.z, hi.z, lo.w, hi.w};
          mma16816<T>(acc, a0, bf[set][c][0]);
          mma16816<T>(acc, a1, bf[set][c][1]);
        }
        // acc[0], acc[1]: row g, projections 2t, 2t+1;  acc[2], acc[3]: row g+8
        const uint32_t b0 = __ballot_sync(0xffffffffu, acc[0] > 0.f), b1 = __ballot_sync(0xffffffffu, acc[1] > 0.f);
        const uint32_t b2 = __ballot_sync(0xffffffffu, acc[2] > 0.f), b3 = __ballot_sync(0xffffffffu, acc[3] > 0.f);
        const int sh4 = 4 * g;
        code_lo |= (spread4((b0 >> sh4) & 0xFu) | (spread4((b1 >> sh4) & 0xFu) << 1)) << (8 * set);
        code_hi |= (spread4((b2 >> sh4) & 0xFu) | (spread4((b3 >> sh4) & 0xFu) << 1)) << (8 * set);
      }
      if (t == 0) {
        const long long row = base + u * 16 + g;
        if (row < total_rows) codes[row] = (int32_t)(code_lo ^ (code_lo >> 1));
        if (row + 8 < total_rows) codes[row + 8] = (int32_t)(code_hi ^ (code_hi >> 1));
      }
    }
  }
}

template <typename T, int CH>
static void launch_hash_mma(const T* x, int64_t sb, int64_t sh, int64_t sn, int H, int n, const float* proj, int r, int32_t* codes,
                            long long total, cudaStream_t st) {
  constexpr int UNROLL = CH <= 2 ? 2 : 1;   // 64 registers -> four CTAs (32 warps) per SM, each with its loads in flight
  const long long rows_per_cta = 8LL * 16 * UNROLL;
  long long want = (total + rows_per_cta - 1) / rows_per_cta;
  const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
  if (r <= 8)
    lsh_hash_mma_kernel<T, CH, 1, UNROLL><<<grid, 256, 0, st>>>(x, sb, sh, sn, H, n, proj, r, codes, total);
  else
    lsh_hash_mma_kernel<T, CH, 2, UNROLL><<<grid, 256, 0, st>>>(x, sb, sh, sn, H, n, proj, r, codes, total);
}

// Generic path (any d <= 256, any element alignment): one warp per row, lane-strided elements.
template <typename T>
__global__ void __launch_bounds__(256) lsh_hash_generic_kernel(const T* __restrict__ x, int64_t sb, int64_t sh, int64_t sn, int H, int n,
                                                               int d, const float* __restrict__ proj, int r, int32_t* __restrict__ codes,
                                                               long long total_rows) {
  extern __shared__ float sproj[];
  for (int i = threadIdx.x; i < d * r; i += blockDim.x) sproj[i] = proj[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp_id; row < total_rows; row += n_warps) {
    long long bh = row / n;
    int i = (int)(row - bh * n);
    const T* p = x + (bh / H) * sb + (bh % H) * sh + (long long)i * sn;
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    for (int e = lane; e < d; e += 32) {
      float xv = to_f32<T>(p[e]);
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < r) acc[j] = fmaf(xv, sproj[e * r + j], acc[j]);
    }
    uint32_t code = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if (j < r) {
        float s = acc[j];
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        code |= (s > 0.f ? 1u : 0u) << j;
      }
    }
    if (lane == 0) codes[row] = (int32_t)(code ^ (code >> 1));
  }
}

template <typename T>
static int launch_hash(const void* x, int64_t sb, int64_t sh, int64_t sn, int B, int H, int n, int d, const float* proj, int r,
                       int32_t* codes, cudaStream_t st) {
  const long long total = (long long)B * H * n;
  if (total == 0) return HA_OK;
  constexpr int EPC = Vec16<T>::N;
  const int lpr = d / EPC;
  const bool vec_ok = (d % EPC == 0) && (lpr == 4 || lpr == 8 || lpr == 16 || lpr == 32) && (sb % EPC == 0) && (sh % EPC == 0) &&
                      (sn % EPC == 0) && ((uintptr_t)x % 16 == 0);
  int sms = 148;
  if constexpr (!std::is_same<T, float>::value) {
    // tensor-core path: 16-byte aligned rows, d a multiple of 32 up to 128.  The projection is rounded to the input
    // dtype, which is the dtype the reference requires it to have (src/angular_lsh_triton.py:104).
    if (vec_ok && (d == 32 || d == 64 || d == 128)) {
      if (d == 32) launch_hash_mma<T, 1>((const T*)x, sb, sh, sn, H, n, proj, r, codes, total, st);
      else if (d == 64) launch_hash_mma<T, 2>((const T*)x, sb, sh, sn, H, n, proj, r, codes, total, st);
      else launch_hash_mma<T, 4>((const T*)x, sb, sh, sn, H, n, proj, r, codes, total, st);
      HA_LAUNCHED("ha_lsh_hash");
      return HA_OK;
    }
  }
  if (vec_ok && lpr >= 8) {
    const int rows_per_cta = 8 * (32 / lpr) * 4;
    long long want = (total + rows_per_cta - 1) / rows_per_cta;
    int grid = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    if (r <= 8)
      lsh_hash_vec_kernel<T, 8, 4><<<grid, 256, 0, st>>>((const T*)x, sb, sh, sn, H, n, d, proj, r, codes, total);
    else
      lsh_hash_vec_kernel<T, 16, 2><<<grid, 256, 0, st>>>((const T*)x, sb, sh, sn, H, n, d, proj, r, codes, total);
  } else {
    long long want = (total + 7) / 8;
    int grid = (int)(want < (long long)sms * 8 ? want : (long long)sms * 8);
    lsh_hash_generic_kernel<T><<<grid, 256, d * r * sizeof(float), st>>>((const T*)x, sb, sh, sn, H, n, d, proj, r, codes, total);
  }
  HA_LAUNCHED("ha_lsh_hash");
  return HA_OK;
}

// ---------------------------------------------------------------------------------------------------
// Row gather: one 16-byte chunk per thread when rows allow it, element-wise otherwise.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gather_rows_vec_kernel(const uint8_t* __restrict__ src, int64_t sb_bytes, int64_t sh_bytes,
                                                              int64_t sn_bytes, int H, int chunks_per_row, const int32_t* __restrict__ idx,
                                                              int n_idx, uint8_t* __restrict__ dst, long long total_chunks) {
  constexpr int UN = 4;   // independent copies in flight per thread
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; t0 < total_chunks; t0 += stride * UN) {
    uint4 v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const long long t = t0 + u * stride;
      v[u] = make_uint4(0, 0, 0, 0);
      if (t < total_chunks) {
        const long long orow = t / chunks_per_row;
        const int c = (int)(t - orow * chunks_per_row);
        const long long bh = orow / n_idx;
        const int srow = __ldg(idx + orow);
        v[u] = __ldg(reinterpret_cast<const uint4*>(src + (bh / H) * sb_bytes + (bh % H) * sh_bytes + (long long)srow * sn_bytes) + c);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const long long t = t0 + u * stride;
      if (t < total_chunks) reinterpret_cast<uint4*>(dst)[t] = v[u];
    }
  }
}
template <typename T>
__global__ void __launch_bounds__(256) gather_rows_elem_kernel(const T* __restrict__ src, int64_t sb, int64_t sh, int64_t sn, int H, int width,
                                                               const int32_t* __restrict__ idx, int n_idx, T* __restrict__ dst,
                                                               long long total) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    long long orow = t / width;
    int c = (int)(t - orow * width);
    long long bh = orow / n_idx;
    dst[t] = src[(bh / H) * sb + (bh % H) * sh + (long long)idx[orow] * sn + c];
  }
}

// ---------------------------------------------------------------------------------------------------
// delta = rowwise sum(o * do); one warp per row
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) delta_kernel(const T* __restrict__ o, int64_t osb, int64_t osh, int64_t osn, const T* __restrict__ go,
                                                    int64_t gsb, int64_t gsh, int64_t gsn, int H, int n, int dv, float* __restrict__ delta,
                                                    long long total_rows) {
  const int lane = threadIdx.x & 31;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp_id; row < total_rows; row += n_warps) {
    long long bh = row / n;
    int i = (int)(row - bh * n);
    const T* po = o + (bh / H) * osb + (bh % H) * osh + (long long)i * osn;
    const T* pg = go + (bh / H) * gsb + (bh % H) * gsh + (long long)i * gsn;
    float s = 0.f;
    for (int e = lane; e < dv; e += 32) s = fmaf(to_f32<T>(po[e]), to_f32<T>(pg[e]), s);
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) delta[row] = s;
  }
}


// delta, vectorised: rows of dv elements read as 16-byte chunks, LPR = dv*sizeof(T)/16 lanes per row.
template <typename T>
__global__ void __launch_bounds__(256) delta_vec_kernel(const T* __restrict__ o, int64_t osb, int64_t osh, int64_t osn, const T* __restrict__ go,
                                                        int64_t gsb, int64_t gsh, int64_t gsn, int H, int n, int lpr, float* __restrict__ delta,
                                                        long long total_rows) {
  constexpr int EPC = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int rpw = 32 / lpr, chunk = lane % lpr, sub = lane / lpr;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  constexpr int UN = 4;
  for (long long base = warp_id * rpw * UN; base < total_rows; base += n_warps * rpw * UN) {
    uint4 a[UN], b[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const long long row = base + u * rpw + sub;
      a[u] = b[u] = make_uint4(0, 0, 0, 0);
      if (row < total_rows) {
        const long long bh = row / n;
        const int i = (int)(row - bh * n);
        a[u] = __ldg(reinterpret_cast<const uint4*>(o + (bh / H) * osb + (bh % H) * osh + (long long)i * osn + chunk * EPC));
        b[u] = __ldg(reinterpret_cast<const uint4*>(go + (bh / H) * gsb + (bh % H) * gsh + (long long)i * gsn + chunk * EPC));
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      float fa[EPC], fb[EPC];
      unpack16<T>(a[u], fa);
      unpack16<T>(b[u], fb);
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < EPC; ++e) s = fmaf(fa[e], fb[e], s);
      for (int off = lpr >> 1; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      const long long row = base + u * rpw + sub;
      if (chunk == 0 && row < total_rows) delta[row] = s;
    }
  }
}

template <typename T>
static bool launch_delta_vec(const void* o, int64_t osb, int64_t osh, int64_t osn, const void* go, int64_t gsb, int64_t gsh, int64_t gsn,
                             int H, int n, int dv, float* delta, long long rows, cudaStream_t st) {
  constexpr int EPC = Vec16<T>::N;
  const int lpr = dv / EPC;
  const bool ok = dv % EPC == 0 && (lpr == 2 || lpr == 4 || lpr == 8 || lpr == 16 || lpr == 32) && osb % EPC == 0 && osh % EPC == 0 &&
                  osn % EPC == 0 && gsb % EPC == 0 && gsh % EPC == 0 && gsn % EPC == 0 && (uintptr_t)o % 16 == 0 && (uintptr_t)go % 16 == 0;
  if (!ok) return false;
  const long long per_cta = 8LL * (32 / lpr) * 4;
  long long want = (rows + per_cta - 1) / per_cta;
  const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
  delta_vec_kernel<T><<<grid, 256, 0, st>>>((const T*)o, osb, osh, osn, (const T*)go, gsb, gsh, gsn, H, n, lpr, delta, rows);
  return true;
}

template <typename T>
__global__ void __launch_bounds__(256) cast_kernel(const float* __restrict__ src, T* __restrict__ dst, long long count) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < count; t += (long long)gridDim.x * blockDim.x)
    dst[t] = from_f32<T>(src[t]);
}

// ---------------------------------------------------------------------------------------------------
// LSE merge of two partial attentions, in place into (o1, lse1); one warp per row.
//   reference form: c = round_T(1 / (1 + exp(lse2 - lse1))); o = c*o1 + (1-c)*o2; lse = lse1 - log(c + eps_f32)
//   exact form:     lse = logaddexp(lse1, lse2); o = o1*exp(lse1-lse) + o2*exp(lse2-lse)
// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) merge_kernel(T* __restrict__ o1, float* __restrict__ lse1, const T* __restrict__ o2,
                                                    const float* __restrict__ lse2, long long rows, int dv, int exact) {
  const int lane = threadIdx.x & 31;
  const long long warp_id = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp_id; row < rows; row += n_warps) {
    float l1 = lse1[row], l2 = lse2[row];
    float w1, w2, ln;
    if (exact) {
      float m = fmaxf(l1, l2);
      if (m == -INFINITY) { w1 = 0.5f; w2 = 0.5f; ln = m; }
      else {
        float e1 = __expf(l1 - m), e2 = __expf(l2 - m);
        w1 = e1 / (e1 + e2); w2 = e2 / (e1 + e2);
        ln = m + __logf(e1 + e2);
      }
    } else {
      float c = round_to<T>(1.f / (1.f + expf(l2 - l1)));
      w1 = c; w2 = round_to<T>(1.f - c);
      ln = l1 - logf(c + 1.1920929e-07f);
    }
    for (int e = lane; e < dv; e += 32) {
      float a = to_f32<T>(o1[row * dv + e]), b = to_f32<T>(o2[row * dv + e]);
      o1[row * dv + e] = from_f32<T>(w1 * a + w2 * b);
    }
    __syncwarp();
    if (lane == 0) lse1[row] = ln;
  }
}

static inline int grid_for(long long items, int per_cta) {
  long long want = (items + per_cta - 1) / per_cta;
  long long cap = 148LL * 16;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace ha

using namespace ha;


// ---------------------------------------------------------------------------------------------------
// Weights of uniformly sampled key columns: inverse key permutation, then per query tile the dropped slots
// (keys already inside the tile's block window) and the log importance weight of the kept ones.
// ---------------------------------------------------------------------------------------------------
__global__ void invert_perm_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ inv, int m, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long seg = i / m;
  inv[seg * m + idx[i]] = (int32_t)(i - seg * m);
}

__global__ void __launch_bounds__(128) sample_weights_kernel(const int32_t* __restrict__ inv, const int32_t* __restrict__ sample_idx,
                                                             int m, int bs, int S, int smooth, float* __restrict__ tile_logw,
                                                             uint32_t* __restrict__ tile_mask) {
  const int t = blockIdx.x, T_ = gridDim.x;
  const long long seg = blockIdx.y;
  const ha::Window w = ha::block_window(t, bs, m, smooth != 0);
  int kept = 0;
  for (int s0 = 0; s0 < S; s0 += 128) {           // S is a multiple of 128: every thread makes every trip
    const int s = s0 + threadIdx.x;
    const int row = sample_idx ? sample_idx[seg * S + s] : s;
    int off = inv[seg * m + row] - w.first;
    if (off < 0) off += m;
    const bool dropped = off < w.count;
    const unsigned bits = __ballot_sync(0xffffffffu, dropped);
    if ((threadIdx.x & 31) == 0) tile_mask[(seg * T_ + t) * (S / 32) + (s >> 5)] = bits;
    kept += __syncthreads_count(!dropped);
  }
  if (threadIdx.x == 0) tile_logw[seg * T_ + t] = kept > 0 ? logf((float)(m - w.count) / (float)kept) : -INFINITY;
}

extern "C" {

const char* ha_version(void) { return "hyperattn_b200 0.1 (sm_100a)"; }
const char* ha_last_cuda_error(void) {
  static thread_local std::string copy;
  std::lock_guard<std::mutex> lk(g_err_mu);
  copy = g_err;
  return copy.c_str();
}
int64_t ha_launch_count(void) { return (int64_t)g_launches.load(); }

int ha_lsh_hash(const void* x, int64_t sb, int64_t sh, int64_t sn, int32_t B, int32_t H, int32_t n, int32_t d, int32_t dtype,
                const float* proj, int32_t r, int32_t* codes, void* stream) {
  if (B < 0 || H < 0 || n < 0 || d <= 0 || d > 256 || r < 1 || r > 16) return HA_ERR_INVALID;
  if ((long long)B * H * n == 0) return HA_OK;
  if (!x || !proj || !codes) return HA_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case HA_BF16: return launch_hash<__nv_bfloat16>(x, sb, sh, sn, B, H, n, d, proj, r, codes, st);
    case HA_FP16: return launch_hash<__half>(x, sb, sh, sn, B, H, n, d, proj, r, codes, st);
    case HA_FP32: return launch_hash<float>(x, sb, sh, sn, B, H, n, d, proj, r, codes, st);
  }
  return HA_ERR_DTYPE;
}

int ha_gather_rows(const void* src, int64_t sb, int64_t sh, int64_t sn, int32_t B, int32_t H, int32_t width, int32_t dtype,
                   const int32_t* idx, int32_t n_idx, void* dst, void* stream) {
  if (!src || !idx || !dst || width <= 0 || B < 0 || H < 0 || n_idx < 0) return HA_ERR_INVALID;
  if (dtype != HA_BF16 && dtype != HA_FP16 && dtype != HA_FP32) return HA_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int es = dtype_size(dtype);
  const long long rows = (long long)B * H * n_idx;
  if (rows == 0) return HA_OK;
  const bool vec = (width * es) % 16 == 0 && (sb * es) % 16 == 0 && (sh * es) % 16 == 0 && (sn * es) % 16 == 0 &&
                   (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0;
  if (vec) {
    const int cpr = width * es / 16;
    const long long total = rows * cpr;
    gather_rows_vec_kernel<<<grid_for(total, 256 * 4), 256, 0, st>>>((const uint8_t*)src, sb * es, sh * es, sn * es, H, cpr, idx, n_idx,
                                                                    (uint8_t*)dst, total);
  } else {
    const long long total = rows * width;
    if (es == 2)
      gather_rows_elem_kernel<uint16_t><<<grid_for(total, 256 * 4), 256, 0, st>>>((const uint16_t*)src, sb, sh, sn, H, width, idx, n_idx,
                                                                                 (uint16_t*)dst, total);
    else
      gather_rows_elem_kernel<uint32_t><<<grid_for(total, 256 * 4), 256, 0, st>>>((const uint32_t*)src, sb, sh, sn, H, width, idx, n_idx,
                                                                                 (uint32_t*)dst, total);
  }
  HA_LAUNCHED("ha_gather_rows");
  return HA_OK;
}

int ha_delta(const void* o, int64_t osb, int64_t osh, int64_t osn, const void* go, int64_t gsb, int64_t gsh, int64_t gsn, int32_t B,
             int32_t H, int32_t n, int32_t dv, int32_t dtype, float* delta, void* stream) {
  if (!o || !go || !delta || dv <= 0) return HA_ERR_INVALID;
  cudaStream_t st = (cudaStream_t)stream;
  const long long rows = (long long)B * H * n;
  if (rows == 0) return HA_OK;
  bool done = false;
  switch (dtype) {
    case HA_BF16: done = launch_delta_vec<__nv_bfloat16>(o, osb, osh, osn, go, gsb, gsh, gsn, H, n, dv, delta, rows, st); break;
    case HA_FP16: done = launch_delta_vec<__half>(o, osb, osh, osn, go, gsb, gsh, gsn, H, n, dv, delta, rows, st); break;
    case HA_FP32: done = launch_delta_vec<float>(o, osb, osh, osn, go, gsb, gsh, gsn, H, n, dv, delta, rows, st); break;
    default: return HA_ERR_DTYPE;
  }
  if (done) {
    HA_LAUNCHED("ha_delta");
    return HA_OK;
  }
  const int grid = grid_for(rows, 8);
  switch (dtype) {
    case HA_BF16: delta_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)o, osb, osh, osn, (const __nv_bfloat16*)go, gsb, gsh, gsn, H, n, dv, delta, rows); break;
    case HA_FP16: delta_kernel<__half><<<grid, 256, 0, st>>>((const __half*)o, osb, osh, osn, (const __half*)go, gsb, gsh, gsn, H, n, dv, delta, rows); break;
    case HA_FP32: delta_kernel<float><<<grid, 256, 0, st>>>((const float*)o, osb, osh, osn, (const float*)go, gsb, gsh, gsn, H, n, dv, delta, rows); break;
    default: return HA_ERR_DTYPE;
  }
  HA_LAUNCHED("ha_delta");
  return HA_OK;
}

int ha_cast_from_f32(const float* src, void* dst, int64_t count, int32_t dtype, void* stream) {
  if (!src || !dst || count < 0) return HA_ERR_INVALID;
  if (count == 0) return HA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for(count, 256 * 8);
  switch (dtype) {
    case HA_BF16: cast_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(src, (__nv_bfloat16*)dst, count); break;
    case HA_FP16: cast_kernel<__half><<<grid, 256, 0, st>>>(src, (__half*)dst, count); break;
    case HA_FP32: cast_kernel<float><<<grid, 256, 0, st>>>(src, (float*)dst, count); break;
    default: return HA_ERR_DTYPE;
  }
  HA_LAUNCHED("ha_cast_from_f32");
  return HA_OK;
}

int ha_lse_merge(void* o1, float* lse1, const void* o2, const float* lse2, int64_t rows, int32_t dv, int32_t dtype, int32_t exact,
                 void* stream) {
  if (!o1 || !lse1 || !o2 || !lse2 || rows < 0 || dv <= 0) return HA_ERR_INVALID;
  if (rows == 0) return HA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for(rows, 8);
  switch (dtype) {
    case HA_BF16: merge_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((__nv_bfloat16*)o1, lse1, (const __nv_bfloat16*)o2, lse2, rows, dv, exact); break;
    case HA_FP16: merge_kernel<__half><<<grid, 256, 0, st>>>((__half*)o1, lse1, (const __half*)o2, lse2, rows, dv, exact); break;
    case HA_FP32: merge_kernel<float><<<grid, 256, 0, st>>>((float*)o1, lse1, (const float*)o2, lse2, rows, dv, exact); break;
    default: return HA_ERR_DTYPE;
  }
  HA_LAUNCHED("ha_lse_merge");
  return HA_OK;
}

int ha_sample_weights(const int32_t* k_idx, const int32_t* sample_idx, int32_t segs, int32_t m, int32_t block_size,
                      int32_t sample_size, int32_t smooth, int32_t* inv_workspace, float* tile_logw, uint32_t* tile_mask,
                      void* stream) {
  if (segs < 0 || m < 0 || block_size <= 0 || sample_size < 0) return HA_ERR_INVALID;
  if (m % TILE || sample_size % TILE || sample_size > m) return HA_ERR_INVALID;
  if (segs == 0 || m == 0 || sample_size == 0) return HA_OK;
  if (!k_idx || !inv_workspace || !tile_logw || !tile_mask) return HA_ERR_INVALID;
  if (segs > 65535) return HA_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)segs * m;
  if ((total + 255) / 256 > 0x7fffffffLL) return HA_ERR_TOO_LARGE;
  invert_perm_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(k_idx, inv_workspace, m, total);
  HA_LAUNCHED("ha_sample_weights (invert)");
  sample_weights_kernel<<<dim3(m / TILE, segs), 128, 0, st>>>(inv_workspace, sample_idx, m, (block_size + TILE - 1) / TILE,
                                                             sample_size, smooth, tile_logw, tile_mask);
  HA_LAUNCHED("ha_sample_weights");
  return HA_OK;
}

}  // extern "C"
