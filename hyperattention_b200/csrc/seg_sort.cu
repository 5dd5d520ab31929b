// Segmented stable argsort of small integer keys (LSH bucket codes) by counting sort.
//
// The keys have at most 16 significant bits (8 by default), so a stable sort is one counting pass per 8-bit digit:
//   hist    : every warp counts the 256 digit values of its sub-chunk (SUB consecutive keys of one segment)
//   scan    : per segment, exclusive prefix over (digit value major, sub-chunk minor) -> start of every
//             (sub-chunk, digit value) run in the output
//   scatter : every warp walks its sub-chunk in order, 32 keys at a time; a key's output slot is the run start plus
//             the number of equal keys before it (match_any + popc within the warp step, a running counter across
//             steps), which keeps ties in original order.
// Traffic per digit pass: keys read twice (4 B each) + one 4 B index written, plus 1 KB of counters per sub-chunk.
#include "common.cuh"

#include <mutex>

namespace ha {

constexpr int SUB = 1024;          // keys per warp
constexpr int WARPS = 8;           // warps per CTA

__device__ __forceinline__ int load_key(const int32_t* __restrict__ seg_codes, const int32_t* __restrict__ idx_in, int i, int shift) {
  int src = idx_in ? idx_in[i] : i;
  return (seg_codes[src] >> shift) & 0xFF;
}

// grid: (ceil(n_sub / WARPS), n_segs)
__global__ void __launch_bounds__(WARPS * 32) sort_hist_kernel(const int32_t* __restrict__ codes, int n, int span, int seg_off, int seg_len,
                                                              int parts, int n_sub, int shift, const int32_t* __restrict__ idx_in,
                                                              uint32_t* __restrict__ hist) {
  __shared__ uint32_t h[WARPS][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = blockIdx.x * WARPS + warp;
  const int seg = blockIdx.y;
  for (int b = lane; b < 256; b += 32) h[warp][b] = 0;
  __syncwarp();
  if (sub < n_sub) {
    const int32_t* seg_codes = codes + (long long)(seg / parts) * n + (long long)(seg % parts) * span + seg_off;
    const int32_t* seg_idx = idx_in ? idx_in + (long long)seg * seg_len : nullptr;
    const int begin = sub * SUB, end = min(seg_len, begin + SUB);
    for (int i = begin + lane; i < end; i += 32) atomicAdd(&h[warp][load_key(seg_codes, seg_idx, i, shift)], 1u);
    __syncwarp();
    uint32_t* out = hist + ((long long)seg * n_sub + sub) * 256;
    for (int b = lane; b < 256; b += 32) out[b] = h[warp][b];
  }
}

// grid: n_segs, 256 threads (one per digit value)
__global__ void __launch_bounds__(256) sort_scan_kernel(uint32_t* __restrict__ hist, int n_sub) {
  __shared__ uint32_t totals[256];
  const int b = threadIdx.x;
  uint32_t* h = hist + (long long)blockIdx.x * n_sub * 256;
  uint32_t run = 0;
  for (int s = 0; s < n_sub; ++s) {
    uint32_t c = h[s * 256 + b];
    h[s * 256 + b] = run;
    run += c;
  }
  totals[b] = run;
  __syncthreads();
  // exclusive scan of 256 totals (Hillis-Steele on shared memory)
  uint32_t mine = run;
  for (int off = 1; off < 256; off <<= 1) {
    uint32_t add = b >= off ? totals[b - off] : 0;
    __syncthreads();
    totals[b] += add;
    __syncthreads();
  }
  const uint32_t base = totals[b] - mine;
  for (int s = 0; s < n_sub; ++s) h[s * 256 + b] += base;
}

__global__ void __launch_bounds__(WARPS * 32) sort_scatter_kernel(const int32_t* __restrict__ codes, int n, int span, int seg_off, int seg_len,
                                                                 int parts, int n_sub, int shift, const int32_t* __restrict__ idx_in,
                                                                 const uint32_t* __restrict__ hist, int32_t* __restrict__ idx_out) {
  __shared__ uint32_t off[WARPS][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = blockIdx.x * WARPS + warp;
  const int seg = blockIdx.y;
  if (sub >= n_sub) return;
  const uint32_t* hin = hist + ((long long)seg * n_sub + sub) * 256;
  for (int b = lane; b < 256; b += 32) off[warp][b] = hin[b];
  __syncwarp();
  const int32_t* seg_codes = codes + (long long)(seg / parts) * n + (long long)(seg % parts) * span + seg_off;
  const int32_t* seg_idx = idx_in ? idx_in + (long long)seg * seg_len : nullptr;
  int32_t* out = idx_out + (long long)seg * seg_len;
  const int begin = sub * SUB, end = min(seg_len, begin + SUB);
  const uint32_t lt = (1u << lane) - 1u;
  for (int i0 = begin; i0 < end; i0 += 32) {
    const int i = i0 + lane;
    const bool valid = i < end;
    int src = 0, key = 256 + lane;  // inactive lanes get keys nobody shares
    if (valid) {
      src = seg_idx ? seg_idx[i] : i;
      key = (seg_codes[src] >> shift) & 0xFF;
    }
    const uint32_t same = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(same & lt);
    uint32_t pos = 0;
    if (valid) pos = off[warp][key] + rank;
    __syncwarp();
    if (valid && rank == 0) off[warp][key] += __popc(same);
    __syncwarp();
    if (valid) out[pos] = src;
  }
}

}  // namespace ha

using namespace ha;

extern "C" {

int64_t ha_seg_sort_workspace_bytes(int32_t rows, int32_t n, int32_t span, int32_t seg_len, int32_t key_bits) {
  if (rows <= 0 || n <= 0 || span <= 0 || seg_len <= 0) return 0;
  const long long segs = (long long)rows * (n / span);
  const long long n_sub = (seg_len + SUB - 1) / SUB;
  long long bytes = segs * n_sub * 256 * 4;
  if (key_bits > 8) bytes += segs * seg_len * 4;
  return (bytes + 255) / 256 * 256;
}

int ha_seg_sort(const int32_t* codes, int32_t rows, int32_t n, int32_t span, int32_t seg_off, int32_t seg_len, int32_t key_bits,
                int32_t* idx_out, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!codes || !idx_out || rows < 0 || n < 0 || span <= 0 || seg_len < 0 || seg_off < 0 || key_bits < 1 || key_bits > 16)
    return HA_ERR_INVALID;
  if (n % span != 0 || seg_off + seg_len > span) return HA_ERR_INVALID;
  if (rows == 0 || n == 0 || seg_len == 0) return HA_OK;
  if (!workspace || workspace_bytes < ha_seg_sort_workspace_bytes(rows, n, span, seg_len, key_bits)) return HA_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int parts = n / span;
  const long long segs = (long long)rows * parts;
  const int n_sub = (seg_len + SUB - 1) / SUB;
  uint32_t* hist = (uint32_t*)workspace;
  int32_t* tmp = (int32_t*)((uint8_t*)workspace + segs * n_sub * 256 * 4);
  const int passes = key_bits > 8 ? 2 : 1;
  // gridDim.y is limited to 65535: larger segment counts are folded over several launches, each starting at a
  // row boundary (a multiple of `parts` segments) so that the kernels' row/part arithmetic stays valid.
  if (parts > 65535) return HA_ERR_INVALID;
  const long long fold = (65535 / parts) * (long long)parts;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = pass * 8;
    const int32_t* in = pass == 0 ? nullptr : tmp;
    int32_t* out = (passes == 2 && pass == 0) ? tmp : idx_out;
    for (long long s0 = 0; s0 < segs; s0 += fold) {
      const int ns = (int)((segs - s0) < fold ? (segs - s0) : fold);
      dim3 grid((n_sub + WARPS - 1) / WARPS, ns);
      const int32_t* c = codes + (s0 / parts) * (long long)n;
      sort_hist_kernel<<<grid, WARPS * 32, 0, st>>>(c, n, span, seg_off, seg_len, parts, n_sub, shift,
                                                   in ? in + s0 * seg_len : nullptr, hist + s0 * n_sub * 256);
      HA_LAUNCHED("ha_seg_sort hist");
      sort_scan_kernel<<<ns, 256, 0, st>>>(hist + s0 * n_sub * 256, n_sub);
      HA_LAUNCHED("ha_seg_sort scan");
      sort_scatter_kernel<<<grid, WARPS * 32, 0, st>>>(c, n, span, seg_off, seg_len, parts, n_sub, shift,
                                                      in ? in + s0 * seg_len : nullptr, hist + s0 * n_sub * 256, out + s0 * seg_len);
      HA_LAUNCHED("ha_seg_sort scatter");
    }
  }
  return HA_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of ha_seg_sort.
//
// Some hosts of this library are not in a position to hand over a workspace: an inference server that has already
// given all of HBM to its own pools, a plug-in loaded without any allocator of its own (no torch, no cudaMalloc
// rights inside a captured or latency-critical region, where cudaMalloc would also synchronise the device).  For
// them the counters (and, for keys wider than 8 bits, the intermediate permutation) live in a fixed array that is
// part of the library image, HA_SEG_SORT_STATIC_BYTES bytes on every GPU that loads the library, until exit.
//
// g_sort_scratch names device memory only in device code.  On the host the identifier is a handle, not an address a
// kernel may be given; the address is looked up once per device with cudaGetSymbolAddress while that device is
// current, and that pointer is what the kernels receive.
// ---------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_sort_scratch[HA_SEG_SORT_STATIC_BYTES];

namespace ha {
constexpr int MAX_DEVICES = 64;
static std::mutex g_scratch_mu;
static void* g_scratch_ptr[MAX_DEVICES] = {nullptr};
}  // namespace ha

extern "C" int ha_seg_sort_noalloc(const int32_t* codes, int32_t rows, int32_t n, int32_t span, int32_t seg_off, int32_t seg_len,
                                   int32_t key_bits, int32_t* idx_out, void* stream) {
  if (rows < 0 || n < 0 || span <= 0 || seg_len < 0 || seg_off < 0 || key_bits < 1 || key_bits > 16) return HA_ERR_INVALID;
  if (n % span != 0 || seg_off + seg_len > span) return HA_ERR_INVALID;
  if (rows == 0 || n == 0 || seg_len == 0) return HA_OK;
  if (ha_seg_sort_workspace_bytes(rows, n, span, seg_len, key_bits) > (int64_t)HA_SEG_SORT_STATIC_BYTES) return HA_ERR_TOO_LARGE;
  int dev = -1;
  HA_CUDA_OK(cudaGetDevice(&dev), "ha_seg_sort_noalloc cudaGetDevice");
  if (dev < 0 || dev >= ha::MAX_DEVICES) return HA_ERR_INVALID;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(ha::g_scratch_mu);
    if (!ha::g_scratch_ptr[dev]) {
      void* ptr = nullptr;
      HA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_sort_scratch), "ha_seg_sort_noalloc cudaGetSymbolAddress");
      if (!ptr) return HA_ERR_CUDA;
      ha::g_scratch_ptr[dev] = ptr;
    }
    scratch = ha::g_scratch_ptr[dev];
  }
  // Nothing in the array has to start at zero: every counter block and every intermediate index a pass reads is
  // written by that same call first, so the previous call's contents are simply overwritten.
  return ha_seg_sort(codes, rows, n, span, seg_off, seg_len, key_bits, idx_out, scratch, (int64_t)HA_SEG_SORT_STATIC_BYTES, stream);
}

