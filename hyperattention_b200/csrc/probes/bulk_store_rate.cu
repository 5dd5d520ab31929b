// Rate at which a CTA can write a 128 x 128-byte tile from shared to global memory, by six methods (stand-alone; not part
// of the library).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o bulk_store_rate bulk_store_rate.cu && ./bulk_store_rate
//
// One CTA of 128 threads per SM writes a 16 KB tile `iters` times; every thread owns one 128-byte row (as a thread that
// drains a TMEM accumulator does).  Methods: a bulk copy per row (cp.async.bulk, 128 B), one bulk copy of the whole tile,
// the same two as fp32 additions (cp.reduce.async.bulk .add.f32), per-lane st.global.v4 of the lane's own row (32
// different lines per instruction), per-lane red.global.add.v4.f32.  Each round waits until the copy engine has read the
// tile (as a producer that reuses its staging buffer must).  `spread` = how many different 16 KB destinations a CTA cycles
// through (1: stays in L2; 64: 1 MB per CTA).  Printed: cycles per tile and bytes per clock per SM.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
template <int MODE>   // 0: 128 x 128 B stores, 1: one 16 KB store, 2: 128 x 128 B adds, 3: one 16 KB add, 4: per-lane st.global.v4 rows, 5: red.v4 rows
__global__ void k(float* out, long long* cyc, int iters, int spread) {
  __shared__ __align__(128) uint8_t tile[16384];
  const int t = threadIdx.x;
  for (int i = t; i < 4096; i += 128) ((float*)tile)[i] = 1.0f;
  __syncthreads();
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
    // destination: a 16 KB block of this CTA's region; `spread` blocks are cycled through
    float* dst = out + ((long long)blockIdx.x * spread + (it % spread)) * 4096;
    if (MODE == 0 || MODE == 2) {
      // scattered rows: thread t -> row (t * 37) % 128 of the block
      float* d = dst + ((t * 37) & 127) * 32;
      if (MODE == 0) asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 128;" ::"l"(d), "r"(s32(tile + t * 128)) : "memory");
      else asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], 128;" ::"l"(d), "r"(s32(tile + t * 128)) : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    } else if (MODE == 1 || MODE == 3) {
      if (t == 0) {
        if (MODE == 1) asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], 16384;" ::"l"(dst), "r"(s32(tile)) : "memory");
        else asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], 16384;" ::"l"(dst), "r"(s32(tile)) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      }
      __syncthreads();
    } else {
      float* d = dst + ((t * 37) & 127) * 32;
      const float4 v = ((float4*)tile)[t];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (MODE == 4) ((float4*)d)[c] = v;
        else asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(d + 4 * c), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
      }
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncthreads();
  if (t == 0) cyc[blockIdx.x] = clock64() - t0;
}
int main() {
  const int grid = 148, iters = 2000;
  float* out; long long* cyc;
  long long h[148];
  for (int spread : {1, 64}) {
    cudaMalloc(&out, (size_t)grid * spread * 16384); cudaMemset(out, 0, (size_t)grid * spread * 16384);
    cudaMalloc(&cyc, sizeof(h));
    const char* names[6] = {"128 x 128 B bulk stores", "one 16 KB bulk store", "128 x 128 B bulk adds", "one 16 KB bulk add", "per-lane st.global.v4 rows", "per-lane red.v4 rows"};
    for (int m = 0; m < 6; ++m) {
      for (int rep = 0; rep < 2; ++rep) {
        switch (m) {
          case 0: k<0><<<grid, 128>>>(out, cyc, iters, spread); break;
          case 1: k<1><<<grid, 128>>>(out, cyc, iters, spread); break;
          case 2: k<2><<<grid, 128>>>(out, cyc, iters, spread); break;
          case 3: k<3><<<grid, 128>>>(out, cyc, iters, spread); break;
          case 4: k<4><<<grid, 128>>>(out, cyc, iters, spread); break;
          case 5: k<5><<<grid, 128>>>(out, cyc, iters, spread); break;
        }
        if (cudaDeviceSynchronize() != cudaSuccess) { printf("error %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
      }
      cudaMemcpy(h, cyc, sizeof(h), cudaMemcpyDeviceToHost);
      double s = 0; for (int i = 0; i < grid; ++i) s += h[i];
      printf("spread %2d  %-28s %8.1f cycles per 16 KB tile per CTA  (%.1f B/clk/SM)\n", spread, names[m], s / grid / iters, 16384.0 / (s / grid / iters));
    }
    cudaFree(out); cudaFree(cyc);
  }
  return 0;
}
