// tcgen05.mma issue / completion rate probe (stand-alone; not part of the library).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o mma_issue_rate mma_issue_rate.cu && ./mma_issue_rate
//
// n_iss threads of one CTA (one per warp) each issue R back-to-back tcgen05.mma (cta_group::1, kind::f16, M 128, K 16) of one
// shape into an accumulator of their own, then commit; one CTA per SM.  Printed per configuration: cycles per instruction
// seen by an issuing thread until its last instruction is accepted ("issue") and until its commit arrives ("complete").
// With n issuers the tensor pipe's throughput is that figure divided by n.  Operands are zero-filled shared memory; every
// descriptor stays inside the 64 KB operand area (A: 32 KB, B: 32 KB; N <= 128 for MN-major B, N <= 256 for K-major B).
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 2; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int limit) {
  for (int i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// mode: a_tmem (0/1), a_mn, b_mn; N; R instr; ld_warps = number of extra warps hammering tcgen05.ld meanwhile; distinct = rotate accumulators
__global__ void __launch_bounds__(256) rate(long long* out, int N, int R, int a_tmem, int a_mn, int b_mn, int ld_load, int distinct, int* err, int n_iss) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int stop;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < 69000 / 4 - 256; i += 256) ((uint32_t*)smem)[i] = 0;
  if (tid == 0) {
    stop = 0;
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(&mbar)), "r"(n_iss));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&tmem_slot)), "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tbase = tmem_slot;
  const uint32_t sA = smem_u32(smem), sB = sA + 32768;
  if ((tid & 31) == 0 && warp < n_iss) {
    uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    if (a_mn) idesc |= (1u << 15);
    if (b_mn) idesc |= (1u << 16);
    long long t0 = clock64();
    for (int i = 0; i < R; ++i) {
      const int kk = i & 3;
      uint64_t adesc = a_mn ? make_desc(sA + kk * 2048, 16384, 1024) : make_desc(sA + kk * 32, 16, 1024);
      uint64_t bdesc = b_mn ? make_desc(sB + kk * 2048, 16384, 1024) : make_desc(sB + kk * 32, 16, 1024);
      uint32_t tD = tbase + (distinct ? ((i / 8) & 1) * 256 : 0) + warp * 128 * (N <= 128);
      uint32_t acc = 1;
      if (a_tmem) {
        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                     :: "r"(tD), "r"(tbase + 448 + kk * 8), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
      } else {
        asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                     :: "r"(tD), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
      }
    }
    long long t1 = clock64();
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(&mbar)) : "memory");
    bool ok = mbar_wait(smem_u32(&mbar), 0, 4000000);
    long long t2 = clock64();
    stop = 1;
    if (!ok) *err = 1;
    if (blockIdx.x == 0 && warp == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  } else if (warp >= 4 && ld_load) {
    // four warps reading TMEM columns [256, 384) over and over (and writing some back) while the MMAs run
    uint32_t addr = tbase + 256 + ((uint32_t)((warp & 3) * 32) << 16);
    uint32_t sink = 0;
    int iters = 0;
    while (!stop && iters < 200000) {
      uint32_t r[32];
      asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                   : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                     "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                     "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                     "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                   : "r"(addr + (iters & 3) * 32) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      sink += r[0] + r[31];
      ++iters;
    }
    if (sink == 0x12345678u) out[7] = sink;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tbase), "r"(512));
}
int main() {
  long long* out; int* err;
  CK(cudaMalloc(&out, 64)); CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4));
  CK(cudaFuncSetAttribute(rate, cudaFuncAttributeMaxDynamicSharedMemorySize, 70000));
  struct Cfg { const char* name; int N, a_tmem, a_mn, b_mn, ld, distinct, n_iss; };
  Cfg cfgs[] = {
    {"SS N64  K-major A, K-major B, 1 issuer", 64, 0, 0, 0, 0, 0, 1},  {"SS N128 K-major A, K-major B, 1 issuer", 128, 0, 0, 0, 0, 0, 1},
    {"SS N256 K-major A, K-major B, 1 issuer", 256, 0, 0, 0, 0, 0, 1}, {"SS N64  MN-major A and B, 1 issuer", 64, 0, 1, 1, 0, 0, 1},
    {"TS N64  MN-major B, 1 issuer", 64, 1, 0, 1, 0, 0, 1},            {"TS N128 MN-major B, 1 issuer", 128, 1, 0, 1, 0, 0, 1},
    {"SS N64  K/K, 1 issuer + 4 warps of tcgen05.ld", 64, 0, 0, 0, 1, 0, 1},
    {"SS N64  K/K, 2 issuers", 64, 0, 0, 0, 0, 0, 2},                  {"SS N64  K/K, 4 issuers", 64, 0, 0, 0, 0, 0, 4},
    {"SS N128 K/K, 2 issuers", 128, 0, 0, 0, 0, 0, 2},                 {"SS N128 K/K, 3 issuers", 128, 0, 0, 0, 0, 0, 3},
    {"TS N64  MN-major B, 2 issuers", 64, 1, 0, 1, 0, 0, 2},
  };
  for (auto& c : cfgs) {
    for (int R : {64, 512}) {
      rate<<<148, 256, 70000>>>(out, c.N, R, c.a_tmem, c.a_mn, c.b_mn, c.ld, c.distinct, err, c.n_iss);
      CK(cudaDeviceSynchronize());
      long long h[2]; int e;
      CK(cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost)); CK(cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost));
      printf("%-34s R=%4d  issue %7.1f clk/instr  complete %7.1f clk/instr  (ideal %d) err=%d\n", c.name, R, (double)h[0] / R, (double)h[1] / R, c.N / 2, e);
    }
  }
  return 0;
}
