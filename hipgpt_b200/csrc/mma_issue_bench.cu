// Standalone measurement program (not part of the library): cycles per tcgen05.mma kind::tf32, M=128 K=8, for
// several N, operand A from shared memory (SS) or from TMEM (TS), B K-major or N-major.  One thread issues
// `count` instructions back to back, then commits and waits.  Build and run on a B200:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_issue_bench hipgpt_b200/csrc/mma_issue_bench.cu && ./mma_issue_bench
// Every wait is bounded.  The figures it gave are recorded in profiles/tcgen05_mma_issue_cost.md.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_desc(uint32_t a, uint32_t lbo, uint32_t sbo, uint32_t lt) {
  uint64_t d = 0; d |= (uint64_t)((a >> 4) & 0x3FFF); d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16; d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32; d |= 1ull << 46; d |= (uint64_t)lt << 61; return d; }
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int bn) { return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)bn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  uint32_t addr = smem_u32(bar);
  for (long long i = 0; i < (1ll<<22); ++i) { uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true; }
  return false; }
template <int N, bool TS, bool BN>
__global__ void bench(long long *out, int count) {
  extern __shared__ __align__(1024) uint8_t raw[];
  float *base = (float *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t mbar; __shared__ uint32_t slot;
  int tid = threadIdx.x;
  for (int i = tid; i < 40 * 1024; i += blockDim.x) base[i] = 0.001f * (i & 255);
  if (tid < 32) { asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(&slot)), "r"(512u) : "memory");
                  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
  if (tid == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&mbar)) : "memory"); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  uint32_t tmem = slot;
  if (tid == 0) {
    uint64_t da = make_desc(smem_u32(base), 16, 1024, 2);
    uint64_t db = BN ? make_desc(smem_u32(base + 4096), 8192, 512, 1) : make_desc(smem_u32(base + 4096), 16, 1024, 2);
    constexpr uint32_t idesc = make_idesc(128, N, BN ? 1 : 0);
    for (int rep = 0; rep < 3; ++rep) {
      long long t0 = clock64();
      for (int i = 0; i < count; ++i) {
        uint32_t acc = i ? 1u : 0u;
        if (TS) asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" :: "r"(tmem), "r"(tmem + 256 + (i & 7) * 8), "l"(db + (uint64_t)((i & 3) * (BN ? 64 : 2))), "r"(idesc), "r"(acc) : "memory");
        else    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" :: "r"(tmem), "l"(da + (uint64_t)((i & 3) * 2)), "l"(db + (uint64_t)((i & 3) * (BN ? 64 : 2))), "r"(idesc), "r"(acc) : "memory");
      }
      long long t1 = clock64();
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(&mbar)) : "memory");
      bool ok = mbar_wait(&mbar, rep & 1);
      long long t2 = clock64();
      out[rep * 3 + 0] = t1 - t0; out[rep * 3 + 1] = t2 - t0; out[rep * 3 + 2] = ok;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem), "r"(512u) : "memory");
}
template <int N, bool TS, bool BN> void run(const char *name, int count) {
  long long *d; cudaMalloc(&d, 9 * 8); cudaMemset(d, 0, 72);
  cudaFuncSetAttribute(bench<N, TS, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  bench<N, TS, BN><<<1, 128, 200 * 1024>>>(d, count);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[9]; cudaMemcpy(h, d, 72, cudaMemcpyDeviceToHost);
  printf("%-22s count=%d err=%d issue=%lld total=%lld ok=%lld | issue/mma=%.1f total/mma=%.1f\n", name, count, (int)e, h[6], h[7], h[8], (double)h[6] / count, (double)h[7] / count);
  cudaFree(d);
}
int main() {
  for (int count : {1, 12, 48}) {
    run<32, false, false>("SS N=32 Kmajor", count);
    run<64, false, false>("SS N=64 Kmajor", count);
    run<128, false, false>("SS N=128 Kmajor", count);
    run<256, false, false>("SS N=256 Kmajor", count);
    run<32, false, true>("SS N=32 Nmajor", count);
    run<64, false, true>("SS N=64 Nmajor", count);
    run<32, true, true>("TS N=32 Nmajor", count);
    run<64, true, true>("TS N=64 Nmajor", count);
    run<128, true, true>("TS N=128 Nmajor", count);
  }
  return 0;
}
