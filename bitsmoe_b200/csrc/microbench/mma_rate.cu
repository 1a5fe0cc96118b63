// Micro-benchmark: cycles per tcgen05.mma (M = 128, K = 16, fp16) for the operand layouts and N the library uses.
// Build and run:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate mma_rate.cu && ./mma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../tc05.cuh"
using namespace bm;
__global__ void __launch_bounds__(128, 1) rate_kernel(int layout, int N, int lboA, int sboA, int lboB, int sboB, int iters, long long* out) {
  extern __shared__ unsigned char raw[];
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar;
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(base)[i] = 0x3c003c00u;  // fp16 ones
  if (threadIdx.x == 0) { tc::mbar_init(&bar, 1); tc::mbar_init_fence(); }
  if (threadIdx.x < 32) tc::tmem_alloc(&tmem_slot, 512);
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tm = tmem_slot;
  if (threadIdx.x == 0) {
    const uint32_t idesc = tc::idesc_f16(128, N);
    uint64_t ad = tc::smem_desc_kmajor(tc::smem_u32(base), lboA, sboA) | (static_cast<uint64_t>(layout) << 61);
    uint64_t bd = tc::smem_desc_kmajor(tc::smem_u32(base + 64 * 1024), lboB, sboB) | (static_cast<uint64_t>(layout) << 61);
    // warm
    tc::mma_f16(tm, ad, bd, idesc, 0);
    tc::mma_commit(&bar);
    tc::mbar_wait(&bar, 0);
    const long long t0 = clock64();
    for (int i = 0; i < iters; ++i) tc::mma_f16(tm, ad + ((i & 3) * 2), bd + ((i & 3) * 2), idesc, 1);
    const long long t1 = clock64();
    tc::mma_commit(&bar);
    tc::mbar_wait(&bar, 1);
    const long long t2 = clock64();
    out[0] = t1 - t0;
    out[1] = t2 - t0;
  }
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x < 32) tc::tmem_dealloc(tm, 512);
}
int main() {
  long long* d; cudaMalloc(&d, 16);
  cudaFuncSetAttribute(rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  struct Cfg { const char* name; int layout, N, lboA, sboA, lboB, sboB; } cfgs[] = {
    {"none N=64 lbo2080/1040", 0, 64, 2080, 128, 1040, 128},
    {"none N=64 lbo2048/1024", 0, 64, 2048, 128, 1024, 128},
    {"none N=128 lbo2048", 0, 128, 2048, 128, 2048, 128},
    {"none N=256 lbo2048/4096", 0, 256, 2048, 128, 4096, 128},
    {"sw128 N=64", 2, 64, 16, 1024, 16, 1024},
    {"sw128 N=128", 2, 128, 16, 1024, 16, 1024},
    {"sw128 N=256", 2, 256, 16, 1024, 16, 1024},
  };
  for (auto& c : cfgs) {
    const int iters = 2000;
    rate_kernel<<<1, 128, 180 * 1024>>>(c.layout, c.N, c.lboA, c.sboA, c.lboB, c.sboB, iters, d);
    cudaError_t e = cudaDeviceSynchronize();
    long long h[2] = {0, 0};
    cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
    printf("%-28s issue %.1f cyc/mma  complete %.1f cyc/mma  (%s)\n", c.name, double(h[0]) / iters, double(h[1]) / iters, cudaGetErrorString(e));
    if (e != cudaSuccess) return 1;
  }
  return 0;
}
