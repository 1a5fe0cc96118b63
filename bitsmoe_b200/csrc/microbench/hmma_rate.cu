// Micro-benchmark: throughput of the legacy warp-level tensor-core path (mma.sync.m16n8k16 f16 -> f32) on one SM, for
// 1..4 independent accumulator chains per warp and 4..32 warps.
// Build and run:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o hmma_rate hmma_rate.cu && ./hmma_rate
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>
__device__ __forceinline__ void mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int CHAINS>
__global__ void rate_kernel(int iters, long long* out, float* sink) {
  float acc[CHAINS][4];
#pragma unroll
  for (int c = 0; c < CHAINS; ++c)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[c][j] = 0.f;
  const uint32_t a = 0x3c003c00u + threadIdx.x, b = 0x3c003c00u;
  __syncthreads();
  const long long t0 = clock64();
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int c = 0; c < CHAINS; ++c) mma(acc[c], a, a + c, a, a, b, b + i);
  }
  __syncthreads();
  const long long t1 = clock64();
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < CHAINS; ++c) s += acc[c][0] + acc[c][3];
  if (s == 123.f) sink[0] = s;
  if (threadIdx.x == 0) out[0] = t1 - t0;
}
template <int CHAINS>
void run(int warps, long long* d, float* sink) {
  const int iters = 4096;
  rate_kernel<CHAINS><<<1, warps * 32>>>(iters, d, sink);
  cudaDeviceSynchronize();
  long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  const double per_sm = double(h) / (double(iters) * CHAINS * warps);
  printf("warps %2d chains %d : %.2f cycles per HMMA per SM  (%.0f FLOP/clk/SM), %.1f cycles per HMMA per warp\n", warps, CHAINS, per_sm,
         4096.0 / per_sm, double(h) / (double(iters) * CHAINS));
}
int main() {
  long long* d; float* sink;
  cudaMalloc(&d, 8); cudaMalloc(&sink, 4);
  for (int w : {4, 8, 16, 32}) { run<1>(w, d, sink); run<2>(w, d, sink); run<4>(w, d, sink); }
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
