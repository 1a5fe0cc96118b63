// Check of tcgen05.mma with the A operand in tensor memory (written from registers with tcgen05.st), B in shared
// memory: D[128 x 16] = A[128 x 16] * B[16 x 16]^T, fp16 inputs, fp32 accumulators.  Thread of TMEM lane m writes row m
// of A as eight 32-bit columns (two fp16 each, k ascending).  Prints the largest deviation from the host product.
// Build and run:  nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tmem_a_operand tmem_a_operand.cu && ./tmem_a_operand
#include <cstdint>
#include <cstdio>
#include <cmath>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include "../tc05.cuh"
using namespace bm;

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __launch_bounds__(128, 1) check_kernel(const __half* __restrict__ A, const __half* __restrict__ B, float* __restrict__ D) {
  __shared__ __align__(1024) unsigned char bsm[16 * 16 * 2];   // B: 16 rows (n) x 16 k, K-major core matrices
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(8) uint64_t bar;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, m = threadIdx.x;
  if (threadIdx.x == 0) { tc::mbar_init(&bar, 1); tc::mbar_init_fence(); }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 64);
  // B in the canonical layout: chunk kc (8 k) of row n at kc * 16 rows * 16 B + (n / 8) * 128 + (n % 8) * 16
  for (int i = threadIdx.x; i < 16 * 16; i += blockDim.x) {
    const int n = i / 16, k = i % 16;
    reinterpret_cast<__half*>(bsm)[((k >> 3) * 16 * 16 + (n >> 3) * 128 + (n & 7) * 16) / 2 + (k & 7)] = B[n * 16 + k];
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tm = tmem_slot;
  const uint32_t d_cols = tm, a_cols = tm + 32;
  uint32_t r[8];
  for (int j = 0; j < 8; ++j) {
    const __half2 h = __halves2half2(A[m * 16 + 2 * j], A[m * 16 + 2 * j + 1]);
    r[j] = *reinterpret_cast<const uint32_t*>(&h);
  }
  tmem_st8(a_cols + (static_cast<uint32_t>(32 * warp) << 16), r);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  if (threadIdx.x == 0) {
    const uint64_t bd = tc::smem_desc_kmajor(tc::smem_u32(bsm), 16 * 16, 128);
    mma_f16_ta(d_cols, a_cols, bd, tc::idesc_f16(128, 16), 0);
    tc::mma_commit(&bar);
  }
  const bool done = tc::mbar_wait(&bar, 0);
  tc::fence_after_sync();
  float v[16];
  tmem_ld16(d_cols + (static_cast<uint32_t>(32 * warp) << 16), v);
  for (int n = 0; n < 16; ++n) D[m * 16 + n] = done ? v[n] : -12345.f;
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tm, 64);
}

int main() {
  __half hA[128 * 16], hB[16 * 16];
  for (int i = 0; i < 128 * 16; ++i) hA[i] = __float2half(static_cast<float>((i * 7 + 3) % 13 - 6));
  for (int i = 0; i < 16 * 16; ++i) hB[i] = __float2half(static_cast<float>((i * 5 + 1) % 11 - 5) * 0.25f);
  __half *dA, *dB; float* dD;
  cudaMalloc(&dA, sizeof(hA)); cudaMalloc(&dB, sizeof(hB)); cudaMalloc(&dD, 128 * 16 * 4);
  cudaMemcpy(dA, hA, sizeof(hA), cudaMemcpyHostToDevice); cudaMemcpy(dB, hB, sizeof(hB), cudaMemcpyHostToDevice);
  check_kernel<<<1, 128>>>(dA, dB, dD);
  cudaError_t e = cudaDeviceSynchronize();
  float hD[128 * 16];
  cudaMemcpy(hD, dD, sizeof(hD), cudaMemcpyDeviceToHost);
  double worst = 0;
  for (int m = 0; m < 128; ++m)
    for (int n = 0; n < 16; ++n) {
      double ref = 0;
      for (int k = 0; k < 16; ++k) ref += double(__half2float(hA[m * 16 + k])) * double(__half2float(hB[n * 16 + k]));
      worst = fmax(worst, fabs(ref - hD[m * 16 + n]));
    }
  printf("A-from-TMEM MMA: max |D - ref| = %g  (%s)  D[0][0..3] = %g %g %g %g\n", worst, cudaGetErrorString(e), hD[0], hD[1], hD[2], hD[3]);
  return e == cudaSuccess ? 0 : 1;
}
