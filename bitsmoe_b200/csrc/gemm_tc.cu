// Shared-basis products for large token counts on the 5th-generation tensor cores:
//   C[m][n] = sum_k X[m][k] * W[n][k],  X = activations (rows = tokens), W = fp16 basis matrix.
//   h_gate / h_up = x . Vh^T  (bitsmoe/models/qwen3moe/bitsmoe_block.py:63-64)
//   y = fp16(rank_accum) . U_down^T (+ residual)  (bitsmoe/models/base_block.py:414)
// One CTA computes a 128 x 256 tile: tokens on the 128 TMEM lanes, 256 fp32 accumulator columns.
// All 8 warps stream K in slices of 64: global -> registers (converted to fp16 on the way) -> shared
// memory in the K-major canonical layout of 8x16-byte core matrices; one elected thread issues
// tcgen05.mma (M=128, N=256, K=16) four times per slice and commits to the slice's mbarrier, so the
// next slice is being loaded while the tensor core works on this one.  The epilogue reads the
// accumulators with tcgen05.ld and stores rows of C.
#include "common.cuh"
#include "tc05.cuh"

namespace bm {

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 64, TC_THREADS = 256, TC_STAGES = 2;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
constexpr int TC_B_BYTES = TC_BN * TC_BK * 2;   // 32 KB
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;

struct GemmTcArgs {
  const void* X;          // [M, K]
  const __half* W[2];     // [N, K] each
  void* C[2];             // [M, N] each
  const void* residual;   // [M, N] (W[0] only) or null
  int M, N, K;
  int x_dtype, c_dtype;
  int* status;
};

// 8 consecutive K elements of row r, chunk kc, converted to fp16 and returned as one 16-byte vector
__device__ __forceinline__ uint4 load_chunk_f16(const void* base, int dtype, size_t elem) {
  if (dtype == BM_F16) return *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem);
  __half out[8];
  if (dtype == BM_BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + elem);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __float2half_rn(__uint_as_float(w[i] << 16));
      out[2 * i + 1] = __float2half_rn(__uint_as_float(w[i] & 0xffff0000u));
    }
  } else {
    const float4 f0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem);
    const float4 f1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem + 4);
    out[0] = __float2half_rn(f0.x); out[1] = __float2half_rn(f0.y); out[2] = __float2half_rn(f0.z); out[3] = __float2half_rn(f0.w);
    out[4] = __float2half_rn(f1.x); out[5] = __float2half_rn(f1.y); out[6] = __float2half_rn(f1.z); out[7] = __float2half_rn(f1.w);
  }
  return *reinterpret_cast<uint4*>(out);
}

// canonical K-major tile of `rows` rows x 64 K: chunk kc (8 K elements) of row r lives at
//   kc * rows * 16 + (r / 8) * 128 + (r % 8) * 16
__device__ __forceinline__ uint32_t canon_off(int rows, int r, int kc) { return kc * rows * 16 + (r >> 3) * 128 + (r & 7) * 16; }

__global__ void __launch_bounds__(TC_THREADS) gemm_tc_kernel(GemmTcArgs a) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ __align__(8) uint64_t bar_free[TC_STAGES];   // MMAs that read stage s are complete
  __shared__ __align__(8) uint64_t bar_done;              // all MMAs of the tile are complete
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * TC_BM, n0 = blockIdx.y * TC_BN, z = blockIdx.z;
  const __half* W = a.W[z];
  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) tc::mbar_init(&bar_free[s], 1);
    tc::mbar_init(&bar_done, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, TC_BN);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_d = tmem_slot;
  const uint32_t idesc = tc::idesc_f16(TC_BM, TC_BN);
  const int nslices = a.K / TC_BK;
  bool ok = true;
  // lane -> (row within an 8-row group, one of 4 chunks): a quarter warp fills one 128-byte core matrix
  const int r8 = lane & 7, kq = lane >> 3;
  for (int s = 0; s < nslices; ++s) {
    const int buf = s % TC_STAGES;
    unsigned char* As = tc_smem + buf * TC_STAGE_BYTES;
    unsigned char* Bs = As + TC_A_BYTES;
    if (s >= TC_STAGES && !tc::mbar_wait(&bar_free[buf], ((s / TC_STAGES) - 1) & 1)) { ok = false; break; }
    const int k0 = s * TC_BK;
    // A: 128 rows x 8 chunks = 1024 vectors; B: 256 rows x 8 chunks = 2048 vectors; 32 vectors per warp step
    for (int v = warp; v < (TC_BM + TC_BN) / 8 * 2; v += TC_THREADS / 32) {
      // v enumerates (8-row group, pair of 4-chunk halves)
      const int grp = v >> 1, kc = (v & 1) * 4 + kq;
      if (grp < TC_BM / 8) {
        const int r = grp * 8 + r8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (m0 + r < a.M) val = load_chunk_f16(a.X, a.x_dtype, static_cast<size_t>(m0 + r) * a.K + k0 + kc * 8);
        *reinterpret_cast<uint4*>(As + canon_off(TC_BM, r, kc)) = val;
      } else {
        const int r = (grp - TC_BM / 8) * 8 + r8;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (n0 + r < a.N) val = *reinterpret_cast<const uint4*>(W + static_cast<size_t>(n0 + r) * a.K + k0 + kc * 8);
        *reinterpret_cast<uint4*>(Bs + canon_off(TC_BN, r, kc)) = val;
      }
    }
    tc::fence_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc::fence_after_sync();
      const uint32_t a_base = tc::smem_u32(As), b_base = tc::smem_u32(Bs);
#pragma unroll
      for (int kk = 0; kk < TC_BK / 16; ++kk) {
        const uint64_t ad = tc::smem_desc_kmajor(a_base + 2 * kk * TC_BM * 16, TC_BM * 16, 128);
        const uint64_t bd = tc::smem_desc_kmajor(b_base + 2 * kk * TC_BN * 16, TC_BN * 16, 128);
        tc::mma_f16(tmem_d, ad, bd, idesc, (s > 0 || kk > 0) ? 1u : 0u);
      }
      tc::mma_commit(&bar_free[buf]);
      if (s == nslices - 1) tc::mma_commit(&bar_done);
    }
  }
  if (ok && !tc::mbar_wait(&bar_done, 0)) ok = false;
  tc::fence_after_sync();
  if (ok) {
    // warp w reads TMEM lanes 32*(w%4).., columns 128*(w/4) .. +127
    const int row = m0 + 32 * (warp & 3) + lane;
    const int col_half = (warp >> 2) * (TC_BN / 2);
#pragma unroll 1
    for (int c = 0; c < TC_BN / 2; c += 32) {
      float v[32];
      tc::tmem_ld32(tmem_d + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + col_half + c, v);
      if (row < a.M) {
        const int n = n0 + col_half + c;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (n + i < a.N) {
            const size_t idx = static_cast<size_t>(row) * a.N + n + i;
            float val = v[i];
            if (a.residual && z == 0) val += load_act(a.residual, a.c_dtype, idx);
            store_act(a.C[z], a.c_dtype, idx, val);
          }
        }
      }
    }
  } else if (threadIdx.x == 0 && a.status) {
    atomicExch(a.status, BM_ERR_TIMEOUT);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_d, TC_BN);
}

int launch_gemm_tc(const GemmTcArgs& a, int problems, cudaStream_t st) {
  BM_REQUIRE(a.K % TC_BK == 0, BM_ERR_UNSUPPORTED, "gemm_tc: K=%d must be a multiple of %d", a.K, TC_BK);
  BM_REQUIRE((reinterpret_cast<uintptr_t>(a.X) & 15u) == 0, BM_ERR_UNSUPPORTED, "gemm_tc: activations must be 16-byte aligned");
  static bool attr_done = false;
  const int smem = TC_STAGES * TC_STAGE_BYTES;
  if (!attr_done) {
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_done = true;
  }
  dim3 grid((a.M + TC_BM - 1) / TC_BM, (a.N + TC_BN - 1) / TC_BN, problems);
  gemm_tc_kernel<<<grid, TC_THREADS, smem, st>>>(a);
  BM_LAUNCH_CHECK("gemm_tc_kernel");
  return BM_OK;
}

}  // namespace bm
