// Shared-basis products:  C[M,N] = A[M,K] . B[N,K]^T  with B the fp16 basis matrix.
//   h_gate / h_up = x . Vh^T      (bitsmoe/models/qwen3moe/bitsmoe_block.py:63-64)
//   y = fp16(rank_accum) . U_down^T (+ residual)   (bitsmoe/models/base_block.py:414)
// fp32 accumulation, one rounding on store.  This file holds the CUDA-core version that
// serves every shape; it tiles A and B through shared memory with 16-byte loads.
#include "common.cuh"

namespace bm {

constexpr int G_BK = 32;
constexpr int G_THREADS = 256;


__device__ __forceinline__ void load8(const void* base, int dtype, int64_t idx, bool ok, int round_f16, float (&v)[8]) {
  if (!ok) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    return;
  }
  if (dtype == BM_F32) {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    const float4 b = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    if (round_f16) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = __half2float(__float2half_rn(v[i]));
    }
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + idx);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (dtype == BM_F16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
      } else {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  }
}

template <int BM, int BN>
__global__ void __launch_bounds__(G_THREADS) gemm_nt_kernel(GemmArgs g) {
  constexpr int TX = BN / 4;            // threads along N, 4 columns each
  constexpr int TY = G_THREADS / TX;    // threads along M
  constexpr int RM = BM / TY;           // rows per thread
  static_assert(BM % TY == 0 && RM >= 1, "tile shape");
  __shared__ float As[G_BK][BM + 4];
  __shared__ float Bs[G_BK][BN + 4];
  const int z = blockIdx.z;
  const void* A = g.A[z];
  const __half* B = g.B[z];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % TX, ty = threadIdx.x / TX;
  float acc[RM][4];
#pragma unroll
  for (int i = 0; i < RM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += G_BK) {
    // A tile: BM x 32 -> BM*4 vectors of 8
    for (int v = threadIdx.x; v < BM * (G_BK / 8); v += G_THREADS) {
      const int r = v / (G_BK / 8), kc = (v % (G_BK / 8)) * 8;
      float f[8];
      const bool ok = (m0 + r < g.M) && (k0 + kc < g.K);
      load8(A, g.a_dtype, static_cast<int64_t>(m0 + r) * g.K + k0 + kc, ok, g.round_a_f16, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) As[kc + i][r] = f[i];
    }
    for (int v = threadIdx.x; v < BN * (G_BK / 8); v += G_THREADS) {
      const int r = v / (G_BK / 8), kc = (v % (G_BK / 8)) * 8;
      float f[8];
      const bool ok = (n0 + r < g.N) && (k0 + kc < g.K);
      load8(B, BM_F16, static_cast<int64_t>(n0 + r) * g.K + k0 + kc, ok, 0, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) Bs[kc + i][r] = f[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < G_BK; ++kk) {
      float a[RM], b[4];
#pragma unroll
      for (int i = 0; i < RM; ++i) a[i] = As[kk][ty * RM + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int m = m0 + ty * RM + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      const int64_t idx = static_cast<int64_t>(m) * g.N + n;
      float v = acc[i][j];
      if (g.residual && z == 0) v += load_act(g.residual, g.c_dtype, idx);
      store_act(g.C[z], g.c_dtype, idx, v);
    }
  }
}

int launch_gemm_nt(const GemmArgs& g, int problems, cudaStream_t st) {
  BM_REQUIRE(g.K % 8 == 0, BM_ERR_UNSUPPORTED, "gemm_nt: K=%d must be a multiple of 8", g.K);
  if (g.M == 0 || g.N == 0) return BM_OK;
  if (g.M <= 64) {
    dim3 grid((g.N + 15) / 16, (g.M + 63) / 64, problems);
    gemm_nt_kernel<64, 16><<<grid, G_THREADS, 0, st>>>(g);
  } else {
    dim3 grid((g.N + 63) / 64, (g.M + 63) / 64, problems);
    gemm_nt_kernel<64, 64><<<grid, G_THREADS, 0, st>>>(g);
  }
  BM_LAUNCH_CHECK("gemm_nt_kernel");
  return BM_OK;
}

}  // namespace bm
