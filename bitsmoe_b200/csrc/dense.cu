// Dense products around the packed experts, so that a whole MoE block runs inside the library:
//   router logits   logits = x . W_gate^T          (bitsmoe/models/qwen3moe/bitsmoe_block.py:45)
//   shared expert   y = (silu(x . Wg^T) * (x . Wu^T)) . Wd^T, optionally scaled per token by sigmoid(x . w)
//                   (bitsmoe/models/deepseekv2/bitsmoe_block.py:123-124, bitsmoe/models/qwen3next/bitsmoe_block.py:144-147)
// The products run on the same kernels as the shared-basis projections: the cluster split-K kernel for decode-sized
// batches, the tcgen05 GEMM above that, a CUDA-core GEMM for shapes neither takes.
#include "common.cuh"

namespace bm {

struct SkinnyArgs {
  const __half* W[2];
  void* C[2];
  const void* X;
  const void* residual;
  int rows_per_w, n_w;
  int N, K;
  int x_dtype, c_dtype;
  int round_x_f16;
  int splits;
  int mrows;
  float4* zero;
  int zero_n;
};
int launch_skinny_nt(SkinnyArgs a, cudaStream_t st);
int launch_gemm_nt(const GemmArgs& g, int problems, cudaStream_t st);

constexpr int DENSE_SKINNY_MAX_TOKENS = 256;

// C_i [T, N] = X [T, K] . W_i [N, K]^T for `problems` (1 or 2) weight matrices sharing X; residual (problem 0 only) may
// be null.  Chooses the kernel by shape.
int dense_xwT(const void* X, int x_dtype, const __half* W0, const __half* W1, void* C0, void* C1, int c_dtype,
              const void* residual, int T, int N, int K, int problems, int* status, cudaStream_t st) {
  if (T == 0) return BM_OK;
  const bool aligned = (reinterpret_cast<uintptr_t>(X) & 15u) == 0;
  if (T <= DENSE_SKINNY_MAX_TOKENS && aligned && N % 32 == 0) {
    // the fewest k-splits whose slice fits shared memory; 32 output rows per CTA when the cluster splits k
    for (int splits = 1; splits <= 8; splits *= 2) {
      if (K % (16 * splits)) continue;
      const int mrows = splits == 1 ? 16 : 32;
      const size_t smem = static_cast<size_t>(mrows + 64) * (K / splits + 8) * 2 + (splits > 1 ? static_cast<size_t>(mrows) * 64 * 4 : 0);
      const int ctas = (N * problems / mrows) * splits;
      if (smem > 160 * 1024 || (splits < 8 && ctas < 96 && K / splits > 256)) continue;   // spread small products over the SMs
      SkinnyArgs a{};
      a.W[0] = W0; a.W[1] = problems > 1 ? W1 : W0;
      a.C[0] = C0; a.C[1] = problems > 1 ? C1 : C0;
      a.X = X; a.residual = residual;
      a.rows_per_w = N; a.n_w = problems;
      a.N = T; a.K = K;
      a.x_dtype = x_dtype; a.c_dtype = c_dtype; a.round_x_f16 = 1;
      a.splits = splits; a.mrows = mrows;
      const int rc = launch_skinny_nt(a, st);
      if (rc != BM_ERR_UNSUPPORTED) return rc;
    }
  }
  if (aligned && K % 64 == 0 && N % 8 == 0) {
    GemmTcArgs t{};
    t.X = X; t.W[0] = W0; t.W[1] = problems > 1 ? W1 : W0; t.C[0] = C0; t.C[1] = problems > 1 ? C1 : C0;
    t.residual = residual; t.M = T; t.N = N; t.K = K; t.x_dtype = x_dtype; t.c_dtype = c_dtype; t.status = status;
    return launch_gemm_basis(t, problems, st);
  }
  GemmArgs g{};
  g.A[0] = g.A[1] = X;
  g.B[0] = W0; g.B[1] = problems > 1 ? W1 : W0;
  g.C[0] = C0; g.C[1] = problems > 1 ? C1 : C0;
  g.residual = residual;
  g.a_dtype = x_dtype; g.c_dtype = c_dtype; g.round_a_f16 = x_dtype == BM_F32 ? 1 : 0;
  g.M = T; g.N = N; g.K = K;
  return launch_gemm_nt(g, problems, st);
}

// gate[t] = sigmoid(x[t] . w): one warp per token.
__global__ void __launch_bounds__(256) row_gate_kernel(const void* __restrict__ x, int x_dtype, const __half* __restrict__ w, int T,
                                                       int H, float* __restrict__ gate) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float acc = 0.f;
  for (int i = lane; i < H; i += 32) acc += load_act(x, x_dtype, static_cast<int64_t>(t) * H + i) * __half2float(w[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) gate[t] = 1.f / (1.f + __expf(-acc));
}

// z[t, c] = fp16(silu(g) * u * gate[t]); g, u fp16 [T, I].
__global__ void __launch_bounds__(256) silu_mul_kernel(const __half2* __restrict__ g, const __half2* __restrict__ u,
                                                       const float* __restrict__ gate, int64_t n_pairs, int pairs_per_row,
                                                       __half2* __restrict__ z) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_pairs; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const float2 gv = __half22float2(g[i]), uv = __half22float2(u[i]);
    const float s = gate ? gate[i / pairs_per_row] : 1.f;
    z[i] = __floats2half2_rn(__fdividef(gv.x, 1.f + __expf(-gv.x)) * uv.x * s, __fdividef(gv.y, 1.f + __expf(-gv.y)) * uv.y * s);
  }
}

}  // namespace bm

using namespace bm;

extern "C" int bm_gate_logits(const void* x, int x_dtype, const uint16_t* gate_w, int32_t T, int32_t num_routed, int32_t hidden,
                              void* logits, int logits_dtype, void* stream) {
  bm::NvtxRange nvtx_range("bm_gate_logits");
  BM_REQUIRE(T >= 0 && num_routed > 0 && hidden > 0, BM_ERR_INVALID_ARG, "gate_logits: bad sizes");
  BM_REQUIRE(x_dtype >= BM_F16 && x_dtype <= BM_F32 && logits_dtype >= BM_F16 && logits_dtype <= BM_F32, BM_ERR_INVALID_ARG,
             "gate_logits: bad dtype");
  if (T == 0) return BM_OK;
  BM_REQUIRE(x && gate_w && logits, BM_ERR_INVALID_ARG, "gate_logits: null pointer");
  return dense_xwT(x, x_dtype, reinterpret_cast<const __half*>(gate_w), nullptr, logits, nullptr, logits_dtype, nullptr, T, num_routed,
                   hidden, 1, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" size_t bm_dense_mlp_workspace_bytes(int32_t T, int32_t intermediate) {
  if (T < 0 || intermediate <= 0) return 0;
  // g, u, z fp16 [T, I] and the per-token gate
  return align_up(static_cast<size_t>(T) * intermediate * 2, 256) * 3 + align_up(static_cast<size_t>(T) * 4, 256);
}

extern "C" int bm_dense_mlp_forward(const void* x, int x_dtype, const uint16_t* w_gate, const uint16_t* w_up, const uint16_t* w_down,
                                    const uint16_t* token_gate_w, int32_t T, int32_t hidden, int32_t intermediate,
                                    const void* residual, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
  bm::NvtxRange nvtx_range("bm_dense_mlp_forward");
  BM_REQUIRE(T >= 0 && hidden > 0 && intermediate > 0 && intermediate % 2 == 0, BM_ERR_INVALID_ARG, "dense_mlp: bad sizes");
  BM_REQUIRE(x_dtype >= BM_F16 && x_dtype <= BM_F32 && y_dtype >= BM_F16 && y_dtype <= BM_F32, BM_ERR_INVALID_ARG, "dense_mlp: bad dtype");
  if (T == 0) return BM_OK;
  BM_REQUIRE(x && w_gate && w_up && w_down && y, BM_ERR_INVALID_ARG, "dense_mlp: null pointer");
  const size_t need = bm_dense_mlp_workspace_bytes(T, intermediate);
  BM_REQUIRE(workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, BM_ERR_WORKSPACE,
             "dense_mlp: workspace must be 256-byte aligned and hold %zu bytes (%zu given)", need, workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const size_t mat = align_up(static_cast<size_t>(T) * intermediate * 2, 256);
  __half* g = reinterpret_cast<__half*>(ws);
  __half* u = reinterpret_cast<__half*>(ws + mat);
  __half* z = reinterpret_cast<__half*>(ws + 2 * mat);
  float* gate = reinterpret_cast<float*>(ws + 3 * mat);
  int rc = dense_xwT(x, x_dtype, reinterpret_cast<const __half*>(w_gate), reinterpret_cast<const __half*>(w_up), g, u, BM_F16, nullptr,
                     T, intermediate, hidden, 2, nullptr, st);
  if (rc) return rc;
  if (token_gate_w) {
    row_gate_kernel<<<(T + 7) / 8, 256, 0, st>>>(x, x_dtype, reinterpret_cast<const __half*>(token_gate_w), T, hidden, gate);
    BM_LAUNCH_CHECK("row_gate_kernel");
  }
  const int64_t pairs = static_cast<int64_t>(T) * intermediate / 2;
  const int blocks = static_cast<int>((pairs + 255) / 256 < 148 * 8 ? (pairs + 255) / 256 : 148 * 8);
  silu_mul_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __half2*>(g), reinterpret_cast<const __half2*>(u),
                                          token_gate_w ? gate : nullptr, pairs, intermediate / 2, reinterpret_cast<__half2*>(z));
  BM_LAUNCH_CHECK("silu_mul_kernel");
  return dense_xwT(z, BM_F16, reinterpret_cast<const __half*>(w_down), nullptr, y, nullptr, y_dtype, residual, T, hidden, intermediate, 1,
                   nullptr, st);
}
