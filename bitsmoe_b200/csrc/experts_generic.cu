// Packed routed-expert forward, general path: reads the reference's buffers in place
// (any mix of 1/2/3/4/6/8-bit and raw-fp16 slabs, tail slabs, tail tiles), fp32 math.
//
// Computes, per assignment a = (token t, expert e) and per 128-column tile of the
// intermediate dimension (bitsmoe/algorithms/cpp/mlp_forward.cu:722-764, :1478-1501, :2036-2066):
//   g[c] = sum_k  h_gate[t, rank_idx[k]] * s[k] * scale[tile, k] * q[k, c]      (same for u)
//   z[c] = silu(g[c]) * u[c]
//   rank_accum[t, rank_idx_d[k]] += route_w[a] * s_d[k] * scale_d[tile, k] * sum_c q_d[k, c] * z[c]
// One CTA owns one (expert, tile) and walks that expert's assignments eight at a time; the
// per-tile partial sums of the down product meet in rank_accum through fp32 atomics, as in
// the reference.  The scale of a (tile, row) group is folded into the activation operand,
// so the inner loops multiply by integer codes only.
#include "common.cuh"

namespace bm {

constexpr int GEN_NA = 8;
constexpr int GEN_THREADS = 128;

template <int BITS>
__device__ __forceinline__ float decode_elem(const uint32_t* __restrict__ w, int lane) {
  if constexpr (BITS == 16) {
    const uint32_t word = w[lane >> 1];
    const uint16_t hb = (lane & 1) ? static_cast<uint16_t>(word >> 16) : static_cast<uint16_t>(word & 0xffffu);
    return __half2float(__ushort_as_half(hb));
  } else {
    int u = 0;
#pragma unroll
    for (int p = 0; p < BITS; ++p) u |= static_cast<int>((w[p] >> lane) & 1u) << p;
    return static_cast<float>(BITS == 1 ? 2 * u - 1 : u - (1 << (BITS - 1)));
  }
}

template <int BITS>
__device__ __forceinline__ void gate_up_slab(const uint32_t* __restrict__ tile_payload, int k_slab, int micro, int lane,
                                             const float* __restrict__ hs /*[GEN_NA][stride] at rank_off*/, int stride,
                                             float (&acc)[GEN_NA]) {
  constexpr int WPR = BITS == 16 ? 16 : BITS;
  for (int s0 = 0; s0 < k_slab; s0 += K_STAGE) {
    const int rows_cur = min(K_STAGE, k_slab - s0);
    const uint32_t* base = tile_payload + s0 * MICROS * WPR + micro * rows_cur * WPR;
    for (int r = 0; r < rows_cur; ++r) {
      const float q = decode_elem<BITS>(base + r * WPR, lane);
#pragma unroll
      for (int a = 0; a < GEN_NA; ++a) acc[a] = fmaf(hs[a * stride + s0 + r], q, acc[a]);
    }
  }
}

template <int BITS>
__device__ __forceinline__ void down_row(const uint32_t* __restrict__ tile_payload, int k_slab, int r_in_slab,
                                         const float* __restrict__ z /*[GEN_NA][N_TILE]*/, float (&acc)[GEN_NA]) {
  constexpr int WPR = BITS == 16 ? 16 : BITS;
  const int s0 = (r_in_slab / K_STAGE) * K_STAGE;
  const int r = r_in_slab - s0;
  const int rows_cur = min(K_STAGE, k_slab - s0);
#pragma unroll 1
  for (int micro = 0; micro < MICROS; ++micro) {
    const uint32_t* src = tile_payload + s0 * MICROS * WPR + micro * rows_cur * WPR + r * WPR;
    uint32_t w[WPR];
#pragma unroll
    for (int p = 0; p < WPR; ++p) w[p] = src[p];
#pragma unroll 8
    for (int l = 0; l < N_MICRO; ++l) {
      const float q = decode_elem<BITS>(w, l);
#pragma unroll
      for (int a = 0; a < GEN_NA; ++a) acc[a] = fmaf(q, z[a * N_TILE + micro * N_MICRO + l], acc[a]);
    }
  }
}

#define BM_BITS_SWITCH(bits, CALL)         \
  switch (bits) {                          \
    case 1: { constexpr int B_ = 1; CALL; } break;   \
    case 2: { constexpr int B_ = 2; CALL; } break;   \
    case 3: { constexpr int B_ = 3; CALL; } break;   \
    case 4: { constexpr int B_ = 4; CALL; } break;   \
    case 6: { constexpr int B_ = 6; CALL; } break;   \
    case 8: { constexpr int B_ = 8; CALL; } break;   \
    case 16: { constexpr int B_ = 16; CALL; } break; \
    default: break;                        \
  }

__global__ void __launch_bounds__(GEN_THREADS) experts_generic_kernel(
    const ExpertDev* __restrict__ experts, const __half* __restrict__ h_gate, const __half* __restrict__ h_up, int h_rank,
    const int32_t* __restrict__ token_indices, const int32_t* __restrict__ expert_offsets,
    const float* __restrict__ route_w, int rank_out, int max_rows, int T, float* __restrict__ rank_accum, long long* __restrict__ acc64) {
  extern __shared__ float sm[];
  float* hs = sm;                               // [2][GEN_NA][max_rows]
  float* z = sm + 2 * GEN_NA * max_rows;        // [GEN_NA][N_TILE]
  __shared__ int tok[GEN_NA];
  __shared__ float rw[GEN_NA];

  const int e = blockIdx.y, tile = blockIdx.x;
  const int a_begin = expert_offsets[e], a_end = expert_offsets[e + 1];
  if (a_begin >= a_end) return;
  const ExpertDev& ex = experts[e];
  const int c = threadIdx.x, micro = c >> 5, lane = c & 31;

  for (int a0 = a_begin; a0 < a_end; a0 += GEN_NA) {
    const int na = min(GEN_NA, a_end - a0);
    if (threadIdx.x < GEN_NA) {
      const bool ok = threadIdx.x < na;
      int t = ok ? token_indices[a0 + threadIdx.x] : 0;
      if (t < 0 || t >= T) t = 0;   // a bad index contributes to token 0 with weight 0
      tok[threadIdx.x] = t;
      rw[threadIdx.x] = (ok && token_indices[a0 + threadIdx.x] == t) ? route_w[a0 + threadIdx.x] : 0.f;
    }
    __syncthreads();
    // stage  hs[m][a][row] = h[t_a, rank_idx[row]] * s[row] * scale[tile, row]
    for (int m = 0; m < 2; ++m) {
      const MatDev& md = ex.m[m];
      const __half* h = m == 0 ? h_gate : h_up;
      float* dst = hs + m * GEN_NA * max_rows;
      for (int sl = 0; sl < md.n_slabs; ++sl) {
        const int bits = md.slab_meta[sl * 4 + 0], k_slab = md.slab_meta[sl * 4 + 1];
        const int rank_off = md.slab_meta[sl * 4 + 2], tile_off = md.slab_meta[sl * 4 + 3];
        const int tile_end = (sl + 1 < md.n_slabs) ? md.slab_meta[(sl + 1) * 4 + 3] : md.n_tile_rows;
        const int t = tile_off + tile;
        const bool has_tile = t < tile_end;
        const int scale_off = has_tile ? md.tile_meta[t * 3 + 1] : 0;
        for (int i = threadIdx.x; i < GEN_NA * k_slab; i += GEN_THREADS) {
          const int a = i / k_slab, r = i - a * k_slab;
          const int row = rank_off + r;
          float v = 0.f;
          if (has_tile && a < na) {
            const int rk = md.rank_idx[row];
            if (rk >= 0 && rk < h_rank) {
              v = __half2float(h[static_cast<int64_t>(tok[a]) * h_rank + rk]) * __half2float(md.s[row]);
              if (bits != 16) v *= __half2float(md.scale[scale_off + r]);
            }
          }
          dst[a * max_rows + row] = v;
        }
      }
    }
    __syncthreads();
    // gate / up for column c of this tile
    float gu[2][GEN_NA];
    int n_valid = 0;
    for (int m = 0; m < 2; ++m) {
      const MatDev& md = ex.m[m];
#pragma unroll
      for (int a = 0; a < GEN_NA; ++a) gu[m][a] = 0.f;
      for (int sl = 0; sl < md.n_slabs; ++sl) {
        const int bits = md.slab_meta[sl * 4 + 0], k_slab = md.slab_meta[sl * 4 + 1];
        const int rank_off = md.slab_meta[sl * 4 + 2], tile_off = md.slab_meta[sl * 4 + 3];
        const int tile_end = (sl + 1 < md.n_slabs) ? md.slab_meta[(sl + 1) * 4 + 3] : md.n_tile_rows;
        const int t = tile_off + tile;
        if (t >= tile_end) continue;
        const uint32_t* tp = md.payload + md.tile_meta[t * 3 + 0];
        n_valid = md.tile_meta[t * 3 + 2];
        const float* hsm = hs + m * GEN_NA * max_rows + rank_off;
        BM_BITS_SWITCH(bits, gate_up_slab<B_>(tp, k_slab, micro, lane, hsm, max_rows, gu[m]));
      }
    }
#pragma unroll
    for (int a = 0; a < GEN_NA; ++a) {
      const float g = gu[0][a];
      z[a * N_TILE + c] = (c < n_valid) ? (g / (1.f + expf(-g))) * gu[1][a] : 0.f;
    }
    __syncthreads();
    // down: one stored row per thread
    const MatDev& dd = ex.m[2];
    for (int row = threadIdx.x; row < dd.n_rows; row += GEN_THREADS) {
      int sl = 0;
      for (; sl < dd.n_slabs; ++sl) {
        const int ro = dd.slab_meta[sl * 4 + 2];
        if (row >= ro && row < ro + dd.slab_meta[sl * 4 + 1]) break;
      }
      if (sl >= dd.n_slabs) continue;
      const int bits = dd.slab_meta[sl * 4 + 0], k_slab = dd.slab_meta[sl * 4 + 1];
      const int rank_off = dd.slab_meta[sl * 4 + 2], tile_off = dd.slab_meta[sl * 4 + 3];
      const int tile_end = (sl + 1 < dd.n_slabs) ? dd.slab_meta[(sl + 1) * 4 + 3] : dd.n_tile_rows;
      const int t = tile_off + tile;
      if (t >= tile_end) continue;
      const int logical = dd.rank_idx[row];
      if (logical < 0 || logical >= rank_out) continue;
      const uint32_t* tp = dd.payload + dd.tile_meta[t * 3 + 0];
      float acc[GEN_NA];
#pragma unroll
      for (int a = 0; a < GEN_NA; ++a) acc[a] = 0.f;
      BM_BITS_SWITCH(bits, down_row<B_>(tp, k_slab, row - rank_off, z, acc));
      float f = __half2float(dd.s[row]);
      if (bits != 16) f *= __half2float(dd.scale[dd.tile_meta[t * 3 + 1] + row - rank_off]);
#pragma unroll
      for (int a = 0; a < GEN_NA; ++a) {
        if (a < na) {
          const float v = acc[a] * f * rw[a];
          if (v != 0.f) acc_add(rank_accum, acc64, static_cast<int64_t>(tok[a]) * rank_out + logical, v);
        }
      }
    }
    __syncthreads();
  }
}

int launch_experts_generic(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                           const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum,
                           long long* acc64, cudaStream_t st) {
  const size_t smem = sizeof(float) * (2 * GEN_NA * L->max_rows + GEN_NA * N_TILE);
  BM_REQUIRE(smem <= 200 * 1024, BM_ERR_UNSUPPORTED, "experts_generic: %d stored rows per matrix exceed shared memory",
             L->max_rows);
  if (smem > 48 * 1024) {
    BM_CUDA(cudaFuncSetAttribute(experts_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(smem)));
  }
  dim3 grid(L->n_tiles, L->num_experts);
  experts_generic_kernel<<<grid, GEN_THREADS, smem, st>>>(L->experts_dev, h_gate, h_up, L->rank_in, token_indices,
                                                         expert_offsets, route_w, L->rank_out, L->max_rows, T,
                                                         rank_accum, acc64);
  BM_LAUNCH_CHECK("experts_generic_kernel");
  return BM_OK;
}

}  // namespace bm
