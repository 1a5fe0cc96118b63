// Shared-basis products for small token counts:  C[n][m] = sum_k W[m][k] * X[n][k]
//   h_gate / h_up = x . Vh^T        (W = Vh_gate | Vh_up, K = hidden, split over a cluster)
//   y = fp16(rank_accum) . U_down^T  (W = U_down, K = rank_out) (+ residual)
// These are weight-streaming GEMVs: every CTA reads a [rows x k-slice] block of W exactly once,
// keeps it in shared memory and multiplies it with the (few) token rows on the tensor cores
// (mma.sync m16n8k16, W rows as the A operand, tokens as N).  When the contraction is long
// (hidden = 2048) it is split over the CTAs of a thread-block cluster, whose partial sums are
// reduced through distributed shared memory, so no atomics and no second pass are needed.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace bm {

constexpr int SK_THREADS = 256;
constexpr int SK_NTOK = 64;   // tokens per chunk

struct SkinnyArgs {
  const __half* W[2];    // up to two weight matrices stacked along m (rows_per_w rows each)
  void* C[2];            // C[i] is [N, rows_per_w]
  const void* X;         // [N, K]
  const void* residual;  // [N, rows_per_w] or null (W[0] only)
  int rows_per_w, n_w;   // total m = rows_per_w * n_w
  int N, K;
  int x_dtype, c_dtype;
  int round_x_f16;       // X is fp32 and is rounded through fp16 (always true for fp32 here)
  int splits;            // cluster size along k
  int mrows;             // W rows per CTA: 16 or 32
  float4* zero;          // optional buffer the grid clears on its way (the next kernel's accumulator), 16-byte units
  int zero_n;
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldsm_x4(const __half* p, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(p))));
}

// smem: Ws [mrows][ks + 8] half | Xs [64][ks + 8] half | recv [splits][mrows / splits][64] float (only when splits > 1)
__global__ void __launch_bounds__(SK_THREADS) skinny_nt_kernel(SkinnyArgs a) {
  extern __shared__ __align__(16) unsigned char sk_smem[];
  const int ks = a.K / a.splits;
  const int stride = ks + 8;
  __half* Ws = reinterpret_cast<__half*>(sk_smem);
  __half* Xs = Ws + static_cast<size_t>(a.mrows) * stride;
  float* recv = reinterpret_cast<float*>(Xs + static_cast<size_t>(SK_NTOK) * stride);
  const int split = blockIdx.x % a.splits;
  const int m0 = (blockIdx.x / a.splits) * a.mrows;     // first global output row of this CTA
  const int wsel = m0 / a.rows_per_w;                    // which stacked matrix
  const int mloc0 = m0 - wsel * a.rows_per_w;
  const __half* W = a.W[wsel] + static_cast<size_t>(mloc0) * a.K + static_cast<size_t>(split) * ks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;

  // peers' shared memory may be written only once every CTA of the cluster runs: arrive now, wait before the first push
  bool peers_up = a.splits == 1;
  cg::cluster_group::arrival_token started;
  if (a.splits > 1) started = cg::this_cluster().barrier_arrive();
  // W slice -> smem with cp.async (16-byte vectors), so it streams in while the token rows are converted
  const int vec_per_row = ks / 8;
  for (int v = threadIdx.x; v < a.mrows * vec_per_row; v += SK_THREADS) {
    const int r = v / vec_per_row, c = (v - r * vec_per_row) * 8;
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(Ws + static_cast<size_t>(r) * stride + c));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(W + static_cast<size_t>(r) * a.K + c) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  if (a.zero != nullptr) {
    for (int i = blockIdx.x * SK_THREADS + threadIdx.x; i < a.zero_n; i += gridDim.x * SK_THREADS) a.zero[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int mblocks = a.mrows / 16;
  for (int n0 = 0; n0 < a.N; n0 += SK_NTOK) {
    const int nn = min(SK_NTOK, a.N - n0);
    const int nblocks = (nn + 7) / 8;
    __syncthreads();   // previous chunk's readers of Xs / part are done
    // X slice -> fp16 smem; the loads of eight vectors are issued before the first conversion
    const int nvec = nblocks * 8 * vec_per_row;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += 8 * SK_THREADS) {
      uint4 raw[8][2];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + u * SK_THREADS;
        const int r = v / vec_per_row, c = (v - r * vec_per_row) * 8;
        raw[u][0] = raw[u][1] = make_uint4(0u, 0u, 0u, 0u);
        if (v < nvec && r < nn) {
          const size_t idx = static_cast<size_t>(n0 + r) * a.K + static_cast<size_t>(split) * ks + c;
          if (a.x_dtype == BM_F32) {
            raw[u][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.X) + idx);
            raw[u][1] = *reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.X) + idx + 4);
          } else {
            raw[u][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.X) + idx);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int v = v0 + u * SK_THREADS;
        if (v >= nvec) break;
        const int r = v / vec_per_row, c = (v - r * vec_per_row) * 8;
        uint4 out = raw[u][0];
        if (a.x_dtype == BM_BF16) {
          const uint32_t w[4] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __half2 h2 = __floats2half2_rn(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
            o[i] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          out = make_uint4(o[0], o[1], o[2], o[3]);
        } else if (a.x_dtype == BM_F32) {
          const uint32_t w[8] = {raw[u][0].x, raw[u][0].y, raw[u][0].z, raw[u][0].w, raw[u][1].x, raw[u][1].y, raw[u][1].z, raw[u][1].w};
          uint32_t o[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __half2 h2 = __floats2half2_rn(__uint_as_float(w[2 * i]), __uint_as_float(w[2 * i + 1]));
            o[i] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          out = make_uint4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<uint4*>(Xs + static_cast<size_t>(r) * stride + c) = out;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    // (mblock, nblock) items round-robin over the warps, two at a time: items `it` and `it + 8` share the W rows when
    // mblocks divides the warp count, so one A fragment feeds two MMAs; a lone item splits its contraction over two
    // accumulators instead.  Fragments come from ldmatrix (rows are 16-byte aligned and 16 bytes apart modulo 128).
    const int n_items = mblocks * nblocks;
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_kofs = 8 * (lane >> 4);   // ldmatrix.x4 address roles, A operand
    const int b_row = lane & 7, b_sel = lane >> 3;                                     // B operand: matrix b_sel of four
    for (int it = warp; it < n_items; it += 2 * (SK_THREADS / 32)) {
      const int it2 = it + SK_THREADS / 32;
      const int mb = it % mblocks, nb = it / mblocks;
      const bool pair = it2 < n_items && (it2 % mblocks) == mb;
      const int nb2 = pair ? it2 / mblocks : nb;
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const __half* wa = Ws + static_cast<size_t>(mb * 16 + a_row) * stride + a_kofs;
      if (pair) {
        // B matrices: (nb, k 0-7) (nb, k 8-15) (nb2, k 0-7) (nb2, k 8-15)
        const __half* xb = Xs + static_cast<size_t>((b_sel < 2 ? nb : nb2) * 8 + b_row) * stride + 8 * (b_sel & 1);
#pragma unroll 4
        for (int k = 0; k < ks; k += 16) {
          uint32_t a0, a1, a2, a3, b0, b1, c0, c1;
          ldsm_x4(wa + k, a0, a1, a2, a3);
          ldsm_x4(xb + k, b0, b1, c0, c1);
          mma16816(acc[0], a0, a1, a2, a3, b0, b1);
          mma16816(acc[1], a0, a1, a2, a3, c0, c1);
        }
      } else {
        // B matrices: (nb, k 0-7) (nb, k 8-15) (nb, k 16-23) (nb, k 24-31); even / odd 16-steps in separate accumulators
        const __half* xb = Xs + static_cast<size_t>(nb * 8 + b_row) * stride + 8 * b_sel;
        int k = 0;
#pragma unroll 2
        for (; k + 32 <= ks; k += 32) {
          uint32_t a0, a1, a2, a3, e0, e1, e2, e3, b0, b1, c0, c1;
          ldsm_x4(wa + k, a0, a1, a2, a3);
          ldsm_x4(wa + k + 16, e0, e1, e2, e3);
          ldsm_x4(xb + k, b0, b1, c0, c1);
          mma16816(acc[0], a0, a1, a2, a3, b0, b1);
          mma16816(acc[1], e0, e1, e2, e3, c0, c1);
        }
        if (k < ks) {   // one 16-step left: the upper two B matrices repeat the lower ones instead of reading past the row
          uint32_t a0, a1, a2, a3, b0, b1, c0, c1;
          ldsm_x4(wa + k, a0, a1, a2, a3);
          ldsm_x4(Xs + static_cast<size_t>(nb * 8 + b_row) * stride + 8 * (b_sel & 1) + k, b0, b1, c0, c1);
          mma16816(acc[0], a0, a1, a2, a3, b0, b1);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[0][j] += acc[1][j]; acc[1][j] = 0.f; }
      }
      // D: rows m = mb*16 + g (+8), cols n = nb*8 + 2t (+1)
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        if (q == 1 && !pair) break;
        const int nbq = q ? nb2 : nb;
        if (a.splits == 1) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int m = mloc0 + mb * 16 + g + (j >= 2 ? 8 : 0), n = nbq * 8 + 2 * t + (j & 1);
            if (n < nn) {
              const size_t idx = static_cast<size_t>(n0 + n) * a.rows_per_w + m;
              float v = acc[q][j];
              if (a.residual && wsel == 0) v += load_act(a.residual, a.c_dtype, idx);
              store_act(a.C[wsel], a.c_dtype, idx, v);
            }
          }
        } else {
          // push the partial sums into the shared memory of the CTA that owns these output rows
          if (!peers_up) { cg::this_cluster().barrier_wait(std::move(started)); peers_up = true; }
          const int rows_per_owner = a.mrows / a.splits;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int m = mb * 16 + g + 8 * h;
            float* dst = cg::this_cluster().map_shared_rank(recv, m / rows_per_owner) +
                         (static_cast<size_t>(split) * rows_per_owner + m % rows_per_owner) * SK_NTOK + nbq * 8 + 2 * t;
            *reinterpret_cast<float2*>(dst) = make_float2(acc[q][2 * h], acc[q][2 * h + 1]);
          }
        }
      }
    }
    if (a.splits > 1) {
      cg::cluster_group cluster = cg::this_cluster();
      if (!peers_up) { cluster.barrier_wait(std::move(started)); peers_up = true; }
      cluster.sync();   // every CTA's partial sums have landed in their owners
      // this CTA owns rows [split * rows_per_owner, +rows_per_owner) of the mrows x nn tile: sum the `splits` copies
      const int rows_per_owner = a.mrows / a.splits;
      const int total = rows_per_owner * nblocks * 8;
      for (int o = threadIdx.x; o < total; o += SK_THREADS) {
        const int r = o / (nblocks * 8), n = o - r * (nblocks * 8);
        float pv[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) pv[c] = c < a.splits ? recv[(static_cast<size_t>(c) * rows_per_owner + r) * SK_NTOK + n] : 0.f;
        float v = ((pv[0] + pv[1]) + (pv[2] + pv[3])) + ((pv[4] + pv[5]) + (pv[6] + pv[7]));
        if (n < nn) {
          const size_t idx = static_cast<size_t>(n0 + n) * a.rows_per_w + mloc0 + split * rows_per_owner + r;
          if (a.residual && wsel == 0) v += load_act(a.residual, a.c_dtype, idx);
          store_act(a.C[wsel], a.c_dtype, idx, v);
        }
      }
      if (n0 + SK_NTOK < a.N) cluster.sync();   // the next chunk overwrites the receive buffers
    }
  }
}

// Returns BM_ERR_UNSUPPORTED when the shape does not fit; the caller then uses the general GEMM.
int launch_skinny_nt(SkinnyArgs a, cudaStream_t st) {
  BM_REQUIRE(a.K % (16 * a.splits) == 0 && a.rows_per_w % a.mrows == 0 && a.splits <= 8 && a.mrows % a.splits == 0, BM_ERR_UNSUPPORTED, "skinny_nt: shape does not tile");
  const int ks = a.K / a.splits;
  size_t smem = static_cast<size_t>(a.mrows + SK_NTOK) * (ks + 8) * 2;
  if (a.splits > 1) smem += static_cast<size_t>(a.mrows) * SK_NTOK * 4;
  BM_REQUIRE(smem <= 160 * 1024, BM_ERR_UNSUPPORTED, "skinny_nt: k-slice of %d does not fit shared memory", ks);
  static PerDeviceOnce attr_once;
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  if (!attr_once.is_done(dev)) {
    BM_CUDA(cudaFuncSetAttribute(skinny_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    attr_once.mark(dev);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((a.rows_per_w * a.n_w / a.mrows) * a.splits);
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = a.splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  count_launch();
  BM_CUDA(cudaLaunchKernelEx(&cfg, skinny_nt_kernel, a));
  return BM_OK;
}

}  // namespace bm
