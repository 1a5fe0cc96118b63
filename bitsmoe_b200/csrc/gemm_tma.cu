// Shared-basis products for large token counts, warp-specialised: tiled TMA loads, tcgen05.mma, persistent CTAs.
//   C[m][n] = sum_k X[m][k] * W[n][k],  X = activations (rows = tokens), W = fp16 basis matrix.
//   h_gate / h_up = x . Vh^T  (bitsmoe/models/qwen3moe/bitsmoe_block.py:63-64)
//   y = fp16(rank_accum) . U_down^T (+ residual)  (bitsmoe/models/base_block.py:414)
// A CTA walks 128 x BN output tiles (BN = 256, or 64 when the wide tile would leave most SMs idle).  Per tile, K is
// streamed in slices of 64 through a ring of stages, both operands K-major with the 128-byte swizzle that the tensor
// map writes and the MMA descriptor reads:
//   warp 0      producer: cp.async.bulk.tensor (2-D tiles) of the X and W slices, completing on the stage's mbarrier
//   warp 1      MMA issue: four tcgen05.mma (M = 128, N = BN, K = 16) per slice, tcgen05.commit frees the stage; the
//               accumulator alternates between two TMEM buffers, so the next tile's products run while this tile's
//               accumulator is read out
//   warps 4-11  epilogue: tcgen05.ld, residual, rounding, stores of whole 64- or 128-byte row pieces
//   warps 12-15, 2, 3  only for bf16 / fp32 activations: round the landed X slice to fp16 in place (both MMA operands have to
//               be fp16: a bf16 A with an fp16 B is not an encodable instruction).  bf16 -> fp16 is element for
//               element; an fp32 slice is twice as large as its fp16 result, and the eight lanes that hold a row read
//               the row's 256 bytes before any of them writes its 16-byte piece of the 128-byte result row.
// Every wait is bounded; a time-out raises the status word.
#include <cuda.h>

#include "common.cuh"
#include "tc05.cuh"

namespace bm {


constexpr int GT_BM = 128, GT_BK = 64, GT_THREADS = 512, GT_MAX_STAGES = 8;
constexpr int GT_WARP_EPI0 = 4, GT_EPI_WARPS = 8, GT_WARP_TR0 = 12, GT_TR_WARPS = 6;    // transform: warps 12-15 and 2, 3

__host__ __device__ constexpr int gt_a_bytes(int xd) { return xd == BM_F32 ? GT_BM * GT_BK * 4 : GT_BM * GT_BK * 2; }
__host__ __device__ constexpr int gt_stage_bytes(int bn, int xd) { return gt_a_bytes(xd) + bn * GT_BK * 2; }
__host__ __device__ constexpr int gt_stages(int bn, int xd) {
  return (216 * 1024) / gt_stage_bytes(bn, xd) < GT_MAX_STAGES ? (216 * 1024) / gt_stage_bytes(bn, xd) : GT_MAX_STAGES;
}

struct GtParams {
  void* C[2];
  const void* residual;
  int M, N, K, c_dtype, problems, tiles_n, ntiles;
  int* status;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   tc::smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(tc::smem_u32(bar))
               : "memory");
}
// K-major operand tile of 128-byte rows, 8-row groups 1024 bytes apart, 128-byte swizzle
__device__ __forceinline__ uint64_t gt_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;              // leading byte offset: unused with swizzled K-major tiles
  d |= static_cast<uint64_t>(1024 >> 4) << 32;      // stride between 8-row groups
  d |= 1ull << 46;                                  // descriptor version of this architecture
  d |= 2ull << 61;                                  // 128-byte swizzle
  return d;
}

template <int BN, int XD>
__global__ void __launch_bounds__(GT_THREADS, 1) gemm_tma_kernel(const __grid_constant__ CUtensorMap map_x,
                                                                 const __grid_constant__ CUtensorMap map_w0,
                                                                 const __grid_constant__ CUtensorMap map_w1, GtParams p) {
  constexpr int A_BYTES = gt_a_bytes(XD), B_BYTES = BN * GT_BK * 2, STAGE = A_BYTES + B_BYTES, NST = gt_stages(BN, XD);
  constexpr uint32_t TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  extern __shared__ unsigned char gt_raw[];
  __shared__ __align__(8) uint64_t loaded[GT_MAX_STAGES], ready[GT_MAX_STAGES], empty[GT_MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gt_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < GT_MAX_STAGES; ++i) {
      tc::mbar_init(&loaded[i], 1);
      tc::mbar_init(&ready[i], GT_TR_WARPS);
      tc::mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&acc_full[i], 1);
      tc::mbar_init(&acc_empty[i], GT_EPI_WARPS);
    }
    tc::mbar_init_fence();
  }
  if (warp == 2) tc::tmem_alloc(&tmem_slot, TMEM_COLS);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const int nslices = p.K / GT_BK;
  bool ok = true;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t st = 0, ph = 0;
      for (int tile = blockIdx.x; tile < p.ntiles && ok; tile += gridDim.x) {
        const int per_m = p.tiles_n * p.problems, m_t = tile / per_m, rem = tile - m_t * per_m;
        const int z = rem / p.tiles_n, n_t = rem - z * p.tiles_n;
        const CUtensorMap* mw = z ? &map_w1 : &map_w0;
        for (int s = 0; s < nslices; ++s) {
          if (!(ok = tc::mbar_wait(&empty[st], ph ^ 1))) break;
          unsigned char* sa = smem + st * STAGE;
          tc::mbar_expect_tx(&loaded[st], A_BYTES + B_BYTES);
          if (XD == BM_F32) {
            // an fp32 row of 64 values is two 128-byte boxes
            tma_load_2d(sa, &map_x, s * GT_BK, m_t * GT_BM, &loaded[st]);
            tma_load_2d(sa + A_BYTES / 2, &map_x, s * GT_BK + 32, m_t * GT_BM, &loaded[st]);
          } else {
            tma_load_2d(sa, &map_x, s * GT_BK, m_t * GT_BM, &loaded[st]);
          }
          tma_load_2d(sa + A_BYTES, mw, s * GT_BK, n_t * BN, &loaded[st]);
          if (++st == NST) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue (the whole warp waits, lane 0 issues)
    uint32_t st = 0, ph = 0, ti = 0;
    const uint32_t idesc = tc::idesc_f16(GT_BM, BN);
    for (int tile = blockIdx.x; tile < p.ntiles && ok; tile += gridDim.x, ++ti) {
      const uint32_t ab = ti & 1u;
      if (ti >= 2 && !(ok = tc::mbar_wait(&acc_empty[ab], ((ti >> 1) - 1) & 1))) break;    // read out two tiles ago
      tc::fence_after_sync();
      for (int s = 0; s < nslices; ++s) {
        if (!(ok = tc::mbar_wait(XD == BM_F16 ? &loaded[st] : &ready[st], ph))) break;
        if (lane == 0) {
          const uint32_t sa = tc::smem_u32(smem + st * STAGE);
          const uint64_t ad = gt_desc_sw128(sa), bd = gt_desc_sw128(sa + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < GT_BK / 16; ++kk)
            tc::mma_f16(tmem_base + ab * BN, ad + 2 * kk, bd + 2 * kk, idesc, (s > 0 || kk > 0) ? 1u : 0u);
          tc::mma_commit(&empty[st]);
        }
        __syncwarp();
        if (++st == NST) { st = 0; ph ^= 1; }
      }
      if (ok && lane == 0) tc::mma_commit(&acc_full[ab]);
      __syncwarp();
    }
  } else if (warp >= GT_WARP_TR0 || warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ rounding of the X slice to fp16, in place
    if (XD != BM_F16) {
      const int tw = warp >= GT_WARP_TR0 ? warp - GT_WARP_TR0 : warp + 2;      // 0 .. 5
      uint32_t st = 0, ph = 0;
      for (int tile = blockIdx.x; tile < p.ntiles && ok; tile += gridDim.x) {
        for (int s = 0; s < nslices; ++s) {
          if (!(ok = tc::mbar_wait(&loaded[st], ph))) break;
          unsigned char* sa = smem + st * STAGE;
          if (XD == BM_BF16) {
            // 1024 pieces of 16 bytes, element for element (the swizzle only permutes whole pieces)
#pragma unroll 2
            for (int i = tw * 32 + lane; i < GT_BM * GT_BK * 2 / 16; i += GT_TR_WARPS * 32) {
              uint4* q = reinterpret_cast<uint4*>(sa) + i;
              const uint4 v = *q;
              const uint32_t w[4] = {v.x, v.y, v.z, v.w};
              __half2 h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xffff0000u));
              *q = *reinterpret_cast<uint4*>(h);
            }
          } else {
            // row r, values 8 j .. 8 j + 7: two 16-byte pieces of box j / 4 -> piece j of the result row
            const int j = lane & 7;
#pragma unroll 2
            for (int rg = tw; rg < GT_BM / 4; rg += GT_TR_WARPS) {
              const int r = rg * 4 + (lane >> 3), sw = r & 7;
              const unsigned char* box = sa + (j >> 2) * (A_BYTES / 2) + r * 128;
              const int c4 = 2 * (j & 3);
              const float4 lo = *reinterpret_cast<const float4*>(box + ((c4 ^ sw) << 4));
              const float4 hi = *reinterpret_cast<const float4*>(box + (((c4 + 1) ^ sw) << 4));
              __half2 h[4] = {__floats2half2_rn(lo.x, lo.y), __floats2half2_rn(lo.z, lo.w), __floats2half2_rn(hi.x, hi.y),
                              __floats2half2_rn(hi.z, hi.w)};
              __syncwarp();          // the row's eight lanes have read before any of them overwrites the row's start
              *reinterpret_cast<uint4*>(sa + r * 128 + ((j ^ sw) << 4)) = *reinterpret_cast<uint4*>(h);
            }
          }
          tc::fence_async_smem();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&ready[st]);
          if (++st == NST) { st = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp >= GT_WARP_EPI0) {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3, half = (warp - GT_WARP_EPI0) >> 2;
    uint32_t ti = 0;
    for (int tile = blockIdx.x; tile < p.ntiles && ok; tile += gridDim.x, ++ti) {
      const int per_m = p.tiles_n * p.problems, m_t = tile / per_m, rem = tile - m_t * per_m;
      const int z = rem / p.tiles_n, n_t = rem - z * p.tiles_n;
      const uint32_t ab = ti & 1u;
      if (!(ok = tc::mbar_wait(&acc_full[ab], (ti >> 1) & 1))) break;
      tc::fence_after_sync();
      const int row = m_t * GT_BM + 32 * q + lane;
      // N is a multiple of 8, so whole 16-byte accesses only need aligned bases
      const bool vec_ok = ((reinterpret_cast<uintptr_t>(p.C[z]) | reinterpret_cast<uintptr_t>(p.residual)) & 15u) == 0;
      const bool with_res = p.residual != nullptr && z == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 2; c += 32) {
        float v[32];
        const int col = half * (BN / 2) + c;
        tc::tmem_ld32(tmem_base + (static_cast<uint32_t>(32 * q) << 16) + ab * BN + col, v);
        const int n = n_t * BN + col;
        if (row < p.M && n + 32 <= p.N && vec_ok) {
          const size_t idx = static_cast<size_t>(row) * p.N + n;
          if (with_res) {
            if (p.c_dtype == BM_F32) {
              const float4* rs = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.residual) + idx);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 r4 = __ldg(rs + i);
                v[4 * i] += r4.x; v[4 * i + 1] += r4.y; v[4 * i + 2] += r4.z; v[4 * i + 3] += r4.w;
              }
            } else {
              const uint4* rs = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.residual) + idx);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint4 r4 = __ldg(rs + i);
                const uint32_t w[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 f;
                  if (p.c_dtype == BM_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                  else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                  v[8 * i + 2 * j] += f.x;
                  v[8 * i + 2 * j + 1] += f.y;
                }
              }
            }
          }
          if (p.c_dtype == BM_F32) {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C[z]) + idx + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          } else {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (p.c_dtype == BM_F16) {
                const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                pk[i] = *reinterpret_cast<const uint32_t*>(&h);
              } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                pk[i] = *reinterpret_cast<const uint32_t*>(&h);
              }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.C[z]) + idx);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
          }
        } else if (row < p.M) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (n + i < p.N) {
              const size_t idx = static_cast<size_t>(row) * p.N + n + i;
              float val = v[i];
              if (with_res) val += load_act(p.residual, p.c_dtype, idx);
              store_act(p.C[z], p.c_dtype, idx, val);
            }
          }
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[ab]);
    }
  }
  if (!ok && lane == 0 && p.status) atomicExch(p.status, BM_ERR_TIMEOUT);
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 2) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- host side -------------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// [rows, cols] row-major, 128-byte-swizzled boxes of box_rows x 128 bytes
static bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int elem_bytes, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims,
            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int XD>
static int launch_one(const CUtensorMap& mx, const CUtensorMap& mw0, const CUtensorMap& mw1, const GtParams& p, int grid, cudaStream_t st) {
  const int smem = gt_stages(BN, XD) * gt_stage_bytes(BN, XD) + 1024;
  static PerDeviceOnce once;
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  if (!once.is_done(dev)) {
    BM_CUDA(cudaFuncSetAttribute(gemm_tma_kernel<BN, XD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    once.mark(dev);
  }
  gemm_tma_kernel<BN, XD><<<grid, GT_THREADS, smem, st>>>(mx, mw0, mw1, p);
  BM_LAUNCH_CHECK("gemm_tma_kernel");
  return BM_OK;
}

// Returns BM_ERR_UNSUPPORTED (without having launched anything) when the shape or the pointers do not suit tiled
// copies; the caller then takes the cp.async kernel.
int launch_gemm_tma(const GemmTcArgs& a, int problems, cudaStream_t st) {
  const int xb = a.x_dtype == BM_F32 ? 4 : 2;
  if (a.K % GT_BK != 0 || a.N % 8 != 0 || a.M <= 0 || problems < 1 || problems > 2) return BM_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a.X) | reinterpret_cast<uintptr_t>(a.W[0]) | reinterpret_cast<uintptr_t>(a.W[problems - 1])) & 15u)
    return BM_ERR_UNSUPPORTED;
  static PerDeviceOnce once;
  static int sm_counts[MAX_DEVICES];
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= MAX_DEVICES) return BM_ERR_UNSUPPORTED;
  if (!once.is_done(dev)) {
    BM_CUDA(cudaDeviceGetAttribute(&sm_counts[dev], cudaDevAttrMultiProcessorCount, dev));
    once.mark(dev);
  }
  const int tiles_m = (a.M + GT_BM - 1) / GT_BM;
  const bool narrow = tiles_m * ((a.N + 255) / 256) * problems < sm_counts[dev] / 2;   // the wide tile would leave most SMs idle
  const int bn = narrow ? 64 : 256;
  CUtensorMap mx, mw0, mw1;
  if (!make_map(&mx, a.X, a.M, a.K, xb, GT_BM) || !make_map(&mw0, a.W[0], a.N, a.K, 2, bn) ||
      !make_map(&mw1, a.W[problems - 1], a.N, a.K, 2, bn))
    return BM_ERR_UNSUPPORTED;
  GtParams p{};
  p.C[0] = a.C[0]; p.C[1] = a.C[problems - 1];
  p.residual = a.residual;
  p.M = a.M; p.N = a.N; p.K = a.K; p.c_dtype = a.c_dtype; p.problems = problems;
  p.tiles_n = (a.N + bn - 1) / bn;
  p.ntiles = tiles_m * p.tiles_n * problems;
  p.status = a.status;
  const int grid = p.ntiles < sm_counts[dev] ? p.ntiles : sm_counts[dev];
  if (narrow) {
    if (a.x_dtype == BM_F32) return launch_one<64, BM_F32>(mx, mw0, mw1, p, grid, st);
    if (a.x_dtype == BM_BF16) return launch_one<64, BM_BF16>(mx, mw0, mw1, p, grid, st);
    return launch_one<64, BM_F16>(mx, mw0, mw1, p, grid, st);
  }
  if (a.x_dtype == BM_F32) return launch_one<256, BM_F32>(mx, mw0, mw1, p, grid, st);
  if (a.x_dtype == BM_BF16) return launch_one<256, BM_BF16>(mx, mw0, mw1, p, grid, st);
  return launch_one<256, BM_F16>(mx, mw0, mw1, p, grid, st);
}

}  // namespace bm
