// Shared-basis products for large token counts on the 5th-generation tensor cores: the cp.async variant, taken when
// a shape or a pointer does not suit the tiled copies of gemm_tma.cu (which is tried first, see launch_gemm_basis).
//   C[m][n] = sum_k X[m][k] * W[n][k],  X = activations (rows = tokens), W = fp16 basis matrix.
//   h_gate / h_up = x . Vh^T  (bitsmoe/models/qwen3moe/bitsmoe_block.py:63-64)
//   y = fp16(rank_accum) . U_down^T (+ residual)  (bitsmoe/models/base_block.py:414)
// One CTA computes a 128 x 256 tile: tokens on the 128 TMEM lanes, 256 fp32 accumulator columns.
// All 8 warps stream K in slices of 64 through a 4-stage ring (cp.async for fp16 data, registers + rounding for
// bf16 / fp32 activations) into shared memory in the K-major canonical layout of 8x16-byte core matrices; one elected thread issues
// tcgen05.mma (M=128, N=256, K=16) four times per slice and commits to the slice's mbarrier, so the
// next slice is being loaded while the tensor core works on this one.  The epilogue reads the
// accumulators with tcgen05.ld and stores rows of C.
#include "common.cuh"
#include "tc05.cuh"

namespace bm {

constexpr int TC_BM = 128, TC_BK = 64, TC_THREADS = 256, TC_STAGES = 4, TC_AHEAD = 3;
constexpr int TC_A_BYTES = TC_BM * TC_BK * 2;   // 16 KB
// The tile is 128 x BN with BN = 256, or 64 when the wide tile would leave most SMs without a CTA (few tokens and a
// narrow output, e.g. the basis projection of 2048 tokens: 32 CTAs against 128).
__host__ __device__ constexpr int tc_stage_bytes(int bn) { return TC_A_BYTES + bn * TC_BK * 2; }


__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t dst = tc::smem_u32(smem);
  const int bytes = valid ? 16 : 0;   // src-size 0 zero-fills the 16 bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// canonical K-major tile of `rows` rows x 64 K: chunk kc (8 K elements) of row r lives at
//   kc * rows * 16 + (r / 8) * 128 + (r % 8) * 16
__device__ __forceinline__ uint32_t canon_off(int rows, int r, int kc) { return kc * rows * 16 + (r >> 3) * 128 + (r & 7) * 16; }

// XD = BM_F16: activations go to shared memory untouched with cp.async.  XD = BM_BF16 / BM_F32: they are loaded
// to registers (all loads of a slice first), rounded to fp16 and stored; both MMA operands are always fp16
// (an instruction descriptor that mixed a bf16 A with an fp16 B raised "illegal instruction" on a B200).
template <int XD, int TC_BN>
__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(GemmTcArgs a) {
  constexpr int TC_STAGE_BYTES = tc_stage_bytes(TC_BN);
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

  constexpr int AV = (TC_BM / 8 * 2) / (TC_THREADS / 32);   // 16-byte vectors of the A slice per thread
  // A operand, fp16 activations: straight to shared memory
  auto issue_a_async = [&](int s) {
    unsigned char* As = tc_smem + (s % TC_STAGES) * TC_STAGE_BYTES;
    const int k0 = s * TC_BK;
    const uint16_t* X = reinterpret_cast<const uint16_t*>(a.X);
#pragma unroll
    for (int i = 0; i < AV; ++i) {
      const int v = warp + i * (TC_THREADS / 32), grp = v >> 1, kc = (v & 1) * 4 + kq, r = grp * 8 + r8;
      const bool valid = m0 + r < a.M;
      cp_async16(As + canon_off(TC_BM, r, kc), X + static_cast<size_t>(valid ? m0 + r : 0) * a.K + k0 + kc * 8, valid);
    }
  };
  // A operand, bf16 / fp32 activations: loaded to registers one slice ahead of the slice being stored, so that the
  // load latency overlaps a whole loop iteration; rounded to fp16 on the way to shared memory
  uint4 raw[AV][XD == BM_F32 ? 2 : 1];
  auto load_a_regs = [&](int s) {
    const int k0 = s * TC_BK;
#pragma unroll
    for (int i = 0; i < AV; ++i) {
      const int v = warp + i * (TC_THREADS / 32), grp = v >> 1, kc = (v & 1) * 4 + kq, r = grp * 8 + r8;
      raw[i][0] = make_uint4(0, 0, 0, 0);
      if (XD == BM_F32) raw[i][XD == BM_F32 ? 1 : 0] = make_uint4(0, 0, 0, 0);
      if (m0 + r < a.M) {
        if (XD == BM_BF16) {
          raw[i][0] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.X) + static_cast<size_t>(m0 + r) * a.K + k0 + kc * 8);
        } else {
          const float* src = reinterpret_cast<const float*>(a.X) + static_cast<size_t>(m0 + r) * a.K + k0 + kc * 8;
          raw[i][0] = *reinterpret_cast<const uint4*>(src);
          raw[i][XD == BM_F32 ? 1 : 0] = *reinterpret_cast<const uint4*>(src + 4);
        }
      }
    }
  };
  auto store_a_regs = [&](int s) {
    unsigned char* As = tc_smem + (s % TC_STAGES) * TC_STAGE_BYTES;
#pragma unroll
    for (int i = 0; i < AV; ++i) {
      const int v = warp + i * (TC_THREADS / 32), grp = v >> 1, kc = (v & 1) * 4 + kq, r = grp * 8 + r8;
      __half2 h[4];
      if (XD == BM_BF16) {
        const uint32_t w[4] = {raw[i][0].x, raw[i][0].y, raw[i][0].z, raw[i][0].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(__uint_as_float(w[j] << 16), __uint_as_float(w[j] & 0xffff0000u));
      } else {
        const uint4 lo = raw[i][0], hi = raw[i][XD == BM_F32 ? 1 : 0];
        h[0] = __floats2half2_rn(__uint_as_float(lo.x), __uint_as_float(lo.y));
        h[1] = __floats2half2_rn(__uint_as_float(lo.z), __uint_as_float(lo.w));
        h[2] = __floats2half2_rn(__uint_as_float(hi.x), __uint_as_float(hi.y));
        h[3] = __floats2half2_rn(__uint_as_float(hi.z), __uint_as_float(hi.w));
      }
      *reinterpret_cast<uint4*>(As + canon_off(TC_BM, r, kc)) = *reinterpret_cast<uint4*>(h);
    }
  };
  auto issue_b = [&](int s) {
    unsigned char* Bs = tc_smem + (s % TC_STAGES) * TC_STAGE_BYTES + TC_A_BYTES;
    const int k0 = s * TC_BK;
#pragma unroll
    for (int i = 0; i < (TC_BN / 8 * 2) / (TC_THREADS / 32); ++i) {
      const int v = warp + i * (TC_THREADS / 32), grp = v >> 1, kc = (v & 1) * 4 + kq, r = grp * 8 + r8;
      const bool valid = n0 + r < a.N;
      cp_async16(Bs + canon_off(TC_BN, r, kc), W + static_cast<size_t>(valid ? n0 + r : 0) * a.K + k0 + kc * 8, valid);
    }
  };

  for (int s = 0; s < TC_AHEAD; ++s) {
    if (s < nslices) {
      if (XD == BM_F16) issue_a_async(s);
      else { load_a_regs(s); store_a_regs(s); }
      issue_b(s);
    }
    cp_async_commit();
  }
  if (XD != BM_F16 && TC_AHEAD < nslices) load_a_regs(TC_AHEAD);
  for (int s = 0; s < nslices; ++s) {
    const int buf = s % TC_STAGES;
    cp_async_wait<TC_AHEAD - 1>();     // this thread's copies of slice s have landed
    tc::fence_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc::fence_after_sync();
      const uint32_t a_base = tc::smem_u32(tc_smem + buf * TC_STAGE_BYTES), b_base = a_base + TC_A_BYTES;
#pragma unroll
      for (int kk = 0; kk < TC_BK / 16; ++kk) {
        const uint64_t ad = tc::smem_desc_kmajor(a_base + 2 * kk * TC_BM * 16, TC_BM * 16, 128);
        const uint64_t bd = tc::smem_desc_kmajor(b_base + 2 * kk * TC_BN * 16, TC_BN * 16, 128);
        tc::mma_f16(tmem_d, ad, bd, idesc, (s > 0 || kk > 0) ? 1u : 0u);
      }
      tc::mma_commit(&bar_free[buf]);
      if (s == nslices - 1) tc::mma_commit(&bar_done);
    }
    const int nxt = s + TC_AHEAD;
    if (nxt < nslices && ok) {
      // stage nxt % STAGES was last read by the MMAs of slice nxt - STAGES = s - 1
      if (nxt >= TC_STAGES && !tc::mbar_wait(&bar_free[nxt % TC_STAGES], ((nxt / TC_STAGES) - 1) & 1)) ok = false;
      if (ok) {
        if (XD == BM_F16) issue_a_async(nxt);
        else {
          store_a_regs(nxt);                               // loaded during the previous iteration
          if (nxt + 1 < nslices) load_a_regs(nxt + 1);
        }
        issue_b(nxt);
      }
    }
    cp_async_commit();
  }
  cp_async_wait<0>();
  if (ok && !tc::mbar_wait(&bar_done, 0)) ok = false;
  tc::fence_after_sync();
  if (ok) {
    // warp w reads TMEM lanes 32*(w%4).., columns 128*(w/4) .. +127
    const int row = m0 + 32 * (warp & 3) + lane;
    const int col_half = (warp >> 2) * (TC_BN / 2);
    // N is a multiple of 8, so whole 16-byte accesses only need aligned bases
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(a.C[z]) | reinterpret_cast<uintptr_t>(a.residual)) & 15u) == 0;
#pragma unroll 1
    for (int c = 0; c < TC_BN / 2; c += 32) {
      float v[32];
      tc::tmem_ld32(tmem_d + (static_cast<uint32_t>(32 * (warp & 3)) << 16) + col_half + c, v);
      const int n = n0 + col_half + c;
      if (row < a.M && n + 32 <= a.N && vec_ok) {
        const size_t idx = static_cast<size_t>(row) * a.N + n;
        if (a.residual && z == 0) {
          // 16-byte loads: a lane owns 32 consecutive columns of its own row, so scalar loads would cost one
          // memory instruction of 32 distinct sectors per column
          if (a.c_dtype == BM_F32) {
            const float4* rs = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.residual) + idx);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 q = __ldg(rs + i);
              v[4 * i] += q.x; v[4 * i + 1] += q.y; v[4 * i + 2] += q.z; v[4 * i + 3] += q.w;
            }
          } else {
            const uint4* rs = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.residual) + idx);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 q = __ldg(rs + i);
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f;
                if (a.c_dtype == BM_F16) f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                v[8 * i + 2 * j] += f.x;
                v[8 * i + 2 * j + 1] += f.y;
              }
            }
          }
        }
        if (a.c_dtype == BM_F32) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.C[z]) + idx + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        } else {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if (a.c_dtype == BM_F16) {
              const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
              pk[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
              const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
              pk[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
          }
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.C[z]) + idx);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        }
      } else if (row < a.M) {
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
  BM_REQUIRE(a.N % 8 == 0, BM_ERR_UNSUPPORTED, "gemm_tc: N=%d must be a multiple of 8", a.N);
  static PerDeviceOnce attr_once;
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  if (!attr_once.is_done(dev)) {
    const int big = TC_STAGES * tc_stage_bytes(256), small = TC_STAGES * tc_stage_bytes(64);
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_F16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_BF16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_F32, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_F16, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_BF16, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
    BM_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BM_F32, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, small));
    attr_once.mark(dev);
  }
  const int mt = (a.M + TC_BM - 1) / TC_BM;
  const bool narrow = mt * ((a.N + 255) / 256) * problems < 74;     // the wide tile would use fewer than half of the SMs
  if (narrow) {
    const int smem = TC_STAGES * tc_stage_bytes(64);
    dim3 grid(mt, (a.N + 63) / 64, problems);
    if (a.x_dtype == BM_F32) gemm_tc_kernel<BM_F32, 64><<<grid, TC_THREADS, smem, st>>>(a);
    else if (a.x_dtype == BM_BF16) gemm_tc_kernel<BM_BF16, 64><<<grid, TC_THREADS, smem, st>>>(a);
    else gemm_tc_kernel<BM_F16, 64><<<grid, TC_THREADS, smem, st>>>(a);
  } else {
    const int smem = TC_STAGES * tc_stage_bytes(256);
    dim3 grid(mt, (a.N + 255) / 256, problems);
    if (a.x_dtype == BM_F32) gemm_tc_kernel<BM_F32, 256><<<grid, TC_THREADS, smem, st>>>(a);
    else if (a.x_dtype == BM_BF16) gemm_tc_kernel<BM_BF16, 256><<<grid, TC_THREADS, smem, st>>>(a);
    else gemm_tc_kernel<BM_F16, 256><<<grid, TC_THREADS, smem, st>>>(a);
  }
  BM_LAUNCH_CHECK("gemm_tc_kernel");
  return BM_OK;
}

}  // namespace bm
