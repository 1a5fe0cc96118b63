// Packed routed-expert forward for small token counts (decode): bandwidth-bound split-K GEMV.
//
// One CTA owns one (expert, 128-column tile) unit.  Its whole unit block (scales + packed words of
// gate, up and down for that tile, ~30 KB at the Qwen3-30B shape) is pulled into shared memory by
// two cp.async.bulk copies that complete on mbarriers, so every active SM has its bytes in flight
// from the first cycle; the down words land while gate/up are being consumed.  Weights never
// exist as fp16 in memory: each warp rebuilds m16n8k16 A fragments from the bit-plane words in
// registers (see fast_layout.cuh) and multiplies them with the tokens' activations (the B operand,
// up to 16 assignments per pass) on the tensor cores.  The per-(tile,row) scale is folded into the
// activation operand for gate/up and into the epilogue for down; the unsigned-code offset
// 2^(b-1) is removed with a per-token correction term instead of per weight.  The six tiles of an
// expert split the contraction of the down product; their partial sums meet in rank_accum through
// fp32 atomics (as in bitsmoe/algorithms/cpp/mlp_forward.cu:2036-2066).
#include "fast_layout.cuh"

namespace bm {

constexpr int DEC_THREADS = 256;
constexpr uint32_t DEC_SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// Bounded wait: false if the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t i = 0; i < DEC_SPIN_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Four A-fragment registers (fp16 subnormals u * 2^-24) from the BITS plane words of one row pair.
template <int BITS>
__device__ __forceinline__ void planes_to_afrag(const uint32_t* __restrict__ w, int t, uint32_t (&a)[4]) {
  uint32_t y0 = 0, y1 = 0;
#pragma unroll
  for (int p = 0; p < BITS; ++p) {
    const uint32_t word = w[p];
    y0 |= __funnelshift_r(word, word, (t - p) & 31) & (0x01010101u << p);
    y1 |= __funnelshift_r(word, word, (t + 4 - p) & 31) & (0x01010101u << p);
  }
  a[0] = __byte_perm(y0, 0u, 0x4140);
  a[1] = __byte_perm(y0, 0u, 0x4342);
  a[2] = __byte_perm(y1, 0u, 0x4140);
  a[3] = __byte_perm(y1, 0u, 0x4342);
}

// One group of slot blocks of uniform width.  `words` points at the group's first word for this warp's
// operand-row block; consecutive contraction blocks are `stride_kb` words apart; `bfrag` points at the
// B operand row (assignment g of N-block 0) at the first contraction position of the group.
template <int BITS, int NB>
__device__ __forceinline__ void mma_group(const uint32_t* __restrict__ words, int stride_kb, int nkb, int g, int t,
                                          const __half* __restrict__ bop, int b_stride, float (&acc)[2][4]) {
  const uint32_t* wp = words + g * BITS;
  const __half* bp = bop + static_cast<size_t>(g) * b_stride + 2 * t;
  for (int kb = 0; kb < nkb; ++kb) {
    uint32_t w[BITS];
#pragma unroll
    for (int p = 0; p < BITS; ++p) w[p] = wp[p];
    uint32_t a[4];
    planes_to_afrag<BITS>(w, t, a);
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const __half* b = bp + static_cast<size_t>(nb) * 8 * b_stride;
      mma_16816(acc[nb], a, *reinterpret_cast<const uint32_t*>(b), *reinterpret_cast<const uint32_t*>(b + 8));
    }
    wp += stride_kb;
    bp += 16;
  }
}

struct DecSmem {
  unsigned char* unit;
  __half* actp;     // [2][FAST_MAX_TOK][slots_stride]
  __half* zp;       // [FAST_MAX_TOK][N_TILE + 8]
  float* corr;      // [3][FAST_MAX_TOK]
  int* tok;         // [FAST_MAX_TOK]
  float* rw;        // [FAST_MAX_TOK]
  uint64_t* bar;    // [2]
};

constexpr int ZP_STRIDE = N_TILE + 8;   // halves; +8 keeps the B-fragment loads of 8 rows on distinct banks

__host__ __device__ inline int dec_slots_stride(int max_slots) { return max_slots + 8; }

__host__ __device__ inline size_t dec_smem_bytes(int max_unit_bytes, int max_slots) {
  size_t o = align_up_c(static_cast<size_t>(max_unit_bytes), 128);
  o += static_cast<size_t>(2) * FAST_MAX_TOK * dec_slots_stride(max_slots) * 2;
  o += static_cast<size_t>(FAST_MAX_TOK) * ZP_STRIDE * 2;
  o += 3 * FAST_MAX_TOK * 4 + FAST_MAX_TOK * 4 + FAST_MAX_TOK * 4 + 64;
  return align_up_c(o, 128);
}

template <int NB>
__device__ __forceinline__ void decode_pass(const FastExpert& fe, const DecSmem& sm, int slots_stride, int tile, int n_valid,
                                            int npass, int rank_out, float* __restrict__ rank_accum,
                                            const unsigned char* __restrict__ arena, bool first_pass, bool* ok) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // ---- gate / up: this warp owns columns 16*warp .. 16*warp+15 of the tile
  float acc[2][2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][nb][j] = 0.f;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const FastMat& fm = fe.m[m];
    const uint32_t* words = reinterpret_cast<const uint32_t*>(sm.unit + fe.sec_off[3 + m]) + warp * 8 * 4;
    const __half* bop = sm.actp + static_cast<size_t>(m) * FAST_MAX_TOK * slots_stride;
    // [kb][mblock][g][plane]: a contraction block holds 64*b words, this warp's rows start at warp*8*b
    mma_group<4, NB>(words, 64 * 4, fm.nblk[0], g, t, bop, slots_stride, acc[m]);
    words = words - warp * 8 * 4 + fm.nblk[0] * 64 * 4 + warp * 8 * 3;
    bop += fm.nblk[0] * 16;
    mma_group<3, NB>(words, 64 * 3, fm.nblk[1], g, t, bop, slots_stride, acc[m]);
    words = words - warp * 8 * 3 + fm.nblk[1] * 64 * 3 + warp * 8 * 2;
    bop += fm.nblk[1] * 16;
    mma_group<2, NB>(words, 64 * 2, fm.nblk[2], g, t, bop, slots_stride, acc[m]);
  }
  // ---- z = silu(g) * u, written as the down product's B operand; per-token sum of z for the offset term
  float zs[NB][2];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    zs[nb][0] = zs[nb][1] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = 16 * warp + g + (j >= 2 ? 8 : 0);
      const int n = nb * 8 + 2 * t + (j & 1);
      const float gv = acc[0][nb][j] * 16777216.f - sm.corr[n];
      const float uv = acc[1][nb][j] * 16777216.f - sm.corr[FAST_MAX_TOK + n];
      const float z = (c < n_valid && n < npass) ? (gv / (1.f + __expf(-gv))) * uv : 0.f;
      const __half zh = __float2half_rn(z);
      sm.zp[n * ZP_STRIDE + (c & ~15) + kperm16(c & 15)] = zh;
      zs[nb][j & 1] += __half2float(zh);
    }
  }
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float v = zs[nb][h];
      v += __shfl_xor_sync(0xffffffffu, v, 4);
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (g == 0) atomicAdd(&sm.corr[2 * FAST_MAX_TOK + nb * 8 + 2 * t + h], v);
    }
  __syncthreads();
  if (first_pass && !mbar_wait(&sm.bar[1], 0)) { *ok = false; return; }
  // ---- down: slot blocks round-robin over the warps, contraction over the tile's 128 columns
  const FastMat& fd = fe.m[2];
  const uint32_t* dwords = reinterpret_cast<const uint32_t*>(sm.unit + fe.sec_off[5]);
  const __half* scale_d = reinterpret_cast<const __half*>(sm.unit + fe.sec_off[2]);
  const int16_t* rank_d = reinterpret_cast<const int16_t*>(arena + fd.tab_off);
  const __half* s_d = reinterpret_cast<const __half*>(arena + fd.tab_off + fd.nslots * 2);
  const int nblk_total = fd.nslots >> 4;
  for (int mb = warp; mb < nblk_total; mb += 8) {
    float dacc[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int j = 0; j < 4; ++j) dacc[nb][j] = 0.f;
    int bits;
    if (mb < fd.nblk[0]) {
      bits = 4;
      mma_group<4, NB>(dwords + mb * 64 * 4, 8 * 4, 8, g, t, sm.zp, ZP_STRIDE, dacc);
    } else if (mb < fd.nblk[0] + fd.nblk[1]) {
      bits = 3;
      mma_group<3, NB>(dwords + fd.nblk[0] * 64 * 4 + (mb - fd.nblk[0]) * 64 * 3, 8 * 3, 8, g, t, sm.zp, ZP_STRIDE, dacc);
    } else {
      bits = 2;
      mma_group<2, NB>(dwords + fd.nblk[0] * 64 * 4 + fd.nblk[1] * 64 * 3 + (mb - fd.nblk[0] - fd.nblk[1]) * 64 * 2, 8 * 2, 8, g,
                       t, sm.zp, ZP_STRIDE, dacc);
    }
    const float off = static_cast<float>(1 << (bits - 1));
#pragma unroll
    for (int half_rows = 0; half_rows < 2; ++half_rows) {
      const int slot = mb * 16 + g + 8 * half_rows;
      const int rk = rank_d[slot];
      if (rk < 0 || rk >= rank_out) continue;
      const float f = __half2float(s_d[slot]) * __half2float(scale_d[slot]);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int n = nb * 8 + 2 * t + h;
          if (n >= npass) continue;
          const float v = (dacc[nb][2 * half_rows + h] * 16777216.f - off * sm.corr[2 * FAST_MAX_TOK + n]) * f * sm.rw[n];
          atomicAdd(&rank_accum[static_cast<int64_t>(sm.tok[n]) * rank_out + rk], v);
        }
    }
  }
}

__global__ void __launch_bounds__(DEC_THREADS) experts_decode_kernel(
    const FastExpert* __restrict__ fast, const unsigned char* __restrict__ arena, const __half* __restrict__ h_gate,
    const __half* __restrict__ h_up, int h_rank, const int32_t* __restrict__ token_indices,
    const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w, int rank_out, int T, int n_tiles,
    int intermediate, int max_unit_bytes, int max_slots, float* __restrict__ rank_accum, int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int e = blockIdx.x / n_tiles, tile = blockIdx.x - e * n_tiles;
  const int a_begin = expert_offsets[e], a_end = expert_offsets[e + 1];
  if (a_begin >= a_end) return;
  __shared__ FastExpert fe;
  if (threadIdx.x < sizeof(FastExpert) / 4)
    reinterpret_cast<uint32_t*>(&fe)[threadIdx.x] = reinterpret_cast<const uint32_t*>(&fast[e])[threadIdx.x];
  const int slots_stride = dec_slots_stride(max_slots);
  DecSmem sm;
  {
    size_t o = 0;
    sm.unit = smem_raw;
    o += align_up_c(static_cast<size_t>(max_unit_bytes), 128);
    sm.actp = reinterpret_cast<__half*>(smem_raw + o);
    o += static_cast<size_t>(2) * FAST_MAX_TOK * slots_stride * 2;
    sm.zp = reinterpret_cast<__half*>(smem_raw + o);
    o += static_cast<size_t>(FAST_MAX_TOK) * ZP_STRIDE * 2;
    sm.corr = reinterpret_cast<float*>(smem_raw + o);
    o += 3 * FAST_MAX_TOK * 4;
    sm.tok = reinterpret_cast<int*>(smem_raw + o);
    o += FAST_MAX_TOK * 4;
    sm.rw = reinterpret_cast<float*>(smem_raw + o);
    o += FAST_MAX_TOK * 4;
    o = (o + 7) & ~static_cast<size_t>(7);
    sm.bar = reinterpret_cast<uint64_t*>(smem_raw + o);
  }
  if (threadIdx.x == 0) {
    mbar_init(&sm.bar[0], 1);
    mbar_init(&sm.bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned char* src = arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes;
    const uint32_t bytes_a = static_cast<uint32_t>(fe.sec_off[5]);
    const uint32_t bytes_b = static_cast<uint32_t>(fe.m[2].words) * 4u;
    mbar_expect_tx(&sm.bar[0], bytes_a);
    bulk_g2s(sm.unit, src, bytes_a, &sm.bar[0]);
    mbar_expect_tx(&sm.bar[1], bytes_b);
    bulk_g2s(sm.unit + bytes_a, src + bytes_a, bytes_b, &sm.bar[1]);
  }
  const int n_valid = min(N_TILE, intermediate - tile * N_TILE);
  bool ok = true;
  bool first = true;
  for (int a0 = a_begin; a0 < a_end; a0 += FAST_MAX_TOK) {
    const int npass = min(FAST_MAX_TOK, a_end - a0);
    if (threadIdx.x < FAST_MAX_TOK) {
      const int n = threadIdx.x;
      int tk = n < npass ? token_indices[a0 + n] : 0;
      const bool good = n < npass && tk >= 0 && tk < T;
      sm.tok[n] = good ? tk : 0;
      sm.rw[n] = good ? route_w[a0 + n] : 0.f;
    }
    if (threadIdx.x < 3 * FAST_MAX_TOK) sm.corr[threadIdx.x] = 0.f;
    __syncthreads();
    if (first && !mbar_wait(&sm.bar[0], 0)) { ok = false; break; }
    // ---- activation operand: actp[m][n][perm(slot)] = fp16(h[tok_n, rank(slot)] * s(slot) * scale(tile, slot))
    {
      const int pair = threadIdx.x >> 3, l8 = threadIdx.x & 7;
      const int m = pair >> 4, n = pair & 15;
      const int n_rows_used = ((npass + 7) >> 3) << 3;
      if (n < n_rows_used) {
        const FastMat& fm = fe.m[m];
        const int16_t* rank_t = reinterpret_cast<const int16_t*>(arena + fm.tab_off);
        const __half* s_t = reinterpret_cast<const __half*>(arena + fm.tab_off + fm.nslots * 2);
        const __half* scale_t = reinterpret_cast<const __half*>(sm.unit + fe.sec_off[m]);
        const __half* h = (m == 0 ? h_gate : h_up) + static_cast<int64_t>(sm.tok[n]) * h_rank;
        __half* dst = sm.actp + (static_cast<size_t>(m) * FAST_MAX_TOK + n) * slots_stride;
        const int b43 = fm.nblk[0] * 16, b3 = (fm.nblk[0] + fm.nblk[1]) * 16;
        float csum = 0.f;
        for (int slot = l8; slot < fm.nslots; slot += 8) {
          float v = 0.f;
          if (n < npass) {
            const int rk = rank_t[slot];
            if (rk >= 0 && rk < h_rank) v = __half2float(h[rk]) * __half2float(s_t[slot]) * __half2float(scale_t[slot]);
          }
          const __half hv = __float2half_rn(v);
          dst[(slot & ~15) + kperm16(slot & 15)] = hv;
          csum += (slot < b43 ? 8.f : (slot < b3 ? 4.f : 2.f)) * __half2float(hv);
        }
        csum += __shfl_xor_sync(0xffffffffu, csum, 1);
        csum += __shfl_xor_sync(0xffffffffu, csum, 2);
        csum += __shfl_xor_sync(0xffffffffu, csum, 4);
        if (l8 == 0) sm.corr[m * FAST_MAX_TOK + n] = csum;
      } else {
        // keep the shuffles above convergent for the whole warp
        float z = 0.f;
        z += __shfl_xor_sync(0xffffffffu, z, 1);
        z += __shfl_xor_sync(0xffffffffu, z, 2);
        z += __shfl_xor_sync(0xffffffffu, z, 4);
      }
    }
    __syncthreads();
    if (npass <= 8) decode_pass<1>(fe, sm, slots_stride, tile, n_valid, npass, rank_out, rank_accum, arena, first, &ok);
    else decode_pass<2>(fe, sm, slots_stride, tile, n_valid, npass, rank_out, rank_accum, arena, first, &ok);
    if (!ok) break;
    first = false;
    __syncthreads();
  }
  if (!ok) {
    if (threadIdx.x == 0) atomicExch(status, BM_ERR_TIMEOUT);
    // give copies still in flight a bounded chance to land before the CTA's shared memory is released
    mbar_wait(&sm.bar[0], 0);
    mbar_wait(&sm.bar[1], 0);
  }
}

int launch_experts_decode(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                          const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, cudaStream_t st) {
  const size_t smem = dec_smem_bytes(L->max_unit_bytes, L->max_slots);
  BM_REQUIRE(smem <= 220 * 1024, BM_ERR_UNSUPPORTED, "experts_decode: unit of %d bytes does not fit shared memory",
             L->max_unit_bytes);
  static int attr_set_for = -1;
  if (attr_set_for != L->device) {
    BM_CUDA(cudaFuncSetAttribute(experts_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    attr_set_for = L->device;
  }
  experts_decode_kernel<<<L->num_experts * L->n_tiles, DEC_THREADS, smem, st>>>(
      L->fast_dev, static_cast<const unsigned char*>(L->arena), h_gate, h_up, L->rank_in, token_indices, expert_offsets,
      route_w, L->rank_out, T, L->n_tiles, L->intermediate, L->max_unit_bytes, L->max_slots, rank_accum, L->status_dev);
  BM_LAUNCH_CHECK("experts_decode_kernel");
  return BM_OK;
}

}  // namespace bm
