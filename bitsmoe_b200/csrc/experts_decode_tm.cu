// Packed routed-expert forward for small token counts, tensor-memory variant (opt-in, BM_DECODE_TM=1).
//
// Same work decomposition and the same producer / bulk-copy pipeline as experts_decode.cu (one unit = (expert,
// 128-column tile), two shared-memory stages, 8 assignments per pass), but the products run on tcgen05 with the
// WEIGHT operand in tensor memory: every compute thread owns one operand row (= one TMEM lane), expands its row's
// codes from the row-major arena words into exact fp16 integers (mask | 1024, exact subtract) and stores them with
// tcgen05.st; one thread then issues M = 128, N = 16 MMAs against the token-side operand in shared memory.  A unit
// takes 2 * nkb + 8 * n_mt MMAs (60 at the Qwen3-30B shape) instead of ~1500 warp-level mma.sync, no offset
// correction (the codes are signed after the subtract) and no per-MMA operand loads.
#include <cstdlib>

#include "fast_layout.cuh"
#include "tc05.cuh"

namespace bm {

// Optional phase timing (debug builds only): cycles of compute thread 0, accumulated into status[8 + phase].
#ifdef BM_DECODE_TIMING
#define TM_TICK(phase)                                                                                        \
  do {                                                                                                        \
    if (threadIdx.x == 0) {                                                                                   \
      const long long now_ = clock64();                                                                       \
      atomicAdd(reinterpret_cast<unsigned long long*>(status + 8) + (phase), static_cast<unsigned long long>(now_ - tick_)); \
      tick_ = now_;                                                                                           \
    }                                                                                                         \
  } while (0)
#else
#define TM_TICK(phase) do {} while (0)
#endif

constexpr int TM_THREADS = 288;             // 8 compute warps + 1 producer warp
constexpr int TM_CONSUMERS = 256;
constexpr int TM_NTOK = FAST_MAX_TOK;        // assignments per pass
constexpr int TM_N = 16;                     // MMA N (rows 8..15 of the token operand stay zero)
constexpr int TM_CHUNK = TM_N * 16;          // bytes of one 8-position chunk of a token-side operand
constexpr int TM_MAX_E = 1024;

__device__ __forceinline__ void tm_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(TM_CONSUMERS) : "memory"); }

__device__ __forceinline__ void tm_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tm_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tm_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
// D[tmem] (+)= A[tmem] * B[smem]^T, issued by one thread
__device__ __forceinline__ void tm_mma(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// 8 codes of a nibble word / 16 codes of a dense word -> fp16 pairs (k even, k odd) holding the signed codes exactly
__device__ __forceinline__ void tm_expand_nib(uint32_t w, uint32_t* r) {
  const uint32_t bias_u = 0x64006400u + FAST_NIB_OFFSET * 0x00010001u;
  const __half2 bias = *reinterpret_cast<const __half2*>(&bias_u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t v = ((w >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
    const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&v), bias);
    r[j] = *reinterpret_cast<const uint32_t*>(&q);
  }
}
__device__ __forceinline__ void tm_expand_dense(uint32_t w, uint32_t* r) {
  const uint32_t bias_u = 0x64006400u + FAST_DENSE_OFFSET * 0x00010001u;
  const __half2 bias = *reinterpret_cast<const __half2*>(&bias_u);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t v = ((w >> (2 * j)) & 0x00030003u) | 0x64006400u;
    const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&v), bias);
    r[j] = *reinterpret_cast<const uint32_t*>(&q);
  }
}

struct TmStageInfo {
  FastExpert fe;
  int tok[TM_NTOK];
  float rw[TM_NTOK];
  int a_begin, a_end;
};

__host__ __device__ inline size_t tm_stage_bytes(int max_unit_bytes, int max_slots, int h_rank) {
  return align_up_c(static_cast<size_t>(max_unit_bytes), 128) + align_up_c(static_cast<size_t>(3) * (max_slots * 4 + 16), 128) +
         align_up_c(static_cast<size_t>(2) * TM_NTOK * h_rank * 2, 128);
}
__host__ __device__ inline size_t tm_smem_bytes(int max_unit_bytes, int max_slots, int h_rank) {
  size_t o = 2 * tm_stage_bytes(max_unit_bytes, max_slots, h_rank);
  o += static_cast<size_t>(2) * (max_slots / 8) * TM_CHUNK;   // token-side operands of gate and up
  o += static_cast<size_t>(N_TILE / 8) * TM_CHUNK;            // z
  o += TM_MAX_E * 2;
  return align_up_c(o, 128) + 1024;
}

__global__ void __launch_bounds__(TM_THREADS, 1) experts_decode_tm_kernel(
    const FastExpert* __restrict__ fast, const unsigned char* __restrict__ arena, const __half* __restrict__ h_gate,
    const __half* __restrict__ h_up, int h_rank, const int32_t* __restrict__ token_indices,
    const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w, int rank_out, int T, int num_experts,
    int n_tiles, int intermediate, int max_unit_bytes, int max_slots, int a_cols, float* __restrict__ rank_accum,
    int* __restrict__ status) {
  extern __shared__ unsigned char tm_raw[];
  __shared__ TmStageInfo info[2];
  __shared__ __align__(8) uint64_t bar_full[2][2];   // [stage][scales, gate/up words, tables, h rows | down words]
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ __align__(8) uint64_t bar_mma;
  __shared__ int warp_cnt[9];
  __shared__ uint32_t tmem_slot;
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tm_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const size_t unit_bytes_al = align_up_c(static_cast<size_t>(max_unit_bytes), 128);
  const size_t tabs_bytes_al = align_up_c(static_cast<size_t>(3) * (max_slots * 4 + 16), 128);
  const size_t stage_bytes = tm_stage_bytes(max_unit_bytes, max_slots, h_rank);
  const uint32_t act_m_bytes = static_cast<uint32_t>(max_slots / 8) * TM_CHUNK;
  unsigned char* act = base + 2 * stage_bytes;
  unsigned char* zb = act + 2 * act_m_bytes;
  int16_t* active = reinterpret_cast<int16_t*>(zb + (N_TILE / 8) * TM_CHUNK);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      tc::mbar_init(&bar_full[s][0], 1);
      tc::mbar_init(&bar_full[s][1], 1);
      tc::mbar_init(&bar_empty[s], 8);
    }
    tc::mbar_init(&bar_mma, 1);
    tc::mbar_init_fence();
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);
  // rows 8..15 of the token-side operands are never written again: they must read as zero
  for (int i = threadIdx.x; i < static_cast<int>((2 * act_m_bytes + (N_TILE / 8) * TM_CHUNK) / 16); i += TM_THREADS)
    reinterpret_cast<uint4*>(act)[i] = make_uint4(0u, 0u, 0u, 0u);
  // ---- compact the active experts (ascending id)
  int n_active = 0;
  for (int b0 = 0; b0 < num_experts; b0 += TM_THREADS) {
    const int e = b0 + threadIdx.x;
    const bool is_act = e < num_experts && expert_offsets[e + 1] > expert_offsets[e];
    const unsigned m = __ballot_sync(0xffffffffu, is_act);
    if (lane == 0) warp_cnt[warp] = __popc(m);
    __syncthreads();
    int before = n_active;
    for (int w = 0; w < warp; ++w) before += warp_cnt[w];
    if (is_act) active[before + __popc(m & ((1u << lane) - 1u))] = static_cast<int16_t>(e);
    for (int w = 0; w < 9; ++w) n_active += warp_cnt[w];
    __syncthreads();
  }
  tc::fence_async_smem();
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tm = tmem_slot;
  const int n_units = n_active * n_tiles;
  const int nkb_max = max_slots >> 4;
  const uint32_t col_ag = tm, col_au = tm + 8 * nkb_max, col_dg = tm + a_cols, col_du = col_dg + TM_N, col_dd = col_du + TM_N;
  const uint32_t idesc = tc::idesc_f16(128, TM_N);
  bool ok = true;

  if (warp == 8) {
    // ------------------------------------------------------------------ producer warp
    int it = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++it) {
      const int buf = it & 1;
      const int e = active[u / n_tiles], tile = u % n_tiles;
      if (!tc::mbar_wait(&bar_empty[buf], ((it >> 1) & 1) ^ 1)) { ok = false; break; }
      TmStageInfo& si = info[buf];
      for (int i = lane; i < static_cast<int>(sizeof(FastExpert) / 4); i += 32)
        reinterpret_cast<uint32_t*>(&si.fe)[i] = reinterpret_cast<const uint32_t*>(&fast[e])[i];
      const int a_begin = expert_offsets[e], a_end = expert_offsets[e + 1];
      const int npass = min(TM_NTOK, a_end - a_begin);
      int tk = 0;
      if (lane < TM_NTOK) {
        tk = lane < npass ? token_indices[a_begin + lane] : 0;
        const bool good = lane < npass && tk >= 0 && tk < T;
        tk = good ? tk : 0;
        si.tok[lane] = tk;
        si.rw[lane] = good ? route_w[a_begin + lane] : 0.f;
      }
      if (lane == 0) { si.a_begin = a_begin; si.a_end = a_end; }
      __syncwarp();
      const FastExpert& fe = si.fe;
      unsigned char* stage = base + buf * stage_bytes;
      const unsigned char* src = arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes;
      const uint32_t scale_bytes = static_cast<uint32_t>(fe.sec_off[3]);
      const uint32_t gu_bytes = static_cast<uint32_t>(fe.rm_off[2] - fe.rm_off[0]);
      const uint32_t d_bytes = static_cast<uint32_t>(fe.m[2].words) * 4u;
      const uint32_t tb0 = static_cast<uint32_t>(fe.m[0].nslots) * 4u, tb1 = static_cast<uint32_t>(fe.m[1].nslots) * 4u,
                     tb2 = static_cast<uint32_t>(fe.m[2].nslots) * 4u;
      const uint32_t row_bytes = static_cast<uint32_t>(h_rank) * 2u;
      if (lane == 0) {
        tc::mbar_expect_tx(&bar_full[buf][0], scale_bytes + gu_bytes + tb0 + tb1 + tb2 + 2u * npass * row_bytes);
        tc::bulk_g2s(stage, src, scale_bytes, &bar_full[buf][0]);
        tc::bulk_g2s(stage + fe.sec_off[3], src + fe.rm_off[0], gu_bytes, &bar_full[buf][0]);
        tc::bulk_g2s(stage + unit_bytes_al, arena + fe.m[0].tab_off, tb0, &bar_full[buf][0]);
        tc::bulk_g2s(stage + unit_bytes_al + tb0, arena + fe.m[1].tab_off, tb1, &bar_full[buf][0]);
        tc::bulk_g2s(stage + unit_bytes_al + tb0 + tb1, arena + fe.m[2].tab_off, tb2, &bar_full[buf][0]);
        tc::mbar_expect_tx(&bar_full[buf][1], d_bytes);
        tc::bulk_g2s(stage + fe.sec_off[5], src + fe.rm_off[2], d_bytes, &bar_full[buf][1]);
      }
      __syncwarp();
      if (lane < 2 * npass) {
        const int m = lane / npass, n = lane - m * npass;
        const int tkn = __shfl_sync(__activemask(), tk, n);
        const __half* hsrc = (m == 0 ? h_gate : h_up) + static_cast<int64_t>(tkn) * h_rank;
        tc::bulk_g2s(stage + unit_bytes_al + tabs_bytes_al + (static_cast<size_t>(m) * TM_NTOK + n) * row_bytes, hsrc, row_bytes,
                     &bar_full[buf][0]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(status, BM_ERR_TIMEOUT);
  } else {
    // ------------------------------------------------------------------ compute warps
    const int q4 = warp & 3, half = warp >> 2;                    // TMEM lane quarter, warp group
    const uint32_t lane_sel = static_cast<uint32_t>(32 * q4) << 16;
    const int row = 32 * q4 + lane;                                // operand row inside a 128-row tile = TMEM lane
    uint32_t mma_round = 0;
    int it = 0;
    long long tick_ = clock64();
    (void)tick_;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t parity = (it >> 1) & 1;
      const int tile = u % n_tiles;
      const int n_valid = min(N_TILE, intermediate - tile * N_TILE);
      unsigned char* stage = base + buf * stage_bytes;
      if (!tc::mbar_wait(&bar_full[buf][0], parity)) { ok = false; break; }
      TM_TICK(0);
      TmStageInfo& si = info[buf];
      const FastExpert& fe = si.fe;
      const unsigned char* tabs[3];
      tabs[0] = stage + unit_bytes_al;
      tabs[1] = tabs[0] + fe.m[0].nslots * 4;
      tabs[2] = tabs[1] + fe.m[1].nslots * 4;
      const __half* hrows = reinterpret_cast<const __half*>(stage + unit_bytes_al + tabs_bytes_al);
      const int a_begin = si.a_begin, a_end = si.a_end;
      const FastMat& fd = fe.m[2];
      const int n_mt = (fd.nslots + 127) >> 7;
      for (int a0 = a_begin; a0 < a_end && ok; a0 += TM_NTOK) {
        const int npass = min(TM_NTOK, a_end - a0);
        const bool staged = a0 == a_begin;
        if (!staged) {
          tm_consumer_sync();
          if (threadIdx.x < TM_NTOK) {
            const int n = threadIdx.x;
            const int tk = n < npass ? token_indices[a0 + n] : 0;
            const bool good = n < npass && tk >= 0 && tk < T;
            si.tok[n] = good ? tk : 0;
            si.rw[n] = good ? route_w[a0 + n] : 0.f;
          }
          tm_consumer_sync();
        }
        // ---- token-side operand: act[m][slot / 8][n][slot % 8] = fp16(h[tok_n, rank(slot)] * s(slot) * scale(tile, slot))
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const int nslots = fe.m[m].nslots;
          const int16_t* rank_t = reinterpret_cast<const int16_t*>(tabs[m]);
          const __half* s_t = reinterpret_cast<const __half*>(tabs[m] + nslots * 2);
          const __half* scale_t = reinterpret_cast<const __half*>(stage + fe.sec_off[m]);
          const __half* hg = m == 0 ? h_gate : h_up;
          const __half* hs = hrows + static_cast<size_t>(m) * TM_NTOK * h_rank;
          unsigned char* dst = act + m * act_m_bytes;
          for (int slot = threadIdx.x; slot < nslots; slot += TM_CONSUMERS) {
            const int rk = rank_t[slot];
            const float f = __half2float(s_t[slot]) * __half2float(scale_t[slot_pos(slot)]);
            const bool live = rk >= 0 && rk < h_rank;
            __half* d = reinterpret_cast<__half*>(dst + (slot >> 3) * TM_CHUNK + (slot & 7) * 2);
#pragma unroll
            for (int n = 0; n < TM_NTOK; ++n) {
              float hv = 0.f;
              if (live && n < npass)
                hv = __half2float(staged ? hs[n * h_rank + rk] : hg[static_cast<int64_t>(si.tok[n]) * h_rank + rk]);
              d[n * 8] = __float2half_rn(hv * f);
            }
          }
        }
        tc::fence_async_smem();
        TM_TICK(1);
        // ---- weight operand of gate (warps 0-3) and up (warps 4-7): this thread's row -> tensor memory
        {
          const FastMat& fm = fe.m[half];
          const uint32_t* sec = reinterpret_cast<const uint32_t*>(stage + fe.sec_off[3 + half]);
          const int nkb = fm.nslots >> 4, nb0 = fm.nblk[0];
          const uint32_t col_a = (half == 0 ? col_ag : col_au) + lane_sel;
          for (int kb = 0; kb < nkb; ++kb) {
            uint32_t r[8];
            if (kb < nb0) {
              const uint2 w = reinterpret_cast<const uint2*>(sec)[kb * 128 + row];
              tm_expand_nib(w.x, r);
              tm_expand_nib(w.y, r + 4);
            } else {
              tm_expand_dense(sec[nb0 * 256 + (kb - nb0) * 128 + row], r);
            }
            tm_st8(col_a + 8 * kb, r);
          }
          tm_wait_st();
        }
        tc::fence_before_sync();
        tm_consumer_sync();
        TM_TICK(2);
        if (threadIdx.x == 0) {
          tc::fence_after_sync();
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const int nkb = fe.m[m].nslots >> 4;
            const uint64_t bd0 = tc::smem_desc_kmajor(tc::smem_u32(act + m * act_m_bytes), TM_CHUNK, 128);
            for (int kb = 0; kb < nkb; ++kb)
              tm_mma(m == 0 ? col_dg : col_du, (m == 0 ? col_ag : col_au) + 8 * kb, bd0 + ((2 * kb * TM_CHUNK) >> 4), idesc, kb > 0 ? 1u : 0u);
          }
          tc::mma_commit(&bar_mma);
        }
        if (!tc::mbar_wait(&bar_mma, mma_round & 1)) { ok = false; break; }
        ++mma_round;
        tc::fence_after_sync();
        TM_TICK(3);
        // ---- z = silu(g) * u for this thread's column: tokens 4*half .. 4*half+3
        {
          float gv[8], uv[8];
          tm_ld8(col_dg + lane_sel, gv);
          tm_ld8(col_du + lane_sel, uv);
          __half* zc = reinterpret_cast<__half*>(zb + (row >> 3) * TM_CHUNK + (row & 7) * 2);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int n = 4 * half + i;
            const float g = gv[n], z = (row < n_valid && n < npass) ? (g / (1.f + __expf(-g))) * uv[n] : 0.f;
            zc[n * 8] = __float2half_rn(z);
          }
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        tm_consumer_sync();
        TM_TICK(4);
        if (!tc::mbar_wait(&bar_full[buf][1], parity)) { ok = false; break; }
        TM_TICK(5);
        // ---- weight operand of down: 128-row tiles of slots, tile mt by warp group mt % 2
        const uint32_t* dsec = reinterpret_cast<const uint32_t*>(stage + fe.sec_off[5]);
        const int n0 = fd.nblk[0] * 16, n1 = fd.nblk[1] * 16;
        for (int mt = half; mt < n_mt; mt += 2) {
          const int slot = 128 * mt + row;
          for (int kb = 0; kb < 8; ++kb) {
            uint32_t r[8];
            if (slot < n0) {
              const uint2 w = reinterpret_cast<const uint2*>(dsec)[kb * n0 + slot];
              tm_expand_nib(w.x, r);
              tm_expand_nib(w.y, r + 4);
            } else if (slot < n0 + n1) {
              tm_expand_dense(dsec[n0 * 16 + kb * n1 + (slot - n0)], r);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) r[j] = 0u;
            }
            tm_st8(tm + 64 * mt + 8 * kb + lane_sel, r);
          }
        }
        tm_wait_st();
        tc::fence_before_sync();
        tm_consumer_sync();
        TM_TICK(6);
        if (threadIdx.x == 0) {
          tc::fence_after_sync();
          const uint64_t zd0 = tc::smem_desc_kmajor(tc::smem_u32(zb), TM_CHUNK, 128);
          for (int mt = 0; mt < n_mt; ++mt)
            for (int kb = 0; kb < 8; ++kb)
              tm_mma(col_dd + TM_N * mt, tm + 64 * mt + 8 * kb, zd0 + ((2 * kb * TM_CHUNK) >> 4), idesc, kb > 0 ? 1u : 0u);
          tc::mma_commit(&bar_mma);
        }
        if (!tc::mbar_wait(&bar_mma, mma_round & 1)) { ok = false; break; }
        ++mma_round;
        tc::fence_after_sync();
        TM_TICK(7);
        // ---- rank_accum[token, rank(slot)] += acc * s * scale * route weight
        {
          const int16_t* rank_d = reinterpret_cast<const int16_t*>(tabs[2]);
          const __half* s_d = reinterpret_cast<const __half*>(tabs[2] + fd.nslots * 2);
          const __half* scale_d = reinterpret_cast<const __half*>(stage + fe.sec_off[2]);
          for (int mt = half; mt < n_mt; mt += 2) {
            const int slot = 128 * mt + row;
            float v[8];
            tm_ld8(col_dd + TM_N * mt + lane_sel, v);
            if (slot < fd.nslots) {
              const int rk = rank_d[slot];
              if (rk >= 0 && rk < rank_out) {
                const float f = __half2float(s_d[slot]) * __half2float(scale_d[slot]);
#pragma unroll
                for (int n = 0; n < TM_NTOK; ++n)
                  if (n < npass) atomicAdd(&rank_accum[static_cast<int64_t>(si.tok[n]) * rank_out + rk], v[n] * f * si.rw[n]);
              }
            }
          }
        }
        tc::fence_before_sync();
        tm_consumer_sync();
        TM_TICK(8);
      }
      if (lane == 0) tc::mbar_arrive(&bar_empty[buf]);
    }
    if (!ok && threadIdx.x == 0) atomicExch(status, BM_ERR_TIMEOUT);
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tm, 512);
}

bool experts_decode_tm_fits(const bm_layer* L) {
  const int nkb_max = L->max_slots / 16, n_mt_max = (L->max_slots + 127) / 128;
  const int a_cols = nkb_max * 16 > n_mt_max * 64 ? nkb_max * 16 : n_mt_max * 64;
  return a_cols + 2 * TM_N + TM_N * n_mt_max <= 512 && tm_smem_bytes(L->max_unit_bytes, L->max_slots, L->rank_in) <= 220 * 1024 &&
         L->num_experts <= TM_MAX_E && L->rank_in % 8 == 0;
}

int launch_experts_decode_tm(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                             const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, cudaStream_t st) {
  BM_REQUIRE(experts_decode_tm_fits(L), BM_ERR_UNSUPPORTED, "experts_decode_tm: layer with %d slots does not fit", L->max_slots);
  BM_REQUIRE((reinterpret_cast<uintptr_t>(h_gate) & 15u) == 0 && (reinterpret_cast<uintptr_t>(h_up) & 15u) == 0, BM_ERR_INVALID_ARG,
             "experts_decode_tm: h_gate / h_up rows must be 16-byte aligned (rank %d)", L->rank_in);
  const size_t smem = tm_smem_bytes(L->max_unit_bytes, L->max_slots, L->rank_in);
  static int attr_set_for = -1;
  static int sm_count = 148;
  if (attr_set_for != L->device) {
    BM_CUDA(cudaFuncSetAttribute(experts_decode_tm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    BM_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, L->device));
    attr_set_for = L->device;
  }
  const int nkb_max = L->max_slots / 16, n_mt_max = (L->max_slots + 127) / 128;
  const int a_cols = nkb_max * 16 > n_mt_max * 64 ? nkb_max * 16 : n_mt_max * 64;
  int grid = sm_count;   // the kernel takes all 512 tensor-memory columns: one CTA per SM
  const int max_units = L->num_experts * L->n_tiles;
  if (grid > max_units) grid = max_units;
  // at least 116 KB of shared memory per CTA keeps a second CTA (which would wait for tensor memory) off the SM
  const size_t smem_launch = smem < 120 * 1024 ? 120 * 1024 : smem;
  experts_decode_tm_kernel<<<grid, TM_THREADS, smem_launch, st>>>(
      L->fast_dev, static_cast<const unsigned char*>(L->arena), h_gate, h_up, L->rank_in, token_indices, expert_offsets,
      route_w, L->rank_out, T, L->num_experts, L->n_tiles, L->intermediate, L->max_unit_bytes, L->max_slots, a_cols,
      rank_accum, L->status_dev);
  BM_LAUNCH_CHECK("experts_decode_tm_kernel");
  return BM_OK;
}

}  // namespace bm
