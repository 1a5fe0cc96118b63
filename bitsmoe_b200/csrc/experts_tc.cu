// Packed routed-expert forward for large token counts (prefill): fused mixed-bit grouped GEMM on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Work item = (expert, block of up to 64 of its assignments).  One persistent CTA per SM walks the items.
// For an item the three products of every 128-column tile run with the WEIGHTS as the 128-row operand:
//   gate/up:  D_g[c, n] = sum_slot  W_g[c, slot] * act_g[n, slot]      (M = 128 columns c, N = 64 tokens)
//   down:     D_d[slot, n] += sum_c W_d[slot, c] * z[n, c]             (M = 128 row slots x 3, N = 64 tokens)
// so decode-like small N and prefill share one tile shape, and D_d accumulates over all tiles in TMEM.
// Warp roles (576 threads):
//   warps 0-7   epilogue (two per TMEM lane quarter, 32 token columns each): tcgen05.ld D_g/D_u -> z = silu(g)*u -> fp16 Z tile in shared memory; at the end of
//               the item D_d -> * s * route weight -> fp32 atomics into rank_accum
//   warp  8     producer: item descriptor, cp.async.bulk of the packed words + scales of (tile, matrix)
//               sections into a 3-slot ring
//   warp  9     MMA issue (one thread) and tcgen05.commit to the ring / phase mbarriers
//   warps 10-17 converters: arena words (nibble / dense 2-bit codes) -> fp16 (q * scale) A-operand stages of 128 rows x 16 K in the
//               canonical K-major core-matrix layout, 4-stage ring of 4 blocks; they also build the activation operand
//               act[n, slot] = fp16(h[token, rank(slot)] * s(slot)) once per item
// Every mbarrier wait is bounded in time and aborts the whole CTA through a shared flag.
#include "fast_layout.cuh"
#include "tc05.cuh"

namespace bm {

constexpr int XT_NT = 64;                 // tokens (assignments) per item = MMA N
constexpr int XT_THREADS = 576;
constexpr int XT_EPI_WARPS = 8, XT_PRODUCER_WARP = 8, XT_MMA_WARP = 9, XT_DQ_WARP0 = 10, XT_DQ_WARPS = 8;
constexpr int XT_RING = 4;                // A-operand stages
constexpr int XT_STAGE_BLOCKS = 4;        // contraction blocks of 16 per stage (one per dequantiser warp pair)
constexpr int XT_A_CHUNK = 128 * 16 + 32;  // bytes between 8-position chunks of a weight stage (padded: conflict-free 16-byte stores)
constexpr int XT_STAGE_BYTES = 2 * XT_STAGE_BLOCKS * XT_A_CHUNK;
constexpr int XT_CHUNK_STRIDE = XT_NT * 16 + 16;   // bytes between 8-position chunks of the token-side operands (padded: conflict-free stores)
constexpr int XT_MAX_E = 1024;
constexpr int XT_SEC = 5;                 // section slots: (tile, matrix) sections up to five ahead

struct XtBars {
  uint64_t sec_full[XT_SEC], sec_empty[XT_SEC];
  uint64_t w_full[XT_RING], w_empty[XT_RING];
  uint64_t act_ready, gu_done, z_ready, tmem_gu_free, down_done;
};

struct XtItem {
  FastExpert fe;
  int tok[XT_NT];
  float rw[XT_NT];
  int n, expert;
};

__device__ __forceinline__ bool xt_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t backoff_ns = 0) {
  const uint32_t addr = tc::smem_u32(bar);
  uint64_t t0 = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(20000u)
        : "memory");
    if (done) return true;
    if (*abort_flag) return false;
    if (backoff_ns) __nanosleep(backoff_ns);
    if ((i & 15u) == 15u) {
      const uint64_t now = tc::global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > tc::WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
  }
}

// One arena word (a 16x16 block's codes owned by lane (g, t), see fast_layout.cuh) -> four fp16 pairs
// (q * scale): r[0] = row g, k (2t, 2t+1); r[1] = row g+8, same k; r[2] = row g, k (2t+8, 2t+9); r[3] = row g+8.
// The code sits in the mantissa of 1024 (fields at bit 0) or of 64 (fields at bit 4); subtracting
// 1024 + offset or 64 + offset is exact, the multiplication by the scale rounds once, as fp16(q * scale) does.
template <bool DENSE>
__device__ __forceinline__ void dequant_block(uint32_t w, __half2 s0, __half2 s1, __half2 s2, __half2 s3, uint32_t (&r)[4]) {
  constexpr uint32_t mlo = DENSE ? 0x00030003u : 0x000F000Fu, mhi = DENSE ? 0x00300030u : 0x00F000F0u;
  constexpr uint32_t off = DENSE ? FAST_DENSE_OFFSET : FAST_NIB_OFFSET;
  constexpr uint32_t blo_bits = 0x64006400u + off * 0x00010001u;          // fp16x2 of 1024 + offset
  constexpr uint32_t bhi_bits = 0x54005400u + off * 0x00100010u;          // fp16x2 of 64 + offset
  const uint32_t blo_u = blo_bits, bhi_u = bhi_bits;
  const __half2 blo = *reinterpret_cast<const __half2*>(&blo_u), bhi = *reinterpret_cast<const __half2*>(&bhi_u);
  const uint32_t sh = w >> (DENSE ? 2 : 8);
  uint32_t v[4] = {(w & mlo) | 0x64006400u, (w & mhi) | 0x54005400u, (sh & mlo) | 0x64006400u, (sh & mhi) | 0x54005400u};
  const __half2 o0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v[0]), blo), s0);
  const __half2 o1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v[1]), bhi), s1);
  const __half2 o2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v[2]), blo), s2);
  const __half2 o3 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&v[3]), bhi), s3);
  r[0] = *reinterpret_cast<const uint32_t*>(&o0);
  r[1] = *reinterpret_cast<const uint32_t*>(&o1);
  r[2] = *reinterpret_cast<const uint32_t*>(&o2);
  r[3] = *reinterpret_cast<const uint32_t*>(&o3);
}

// The two blocks of a pair -> the two 16-byte chunks (rows 16x+g and 16x+g+8) of K-chunk 4*pair_in_stage + t.
// `word0` / `word1` are the pair's two blocks (dense: the same word, the second shifted by 8).
template <bool DENSE>
__device__ __forceinline__ void dequant_pair_store(uint32_t word0, uint32_t word1, const __half2 (&sa)[4], const __half2 (&sb)[4],
                                                   unsigned char* dst) {
  uint32_t r0[4], r1[4];
  dequant_block<DENSE>(word0, sa[0], sb[0], sa[1], sb[1], r0);
  dequant_block<DENSE>(word1, sa[2], sb[2], sa[3], sb[3], r1);
  *reinterpret_cast<uint4*>(dst) = make_uint4(r0[0], r0[2], r1[0], r1[2]);
  *reinterpret_cast<uint4*>(dst + 128) = make_uint4(r0[1], r0[3], r1[1], r1[3]);
}

struct XtSmem {
  unsigned char* act;     // [2][nchunks][XT_NT rows] canonical K-major, 16-byte chunks
  unsigned char* z;       // [16 chunks][XT_NT rows]
  unsigned char* ring;    // [XT_RING][XT_STAGE_BYTES]
  unsigned char* sec[XT_SEC];  // section buffers: [scale (sec_scale_bytes) | words]
  int* prefix;            // [E + 1] items before each expert
  int16_t* rank_s;        // [2][max_slots] logical rank per slot (gate, up) of the current item's expert
  __half* s_s;            // [2][max_slots]
};

__host__ __device__ inline size_t xt_sec_bytes(int max_slots, int max_words) {
  return align_up_c(static_cast<size_t>(max_slots) * 2, 128) + align_up_c(static_cast<size_t>(max_words) * 4, 128);
}
__host__ __device__ inline size_t xt_smem_bytes(int max_slots, int max_words, int num_experts) {
  size_t o = 0;
  o += static_cast<size_t>(2) * (max_slots / 8) * XT_CHUNK_STRIDE;   // act
  o += static_cast<size_t>(N_TILE / 8) * XT_CHUNK_STRIDE;            // z
  o = align_up_c(o, 128) + static_cast<size_t>(XT_RING) * XT_STAGE_BYTES;       // ring
  o += XT_SEC * xt_sec_bytes(max_slots, max_words);
  o += align_up_c(static_cast<size_t>(num_experts + 1) * 4, 128);
  o += align_up_c(static_cast<size_t>(2) * max_slots * 4, 128);
  return o + 1024;                                          // slack for the 1024-byte base alignment
}

__global__ void __launch_bounds__(XT_THREADS, 1) experts_tc_kernel(
    const FastExpert* __restrict__ fast, const unsigned char* __restrict__ arena, const __half* __restrict__ h_gate,
    const __half* __restrict__ h_up, int h_rank, const int32_t* __restrict__ token_indices,
    const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w, int rank_out, int T, int num_experts,
    int n_tiles, int max_slots, int max_words, float* __restrict__ rank_accum, long long* __restrict__ acc64,
    int* __restrict__ status) {
  extern __shared__ unsigned char xt_raw[];
  __shared__ __align__(8) XtBars bars;
  __shared__ XtItem item;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  XtSmem sm;
  {
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(xt_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    size_t o = 0;
    sm.act = base; o += static_cast<size_t>(2) * (max_slots / 8) * XT_CHUNK_STRIDE;
    sm.z = base + o; o += static_cast<size_t>(N_TILE / 8) * XT_CHUNK_STRIDE;
    o = align_up_c(o, 128);
    sm.ring = base + o; o += static_cast<size_t>(XT_RING) * XT_STAGE_BYTES;
    for (int i = 0; i < XT_SEC; ++i) { sm.sec[i] = base + o; o += xt_sec_bytes(max_slots, max_words); }
    sm.prefix = reinterpret_cast<int*>(base + o); o += align_up_c(static_cast<size_t>(num_experts + 1) * 4, 128);
    sm.rank_s = reinterpret_cast<int16_t*>(base + o);
    sm.s_s = reinterpret_cast<__half*>(base + o + static_cast<size_t>(2) * max_slots * 2);
  }
  const size_t sec_scale_bytes = align_up_c(static_cast<size_t>(max_slots) * 2, 128);
  if (threadIdx.x == 0) {
    for (int i = 0; i < XT_SEC; ++i) { tc::mbar_init(&bars.sec_full[i], 1); tc::mbar_init(&bars.sec_empty[i], XT_DQ_WARPS); }
    for (int i = 0; i < XT_RING; ++i) { tc::mbar_init(&bars.w_full[i], XT_DQ_WARPS / 2); tc::mbar_init(&bars.w_empty[i], 1); }
    tc::mbar_init(&bars.act_ready, 1);
    tc::mbar_init(&bars.gu_done, 1);
    tc::mbar_init(&bars.z_ready, XT_EPI_WARPS);
    tc::mbar_init(&bars.tmem_gu_free, XT_EPI_WARPS);
    tc::mbar_init(&bars.down_done, 1);
    tc::mbar_init_fence();
    abort_flag_s = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);
  // items before each expert (an item = up to XT_NT consecutive assignments of one expert): every thread loads
  // its experts' counts in parallel, one warp then scans them
  for (int e = threadIdx.x; e < num_experts; e += XT_THREADS)
    sm.prefix[e + 1] = (expert_offsets[e + 1] - expert_offsets[e] + XT_NT - 1) / XT_NT;
  __syncthreads();
  if (warp == 1) {
    int carry = 0;
    for (int base = 0; base < num_experts; base += 32) {
      const int e = base + lane;
      int v = e < num_experts ? sm.prefix[e + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += n;
      }
      if (e < num_experts) sm.prefix[e + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) sm.prefix[0] = 0;
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem_base = tmem_slot;
  const int n_items = sm.prefix[num_experts];
  const uint32_t idesc = tc::idesc_f16(128, XT_NT);
  const uint32_t d_gate = tmem_base, d_up = tmem_base + XT_NT, d_down = tmem_base + 2 * XT_NT;

  // running counters shared by construction between roles (every role advances them identically)
  uint32_t ring_i = 0;      // A-operand stages produced / consumed so far
  uint32_t gu_round = 0;    // gate/up rounds (one per tile) so far
  uint32_t sec_round = 0;   // tiles so far (each uses the three section slots once)
  uint32_t item_round = 0;

  for (int it = blockIdx.x; it < n_items; it += gridDim.x, ++item_round) {
    __syncthreads();   // previous item completely finished (TMEM read out, item info free)
    if (warp == XT_PRODUCER_WARP) {
      // locate the item: last expert e with prefix[e] <= it
      int lo = 0, hi = num_experts - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (sm.prefix[mid] <= it) lo = mid; else hi = mid - 1;
      }
      const int e = lo;
      const int a0 = expert_offsets[e] + (it - sm.prefix[e]) * XT_NT;
      const int n = min(XT_NT, expert_offsets[e + 1] - a0);
      for (int i = lane; i < static_cast<int>(sizeof(FastExpert) / 4); i += 32)
        reinterpret_cast<uint32_t*>(&item.fe)[i] = reinterpret_cast<const uint32_t*>(&fast[e])[i];
      for (int i = lane; i < XT_NT; i += 32) {
        int tk = i < n ? token_indices[a0 + i] : 0;
        const bool good = i < n && tk >= 0 && tk < T;
        item.tok[i] = good ? tk : 0;
        item.rw[i] = good ? route_w[a0 + i] : 0.f;
      }
      if (lane == 0) { item.n = n; item.expert = e; }
    }
    __syncthreads();
    const FastExpert& fe = item.fe;
    const int n_tok = item.n;
    const int nblk_d = fe.m[2].nslots >> 4;
    const int n_mt = (nblk_d + 7) >> 3;   // 128-row tiles of the down product (<= 3)

    // ---- activation operand, once per item, by every warp except the producer and the MMA issuer
    if (warp != XT_PRODUCER_WARP && warp != XT_MMA_WARP) {
      constexpr int XT_STAGERS = (XT_EPI_WARPS + XT_DQ_WARPS) * 32;
      const int tid_s = warp < XT_EPI_WARPS ? threadIdx.x : threadIdx.x - 64;
      const uint32_t act_m_bytes = static_cast<uint32_t>(max_slots / 8) * XT_CHUNK_STRIDE;
      // activation operand, once per item: act[m][chunk][n] = 8 consecutive contraction positions of token n
      for (int m = 0; m < 2; ++m) {
        const FastMat& fm = fe.m[m];
        const int16_t* rank_t = reinterpret_cast<const int16_t*>(arena + fm.tab_off);
        const __half* s_t = reinterpret_cast<const __half*>(arena + fm.tab_off + fm.nslots * 2);
        for (int i = tid_s; i < fm.nslots; i += XT_STAGERS) {
          const int rk = rank_t[i];
          const bool live = rk >= 0 && rk < h_rank;
          sm.rank_s[m * max_slots + i] = static_cast<int16_t>(live ? rk : 0);
          sm.s_s[m * max_slots + i] = live ? s_t[i] : __float2half(0.f);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(XT_STAGERS) : "memory");
      for (int m = 0; m < 2; ++m) {
        const FastMat& fm = fe.m[m];
        const __half* h = m == 0 ? h_gate : h_up;
        const int16_t* rk_s = sm.rank_s + m * max_slots;
        const __half* sv_s = sm.s_s + m * max_slots;
        const int nchunks = fm.nslots >> 3;
#pragma unroll 2
        for (int task = tid_s; task < nchunks * XT_NT; task += XT_STAGERS) {
          const int n = task / nchunks, c8 = task % nchunks;
          const __half* hrow = h + static_cast<int64_t>(item.tok[n]) * h_rank;
          const float live = n < n_tok ? 1.f : 0.f;
          int slot[8];
          __half hv[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            slot[j] = ((c8 >> 2) << 5) + pos32_inv((c8 & 3) * 8 + j);   // chunk c8 = positions 8 c8 .. 8 c8 + 7 of the pos32 order
            hv[j] = hrow[rk_s[slot[j]]];
          }
          __half v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __float2half_rn(__half2float(hv[j]) * __half2float(sv_s[slot[j]]) * live);
          *reinterpret_cast<uint4*>(sm.act + m * act_m_bytes + c8 * XT_CHUNK_STRIDE + (n >> 3) * 128 + (n & 7) * 16) =
              *reinterpret_cast<uint4*>(v);
        }
      }
      tc::fence_async_smem();
      asm volatile("bar.sync 1, %0;" ::"n"(XT_STAGERS) : "memory");
      if (tid_s == 0) tc::mbar_arrive(&bars.act_ready);

    }
    if (warp == XT_PRODUCER_WARP) {
      // ------------------------------------------------------------------ producer
      if (lane == 0) {
        uint32_t sr = sec_round;
        for (int tile = 0; tile < n_tiles && !*abort_flag; ++tile, ++sr) {
          const unsigned char* unit = arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes;
          for (int m = 0; m < 3; ++m) {
            const uint32_t use = sr * 3u + m, ss = use % XT_SEC;
            if (!xt_wait(&bars.sec_empty[ss], ((use / XT_SEC) & 1) ^ 1, abort_flag)) break;
            const uint32_t sb = static_cast<uint32_t>(fe.m[m].nslots) * 2u, wb = static_cast<uint32_t>(fe.m[m].words) * 4u;
            tc::mbar_expect_tx(&bars.sec_full[ss], sb + wb);
            tc::bulk_g2s(sm.sec[ss], unit + fe.sec_off[m], sb, &bars.sec_full[ss]);
            tc::bulk_g2s(sm.sec[ss] + sec_scale_bytes, unit + fe.sec_off[3 + m], wb, &bars.sec_full[ss]);
          }
        }
      }
    } else if (warp == XT_MMA_WARP) {
      // ------------------------------------------------------------------ MMA issue
      if (lane == 0) {
        bool ok = xt_wait(&bars.act_ready, item_round & 1, abort_flag);
        uint32_t ri = ring_i, gr = gu_round;
        const uint32_t act_base = tc::smem_u32(sm.act), z_base = tc::smem_u32(sm.z), ring_base = tc::smem_u32(sm.ring);
        const uint32_t act_m_bytes = static_cast<uint32_t>(max_slots / 8) * XT_CHUNK_STRIDE;
        // descriptors: constant upper part, start-address field advanced per block
        const uint64_t a_desc0 = tc::smem_desc_kmajor(ring_base, XT_A_CHUNK, 128);
        const uint64_t b_desc0 = tc::smem_desc_kmajor(act_base, XT_CHUNK_STRIDE, 128);
        const uint64_t z_desc0 = tc::smem_desc_kmajor(z_base, XT_CHUNK_STRIDE, 128);
        for (int tile = 0; tile < n_tiles && ok; ++tile, ++gr) {
          if (gr > 0) ok = xt_wait(&bars.tmem_gu_free, (gr - 1) & 1, abort_flag);
          for (int m = 0; m < 2 && ok; ++m) {
            const int nkb = fe.m[m].nslots >> 4;
            const uint64_t bm_desc = b_desc0 + ((m * act_m_bytes) >> 4);
            for (int kb0 = 0; kb0 < nkb; kb0 += XT_STAGE_BLOCKS, ++ri) {
              const int slot = ri % XT_RING;
              if (!(ok = xt_wait(&bars.w_full[slot], (ri / XT_RING) & 1, abort_flag))) break;
              tc::fence_after_sync();
              const int cnt = min(XT_STAGE_BLOCKS, nkb - kb0);
              for (int j = 0; j < cnt; ++j) {
                const uint64_t ad = a_desc0 + ((slot * XT_STAGE_BYTES + 2 * j * XT_A_CHUNK) >> 4);
                const uint64_t bd = bm_desc + ((2 * (kb0 + j) * XT_CHUNK_STRIDE) >> 4);
                tc::mma_f16(m == 0 ? d_gate : d_up, ad, bd, idesc, (kb0 + j) > 0 ? 1u : 0u);
              }
              tc::mma_commit(&bars.w_empty[slot]);
            }
          }
          if (!ok) break;
          tc::mma_commit(&bars.gu_done);
          ok = xt_wait(&bars.z_ready, gr & 1, abort_flag);
          for (int mt = 0; mt < n_mt && ok; ++mt) {
            for (int kb0 = 0; kb0 < 8; kb0 += XT_STAGE_BLOCKS, ++ri) {
              const int slot = ri % XT_RING;
              if (!(ok = xt_wait(&bars.w_full[slot], (ri / XT_RING) & 1, abort_flag))) break;
              tc::fence_after_sync();
              for (int j = 0; j < XT_STAGE_BLOCKS; ++j) {
                const uint64_t ad = a_desc0 + ((slot * XT_STAGE_BYTES + 2 * j * XT_A_CHUNK) >> 4);
                const uint64_t bd = z_desc0 + ((2 * (kb0 + j) * XT_CHUNK_STRIDE) >> 4);
                tc::mma_f16(d_down + mt * XT_NT, ad, bd, idesc, (tile > 0 || kb0 + j > 0) ? 1u : 0u);
              }
              tc::mma_commit(&bars.w_empty[slot]);
            }
          }
          if (ok) tc::mma_commit(&bars.down_done);
        }
      }
    }
    else if (warp >= XT_DQ_WARP0) {
      // ------------------------------------------------------------------ dequantisers
      const int dw = warp - XT_DQ_WARP0;
      // Two teams of four warps take alternate stages (two pairs of 16-blocks x 128 operand rows); inside a team
      // warp `wt` converts the operand-row blocks x = wt and wt + 4, so two stages are always in flight.
      const int team = dw >> 2, wt = dw & 3, g = lane >> 2, t = lane & 3;
      uint32_t ri = ring_i, sr = sec_round;
      bool ok = true;
      for (int tile = 0; tile < n_tiles && ok; ++tile, ++sr) {
        for (int m = 0; m < 2 && ok; ++m) {
          const uint32_t use = sr * 3u + m, ss = use % XT_SEC;
          ok = xt_wait(&bars.sec_full[ss], (use / XT_SEC) & 1, abort_flag);
          if (!ok) break;
          const FastMat& fm = fe.m[m];
          const uint32_t* words = reinterpret_cast<const uint32_t*>(sm.sec[ss] + sec_scale_bytes);
          const uint4* scale4 = reinterpret_cast<const uint4*>(sm.sec[ss]);    // 8 halves per (pair, t)
          const int npairs = fm.nslots >> 5, nib_pairs = fm.nblk[0] >> 1;
          const uint32_t* dense_words = words + fm.nblk[0] * 256;
          for (int p0 = 0; p0 < npairs; p0 += 2, ++ri) {
            if (static_cast<int>(ri & 1u) != team) continue;
            const int slot = ri % XT_RING;
            if (!(ok = xt_wait(&bars.w_empty[slot], ((ri / XT_RING) & 1) ^ 1, abort_flag))) break;
            unsigned char* stage = sm.ring + slot * XT_STAGE_BYTES;
#pragma unroll
            for (int pp = 0; pp < 2; ++pp) {
              const int pr = p0 + pp;
              if (pr >= npairs) break;
              const uint4 sv = scale4[pr * 4 + t];
              const __half2 sc[4] = {*reinterpret_cast<const __half2*>(&sv.x), *reinterpret_cast<const __half2*>(&sv.y),
                                     *reinterpret_cast<const __half2*>(&sv.z), *reinterpret_cast<const __half2*>(&sv.w)};
              unsigned char* dst = stage + (pp * 4 + t) * XT_A_CHUNK + g * 16;
              if (pr < nib_pairs) {
                const uint2 w0 = reinterpret_cast<const uint2*>(words)[(pr * 8 + wt) * 32 + lane];
                const uint2 w1 = reinterpret_cast<const uint2*>(words)[(pr * 8 + wt + 4) * 32 + lane];
                dequant_pair_store<false>(w0.x, w0.y, sc, sc, dst + wt * 256);
                dequant_pair_store<false>(w1.x, w1.y, sc, sc, dst + (wt + 4) * 256);
              } else {
                const int dp = pr - nib_pairs;
                const uint32_t w0 = dense_words[(dp * 8 + wt) * 32 + lane];
                const uint32_t w1 = dense_words[(dp * 8 + wt + 4) * 32 + lane];
                dequant_pair_store<true>(w0, w0 >> 8, sc, sc, dst + wt * 256);
                dequant_pair_store<true>(w1, w1 >> 8, sc, sc, dst + (wt + 4) * 256);
              }
            }
            tc::fence_async_smem();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bars.w_full[slot]);
          }
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bars.sec_empty[ss]);
        }
        if (!ok) break;
        const uint32_t use_d = sr * 3u + 2u, sd = use_d % XT_SEC;
        ok = xt_wait(&bars.sec_full[sd], (use_d / XT_SEC) & 1, abort_flag);
        if (!ok) break;
        const FastMat& fd = fe.m[2];
        const uint32_t* dwords = reinterpret_cast<const uint32_t*>(sm.sec[sd] + sec_scale_bytes);
        const uint32_t* ddense = dwords + fd.nblk[0] * 256;
        const __half* scale_d = reinterpret_cast<const __half*>(sm.sec[sd]);
        for (int mt = 0; mt < n_mt && ok; ++mt) {
          // this thread's two operand-row blocks: slot blocks 8*mt + wt and 8*mt + wt + 4
          __half2 sg[2], sh[2];
          int mbu[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            mbu[u] = 8 * mt + wt + 4 * u;
            sg[u] = sh[u] = __float2half2_rn(0.f);
            if (mbu[u] < nblk_d) {
              sg[u] = __half2half2(scale_d[16 * mbu[u] + g]);
              sh[u] = __half2half2(scale_d[16 * mbu[u] + g + 8]);
            }
          }
          for (int p0 = 0; p0 < 4; p0 += 2, ++ri) {
            if (static_cast<int>(ri & 1u) != team) continue;
            const int slot = ri % XT_RING;
            if (!(ok = xt_wait(&bars.w_empty[slot], ((ri / XT_RING) & 1) ^ 1, abort_flag))) break;
            unsigned char* stage = sm.ring + slot * XT_STAGE_BYTES;
#pragma unroll
            for (int pp = 0; pp < 2; ++pp) {
              const int pr = p0 + pp;
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                unsigned char* dst = stage + (pp * 4 + t) * XT_A_CHUNK + g * 16 + (wt + 4 * u) * 256;
                const __half2 sa[4] = {sg[u], sg[u], sg[u], sg[u]};
                const __half2 sb[4] = {sh[u], sh[u], sh[u], sh[u]};
                const int mb = mbu[u];
                if (mb >= nblk_d) {
                  *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                  *reinterpret_cast<uint4*>(dst + 128) = make_uint4(0, 0, 0, 0);
                } else if (mb < fd.nblk[0]) {
                  const uint2 w = reinterpret_cast<const uint2*>(dwords)[(mb * 4 + pr) * 32 + lane];
                  dequant_pair_store<false>(w.x, w.y, sa, sb, dst);
                } else {
                  const uint32_t w = ddense[((mb - fd.nblk[0]) * 4 + pr) * 32 + lane];
                  dequant_pair_store<true>(w, w >> 8, sa, sb, dst);
                }
              }
            }
            tc::fence_async_smem();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&bars.w_full[slot]);
          }
        }
        __syncwarp();
        if (ok && lane == 0) tc::mbar_arrive(&bars.sec_empty[sd]);
      }
    } else {
      // ------------------------------------------------------------------ epilogue warps 0-3
      const int q = warp & 3, nhalf = (warp >> 2) * 32;      // lane quarter, first of this warp's 32 token columns
      const uint32_t lane_sel = static_cast<uint32_t>(32 * q) << 16;
      uint32_t gr = gu_round;
      bool ok = true;
      const int c = 32 * q + lane;                                   // row of D_g / D_u = column of the tile
      const int c_pos = slot_pos(c);
      unsigned char* zrow = sm.z + (c_pos >> 3) * XT_CHUNK_STRIDE + (c_pos & 7) * 2;
      for (int tile = 0; tile < n_tiles && ok; ++tile, ++gr) {
        ok = xt_wait(&bars.gu_done, gr & 1, abort_flag, 200);
        if (ok && gr > 0) ok = xt_wait(&bars.down_done, (gr - 1) & 1, abort_flag, 200);
        if (!ok) break;
        tc::fence_after_sync();
        {
          const int n0 = nhalf;
          float gv[32], uv[32];
          tc::tmem_ld32(d_gate + lane_sel + n0, gv);
          tc::tmem_ld32(d_up + lane_sel + n0, uv);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int n = n0 + i;
            const float zf = __fdividef(gv[i] * uv[i], 1.f + __expf(-gv[i]));
            *reinterpret_cast<__half*>(zrow + (n >> 3) * 128 + (n & 7) * 16) = __float2half_rn(n < n_tok ? zf : 0.f);
          }
        }
        tc::fence_before_sync();
        tc::fence_async_smem();
        __syncwarp();
        if (lane == 0) { tc::mbar_arrive(&bars.tmem_gu_free); tc::mbar_arrive(&bars.z_ready); }
      }
      if (ok) ok = xt_wait(&bars.down_done, (gr - 1) & 1, abort_flag, 200);
      if (ok) {
        tc::fence_after_sync();
        const FastMat& fd = fe.m[2];
        const int16_t* rank_d = reinterpret_cast<const int16_t*>(arena + fd.tab_off);
        const __half* s_d = reinterpret_cast<const __half*>(arena + fd.tab_off + fd.nslots * 2);
        for (int mt = 0; mt < n_mt; ++mt) {
          const int slot = 128 * mt + 32 * q + lane;
          int rk = -1;
          float sv = 0.f;
          if (slot < fd.nslots) { rk = rank_d[slot]; sv = __half2float(s_d[slot]); }
          const bool live = rk >= 0 && rk < rank_out;
          {
            const int n0 = nhalf;
            float v[32];
            tc::tmem_ld32(d_down + mt * XT_NT + lane_sel + n0, v);
            if (live) {
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int n = n0 + i;
                if (n < n_tok) acc_add(rank_accum, acc64, static_cast<int64_t>(item.tok[n]) * rank_out + rk, v[i] * sv * item.rw[n]);
              }
            }
          }
        }
        tc::fence_before_sync();
      }
    }
    // every role advances the shared counters identically
    gu_round += n_tiles;
    sec_round += n_tiles;
    ring_i += static_cast<uint32_t>(n_tiles) * ((((fe.m[0].nslots >> 4) + XT_STAGE_BLOCKS - 1) / XT_STAGE_BLOCKS) +
                                                (((fe.m[1].nslots >> 4) + XT_STAGE_BLOCKS - 1) / XT_STAGE_BLOCKS) +
                                                n_mt * (8 / XT_STAGE_BLOCKS));
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && abort_flag_s) atomicExch(status, BM_ERR_TIMEOUT);
}

// Whether the layer's largest expert fits the tensor path's shared- and tensor-memory budget (AUTO falls back to the
// decode path otherwise).
bool experts_tc_fits(const bm_layer* L) {
  return L->num_experts <= XT_MAX_E && L->intermediate % N_TILE == 0 && L->max_slots <= 3 * 128 &&
         xt_smem_bytes(L->max_slots, L->max_words, L->num_experts) <= 224 * 1024;
}

int launch_experts_tc(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                      const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, long long* acc64,
                      cudaStream_t st) {
  BM_REQUIRE(L->num_experts <= XT_MAX_E, BM_ERR_UNSUPPORTED, "experts_tc: more than %d experts", XT_MAX_E);
  BM_REQUIRE(L->intermediate % N_TILE == 0, BM_ERR_UNSUPPORTED, "experts_tc: intermediate size must be a multiple of %d", N_TILE);
  BM_REQUIRE(L->max_slots <= 3 * 128, BM_ERR_UNSUPPORTED, "experts_tc: %d row slots exceed the tensor-memory budget", L->max_slots);
  const size_t smem = xt_smem_bytes(L->max_slots, L->max_words, L->num_experts);
  BM_REQUIRE(smem <= 224 * 1024, BM_ERR_UNSUPPORTED, "experts_tc: layer needs %zu bytes of shared memory", smem);
  static PerDeviceOnce attr_once;
  static int sm_counts[MAX_DEVICES];
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  BM_REQUIRE(dev >= 0 && dev < MAX_DEVICES, BM_ERR_UNSUPPORTED, "experts_tc: device ordinal %d out of range", dev);
  if (!attr_once.is_done(dev)) {
    BM_CUDA(cudaFuncSetAttribute(experts_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
    BM_CUDA(cudaDeviceGetAttribute(&sm_counts[dev], cudaDevAttrMultiProcessorCount, dev));
    attr_once.mark(dev);
  }
  const int sm_count = sm_counts[dev];
  experts_tc_kernel<<<sm_count, XT_THREADS, smem, st>>>(
      L->fast_dev, static_cast<const unsigned char*>(L->arena), h_gate, h_up, L->rank_in, token_indices, expert_offsets,
      route_w, L->rank_out, T, L->num_experts, L->n_tiles, L->max_slots, L->max_words, rank_accum, acc64, L->status_dev);
  BM_LAUNCH_CHECK("experts_tc_kernel");
  return BM_OK;
}

}  // namespace bm
