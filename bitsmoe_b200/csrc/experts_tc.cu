// Packed routed-expert forward for large token counts (prefill): fused mixed-bit grouped GEMM on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Work item = (expert, block of up to NT of its assignments; NT -- 64 where it fits -- is chosen per layer so that the
// activation operand of an item, two z tiles and enough copy / conversion stages fit in shared memory and seven
// accumulators of NT columns fit in tensor memory).  One persistent CTA per SM walks the
// items.  For an item the three products of every 128-column tile run with the WEIGHTS as the 128-row operand:
//   gate/up:  D_g[c, n] = sum_slot  W_g[c, slot] * act_g[n, slot]      (M = 128 columns c, N = the item's tokens)
//   down:     D_d[slot, n] += sum_c W_d[slot, c] * z[n, c]             (M = 128 row slots x 2 or 3, same N)
// N of the MMAs is the item's token count rounded up to 16, so a short item costs a short MMA; every code is converted
// once per item, so the conversion work per token falls with NT.  D_d accumulates over all tiles in TMEM.
// Warp roles (608 threads):
//   warps 0-7   epilogue (two per TMEM lane quarter, alternate 32-token column chunks): tcgen05.ld D_g/D_u ->
//               z = silu(g)*u -> fp16 z tile in shared memory; at the end of the item D_d * s * route weight is
//               transposed through the idle operand ring and added to rank_accum row by row (16-byte vector
//               reductions).  Warp 0 also looks up the next item while the current one runs.
//   warp  8     producer: cp.async.bulk of the packed words + scales of (tile, matrix) sections into a ring of slots
//   warps 9,10  MMA issue, one thread each.  tcgen05.mma blocks its thread until the tensor pipe accepts it, so the
//               waits and commits around a stage cost tensor time when one thread issues everything; two pipelines
//               (9: gate products and the down product's even row tiles, 10: up products and the odd row tiles)
//               hide one another's bookkeeping and never write the same accumulator.
//   warps 11-18 converters, one team of four warps per pipeline: arena words (nibble / dense 2-bit codes) -> fp16
//               (q * scale) operand stages of 128 rows x 64 contraction positions in the canonical K-major
//               core-matrix layout, a ring of stages per pipeline; together with the epilogue warps they also build
//               the activation operand act[n, slot] = fp16(h[token, rank(slot)] * s(slot)) once per item
// Order of the (tile, matrix) sections of an item, the same for the producer, the converters and the MMA issuer:
//   G0 U0 | G1 U1 D0 | G2 U2 D1 | ... | D(last)
// The down product of a tile is issued one tile late, and the gate/up accumulators and the z tile are double-buffered,
// so the tensor pipe works on the next tile's gate/up products while the epilogue warps turn the current tile's
// accumulators into z.
// Every mbarrier wait is bounded in time and aborts the whole CTA through a shared flag.
#include "fast_layout.cuh"
#include "tc05.cuh"

namespace bm {

constexpr int XT_NT_MAX = 96;             // most tokens (assignments) per item = largest MMA N
constexpr int XT_THREADS = 608;
constexpr int XT_EPI_WARPS = 8, XT_PRODUCER_WARP = 8, XT_MMA_WARP0 = 9, XT_DQ_WARP0 = 11, XT_DQ_WARPS = 8;
constexpr int XT_RING_MAX = 8;            // A-operand stages (at most)
constexpr int XT_STAGE_BLOCKS = 4;        // contraction blocks of 16 per stage (one per dequantiser warp pair)
constexpr int XT_A_CHUNK = 128 * 16 + 32;  // bytes between 8-position chunks of a weight stage (padded: conflict-free 16-byte stores)
constexpr int XT_STAGE_BYTES = 2 * XT_STAGE_BLOCKS * XT_A_CHUNK;
// bytes between 8-position chunks of the token-side operands (padded: conflict-free stores)
__host__ __device__ constexpr int xt_chunk_stride(int nt) { return nt * 16 + 16; }
constexpr int XT_MAX_E = 1024;
constexpr int XT_SEC_MAX = 6;             // section slots (at most): (tile, matrix) sections this many ahead

struct XtBars {
  uint64_t sec_full[XT_SEC_MAX], sec_empty[XT_SEC_MAX];
  uint64_t w_full[XT_RING_MAX], w_empty[XT_RING_MAX];
  uint64_t act_ready, down_done;
  // per buffer (running tile number & 1): gate/up accumulators complete / read out, z tile written / consumed
  uint64_t gu_done[2], tmem_gu_free[2], z_ready[2], z_free[2];
};

// Position in a cyclic buffer of n slots with the phase bit of its mbarriers.
struct XtCycle {
  uint32_t i, ph;
  __device__ __forceinline__ void next(uint32_t n) {
    if (++i == n) { i = 0; ph ^= 1u; }
  }
};

struct XtItem {
  FastExpert fe;
  int tok[XT_NT_MAX];
  float rw[XT_NT_MAX];
  int n, expert;
};

__device__ __noinline__ bool xt_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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
    if ((i & 15u) == 15u) {
      const uint64_t now = tc::global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > tc::WAIT_LIMIT_NS) { *abort_flag = 1; return false; }
    }
  }
}
// Bounded wait: one probe inline (the common case in a running pipeline), the time-limited loop out of line.
__device__ __forceinline__ bool xt_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  uint32_t done;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(done)
               : "r"(tc::smem_u32(bar)), "r"(parity)
               : "memory");
  return done ? true : xt_wait_slow(bar, parity, abort_flag);
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
  unsigned char* act;     // [2][nchunks][nt rows] canonical K-major, 16-byte chunks
  unsigned char* z;       // [2 buffers][16 chunks][nt rows]
  unsigned char* ring;    // [2 pipelines][ring_h][XT_STAGE_BYTES]
  unsigned char* sec0;    // sec_n section buffers of sec_stride bytes: [scale (sec_scale_bytes) | words]
  uint32_t sec_stride;
  int* prefix;            // [E + 1] items before each expert
  int32_t* dst_r;         // [2][h_rank] byte offset of a rank's contraction position inside an operand row (gate, up), or -1
  __half* s_r;            // [2][h_rank] its factor s
};

__host__ __device__ inline size_t xt_sec_bytes(int max_slots, int max_words) {
  return align_up_c(static_cast<size_t>(max_slots) * 2, 128) + align_up_c(static_cast<size_t>(max_words) * 4, 128);
}
__host__ __device__ inline size_t xt_smem_bytes(int max_slots, int max_words, int num_experts, int h_rank, int nt, int ring_n, int sec_n) {
  size_t o = 0;
  o += static_cast<size_t>(2) * (max_slots / 8) * xt_chunk_stride(nt);   // act
  o += static_cast<size_t>(2) * (N_TILE / 8) * xt_chunk_stride(nt);      // z, two buffers
  o = align_up_c(o, 128) + static_cast<size_t>(ring_n) * XT_STAGE_BYTES;       // ring
  o += sec_n * xt_sec_bytes(max_slots, max_words);
  o += align_up_c(static_cast<size_t>(num_experts + 1) * 4, 128);
  o += align_up_c(static_cast<size_t>(2) * h_rank * 6, 128);         // per-rank tables of the activation staging
  return o + 1024;                                          // slack for the 1024-byte base alignment
}

// Locates item `it` (last expert e with prefix[e] <= it) and copies what the roles need; one warp.
__device__ __forceinline__ void xt_load_item(XtItem& item, int it, const int* prefix, int num_experts, int nt, int T,
                                             const FastExpert* __restrict__ fast, const int32_t* __restrict__ token_indices,
                                             const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w,
                                             int lane) {
  int lo = 0, hi = num_experts - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= it) lo = mid; else hi = mid - 1;
  }
  const int e = lo;
  const int a0 = expert_offsets[e] + (it - prefix[e]) * nt;
  const int n = min(nt, expert_offsets[e + 1] - a0);
  for (int i = lane; i < static_cast<int>(sizeof(FastExpert) / 4); i += 32)
    reinterpret_cast<uint32_t*>(&item.fe)[i] = reinterpret_cast<const uint32_t*>(&fast[e])[i];
  for (int i = lane; i < nt; i += 32) {
    const int tk = i < n ? token_indices[a0 + i] : 0;
    const bool good = i < n && tk >= 0 && tk < T;
    item.tok[i] = good ? tk : 0;
    item.rw[i] = good ? route_w[a0 + i] : 0.f;
  }
  if (lane == 0) { item.n = n; item.expert = e; }
}

__global__ void __launch_bounds__(XT_THREADS, 1) experts_tc_kernel(
    const FastExpert* __restrict__ fast, const unsigned char* __restrict__ arena, const __half* __restrict__ h_gate,
    const __half* __restrict__ h_up, int h_rank, const int32_t* __restrict__ token_indices,
    const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w, int rank_out, int T, int num_experts,
    int n_tiles, int max_slots, int max_words, int nt, int ring_h, int sec_n, int acc_stride,
    float* __restrict__ rank_accum, long long* __restrict__ acc64, int* __restrict__ status) {
  extern __shared__ unsigned char xt_raw[];
  __shared__ __align__(8) XtBars bars;
  __shared__ XtItem items[2];             // this item and the next one (looked up while this one runs)
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cs = xt_chunk_stride(nt);     // bytes between 8-position chunks of act / z
  XtSmem sm;
  {
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(xt_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    size_t o = 0;
    sm.act = base; o += static_cast<size_t>(2) * (max_slots / 8) * cs;
    sm.z = base + o; o += static_cast<size_t>(2) * (N_TILE / 8) * cs;
    o = align_up_c(o, 128);
    sm.ring = base + o; o += static_cast<size_t>(2 * ring_h) * XT_STAGE_BYTES;
    sm.sec0 = base + o; sm.sec_stride = static_cast<uint32_t>(xt_sec_bytes(max_slots, max_words)); o += static_cast<size_t>(sec_n) * sm.sec_stride;
    sm.prefix = reinterpret_cast<int*>(base + o); o += align_up_c(static_cast<size_t>(num_experts + 1) * 4, 128);
    sm.dst_r = reinterpret_cast<int32_t*>(base + o);
    sm.s_r = reinterpret_cast<__half*>(base + o + static_cast<size_t>(2) * h_rank * 4);
  }
  const size_t sec_scale_bytes = align_up_c(static_cast<size_t>(max_slots) * 2, 128);
  if (threadIdx.x == 0) {
    for (int i = 0; i < XT_SEC_MAX; ++i) { tc::mbar_init(&bars.sec_full[i], 1); tc::mbar_init(&bars.sec_empty[i], XT_DQ_WARPS); }
    for (int i = 0; i < XT_RING_MAX; ++i) { tc::mbar_init(&bars.w_full[i], XT_DQ_WARPS / 2); tc::mbar_init(&bars.w_empty[i], 1); }
    tc::mbar_init(&bars.act_ready, 1);
    tc::mbar_init(&bars.down_done, 2);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.gu_done[i], 2);
      tc::mbar_init(&bars.tmem_gu_free[i], XT_EPI_WARPS);
      tc::mbar_init(&bars.z_ready[i], XT_EPI_WARPS);
      tc::mbar_init(&bars.z_free[i], 2);
    }
    tc::mbar_init_fence();
    abort_flag_s = 0;
  }
  if (warp == 0) tc::tmem_alloc(&tmem_slot, 512);
  // items before each expert (an item = up to nt consecutive assignments of one expert): every thread loads
  // its experts' counts in parallel, one warp then scans them
  for (int e = threadIdx.x; e < num_experts; e += XT_THREADS)
    sm.prefix[e + 1] = (expert_offsets[e + 1] - expert_offsets[e] + nt - 1) / nt;
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
  // accumulators acc_stride columns apart: (gate, up) of buffer 0, of buffer 1, then the down product's row tiles
  const uint32_t d_down = tmem_base + 4 * acc_stride;
  const uint32_t z_bytes = static_cast<uint32_t>(N_TILE / 8) * cs;
  if (warp == 0 && static_cast<int>(blockIdx.x) < n_items)
    xt_load_item(items[0], blockIdx.x, sm.prefix, num_experts, nt, T, fast, token_indices, expert_offsets, route_w, lane);

  // Positions in the cyclic buffers; every role steps through the same sequence of sections and stages, so each keeps
  // its own copy across items.
  XtCycle sec_c{0, 0};      // section slots (producer, converters)
  XtCycle ring_c{0, 0};     // this pipeline's operand stages (converter team / its MMA issuer)
  uint32_t gu_round = 0;    // tiles so far: tile number g uses accumulator / z buffer g & 1 for the (g >> 1)-th time
  uint32_t item_round = 0;

  for (int it = blockIdx.x; it < n_items; it += gridDim.x, ++item_round) {
    __syncthreads();   // previous item completely finished (TMEM read out), this item's description in place
    const XtItem& item = items[item_round & 1];
    const FastExpert& fe = item.fe;
    const int n_tok = item.n;
    const int n_mma = max(16, (n_tok + 15) & ~15);        // N of this item's MMAs; rows n_tok .. n_mma - 1 are zero
    const uint32_t idesc = tc::idesc_f16(128, n_mma);
    const int nblk_d = fe.m[2].nslots >> 4;
    const int n_mt = (nblk_d + 7) >> 3;   // 128-row tiles of the down product (<= 3)

    // ---- activation operand, once per item, by the epilogue and converter warps
    if (warp < XT_EPI_WARPS || warp >= XT_DQ_WARP0) {
      constexpr int XT_STAGERS = (XT_EPI_WARPS + XT_DQ_WARPS) * 32;
      const int tid_s = warp < XT_EPI_WARPS ? threadIdx.x : threadIdx.x - (XT_DQ_WARP0 - XT_EPI_WARPS) * 32;
      const uint32_t act_m_bytes = static_cast<uint32_t>(max_slots / 8) * cs;
      // act[m][chunk][n] = 8 consecutive contraction positions of token n: fp16(h[token, rank(slot)] * s(slot)).
      // A warp takes a token; its lanes read consecutive ranks of the row (reading in slot order instead would touch
      // every 32-byte sector of a row eight times) and store every value where its row slot sits in the operand.
      // Consecutive ranks sit at mostly consecutive positions, so the lanes' 2-byte stores fall into distinct banks.
      // Two tables per matrix, indexed by rank: where the value goes (or -1) and its factor.
      const int warp_s = tid_s >> 5;
      for (int i = tid_s; i < 2 * h_rank; i += XT_STAGERS) {
        sm.dst_r[i] = -1;
        sm.s_r[i] = __float2half(0.f);
      }
      // rows 0 .. n_mma - 1 of every chunk start as zero (padding slots, rows past the item's tokens)
      {
        const int nch0 = fe.m[0].nslots >> 3, nch_all = nch0 + (fe.m[1].nslots >> 3);
        for (int c8 = warp_s; c8 < nch_all; c8 += XT_STAGERS / 32) {
          unsigned char* chunk = sm.act + (c8 >= nch0 ? act_m_bytes + (c8 - nch0) * cs : c8 * cs);
          for (int n = lane; n < n_mma; n += 32) *reinterpret_cast<uint4*>(chunk + n * 16) = make_uint4(0, 0, 0, 0);
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(XT_STAGERS) : "memory");
      for (int m = 0; m < 2; ++m) {
        const FastMat& fm = fe.m[m];
        const int16_t* rank_t = reinterpret_cast<const int16_t*>(arena + fm.tab_off);
        const __half* s_t = reinterpret_cast<const __half*>(arena + fm.tab_off + fm.nslots * 2);
        for (int i = tid_s; i < fm.nslots; i += XT_STAGERS) {
          const int rk = rank_t[i];
          if (rk >= 0 && rk < h_rank) {
            const int pos = slot_pos(i);
            sm.dst_r[m * h_rank + rk] = (pos >> 3) * cs + (pos & 7) * 2;
            sm.s_r[m * h_rank + rk] = s_t[i];
          }
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(XT_STAGERS) : "memory");
      for (int m = 0; m < 2; ++m) {
        const __half* h = m == 0 ? h_gate : h_up;
        for (int r0 = 0; r0 < h_rank; r0 += 256) {        // lane l takes the ranks r0 + l + 32 k
          int dst[8];
          __half sc[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int r = r0 + lane + 32 * k;
            dst[k] = r < h_rank ? sm.dst_r[m * h_rank + r] : -1;
            sc[k] = r < h_rank ? sm.s_r[m * h_rank + r] : __float2half(0.f);
          }
          for (int n = warp_s; n < n_tok; n += 2 * (XT_STAGERS / 32)) {
            // two tokens per round: sixteen loads in flight per lane
            const int n2 = n + XT_STAGERS / 32;
            const __half* row0 = h + static_cast<int64_t>(item.tok[n]) * h_rank + r0 + lane;
            const __half* row1 = h + static_cast<int64_t>(item.tok[n2 < n_tok ? n2 : n]) * h_rank + r0 + lane;
            __half hv0[8], hv1[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              hv0[k] = dst[k] >= 0 ? row0[32 * k] : __float2half(0.f);
              hv1[k] = dst[k] >= 0 ? row1[32 * k] : __float2half(0.f);
            }
            unsigned char* out0 = sm.act + m * act_m_bytes + (n >> 3) * 128 + (n & 7) * 16;
            unsigned char* out1 = sm.act + m * act_m_bytes + (n2 >> 3) * 128 + (n2 & 7) * 16;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (dst[k] >= 0) {
                *reinterpret_cast<__half*>(out0 + dst[k]) = __hmul(hv0[k], sc[k]);      // one rounding of the exact product
                if (n2 < n_tok) *reinterpret_cast<__half*>(out1 + dst[k]) = __hmul(hv1[k], sc[k]);
              }
            }
          }
        }
      }
      tc::fence_async_smem();
      asm volatile("bar.sync 1, %0;" ::"n"(XT_STAGERS) : "memory");
      if (tid_s == 0) tc::mbar_arrive(&bars.act_ready);
      // the next item's description, while this one runs
      if (warp == 0 && it + static_cast<int>(gridDim.x) < n_items)
        xt_load_item(items[(item_round + 1) & 1], it + gridDim.x, sm.prefix, num_experts, nt, T, fast, token_indices,
                     expert_offsets, route_w, lane);
    }
    if (warp == XT_PRODUCER_WARP) {
      // ------------------------------------------------------------------ producer
      if (lane == 0) {
        for (int t = 0; t <= n_tiles && !*abort_flag; ++t) {
          // sections in issue order: gate and up of tile t, then down of tile t - 1
          for (int m = 0; m < 3; ++m) {
            const int tile = m < 2 ? t : t - 1;
            if (tile < 0 || tile >= n_tiles) continue;
            const unsigned char* unit = arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes;
            const uint32_t ss = sec_c.i;
            if (!xt_wait(&bars.sec_empty[ss], sec_c.ph ^ 1, abort_flag)) break;
            const uint32_t sb = static_cast<uint32_t>(fe.m[m].nslots) * 2u, wb = static_cast<uint32_t>(fe.m[m].words) * 4u;
            tc::mbar_expect_tx(&bars.sec_full[ss], sb + wb);
            tc::bulk_g2s(sm.sec0 + ss * sm.sec_stride, unit + fe.sec_off[m], sb, &bars.sec_full[ss]);
            tc::bulk_g2s(sm.sec0 + ss * sm.sec_stride + sec_scale_bytes, unit + fe.sec_off[3 + m], wb, &bars.sec_full[ss]);
            sec_c.next(sec_n);
          }
        }
      }
    } else if (warp == XT_MMA_WARP0 || warp == XT_MMA_WARP0 + 1) {
      // ------------------------------------------------------------------ MMA issue, one thread per pipeline
      // pipeline 0: gate products and the down product's even row tiles; pipeline 1: up products and the odd row tiles
      const int pl = warp - XT_MMA_WARP0;
      // The whole warp waits (a lone waiting lane wakes up several times slower); lane 0 issues.
      {
        bool ok = xt_wait(&bars.act_ready, item_round & 1, abort_flag);
        const uint32_t act_m_bytes = static_cast<uint32_t>(max_slots / 8) * cs;
        // descriptors: constant upper part, start-address field advanced per block
        const uint64_t a_desc0 = tc::smem_desc_kmajor(tc::smem_u32(sm.ring) + pl * ring_h * XT_STAGE_BYTES, XT_A_CHUNK, 128);
        const uint64_t b_desc0 = tc::smem_desc_kmajor(tc::smem_u32(sm.act) + pl * act_m_bytes, cs, 128);
        const uint64_t z_desc0 = tc::smem_desc_kmajor(tc::smem_u32(sm.z), cs, 128);
        uint64_t* w_full = &bars.w_full[pl * ring_h];
        uint64_t* w_empty = &bars.w_empty[pl * ring_h];
        const int nkb = fe.m[pl].nslots >> 4;
        for (int t = 0; t <= n_tiles && ok; ++t) {
          if (t < n_tiles) {
            const uint32_t g = gu_round + t, b = g & 1u, k = g >> 1;
            if (g >= 2) ok = xt_wait(&bars.tmem_gu_free[b], (k - 1) & 1, abort_flag);   // buffer b read out two tiles ago
            tc::fence_after_sync();
            const uint32_t d_acc = tmem_base + (2 * b + pl) * acc_stride;
            for (int kb0 = 0; kb0 < nkb && ok; kb0 += XT_STAGE_BLOCKS) {
              if (!(ok = xt_wait(&w_full[ring_c.i], ring_c.ph, abort_flag))) break;
              if (lane == 0) {
                const int cnt = min(XT_STAGE_BLOCKS, nkb - kb0);
                const uint64_t ad = a_desc0 + ((ring_c.i * XT_STAGE_BYTES) >> 4);
                const uint64_t bd = b_desc0 + ((2 * kb0 * cs) >> 4);
                for (int j = 0; j < cnt; ++j)
                  tc::mma_f16(d_acc, ad + ((2 * j * XT_A_CHUNK) >> 4), bd + ((2 * j * cs) >> 4), idesc, (kb0 + j) > 0 ? 1u : 0u);
                tc::mma_commit(&w_empty[ring_c.i]);
              }
              __syncwarp();
              ring_c.next(ring_h);
            }
            if (!ok) break;
            if (lane == 0) tc::mma_commit(&bars.gu_done[b]);
            __syncwarp();
          }
          if (t > 0) {
            const int tile = t - 1;
            const uint32_t g = gu_round + tile, zb = g & 1u, k = g >> 1;
            ok = xt_wait(&bars.z_ready[zb], k & 1, abort_flag);
            tc::fence_after_sync();
            const uint64_t zd = z_desc0 + ((zb * z_bytes) >> 4);
            for (int mt = pl; mt < n_mt && ok; mt += 2) {
              for (int kb0 = 0; kb0 < 8; kb0 += XT_STAGE_BLOCKS) {
                if (!(ok = xt_wait(&w_full[ring_c.i], ring_c.ph, abort_flag))) break;
                if (lane == 0) {
                  const uint64_t ad = a_desc0 + ((ring_c.i * XT_STAGE_BYTES) >> 4);
                  const uint64_t bd = zd + ((2 * kb0 * cs) >> 4);
                  for (int j = 0; j < XT_STAGE_BLOCKS; ++j)
                    tc::mma_f16(d_down + mt * acc_stride, ad + ((2 * j * XT_A_CHUNK) >> 4), bd + ((2 * j * cs) >> 4), idesc,
                                (tile > 0 || kb0 + j > 0) ? 1u : 0u);
                  tc::mma_commit(&w_empty[ring_c.i]);
                }
                __syncwarp();
                ring_c.next(ring_h);
              }
            }
            if (ok && lane == 0) {
              tc::mma_commit(&bars.z_free[zb]);
              if (t == n_tiles) tc::mma_commit(&bars.down_done);
            }
            __syncwarp();
          }
        }
      }
    } else if (warp >= XT_DQ_WARP0) {
      // ------------------------------------------------------------------ converters
      // Team 0 (four warps) feeds pipeline 0, team 1 pipeline 1; inside a team warp `wt` converts the operand-row
      // blocks x = wt and wt + 4 of every stage (128 operand rows x 4 blocks of 16 contraction positions).
      const int dw = warp - XT_DQ_WARP0;
      const int team = dw >> 2, wt = dw & 3, g = lane >> 2, t = lane & 3;
      unsigned char* ring = sm.ring + team * ring_h * XT_STAGE_BYTES;
      uint64_t* w_full = &bars.w_full[team * ring_h];
      uint64_t* w_empty = &bars.w_empty[team * ring_h];
      bool ok = true;
      for (int tl = 0; tl <= n_tiles && ok; ++tl) {
        for (int m = 0; m < 2 && ok && tl < n_tiles; ++m) {
          const uint32_t ss = sec_c.i;
          // every converter warp waits for and releases every section, also the other team's: a slot's release
          // counts all eight warps whatever the section holds
          ok = xt_wait(&bars.sec_full[ss], sec_c.ph, abort_flag);
          sec_c.next(sec_n);
          if (!ok) break;
          if (m == team) {
            const FastMat& fm = fe.m[m];
            const unsigned char* sec = sm.sec0 + ss * sm.sec_stride;
            const uint32_t* words = reinterpret_cast<const uint32_t*>(sec + sec_scale_bytes);
            const uint4* scale4 = reinterpret_cast<const uint4*>(sec);    // 8 halves per (pair, t)
            const int npairs = fm.nslots >> 5, nib_pairs = fm.nblk[0] >> 1;
            const uint32_t* dense_words = words + fm.nblk[0] * 256;
            for (int p0 = 0; p0 < npairs; p0 += 2) {
              if (!(ok = xt_wait(&w_empty[ring_c.i], ring_c.ph ^ 1, abort_flag))) break;
              unsigned char* stage = ring + ring_c.i * XT_STAGE_BYTES;
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
              if (lane == 0) tc::mbar_arrive(&w_full[ring_c.i]);
              ring_c.next(ring_h);
            }
          }
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(&bars.sec_empty[ss]);
        }
        if (!ok) break;
        if (tl == 0) continue;                      // the down product runs one tile behind
        const uint32_t sd = sec_c.i;
        ok = xt_wait(&bars.sec_full[sd], sec_c.ph, abort_flag);
        sec_c.next(sec_n);
        if (!ok) break;
        const FastMat& fd = fe.m[2];
        const unsigned char* sec = sm.sec0 + sd * sm.sec_stride;
        const uint32_t* dwords = reinterpret_cast<const uint32_t*>(sec + sec_scale_bytes);
        const uint32_t* ddense = dwords + fd.nblk[0] * 256;
        const __half* scale_d = reinterpret_cast<const __half*>(sec);
        for (int mt = team; mt < n_mt && ok; mt += 2) {
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
          for (int p0 = 0; p0 < 4; p0 += 2) {
            if (!(ok = xt_wait(&w_empty[ring_c.i], ring_c.ph ^ 1, abort_flag))) break;
            unsigned char* stage = ring + ring_c.i * XT_STAGE_BYTES;
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
            if (lane == 0) tc::mbar_arrive(&w_full[ring_c.i]);
            ring_c.next(ring_h);
          }
        }
        __syncwarp();
        if (ok && lane == 0) tc::mbar_arrive(&bars.sec_empty[sd]);
      }
    } else {
      // ------------------------------------------------------------------ epilogue warps 0-7
      // warp = (TMEM lane quarter q, parity of the 32-token column chunks it takes)
      const int q = warp & 3, n_first = (warp >> 2) * 32;
      const uint32_t lane_sel = static_cast<uint32_t>(32 * q) << 16;
      bool ok = true;
      const int c = 32 * q + lane;                                   // row of D_g / D_u = column of the tile
      const int c_pos = slot_pos(c);
      unsigned char* zrow = sm.z + (c_pos >> 3) * cs + (c_pos & 7) * 2;
      for (int tile = 0; tile < n_tiles && ok; ++tile) {
        const uint32_t gt = gu_round + tile, b = gt & 1u, k = gt >> 1;
        ok = xt_wait(&bars.gu_done[b], k & 1, abort_flag);
        if (ok && gt >= 2) ok = xt_wait(&bars.z_free[b], (k - 1) & 1, abort_flag);     // z buffer b consumed two tiles ago
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t d_gate = tmem_base + 2 * b * acc_stride, d_up = d_gate + acc_stride;
        unsigned char* zr = zrow + b * z_bytes;
        for (int n0 = n_first; n0 < n_mma; n0 += 64) {
          // 16 columns at a time: two 32-column loads would hold 64 registers per thread
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int nb = n0 + 16 * hh;
            if (nb >= n_mma) break;
            float gv[16], uv[16];
            tc::tmem_ld16(d_gate + lane_sel + nb, gv);
            tc::tmem_ld16(d_up + lane_sel + nb, uv);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int n = nb + i;
              const float zf = __fdividef(gv[i] * uv[i], 1.f + __expf(-gv[i]));
              *reinterpret_cast<__half*>(zr + (n >> 3) * 128 + (n & 7) * 16) = __float2half_rn(n < n_tok ? zf : 0.f);
            }
          }
        }
        tc::fence_before_sync();
        tc::fence_async_smem();
        __syncwarp();
        if (lane == 0) { tc::mbar_arrive(&bars.tmem_gu_free[b]); tc::mbar_arrive(&bars.z_ready[b]); }
      }
      if (ok) ok = xt_wait(&bars.down_done, item_round & 1, abort_flag);
      if (ok) {
        tc::fence_after_sync();
        const FastMat& fd = fe.m[2];
        const int16_t* rank_d = reinterpret_cast<const int16_t*>(arena + fd.tab_off);
        const __half* s_d = reinterpret_cast<const __half*>(arena + fd.tab_off + fd.nslots * 2);
        // A thread owns a row slot, and the slots of a warp map to scattered ranks: adding straight from the registers
        // costs one 32-byte sector per lane and instruction.  With room for it (the operand ring is idle by now) the
        // four warps that share a 32-token chunk transpose it through shared memory and add whole rows, 16 bytes per
        // lane; ranks without a slot add zero.
        const int grp = warp >> 2;
        const bool transpose = acc64 == nullptr && (rank_out & 3) == 0 &&
                               static_cast<size_t>(2) * 32 * rank_out * 4 <= static_cast<size_t>(2 * ring_h) * XT_STAGE_BYTES;
        float* tbuf = reinterpret_cast<float*>(sm.ring) + grp * 32 * rank_out;
        for (int n0 = n_first; n0 < n_mma; n0 += 64) {
          if (transpose) {
            for (int i = (warp & 3) * 32 + lane; i < 8 * rank_out; i += 128) reinterpret_cast<float4*>(tbuf)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          }
          for (int mt = 0; mt < n_mt; ++mt) {
            const int slot = 128 * mt + 32 * q + lane;
            int rk = -1;
            float sv = 0.f;
            if (slot < fd.nslots) { rk = rank_d[slot]; sv = __half2float(s_d[slot]); }
            const bool live = rk >= 0 && rk < rank_out;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              const int nb = n0 + 16 * hh;
              if (nb >= n_mma) break;
              float v[16];
              tc::tmem_ld16(d_down + mt * acc_stride + lane_sel + nb, v);
              if (live) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  const int n = nb + i;
                  if (n < n_tok) {
                    const float val = v[i] * sv * item.rw[n];
                    if (transpose) tbuf[(16 * hh + i) * rank_out + rk] = val;
                    else acc_add(rank_accum, acc64, static_cast<int64_t>(item.tok[n]) * rank_out + rk, val);
                  }
                }
              }
            }
          }
          if (transpose) {
            asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
            for (int i = q; i < 32 && n0 + i < n_tok; i += 4) {
              float* dst = rank_accum + static_cast<int64_t>(item.tok[n0 + i]) * rank_out;
              for (int c0 = lane * 4; c0 < rank_out; c0 += 128) {
                const float4 x = *reinterpret_cast<const float4*>(tbuf + i * rank_out + c0);
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + c0), "f"(x.x), "f"(x.y), "f"(x.z), "f"(x.w) : "memory");
              }
            }
            if (n0 + 64 < n_mma) asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
          }
        }
        tc::fence_before_sync();
      }
    }
    gu_round += n_tiles;
  }
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) tc::tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && abort_flag_s) atomicExch(status, BM_ERR_TIMEOUT);
}

// Item size and pipeline depths for a layer: the first candidate that fits.  Larger items convert every code for more
// tokens at once, but the item's activation operand (1 KB per token at 256 row slots) and the two z tiles compete with
// the copy and conversion stages for shared memory, and tensor memory has to hold two (gate, up) accumulator pairs
// plus the down product's two or three row tiles of nt columns each.
struct XtPlan { int nt, ring_h, sec_n, acc_stride; size_t smem; };
constexpr size_t XT_SMEM_LIMIT = 227 * 1024 - 4096;     // dynamic part: the kernel's static shared memory (two item descriptions, barriers) stays below 4 KB
static bool xt_plan(const bm_layer* L, XtPlan* out) {
  if (L->num_experts > XT_MAX_E || L->intermediate % N_TILE != 0 || L->max_slots > 3 * 128) return false;
  const int n_mt = (L->max_slots + 127) / 128;
  // {tokens per item, operand stages per pipeline, section slots}
  static const int cand[][3] = {{64, 2, 4}, {64, 2, 3}, {64, 2, 2}, {48, 2, 3}, {48, 2, 2}, {32, 2, 3}, {32, 2, 2}, {16, 2, 2}};
  for (const auto& c : cand) {
    const int nt = c[0], ring_h = c[1], sec_n = c[2];
    const bool shape_ok = nt % 16 == 0 && nt >= 16 && nt <= XT_NT_MAX && ring_h >= 1 && 2 * ring_h <= XT_RING_MAX && sec_n >= 2 &&
                          sec_n <= XT_SEC_MAX;
    // the epilogue reads accumulators in 32-column pieces, so the last one may be read up to the next multiple of 32
    const bool tmem_ok = (3 + n_mt) * nt + (nt + 31) / 32 * 32 <= 512;
    const size_t smem = xt_smem_bytes(L->max_slots, L->max_words, L->num_experts, L->rank_in, nt, 2 * ring_h, sec_n);
    if (shape_ok && tmem_ok && smem <= XT_SMEM_LIMIT) {
      *out = XtPlan{nt, ring_h, sec_n, nt, smem};
      return true;
    }
  }
  return false;
}

// Whether the layer's largest expert fits the tensor path's shared- and tensor-memory budget (AUTO falls back to the
// decode path otherwise).
bool experts_tc_fits(const bm_layer* L) {
  XtPlan p;
  return xt_plan(L, &p);
}

int launch_experts_tc(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                      const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, long long* acc64,
                      cudaStream_t st) {
  BM_REQUIRE(L->num_experts <= XT_MAX_E, BM_ERR_UNSUPPORTED, "experts_tc: more than %d experts", XT_MAX_E);
  BM_REQUIRE(L->intermediate % N_TILE == 0, BM_ERR_UNSUPPORTED, "experts_tc: intermediate size must be a multiple of %d", N_TILE);
  BM_REQUIRE(L->max_slots <= 3 * 128, BM_ERR_UNSUPPORTED, "experts_tc: %d row slots exceed the tensor-memory budget", L->max_slots);
  BM_REQUIRE(L->rank_in % 8 == 0 && ((reinterpret_cast<uintptr_t>(h_gate) | reinterpret_cast<uintptr_t>(h_up)) & 15u) == 0,
             BM_ERR_UNSUPPORTED, "experts_tc: rank-space rows must be 16-byte aligned (rank %d)", L->rank_in);
  XtPlan plan;
  BM_REQUIRE(xt_plan(L, &plan), BM_ERR_UNSUPPORTED, "experts_tc: the layer's largest expert does not fit in shared memory");
  const size_t smem = plan.smem;
  static PerDeviceOnce attr_once;
  static int sm_counts[MAX_DEVICES];
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  BM_REQUIRE(dev >= 0 && dev < MAX_DEVICES, BM_ERR_UNSUPPORTED, "experts_tc: device ordinal %d out of range", dev);
  if (!attr_once.is_done(dev)) {
    BM_CUDA(cudaFuncSetAttribute(experts_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(XT_SMEM_LIMIT)));
    BM_CUDA(cudaDeviceGetAttribute(&sm_counts[dev], cudaDevAttrMultiProcessorCount, dev));
    attr_once.mark(dev);
  }
  const int sm_count = sm_counts[dev];
  experts_tc_kernel<<<sm_count, XT_THREADS, smem, st>>>(
      L->fast_dev, static_cast<const unsigned char*>(L->arena), h_gate, h_up, L->rank_in, token_indices, expert_offsets,
      route_w, L->rank_out, T, L->num_experts, L->n_tiles, L->max_slots, L->max_words, plan.nt, plan.ring_h, plan.sec_n,
      plan.acc_stride, rank_accum, acc64, L->status_dev);
  BM_LAUNCH_CHECK("experts_tc_kernel");
  return BM_OK;
}

}  // namespace bm
