// Packed routed-expert forward for small token counts (decode): bandwidth-bound split-K GEMV.
//
// One CTA owns one (expert, 128-column tile) unit.  Its whole unit block (scales + packed words of
// gate, up and down for that tile, ~30 KB at the Qwen3-30B shape) is pulled into shared memory by
// two cp.async.bulk copies that complete on mbarriers, so every active SM has its bytes in flight
// from the first cycle; the down words land while gate/up are being consumed.  Weights never
// exist as fp16 in memory: each warp expands its arena words into m16n8k16 A fragments with one mask
// per register (see fast_layout.cuh) and multiplies them with the tokens' activations (the B operand,
// up to 8 assignments per pass) on the tensor cores.  The per-(tile,row) scale is folded into the
// activation operand for gate/up and into the epilogue for down; the stored codes' offset
// is removed with a per-token correction term instead of per weight.  The six tiles of an
// expert split the contraction of the down product; their partial sums meet in rank_accum through
// fp32 atomics (as in bitsmoe/algorithms/cpp/mlp_forward.cu:2036-2066).
#include "fast_layout.cuh"
#include "tc05.cuh"

namespace bm {

// Optional phase timing (debug builds only): cycles of compute-warp 0, accumulated into status[8 + phase].
#ifdef BM_DECODE_TIMING
#define BM_TICK(phase)                                                                   \
  do {                                                                                   \
    if (threadIdx.x == 0) {                                                              \
      const long long now_ = clock64();                                                  \
      atomicAdd(reinterpret_cast<unsigned long long*>(bm_timing_base) + (phase), static_cast<unsigned long long>(now_ - bm_tick_)); \
      bm_tick_ = now_;                                                                   \
    }                                                                                    \
  } while (0)
#else
#define BM_TICK(phase) do {} while (0)
#endif

constexpr int DEC_THREADS = 288;            // 8 compute warps + 1 producer warp
constexpr int DEC_MAX_E = 1024;
constexpr int DEC_CLASSES = 4;             // active experts are ordered by passes: >= 4, 3, 2, 1
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return tc::mbar_wait(bar, parity); }

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Rows g + 8 of every A fragment carry a factor 16 (see fast_layout.cuh): accumulator registers 2 and 3
// are scaled back with 2^20 instead of 2^24.
constexpr float DEC_UNSCALE_LO = 16777216.f, DEC_UNSCALE_HI = 1048576.f;

__device__ __forceinline__ void nib_afrag(uint32_t w, uint32_t (&a)[4]) {
  const uint32_t s = w >> 8;
  a[0] = w & 0x000F000Fu;
  a[1] = w & 0x00F000F0u;
  a[2] = s & 0x000F000Fu;
  a[3] = s & 0x00F000F0u;
}
__device__ __forceinline__ void dense_afrag(uint32_t w, uint32_t (&a)[4]) {
  const uint32_t s = w >> 2;
  a[0] = w & 0x00030003u;
  a[1] = w & 0x00300030u;
  a[2] = s & 0x00030003u;
  a[3] = s & 0x00300030u;
}

// `npairs` pairs of 16x16 blocks of one group against the token-side operand.  `wp` points at this lane's word(s) of
// the first pair, consecutive pairs are `stride` words apart; `bp` points at this lane's eight halves of the first pair
// (operand row g, position 8 t).  `off` accumulates the same products against a constant fragment holding the
// group's code offset: its column n ends up as offset * sum_k B[k][n], the term that turns sum u*B into sum q*B.
template <bool DENSE>
__device__ __forceinline__ void mma_pairs(const uint32_t* __restrict__ wp, int stride, int npairs, const __half* __restrict__ bp,
                                          float (&acc)[4], float (&off)[4]) {
  constexpr uint32_t kLo = (DENSE ? FAST_DENSE_OFFSET : FAST_NIB_OFFSET) * 0x00010001u;
  const uint32_t offs[4] = {kLo, kLo << 4, kLo, kLo << 4};
#pragma unroll 2
  for (int p = 0; p < npairs; ++p) {
    const uint4 b = *reinterpret_cast<const uint4*>(bp);
    uint32_t a[4];
    if (DENSE) {
      const uint32_t w = *wp;
      dense_afrag(w, a);
      mma_16816(acc, a, b.x, b.y);
      dense_afrag(w >> 8, a);
      mma_16816(acc, a, b.z, b.w);
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(wp);
      nib_afrag(w.x, a);
      mma_16816(acc, a, b.x, b.y);
      nib_afrag(w.y, a);
      mma_16816(acc, a, b.z, b.w);
    }
    mma_16816(off, offs, b.x, b.y);
    mma_16816(off, offs, b.z, b.w);
    wp += stride;
    bp += 32;
  }
}

struct DecSmem {
  unsigned char* unit;         // current unit block
  const unsigned char* tabs[3];   // current expert's [int16 rank | fp16 s] slot tables of gate, up, down
  __half* actp;                // [2][FAST_MAX_TOK][slots_stride]
  __half* zp;                  // [FAST_MAX_TOK][N_TILE + 8]
  int* tok;                    // [FAST_MAX_TOK]
  float* rw;                   // [FAST_MAX_TOK]
};

constexpr int DEC_CONSUMERS = 256;            // 8 compute warps; warp 8 is the producer
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMERS) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

constexpr int ZP_STRIDE = N_TILE + 32;   // halves; rows 64 bytes apart modulo 128: the 16-byte operand loads of a quarter warp hit distinct banks

__host__ __device__ inline int dec_slots_stride(int max_slots) { return (max_slots + 63) / 64 * 64 + 32; }

// One pipeline stage: [unit block | per-expert slot tables | h rows of the first pass's tokens (gate, up)]
__host__ __device__ inline size_t dec_stage_bytes(int max_unit_bytes, int max_slots, int h_rank) {
  return align_up_c(static_cast<size_t>(max_unit_bytes), 128) + align_up_c(static_cast<size_t>(3) * (max_slots * 4 + 16), 128) +
         align_up_c(static_cast<size_t>(2) * FAST_MAX_TOK * h_rank * 2, 128);
}

__host__ __device__ inline size_t dec_smem_bytes(int max_unit_bytes, int max_slots, int h_rank) {
  size_t o = 2 * dec_stage_bytes(max_unit_bytes, max_slots, h_rank);
  o += static_cast<size_t>(2) * FAST_MAX_TOK * dec_slots_stride(max_slots) * 2;
  o += static_cast<size_t>(FAST_MAX_TOK) * ZP_STRIDE * 2;
  o += DEC_MAX_E * 2;
  return align_up_c(o, 128);
}

__device__ __forceinline__ void decode_pass(const FastExpert& fe, const DecSmem& sm, int slots_stride, int tile, int n_valid,
                                            int npass, int rank_out, float* __restrict__ rank_accum,
                                            const unsigned char* __restrict__ arena, uint64_t* bar_down, uint32_t parity,
                                            bool* ok, long long& bm_tick_, int* bm_timing_base) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // ---- gate / up: this warp owns columns 16*warp .. 16*warp+15 of the tile
  float acc[2][4], offa[2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = offa[m][j] = 0.f;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    const FastMat& fm = fe.m[m];
    const uint32_t* sec = reinterpret_cast<const uint32_t*>(sm.unit + fe.sec_off[3 + m]);
    const __half* bop = sm.actp + static_cast<size_t>(m) * FAST_MAX_TOK * slots_stride + static_cast<size_t>(g) * slots_stride + 8 * t;
    // nibble words [pair][x][lane][2], dense words [pair][x][lane]
    mma_pairs<false>(sec + (warp * 32 + lane) * 2, 512, fm.nblk[0] >> 1, bop, acc[m], offa[m]);
    mma_pairs<true>(sec + fm.nblk[0] * 256 + warp * 32 + lane, 256, fm.nblk[1] >> 1, bop + fm.nblk[0] * 16, acc[m], offa[m]);
  }
  BM_TICK(3);
  // ---- z = silu(g) * u, written as the down product's B operand
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = 16 * warp + g + (j >= 2 ? 8 : 0);
    const int n = 2 * t + (j & 1);
    const float unscale = j >= 2 ? DEC_UNSCALE_HI : DEC_UNSCALE_LO;
    const float gv = (acc[0][j] - offa[0][j]) * unscale;
    const float uv = (acc[1][j] - offa[1][j]) * unscale;
    const float z = (c < n_valid && n < npass) ? (gv / (1.f + __expf(-gv))) * uv : 0.f;
    sm.zp[n * ZP_STRIDE + slot_pos(c)] = __float2half_rn(z);
  }
  consumer_sync();
  BM_TICK(4);
  if (!mbar_wait(bar_down, parity)) { *ok = false; return; }
  BM_TICK(5);
  // ---- down: slot blocks round-robin over the warps, contraction over the tile's 128 columns
  const FastMat& fd = fe.m[2];
  const uint32_t* dwords = reinterpret_cast<const uint32_t*>(sm.unit + fe.sec_off[5]);
  const __half* scale_d = reinterpret_cast<const __half*>(sm.unit + fe.sec_off[2]);
  const int16_t* rank_d = reinterpret_cast<const int16_t*>(sm.tabs[2]);
  const __half* s_d = reinterpret_cast<const __half*>(sm.tabs[2] + fd.nslots * 2);
  const int nblk_total = fd.nslots >> 4;
  const __half* zrow = sm.zp + g * ZP_STRIDE + 8 * t;
  for (int mb = warp; mb < nblk_total; mb += 8) {
    float dacc[4], doff[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) dacc[j] = doff[j] = 0.f;
    // nibble words [mblock][pair][lane][2], dense words [mblock][pair][lane]
    if (mb < fd.nblk[0]) mma_pairs<false>(dwords + (mb * 128 + lane) * 2, 64, 4, zrow, dacc, doff);
    else mma_pairs<true>(dwords + fd.nblk[0] * 256 + (mb - fd.nblk[0]) * 128 + lane, 32, 4, zrow, dacc, doff);
#pragma unroll
    for (int half_rows = 0; half_rows < 2; ++half_rows) {
      const int slot = mb * 16 + g + 8 * half_rows;
      const int rk = rank_d[slot];
      if (rk < 0 || rk >= rank_out) continue;
      const float f = __half2float(s_d[slot]) * __half2float(scale_d[slot]) * (half_rows ? DEC_UNSCALE_HI : DEC_UNSCALE_LO);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int n = 2 * t + h;
        if (n >= npass) continue;
        const float v = (dacc[2 * half_rows + h] - doff[2 * half_rows + h]) * f * sm.rw[n];
        atomicAdd(&rank_accum[static_cast<int64_t>(sm.tok[n]) * rank_out + rk], v);
      }
    }
  }
}

// Persistent kernel.  Every CTA first compacts the list of experts that received tokens (from
// expert_offsets, most passes first), then walks the (active expert, tile) units gridDim.x - 1 - blockIdx.x,
// blockIdx.x + gridDim.x, blockIdx.x + 2 * gridDim.x, ...
// Warp 8 is the producer: for each unit it waits until the target stage is released, fetches the expert
// descriptor and the first pass's token ids / route weights, and starts bulk copies of the unit block, the
// expert's slot tables and the tokens' h rows into one of two shared-memory stages; the 8 compute warps
// consume stage `it & 1` while the next unit streams into the other one, so they never wait on global
// memory except for experts with more than FAST_MAX_TOK assignments (later passes gather h directly).
struct DecStageInfo {
  FastExpert fe;
  int tok[FAST_MAX_TOK];
  float rw[FAST_MAX_TOK];
  int a_begin, a_end;
};

__global__ void __launch_bounds__(DEC_THREADS) experts_decode_kernel(
    const FastExpert* __restrict__ fast, const unsigned char* __restrict__ arena, const __half* __restrict__ h_gate,
    const __half* __restrict__ h_up, int h_rank, const int32_t* __restrict__ token_indices,
    const int32_t* __restrict__ expert_offsets, const float* __restrict__ route_w, int rank_out, int T, int num_experts,
    int n_tiles, int intermediate, int max_unit_bytes, int max_slots, float* __restrict__ rank_accum,
    int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ DecStageInfo info[2];
  __shared__ __align__(8) uint64_t bar_full[2][2];   // [stage][everything but down | down words]
  __shared__ __align__(8) uint64_t bar_empty[2];
  __shared__ int warp_cnt[DEC_CLASSES][9];
  const int slots_stride = dec_slots_stride(max_slots);
  const size_t unit_bytes_al = align_up_c(static_cast<size_t>(max_unit_bytes), 128);
  const size_t tabs_bytes_al = align_up_c(static_cast<size_t>(3) * (max_slots * 4 + 16), 128);
  const size_t stage_bytes = dec_stage_bytes(max_unit_bytes, max_slots, h_rank);
  DecSmem sm;
  int16_t* active;
  {
    size_t o = 2 * stage_bytes;
    sm.unit = smem_raw;
    sm.tabs[0] = sm.tabs[1] = sm.tabs[2] = nullptr;
    sm.actp = reinterpret_cast<__half*>(smem_raw + o);
    o += static_cast<size_t>(2) * FAST_MAX_TOK * slots_stride * 2;
    sm.zp = reinterpret_cast<__half*>(smem_raw + o);
    o += static_cast<size_t>(FAST_MAX_TOK) * ZP_STRIDE * 2;
    active = reinterpret_cast<int16_t*>(smem_raw + o);
    sm.tok = nullptr;
    sm.rw = nullptr;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar_full[0][0], 1);
    mbar_init(&bar_full[0][1], 1);
    mbar_init(&bar_full[1][0], 1);
    mbar_init(&bar_full[1][1], 1);
    mbar_init(&bar_empty[0], 8);
    mbar_init(&bar_empty[1], 8);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // ---- compact the active experts by descending number of passes (4 or more, 3, 2, 1 passes of FAST_MAX_TOK
  // assignments), ascending id inside a class.  A CTA's first unit is taken from the END of the grid's first round
  // (unit gridDim - 1 - blockIdx), its later ones from the front (blockIdx + k * gridDim), so the multi-pass units at
  // the head of the list land on CTAs that do not get a unit of the last, partial round.
  int n_active = 0;
  if (num_experts <= DEC_THREADS) {
    const int e = threadIdx.x;
    const int cnt = e < num_experts ? expert_offsets[e + 1] - expert_offsets[e] : 0;
    const int passes = (cnt + FAST_MAX_TOK - 1) / FAST_MAX_TOK;
    const int cls = cnt <= 0 ? -1 : (passes >= DEC_CLASSES ? 0 : DEC_CLASSES - passes);
    unsigned mine = 0;
#pragma unroll
    for (int c = 0; c < DEC_CLASSES; ++c) {
      const unsigned m = __ballot_sync(0xffffffffu, cls == c);
      if (cls == c) mine = m;
      if (lane == 0) warp_cnt[c][warp] = __popc(m);
    }
    __syncthreads();
    int before = 0;
#pragma unroll
    for (int c = 0; c < DEC_CLASSES; ++c)
      for (int w = 0; w < 9; ++w) {
        const int n = warp_cnt[c][w];
        n_active += n;
        if (c < cls || (c == cls && w < warp)) before += n;
      }
    if (cls >= 0) active[before + __popc(mine & ((1u << lane) - 1u))] = static_cast<int16_t>(e);
    __syncthreads();
  } else {
    for (int c = 0; c < DEC_CLASSES; ++c) {
      for (int base = 0; base < num_experts; base += DEC_THREADS) {
        const int e = base + threadIdx.x;
        const int cnt = e < num_experts ? expert_offsets[e + 1] - expert_offsets[e] : 0;
        const int passes = (cnt + FAST_MAX_TOK - 1) / FAST_MAX_TOK;
        const bool act = cnt > 0 && (passes >= DEC_CLASSES ? 0 : DEC_CLASSES - passes) == c;
        const unsigned m = __ballot_sync(0xffffffffu, act);
        if (lane == 0) warp_cnt[0][warp] = __popc(m);
        __syncthreads();
        int before = n_active;
        for (int w = 0; w < warp; ++w) before += warp_cnt[0][w];
        if (act) active[before + __popc(m & ((1u << lane) - 1u))] = static_cast<int16_t>(e);
        for (int w = 0; w < 9; ++w) n_active += warp_cnt[0][w];
        __syncthreads();
      }
    }
  }
  const int n_units = n_active * n_tiles;
  const int first_unit = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  if (first_unit >= n_units) return;
  bool ok = true;
  long long bm_tick_ = clock64();
  int* bm_timing_base = status + 8;
  (void)bm_tick_; (void)bm_timing_base;

  if (warp == 8) {
    // ------------------------------------------------------------------ producer warp
    int it = 0;
    for (int u = first_unit; u < n_units; u = blockIdx.x + (it + 1) * gridDim.x, ++it) {
      const int buf = it & 1;
      const int e = active[u / n_tiles], tile = u % n_tiles;
      if (!mbar_wait(&bar_empty[buf], ((it >> 1) & 1) ^ 1)) { ok = false; break; }
      DecStageInfo& si = info[buf];
      for (int i = lane; i < static_cast<int>(sizeof(FastExpert) / 4); i += 32)
        reinterpret_cast<uint32_t*>(&si.fe)[i] = reinterpret_cast<const uint32_t*>(&fast[e])[i];
      const int a_begin = expert_offsets[e], a_end = expert_offsets[e + 1];
      const int npass = min(FAST_MAX_TOK, a_end - a_begin);
      int tk = 0;
      if (lane < FAST_MAX_TOK) {
        tk = lane < npass ? token_indices[a_begin + lane] : 0;
        const bool good = lane < npass && tk >= 0 && tk < T;
        tk = good ? tk : 0;
        si.tok[lane] = tk;
        si.rw[lane] = good ? route_w[a_begin + lane] : 0.f;
      }
      if (lane == 0) { si.a_begin = a_begin; si.a_end = a_end; }
      __syncwarp();
      const FastExpert& fe = si.fe;
      unsigned char* stage = smem_raw + buf * stage_bytes;
      const unsigned char* src = arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes;
      const uint32_t bytes_a = static_cast<uint32_t>(fe.sec_off[5]);
      const uint32_t bytes_b = static_cast<uint32_t>(fe.m[2].words) * 4u;
      const uint32_t tb0 = static_cast<uint32_t>(fe.m[0].nslots) * 4u, tb1 = static_cast<uint32_t>(fe.m[1].nslots) * 4u,
                     tb2 = static_cast<uint32_t>(fe.m[2].nslots) * 4u;   // [rank | s] of each matrix, the row table stays behind
      const uint32_t row_bytes = static_cast<uint32_t>(h_rank) * 2u;
      if (lane == 0) {
        mbar_expect_tx(&bar_full[buf][0], bytes_a + tb0 + tb1 + tb2 + 2u * npass * row_bytes);
        bulk_g2s(stage, src, bytes_a, &bar_full[buf][0]);
        bulk_g2s(stage + unit_bytes_al, arena + fe.m[0].tab_off, tb0, &bar_full[buf][0]);
        bulk_g2s(stage + unit_bytes_al + tb0, arena + fe.m[1].tab_off, tb1, &bar_full[buf][0]);
        bulk_g2s(stage + unit_bytes_al + tb0 + tb1, arena + fe.m[2].tab_off, tb2, &bar_full[buf][0]);
        mbar_expect_tx(&bar_full[buf][1], bytes_b);
        bulk_g2s(stage + bytes_a, src + bytes_a, bytes_b, &bar_full[buf][1]);
      }
      __syncwarp();
      if (lane < 2 * npass) {
        const int m = lane / npass, n = lane - m * npass;
        const int tkn = __shfl_sync(__activemask(), tk, n);
        const __half* hsrc = (m == 0 ? h_gate : h_up) + static_cast<int64_t>(tkn) * h_rank;
        bulk_g2s(stage + unit_bytes_al + tabs_bytes_al + (static_cast<size_t>(m) * FAST_MAX_TOK + n) * row_bytes, hsrc, row_bytes,
                 &bar_full[buf][0]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) atomicExch(status, BM_ERR_TIMEOUT);
    return;
  }

  // -------------------------------------------------------------------- compute warps
  int it = 0;
  for (int u = first_unit; u < n_units && ok; u = blockIdx.x + (it + 1) * gridDim.x, ++it) {
    const int buf = it & 1;
    const uint32_t parity = (it >> 1) & 1;
    const int tile = u % n_tiles;
    const int n_valid = min(N_TILE, intermediate - tile * N_TILE);
    unsigned char* stage = smem_raw + buf * stage_bytes;
    if (!mbar_wait(&bar_full[buf][0], parity)) { ok = false; break; }
    BM_TICK(0);
    DecStageInfo& si = info[buf];
    const FastExpert& fe = si.fe;
    DecSmem cur = sm;
    cur.unit = stage;
    cur.tabs[0] = stage + unit_bytes_al;
    cur.tabs[1] = cur.tabs[0] + fe.m[0].nslots * 4;
    cur.tabs[2] = cur.tabs[1] + fe.m[1].nslots * 4;
    cur.tok = si.tok;
    cur.rw = si.rw;
    const __half* hrows = reinterpret_cast<const __half*>(stage + unit_bytes_al + tabs_bytes_al);
    const int a_begin = si.a_begin, a_end = si.a_end;
    for (int a0 = a_begin; a0 < a_end && ok; a0 += FAST_MAX_TOK) {
      const int npass = min(FAST_MAX_TOK, a_end - a0);
      const bool staged = a0 == a_begin;
      if (!staged) {
        // later passes of a crowded expert: token ids and h rows come from global memory
        consumer_sync();
        if (threadIdx.x < FAST_MAX_TOK) {
          const int n = threadIdx.x;
          const int tk = n < npass ? token_indices[a0 + n] : 0;
          const bool good = n < npass && tk >= 0 && tk < T;
          si.tok[n] = good ? tk : 0;
          si.rw[n] = good ? route_w[a0 + n] : 0.f;
        }
        consumer_sync();
      }
      // ---- activation operand: actp[m][n][perm(slot)] = fp16(h[tok_n, rank(slot)] * s(slot) * scale(tile, slot))
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const int nslots = fe.m[m].nslots;
        const int16_t* rank_t = reinterpret_cast<const int16_t*>(cur.tabs[m]);
        const __half* s_t = reinterpret_cast<const __half*>(cur.tabs[m] + nslots * 2);
        const __half* scale_t = reinterpret_cast<const __half*>(stage + fe.sec_off[m]);
        const __half* hg = m == 0 ? h_gate : h_up;
        const __half* hs = hrows + static_cast<size_t>(m) * FAST_MAX_TOK * h_rank;
        __half* dst = cur.actp + static_cast<size_t>(m) * FAST_MAX_TOK * slots_stride;
        for (int slot = threadIdx.x; slot < nslots; slot += DEC_CONSUMERS) {
          const int rk = rank_t[slot];
          const int pos = slot_pos(slot);
          const float f = __half2float(s_t[slot]) * __half2float(scale_t[pos]);
          const bool live = rk >= 0 && rk < h_rank;
          float hv[FAST_MAX_TOK];
#pragma unroll
          for (int n = 0; n < FAST_MAX_TOK; ++n) {
            hv[n] = 0.f;
            if (live && n < npass)
              hv[n] = __half2float(staged ? hs[n * h_rank + rk] : hg[static_cast<int64_t>(si.tok[n]) * h_rank + rk]);
          }
#pragma unroll
          for (int n = 0; n < FAST_MAX_TOK; ++n) dst[n * slots_stride + pos] = __float2half_rn(hv[n] * f);
        }
      }
      consumer_sync();
      BM_TICK(1);
      decode_pass(fe, cur, slots_stride, tile, n_valid, npass, rank_out, rank_accum, arena, &bar_full[buf][1], parity, &ok,
                     bm_tick_, bm_timing_base);
      BM_TICK(6);
    }
    consumer_sync();
    if (lane == 0) mbar_arrive(&bar_empty[buf]);
    BM_TICK(7);
  }
  if (!ok && threadIdx.x == 0) atomicExch(status, BM_ERR_TIMEOUT);
}

int launch_experts_decode(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                          const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, cudaStream_t st) {
  const size_t smem = dec_smem_bytes(L->max_unit_bytes, L->max_slots, L->rank_in);
  BM_REQUIRE(smem <= 220 * 1024, BM_ERR_UNSUPPORTED, "experts_decode: unit of %d bytes does not fit shared memory",
             L->max_unit_bytes);
  BM_REQUIRE(L->num_experts <= DEC_MAX_E, BM_ERR_UNSUPPORTED, "experts_decode: more than %d experts", DEC_MAX_E);
  BM_REQUIRE(L->rank_in % 8 == 0 && (reinterpret_cast<uintptr_t>(h_gate) & 15u) == 0 && (reinterpret_cast<uintptr_t>(h_up) & 15u) == 0,
             BM_ERR_INVALID_ARG, "experts_decode: h_gate / h_up rows must be 16-byte aligned (rank %d)", L->rank_in);
  static int attr_set_for = -1;
  static int sm_count = 148;
  if (attr_set_for != L->device) {
    BM_CUDA(cudaFuncSetAttribute(experts_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
    BM_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, L->device));
    attr_set_for = L->device;
  }
  static size_t occ_for_smem = 0;
  static int per_sm = 1;
  if (occ_for_smem != smem) {
    int blocks = 1;
    BM_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, experts_decode_kernel, DEC_THREADS, smem));
    per_sm = blocks < 1 ? 1 : (blocks > 2 ? 2 : blocks);
    occ_for_smem = smem;
  }
  int grid = sm_count * per_sm;
  const int max_units = L->num_experts * L->n_tiles;
  if (grid > max_units) grid = max_units;
  experts_decode_kernel<<<grid, DEC_THREADS, smem, st>>>(
      L->fast_dev, static_cast<const unsigned char*>(L->arena), h_gate, h_up, L->rank_in, token_indices, expert_offsets,
      route_w, L->rank_out, T, L->num_experts, L->n_tiles, L->intermediate, L->max_unit_bytes, L->max_slots, rank_accum,
      L->status_dev);
  BM_LAUNCH_CHECK("experts_decode_kernel");
  return BM_OK;
}

}  // namespace bm
