// Packed routed-expert forward for small token counts (decode): bandwidth-bound split-K GEMV.
//
// Work unit = (expert, pass of up to 8 of its assignments, range of its 128-column tiles).  The ranges are chosen
// per launch so that the units of one launch fill the grid once: at 64 tokens on a 128-expert layer every CTA gets
// half an expert.  A unit streams its tiles' sections (scales + arena words of gate, up, down, ~10 KB each) through a
// ring of shared-memory slots filled by cp.async.bulk copies that complete on mbarriers; a producer warp keeps the
// ring full across tile and unit boundaries, so an SM has its bytes in flight from the moment the unit is known.
//
// Weights never exist as fp16 in memory: each of the 8 compute warps expands its arena words into m16n8k16 A
// fragments with one mask per register (fast_layout.cuh) and multiplies them with the tokens' operand (B, up to 8
// assignments) on the tensor cores.  Per unit the tokens' h rows are gathered once into hs = fp16(h[rank] * S); per
// tile the gate/up operand is hs * scale(tile) (one half2 multiply per two values).  Stored codes carry an offset
// (8 or 2); it is removed after the products with one scalar per (matrix, token, tile): offset * sum of the operand,
// computed while the operand is built (gate/up) or while z is stored (down), so no MMA is spent on it.  The down
// product accumulates in registers over all tiles of the unit and reaches rank_accum with one fp32 atomic per
// (slot, token) per unit (the reference adds per CTA as well: bitsmoe/algorithms/cpp/mlp_forward.cu:2036-2066).
//
// Every wait is bounded (a launch parameter); a wait that gives up raises a CTA-wide abort flag, all threads leave
// through the same barriers, and the layer's status word reports BM_ERR_TIMEOUT.
#include "fast_layout.cuh"
#include "tc05.cuh"

namespace bm {

constexpr int DEC_THREADS = 288;             // 8 compute warps + 1 producer warp
constexpr int DEC_CONSUMERS = 256;
constexpr int DEC_MAX_E = 1024;
constexpr int DEC_MAX_MB = 4;                // 16-slot blocks of the down matrix per warp (8 warps: up to 512 slots)
constexpr int DEC_MAX_RING = 12;
constexpr int DEC_MIN_RING = 3;              // one tile
constexpr int ZP_STRIDE = N_TILE + 32;       // halves; rows 64 bytes apart modulo 128: 16-byte operand loads of a quarter warp hit distinct banks

// Rows g + 8 of every A fragment carry a factor 16 (fast_layout.cuh): accumulator registers 2 and 3 are scaled back
// with 2^20 instead of 2^24.
constexpr float DEC_UNSCALE_LO = 16777216.f, DEC_UNSCALE_HI = 1048576.f;

__host__ __device__ inline int dec_slots_stride(int max_slots) { return (max_slots + 63) / 64 * 64 + 32; }
// one ring slot holds one section = [fp16 scale per slot | arena words] of one matrix of one tile
__host__ __device__ inline int dec_sec_bytes(int max_slots, int max_words) {
  return static_cast<int>(align_up_c(static_cast<size_t>(max_slots) * 2 + static_cast<size_t>(max_words) * 4, 128));
}

// Dynamic shared memory of one CTA.
struct DecLayout {
  int ring, hrows, tab_gu, tab_d, hs, act, zp, soff, pbase, total;   // byte offsets
  int stride, act_bytes, zp_bytes, tab_bytes;
};
__host__ __device__ inline DecLayout dec_layout(int max_slots, int h_rank, int sec_bytes, int ring_slots, int num_experts, int act_bufs) {
  DecLayout L;
  int o = 0;
  L.stride = dec_slots_stride(max_slots);
  L.tab_bytes = static_cast<int>(align_up_c(static_cast<size_t>(max_slots) * 4, 128));
  L.act_bytes = static_cast<int>(align_up_c(static_cast<size_t>(2) * FAST_MAX_TOK * L.stride * 2, 128));
  L.zp_bytes = static_cast<int>(align_up_c(static_cast<size_t>(FAST_MAX_TOK) * ZP_STRIDE * 2, 128));
  L.ring = o;   o += ring_slots * sec_bytes;
  L.hrows = o;  o += static_cast<int>(align_up_c(static_cast<size_t>(2) * FAST_MAX_TOK * h_rank * 2, 128));
  L.tab_gu = o; o += 2 * L.tab_bytes;
  L.tab_d = o;  o += 2 * L.tab_bytes;       // double-buffered: needed until the end of the unit
  L.hs = o;     o += L.act_bytes;
  L.act = o;    o += act_bufs * L.act_bytes;
  L.zp = o;     o += 2 * L.zp_bytes;
  L.soff = o;   o += static_cast<int>(align_up_c(static_cast<size_t>(num_experts + 1) * 4, 16));   // expert_offsets
  L.pbase = o;  o += static_cast<int>(align_up_c(static_cast<size_t>(num_experts + 4) * 2, 16));   // prefix of passes
  L.total = o;
  return L;
}

struct DecParams {
  const FastExpert* fast;
  const unsigned char* arena;
  const __half* h_gate;
  const __half* h_up;
  const int32_t* token_indices;
  const int32_t* expert_offsets;
  const float* route_w;
  float* rank_accum;
  long long* acc64;      // deterministic mode: 64-bit fixed-point accumulators instead of rank_accum (else null)
  int* status;
  int h_rank, rank_out, T, num_experts, n_tiles, intermediate;
  int max_slots, sec_bytes, ring;
  int act_bufs;          // 2: next tile's operand is built before this tile's barrier; 1: a second barrier per tile instead
  unsigned long long wait_limit_ns;
};

struct DecUnitInfo {
  FastExpert fe;
  int tok[FAST_MAX_TOK];
  float rw[FAST_MAX_TOK];
  int npass, tile0, ntiles, pad_;
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMERS) : "memory"); }

// Bounded wait shared by all roles: gives up when another thread of the CTA already did, or after limit_ns.
__device__ __forceinline__ bool dec_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint64_t limit_ns) {
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
    if ((i & 7u) == 7u) {
      const uint64_t now = tc::global_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) { *abort_flag = 1; return false; }
    }
  }
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
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
// the first pair, consecutive pairs are `stride` words apart; `bp` points at this lane's eight halves of the first
// pair (operand row g, position 8 t).  The products are sums over the STORED codes u = q + offset.
template <bool DENSE>
__device__ __forceinline__ void mma_pairs(const uint32_t* __restrict__ wp, int stride, int npairs, const __half* __restrict__ bp,
                                          float (&acc)[4]) {
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
    wp += stride;
    bp += 32;
  }
}

// The same for the gate and up sections of one tile at once (equal group sizes): two independent accumulator chains.
template <bool DENSE>
__device__ __forceinline__ void mma_pairs2(const uint32_t* __restrict__ wp0, const uint32_t* __restrict__ wp1, int stride, int npairs,
                                           const __half* __restrict__ bp0, const __half* __restrict__ bp1, float (&acc0)[4],
                                           float (&acc1)[4]) {
#pragma unroll 2
  for (int p = 0; p < npairs; ++p) {
    const uint4 b0 = *reinterpret_cast<const uint4*>(bp0);
    const uint4 b1 = *reinterpret_cast<const uint4*>(bp1);
    uint32_t a[4], c[4];
    if (DENSE) {
      const uint32_t w0 = *wp0, w1 = *wp1;
      dense_afrag(w0, a);
      dense_afrag(w1, c);
      mma_16816(acc0, a, b0.x, b0.y);
      mma_16816(acc1, c, b1.x, b1.y);
      dense_afrag(w0 >> 8, a);
      dense_afrag(w1 >> 8, c);
      mma_16816(acc0, a, b0.z, b0.w);
      mma_16816(acc1, c, b1.z, b1.w);
    } else {
      const uint2 w0 = *reinterpret_cast<const uint2*>(wp0);
      const uint2 w1 = *reinterpret_cast<const uint2*>(wp1);
      nib_afrag(w0.x, a);
      nib_afrag(w1.x, c);
      mma_16816(acc0, a, b0.x, b0.y);
      mma_16816(acc1, c, b1.x, b1.y);
      nib_afrag(w0.y, a);
      nib_afrag(w1.y, c);
      mma_16816(acc0, a, b0.z, b0.w);
      mma_16816(acc1, c, b1.z, b1.w);
    }
    wp0 += stride;
    wp1 += stride;
    bp0 += 32;
    bp1 += 32;
  }
}

__device__ __forceinline__ float sum8_halves(const uint4& v) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
  const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
  const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
  return ((a.x + a.y) + (b.x + b.y)) + ((c.x + c.y) + (d.x + d.y));
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// MAXMB: 16-slot blocks of the down matrix per warp (2: up to 256 slots, 4: up to 512); the smaller instance keeps the
// kernel's code, which the instruction cache has to hold, short.
template <int MAXMB>
__global__ void __launch_bounds__(DEC_THREADS) experts_decode_kernel(const DecParams P) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ DecUnitInfo info[2];
  __shared__ __align__(8) uint64_t bar_full[DEC_MAX_RING];
  __shared__ __align__(8) uint64_t bar_empty[DEC_MAX_RING];
  __shared__ __align__(8) uint64_t bar_unit_full[2];
  __shared__ __align__(8) uint64_t bar_tail_empty[2];
  __shared__ __align__(8) uint64_t bar_head_empty;
  __shared__ int warp_tot[DEC_THREADS / 32];
  __shared__ float corr[2][2 * FAST_MAX_TOK];    // [buffer][matrix * 8 + token]: offset-weighted operand sums
  __shared__ __align__(16) float zsum_part[2][FAST_MAX_TOK][8]; // [buffer][token][warp]: partial sums of z over the warp's 16 columns
  __shared__ int abort_raw;
  volatile int* abort_flag = &abort_raw;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const DecLayout lay = dec_layout(P.max_slots, P.h_rank, P.sec_bytes, P.ring, P.num_experts, P.act_bufs);
  int* soff = reinterpret_cast<int*>(smem_raw + lay.soff);                 // expert_offsets [E + 1]
  uint16_t* pbase = reinterpret_cast<uint16_t*>(smem_raw + lay.pbase);     // exclusive prefix of passes per expert
  const uint64_t limit = P.wait_limit_ns;

  if (tid == 0) {
    for (int i = 0; i < P.ring; ++i) {
      tc::mbar_init(&bar_full[i], 1);
      tc::mbar_init(&bar_empty[i], 8);
    }
    tc::mbar_init(&bar_unit_full[0], 1);
    tc::mbar_init(&bar_unit_full[1], 1);
    tc::mbar_init(&bar_tail_empty[0], 8);
    tc::mbar_init(&bar_tail_empty[1], 8);
    tc::mbar_init(&bar_head_empty, 8);
    tc::mbar_init_fence();
    abort_raw = 0;
  }
  // ---- passes per expert (ceil(assignments / 8)) and their exclusive prefix: 4 consecutive experts per thread
  int total_passes;
  {
    const int e0 = tid * 4;
    int o[5];
#pragma unroll
    for (int i = 0; i < 5; ++i) o[i] = e0 + i <= P.num_experts ? P.expert_offsets[e0 + i] : 0;
    int pass[4], sum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int cnt = e0 + i < P.num_experts ? o[i + 1] - o[i] : 0;
      pass[i] = cnt > 0 ? (cnt + FAST_MAX_TOK - 1) / FAST_MAX_TOK : 0;
      sum += pass[i];
      if (e0 + i <= P.num_experts) soff[e0 + i] = o[i];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      const int n = warp_tot[w];
      if (w < warp) before += n;
      all += n;
    }
    total_passes = all;
    int run = before + incl - sum;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (e0 + i < P.num_experts) pbase[e0 + i] = static_cast<uint16_t>(run);
      run += pass[i];
    }
    __syncthreads();
  }
  if (total_passes == 0) return;
  // tile ranges: as many splits per expert as keep the number of units within one round of the grid
  int n_split = static_cast<int>(gridDim.x) / total_passes;
  n_split = n_split < 1 ? 1 : (n_split > P.n_tiles ? P.n_tiles : n_split);
  const int tiles_per = (P.n_tiles + n_split - 1) / n_split;
  n_split = (P.n_tiles + tiles_per - 1) / tiles_per;
  const int n_units = total_passes * n_split;
  if (static_cast<int>(blockIdx.x) >= n_units) return;

  unsigned char* ring = smem_raw + lay.ring;
  const uint32_t R = static_cast<uint32_t>(P.ring);

  if (warp == 8) {
    // ------------------------------------------------------------------ producer warp
    // lane m (0..2) owns section m (gate, up, down) of every tile: its ring slot advances by 3 per tile
    uint32_t my_slot = lane < 3 ? static_cast<uint32_t>(lane) : 0u, my_phase = 0;
    bool ok = true;
    int it = 0;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++it) {
      const int ub = it & 1;
      const int pu = u / n_split, sp = u - pu * n_split;
      int lo = 0, hi = P.num_experts - 1;          // last expert whose prefix is <= pu
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (static_cast<int>(pbase[mid]) <= pu) lo = mid; else hi = mid - 1;
      }
      const int e = lo, pass = pu - static_cast<int>(pbase[e]);
      const int tile0 = sp * tiles_per, ntl = min(tiles_per, P.n_tiles - tile0);
      const int a_begin = soff[e] + pass * FAST_MAX_TOK;
      const int npass = min(FAST_MAX_TOK, soff[e + 1] - a_begin);
      // descriptor, token ids and weights travel together (one round trip)
      uint32_t fe_words[(sizeof(FastExpert) / 4 + 31) / 32];
#pragma unroll
      for (int i = 0; i < static_cast<int>((sizeof(FastExpert) / 4 + 31) / 32); ++i) {
        const int w = lane + 32 * i;
        fe_words[i] = w < static_cast<int>(sizeof(FastExpert) / 4) ? reinterpret_cast<const uint32_t*>(&P.fast[e])[w] : 0u;
      }
      int tk = 0;
      float rwv = 0.f;
      if (lane < npass) {
        tk = P.token_indices[a_begin + lane];
        rwv = P.route_w[a_begin + lane];
      }
      ok = __all_sync(0xffffffffu, dec_wait(&bar_tail_empty[ub], ((it >> 1) & 1) ^ 1, abort_flag, limit) &&
                                       dec_wait(&bar_head_empty, (it & 1) ^ 1, abort_flag, limit));
      if (!ok) break;
      DecUnitInfo& si = info[ub];
#pragma unroll
      for (int i = 0; i < static_cast<int>((sizeof(FastExpert) / 4 + 31) / 32); ++i) {
        const int w = lane + 32 * i;
        if (w < static_cast<int>(sizeof(FastExpert) / 4)) reinterpret_cast<uint32_t*>(&si.fe)[w] = fe_words[i];
      }
      if (lane < FAST_MAX_TOK) {
        const bool good = lane < npass && tk >= 0 && tk < P.T;
        tk = good ? tk : 0;
        si.tok[lane] = tk;
        si.rw[lane] = good ? rwv : 0.f;
      }
      if (lane == 0) { si.npass = npass; si.tile0 = tile0; si.ntiles = ntl; }
      __syncwarp();
      const FastExpert& fe = si.fe;
      const uint32_t row_bytes = static_cast<uint32_t>(P.h_rank) * 2u;
      if (lane == 0)
        tc::mbar_expect_tx(&bar_unit_full[ub], static_cast<uint32_t>(fe.m[0].nslots + fe.m[1].nslots + fe.m[2].nslots) * 4u +
                                                   2u * npass * row_bytes);
      __syncwarp();
      const int tkn = __shfl_sync(0xffffffffu, tk, (lane - 8) & 7);
      if (lane < 3) {              // [rank | s] tables of gate, up (per unit) and down (kept until the unit ends)
        unsigned char* dst = lane < 2 ? smem_raw + lay.tab_gu + lane * lay.tab_bytes : smem_raw + lay.tab_d + ub * lay.tab_bytes;
        tc::bulk_g2s(dst, P.arena + fe.m[lane].tab_off, static_cast<uint32_t>(fe.m[lane].nslots) * 4u, &bar_unit_full[ub]);
      } else if (lane >= 8 && lane < 8 + 2 * FAST_MAX_TOK) {
        const int m = (lane - 8) >> 3, n = (lane - 8) & 7;
        if (n < npass) {
          const __half* hsrc = (m == 0 ? P.h_gate : P.h_up) + static_cast<int64_t>(tkn) * P.h_rank;
          tc::bulk_g2s(smem_raw + lay.hrows + (static_cast<size_t>(m) * FAST_MAX_TOK + n) * row_bytes, hsrc, row_bytes,
                       &bar_unit_full[ub]);
        }
      }
      __syncwarp();
      if (lane < 3) {
        const uint32_t bytes = static_cast<uint32_t>(fe.m[lane].nslots) * 2u + static_cast<uint32_t>(fe.m[lane].words) * 4u;
        const unsigned char* src = P.arena + fe.unit_base + static_cast<int64_t>(tile0) * fe.unit_bytes + fe.sec_off[lane];
        for (int i = 0; i < ntl; ++i) {
          if (!dec_wait(&bar_empty[my_slot], my_phase ^ 1u, abort_flag, limit)) { ok = false; break; }
          tc::mbar_expect_tx(&bar_full[my_slot], bytes);
          tc::bulk_g2s(ring + static_cast<size_t>(my_slot) * P.sec_bytes, src, bytes, &bar_full[my_slot]);
          src += fe.unit_bytes;
          my_slot += 3u;
          if (my_slot >= R) { my_slot -= R; my_phase ^= 1u; }
        }
      }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (*abort_flag) {
      // leave only after the copies already started have landed (or their wait ran out): every barrier that still
      // has a transaction pending completes its current phase when the bytes arrive
      __syncwarp();
      if (lane < 3) {
        // the last section this lane issued sits R/3 or fewer tiles back; waiting for the phase it was issued in is enough
        uint32_t s = my_slot, ph = my_phase;
        if (s < 3u) { s += R; ph ^= 1u; }
        s -= 3u;
        tc::mbar_wait(&bar_full[s], ph, limit);
      }
      if (lane == 0) {
        for (int j = it > 2 ? it - 2 : 0; j < it; ++j) tc::mbar_wait(&bar_unit_full[j & 1], (j >> 1) & 1, limit);
        atomicExch(P.status, BM_ERR_TIMEOUT);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- compute warps
  const int g = lane >> 2, t = lane & 3;
  __half* hs = reinterpret_cast<__half*>(smem_raw + lay.hs);
  const int zpos_lo = slot_pos(16 * warp + g), zpos_hi = slot_pos(16 * warp + g + 8);   // where this thread's z values go
  uint32_t rs = 0, rp = 0;      // ring slot and phase of the current tile's gate section
  int it = 0;
  for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++it) {
    const int ub = it & 1;
    bool ok = dec_wait(&bar_unit_full[ub], (it >> 1) & 1, abort_flag, limit);
    const DecUnitInfo& si = info[ub];
    const FastExpert& fe = si.fe;
    const int npass = si.npass, tile0 = si.tile0, ntl = si.ntiles;
    // ---- hs[m][n][pos(slot)] = fp16(h[tok_n, rank(slot)] * S(slot)), once per unit
    if (ok) {
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const int nslots = fe.m[m].nslots;
        const unsigned char* tab = smem_raw + lay.tab_gu + m * lay.tab_bytes;
        const int16_t* rank_t = reinterpret_cast<const int16_t*>(tab);
        const __half* s_t = reinterpret_cast<const __half*>(tab + nslots * 2);
        const __half* hrow = reinterpret_cast<const __half*>(smem_raw + lay.hrows) + static_cast<size_t>(m) * FAST_MAX_TOK * P.h_rank;
        __half* dst = hs + static_cast<size_t>(m) * FAST_MAX_TOK * lay.stride;
        for (int slot = tid; slot < nslots; slot += DEC_CONSUMERS) {
          const int rk = rank_t[slot];
          const int pos = slot_pos(slot);
          const float sv = __half2float(s_t[slot]);
          const bool live = rk >= 0 && rk < P.h_rank;
#pragma unroll
          for (int n = 0; n < FAST_MAX_TOK; ++n) {
            const float hv = (live && n < npass) ? __half2float(hrow[n * P.h_rank + rk]) : 0.f;
            dst[n * lay.stride + pos] = __float2half_rn(hv * sv);
          }
        }
      }
    }
    consumer_sync();
    if (*abort_flag) break;
    if (lane == 0) tc::mbar_arrive(&bar_head_empty);     // h rows and gate/up tables are consumed

    // Operand of one tile: act[buf][m][n][:] = hs[m][n][:] * scale_m(tile)[:], and the offset-weighted sum of every row.
    // Warp w builds rows 2w and 2w+1 of the 16 (matrix, token) rows; a lane owns chunks of 8 positions.  `gs`, `gp`:
    // ring slot and phase of that tile's gate section.
    auto build_operand = [&](int buf, uint32_t gs, uint32_t gp) -> bool {
      const int m = warp >> 2;
      if (m) { gs += 1u; if (gs >= R) { gs -= R; gp ^= 1u; } }
      if (!dec_wait(&bar_full[gs], gp, abort_flag, limit)) return false;
      const unsigned char* sec = ring + static_cast<size_t>(gs) * P.sec_bytes;
      const int nch = fe.m[m].nslots >> 3, nib_ch = fe.m[m].nblk[0] * 2;
      __half* act = reinterpret_cast<__half*>(smem_raw + lay.act + buf * lay.act_bytes);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int row = 2 * warp + j;          // = m * 8 + n
        float sum = 0.f;
        if ((row & 7) < npass) {
          for (int c = lane; c < nch; c += 32) {
            const uint4 hv = *reinterpret_cast<const uint4*>(hs + row * lay.stride + 8 * c);
            const uint4 sv = *reinterpret_cast<const uint4*>(sec + 16 * c);
            uint4 pr;
            pr.x = hmul2_u32(hv.x, sv.x);
            pr.y = hmul2_u32(hv.y, sv.y);
            pr.z = hmul2_u32(hv.z, sv.z);
            pr.w = hmul2_u32(hv.w, sv.w);
            *reinterpret_cast<uint4*>(act + row * lay.stride + 8 * c) = pr;
            sum += (c < nib_ch ? static_cast<float>(FAST_NIB_OFFSET) : static_cast<float>(FAST_DENSE_OFFSET)) * sum8_halves(pr);
          }
        } else {
          for (int c = lane; c < nch; c += 32) *reinterpret_cast<uint4*>(act + row * lay.stride + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) corr[buf][row] = sum;
      }
      return true;
    };

    ok = ok && build_operand(0, rs, rp);
    consumer_sync();
    if (*abort_flag) break;

    float dtot[MAXMB][4];
#pragma unroll
    for (int i = 0; i < MAXMB; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) dtot[i][j] = 0.f;
    const FastMat& fd = fe.m[2];
    const int nblk_d = fd.nslots >> 4;
    const bool twin = fe.m[0].nblk[0] == fe.m[1].nblk[0] && fe.m[0].nblk[1] == fe.m[1].nblk[1];

    for (int i = 0; i < ntl; ++i) {
      const int buf = i & 1;                           // z / zsum buffer
      const int abuf = P.act_bufs == 2 ? buf : 0;      // operand / corr buffer
      const int n_valid = min(N_TILE, P.intermediate - (tile0 + i) * N_TILE);
      // ring positions of this tile's up and down sections and of the next tile's gate section
      uint32_t us = rs + 1u, up_ = rp;
      if (us >= R) { us -= R; up_ ^= 1u; }
      uint32_t ds = us + 1u, dp = up_;
      if (ds >= R) { ds -= R; dp ^= 1u; }
      uint32_t ns = ds + 1u, np = dp;
      if (ns >= R) { ns -= R; np ^= 1u; }
      // ---- gate / up: this warp owns columns 16*warp .. 16*warp+15 of the tile
      float acc[2][4];
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[m][j] = 0.f;
      if (ok) ok = dec_wait(&bar_full[rs], rp, abort_flag, limit) && dec_wait(&bar_full[us], up_, abort_flag, limit);
      if (ok) {
        const __half* act = reinterpret_cast<const __half*>(smem_raw + lay.act + abuf * lay.act_bytes);
        const uint32_t* sec_g = reinterpret_cast<const uint32_t*>(ring + static_cast<size_t>(rs) * P.sec_bytes + fe.m[0].nslots * 2);
        const uint32_t* sec_u = reinterpret_cast<const uint32_t*>(ring + static_cast<size_t>(us) * P.sec_bytes + fe.m[1].nslots * 2);
        const __half* bop_g = act + g * lay.stride + 8 * t;
        const __half* bop_u = bop_g + FAST_MAX_TOK * lay.stride;
        // nibble words [pair][x][lane][2], dense words [pair][x][lane]
        if (twin) {
          const int nb0 = fe.m[0].nblk[0], nb1 = fe.m[0].nblk[1];
          mma_pairs2<false>(sec_g + (warp * 32 + lane) * 2, sec_u + (warp * 32 + lane) * 2, 512, nb0 >> 1, bop_g, bop_u, acc[0], acc[1]);
          mma_pairs2<true>(sec_g + nb0 * 256 + warp * 32 + lane, sec_u + nb0 * 256 + warp * 32 + lane, 256, nb1 >> 1,
                           bop_g + nb0 * 16, bop_u + nb0 * 16, acc[0], acc[1]);
        } else {
          mma_pairs<false>(sec_g + (warp * 32 + lane) * 2, 512, fe.m[0].nblk[0] >> 1, bop_g, acc[0]);
          mma_pairs<true>(sec_g + fe.m[0].nblk[0] * 256 + warp * 32 + lane, 256, fe.m[0].nblk[1] >> 1, bop_g + fe.m[0].nblk[0] * 16, acc[0]);
          mma_pairs<false>(sec_u + (warp * 32 + lane) * 2, 512, fe.m[1].nblk[0] >> 1, bop_u, acc[1]);
          mma_pairs<true>(sec_u + fe.m[1].nblk[0] * 256 + warp * 32 + lane, 256, fe.m[1].nblk[1] >> 1, bop_u + fe.m[1].nblk[0] * 16, acc[1]);
        }
      }
      __syncwarp();
      if (lane == 0) {   // the gate and up sections of this tile are consumed (their scales went into the operand earlier)
        tc::mbar_arrive(&bar_empty[rs]);
        tc::mbar_arrive(&bar_empty[us]);
      }
      // ---- z = silu(g) * u as the down product's operand, and its per-token sums for the offset term
      {
        __half* zp = reinterpret_cast<__half*>(smem_raw + lay.zp + buf * lay.zp_bytes);
        float zs[2] = {0.f, 0.f};
        const float cg0 = corr[abuf][2 * t], cg1 = corr[abuf][2 * t + 1];
        const float cu0 = corr[abuf][FAST_MAX_TOK + 2 * t], cu1 = corr[abuf][FAST_MAX_TOK + 2 * t + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = 16 * warp + g + (j >= 2 ? 8 : 0);
          const int n = 2 * t + (j & 1);
          const float unscale = j >= 2 ? DEC_UNSCALE_HI : DEC_UNSCALE_LO;
          const float gv = acc[0][j] * unscale - ((j & 1) ? cg1 : cg0);
          const float uv = acc[1][j] * unscale - ((j & 1) ? cu1 : cu0);
          const float z = (c < n_valid && n < npass) ? __fdividef(gv, 1.f + __expf(-gv)) * uv : 0.f;
          const __half zh = __float2half_rn(z);
          zp[n * ZP_STRIDE + (j >= 2 ? zpos_hi : zpos_lo)] = zh;
          zs[j & 1] += __half2float(zh);
        }
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          zs[0] += __shfl_xor_sync(0xffffffffu, zs[0], o);
          zs[1] += __shfl_xor_sync(0xffffffffu, zs[1], o);
        }
        if (g == 0) {
          zsum_part[buf][2 * t][warp] = zs[0];
          zsum_part[buf][2 * t + 1][warp] = zs[1];
        }
      }
      // ---- the next tile's operand goes into the other buffer before the barrier; with one buffer it has to wait
      // until every warp is done with this tile's operand
      if (P.act_bufs == 2 && i + 1 < ntl && ok) ok = build_operand(buf ^ 1, ns, np);
      consumer_sync();
      if (*abort_flag) break;
      // ---- down: slot blocks round-robin over the warps, contraction over the tile's 128 columns
      {
        ok = dec_wait(&bar_full[ds], dp, abort_flag, limit);
        if (ok) {
          const unsigned char* sec = ring + static_cast<size_t>(ds) * P.sec_bytes;
          const __half* scale_d = reinterpret_cast<const __half*>(sec);
          const uint32_t* dwords = reinterpret_cast<const uint32_t*>(sec + fd.nslots * 2);
          const __half* zrow = reinterpret_cast<const __half*>(smem_raw + lay.zp + buf * lay.zp_bytes) + g * ZP_STRIDE + 8 * t;
          float zsum[2];
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float4 a = *reinterpret_cast<const float4*>(&zsum_part[buf][2 * t + h][0]);
            const float4 b = *reinterpret_cast<const float4*>(&zsum_part[buf][2 * t + h][4]);
            zsum[h] = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
          }
#pragma unroll
          for (int i2 = 0; i2 < MAXMB; ++i2) {
            const int mb = warp + 8 * i2;
            if (mb < nblk_d) {
              float dacc[4] = {0.f, 0.f, 0.f, 0.f};
              float off;
              // nibble words [mblock][pair][lane][2], dense words [mblock][pair][lane]
              if (mb < fd.nblk[0]) {
                mma_pairs<false>(dwords + (mb * 128 + lane) * 2, 64, 4, zrow, dacc);
                off = static_cast<float>(FAST_NIB_OFFSET);
              } else {
                mma_pairs<true>(dwords + fd.nblk[0] * 256 + (mb - fd.nblk[0]) * 128 + lane, 32, 4, zrow, dacc);
                off = static_cast<float>(FAST_DENSE_OFFSET);
              }
              const float sc_lo = __half2float(scale_d[mb * 16 + g]), sc_hi = __half2float(scale_d[mb * 16 + g + 8]);
              dtot[i2][0] += sc_lo * (dacc[0] * DEC_UNSCALE_LO - off * zsum[0]);
              dtot[i2][1] += sc_lo * (dacc[1] * DEC_UNSCALE_LO - off * zsum[1]);
              dtot[i2][2] += sc_hi * (dacc[2] * DEC_UNSCALE_HI - off * zsum[0]);
              dtot[i2][3] += sc_hi * (dacc[3] * DEC_UNSCALE_HI - off * zsum[1]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(&bar_empty[ds]);
      }
      if (P.act_bufs == 1 && i + 1 < ntl) {
        if (ok) ok = build_operand(0, ns, np);
        consumer_sync();
        if (*abort_flag) break;
      }
      rs = ns;
      rp = np;
    }
    if (*abort_flag) break;
    // ---- unit epilogue: rank_accum[token, logical rank] += sum over the unit's tiles * S * route weight
    {
      const unsigned char* tab = smem_raw + lay.tab_d + ub * lay.tab_bytes;
      const int16_t* rank_d = reinterpret_cast<const int16_t*>(tab);
      const __half* s_d = reinterpret_cast<const __half*>(tab + fd.nslots * 2);
#pragma unroll
      for (int i2 = 0; i2 < MAXMB; ++i2) {
        const int mb = warp + 8 * i2;
        if (mb < nblk_d) {
#pragma unroll
          for (int hr = 0; hr < 2; ++hr) {
            const int slot = mb * 16 + g + 8 * hr;
            const int rk = rank_d[slot];
            if (rk < 0 || rk >= P.rank_out) continue;
            const float sv = __half2float(s_d[slot]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int n = 2 * t + h;
              if (n >= npass) continue;
              acc_add(P.rank_accum, P.acc64, static_cast<int64_t>(si.tok[n]) * P.rank_out + rk, dtot[i2][2 * hr + h] * sv * si.rw[n]);
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) tc::mbar_arrive(&bar_tail_empty[ub]);
  }
  if (*abort_flag && tid == 0) atomicExch(P.status, BM_ERR_TIMEOUT);
}

// Launch geometry of the decode kernel for this layer on the current device: ring depth, shared memory, grid.
// Two CTAs per SM when a ring of at least one tile fits next to the per-unit buffers, else one CTA with a deeper ring.
int plan_experts_decode(bm_layer* L) {
  L->dec_ok = false;
  if (!L->fast_ok) return BM_OK;
  if (L->num_experts > DEC_MAX_E || L->max_slots > 128 * DEC_MAX_MB || L->rank_in % 8 != 0 || L->n_tiles < 1) return BM_OK;
  int dev = -1, sm_count = 0, smem_optin = 0, smem_sm = 0;
  BM_CUDA(cudaGetDevice(&dev));
  BM_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  BM_CUDA(cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  BM_CUDA(cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev));
  const bool small = L->max_slots <= 128 * 2;
  const void* kernel = small ? reinterpret_cast<const void*>(experts_decode_kernel<2>) : reinterpret_cast<const void*>(experts_decode_kernel<DEC_MAX_MB>);
  cudaFuncAttributes fa;
  BM_CUDA(cudaFuncGetAttributes(&fa, kernel));
  const int sec = dec_sec_bytes(L->max_slots, L->max_words);
  const int stat = static_cast<int>(fa.sharedSizeBytes);
  // candidates, best first: (CTAs per SM, operand buffers, ring slots).  More resident warps hide more latency; a ring
  // of two tiles keeps the copies ahead of the compute warps.
  static const int cand[][3] = {{2, 2, 6}, {2, 2, 5}, {2, 2, 4}, {2, 1, 4}, {2, 1, 3}, {1, 2, 12}, {1, 2, 9}, {1, 2, 6}, {1, 2, 3}, {1, 1, 3}};
  const int forced = L->dec_force_ctas;   // 0 = choose; testing and tuning can ask for a number of CTAs per SM
  int pick = -1;
  size_t smem = 0;
  for (int i = 0; i < static_cast<int>(sizeof(cand) / sizeof(cand[0])) + 2 && pick < 0; ++i) {
    int ctas, bufs, ring;
    if (i < 2) {   // three CTAs per SM only on request
      if (forced != 3) continue;
      ctas = 3; bufs = 1; ring = i == 0 ? 4 : 3;
    } else {
      ctas = cand[i - 2][0]; bufs = cand[i - 2][1]; ring = cand[i - 2][2];
      if (forced > 0 && forced < 3 && ctas != forced) continue;
    }
    const int total = dec_layout(L->max_slots, L->rank_in, sec, ring, L->num_experts, bufs).total;
    const int budget = ctas == 1 ? smem_optin - stat : smem_sm / ctas - 1024 - stat;
    if (total <= budget && total <= smem_optin - stat) {
      pick = i;
      smem = static_cast<size_t>(total);
      L->dec_ring = ring;
      L->dec_act_bufs = bufs;
      L->dec_ctas = ctas;
    }
  }
  if (pick < 0) return BM_OK;
  BM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_optin - stat));
  BM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
  int blocks = 0;
  BM_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, DEC_THREADS, smem));
  if (blocks < 1) return BM_OK;
  L->dec_sec_bytes = sec;
  L->dec_smem = smem;
  L->dec_grid = sm_count * (blocks < L->dec_ctas ? blocks : L->dec_ctas);
  L->dec_ok = true;
  return BM_OK;
}

bool experts_decode_fits(const bm_layer* L) { return L->dec_ok; }

int launch_experts_decode(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                          const int32_t* expert_offsets, const float* route_w, int T, int num_assign, float* rank_accum,
                          long long* acc64, cudaStream_t st) {
  BM_REQUIRE(num_assign / FAST_MAX_TOK + L->num_experts < 60000, BM_ERR_UNSUPPORTED,
             "experts_decode: %d assignments are too many passes for the decode path", num_assign);
  BM_REQUIRE(L->dec_ok, BM_ERR_UNSUPPORTED, "experts_decode: a unit of %d slots / %d words does not fit shared memory",
             L->max_slots, L->max_words);
  BM_REQUIRE((reinterpret_cast<uintptr_t>(h_gate) & 15u) == 0 && (reinterpret_cast<uintptr_t>(h_up) & 15u) == 0,
             BM_ERR_INVALID_ARG, "experts_decode: h_gate / h_up rows must be 16-byte aligned");
  DecParams P{};
  P.fast = L->fast_dev;
  P.arena = static_cast<const unsigned char*>(L->arena);
  P.h_gate = h_gate;
  P.h_up = h_up;
  P.token_indices = token_indices;
  P.expert_offsets = expert_offsets;
  P.route_w = route_w;
  P.rank_accum = rank_accum;
  P.acc64 = acc64;
  P.status = L->status_dev;
  P.h_rank = L->rank_in;
  P.rank_out = L->rank_out;
  P.T = T;
  P.num_experts = L->num_experts;
  P.n_tiles = L->n_tiles;
  P.intermediate = L->intermediate;
  P.max_slots = L->max_slots;
  P.sec_bytes = L->dec_sec_bytes;
  P.ring = L->dec_ring;
  P.act_bufs = L->dec_act_bufs;
  P.wait_limit_ns = tc::WAIT_LIMIT_NS;
  if (L->max_slots <= 128 * 2) experts_decode_kernel<2><<<L->dec_grid, DEC_THREADS, L->dec_smem, st>>>(P);
  else experts_decode_kernel<DEC_MAX_MB><<<L->dec_grid, DEC_THREADS, L->dec_smem, st>>>(P);
  BM_LAUNCH_CHECK("experts_decode_kernel");
  return BM_OK;
}

}  // namespace bm
