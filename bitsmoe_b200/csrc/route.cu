// Token routing: softmax -> top-k -> (renorm, rounding), then the expert-contiguous
// permutation with per-expert offsets and the padded tile table, all on the device
// with no host round trip.
//
// Semantics follow bitsmoe/models/qwen3moe/bitsmoe_block.py:47-51 (router tail) and
// bitsmoe/models/base_block.py:258-289 (_build_packed_routing).  Where the reference
// leaves the order open (torch.topk ties, an unstable argsort) this file fixes it:
// ties go to the lower expert id, and inside an expert assignments are ordered by
// ascending flat (token, slot) index.
#include "common.cuh"

namespace bm {

constexpr int ROUTE_MAX_E = 1024;
constexpr int ROUTE_BLOCK = 1024;           // assignments per block of the permutation kernels
constexpr int ROUTE_WARPS = ROUTE_BLOCK / 32;

// ---------------------------------------------------------------- top-k
// One warp per token; probabilities live in a warp-private shared row.
// Top-k of one token by one warp.  Up to ROUTE_REG_E experts stay in registers (lane l holds experts l, l+32, ...);
// `p` is a warp-private shared row of E floats used only beyond that.
constexpr int ROUTE_REG_PER_LANE = 8;
constexpr int ROUTE_REG_E = 32 * ROUTE_REG_PER_LANE;

__device__ __forceinline__ void warp_topk_token(const void* __restrict__ logits, int dtype, int t, int E, int k, int renorm,
                                                int weight_round, float* p, int32_t* __restrict__ idx_out,
                                                float* __restrict__ w_out) {
  const int lane = threadIdx.x & 31;
  float my_w = 0.f;   // lane j keeps the j-th selected weight (k <= 32)
  int my_i = 0;
  float wsum = 0.f;
  if (E <= ROUTE_REG_E) {
    float v[ROUTE_REG_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_REG_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      v[i] = e < E ? load_act(logits, dtype, static_cast<int64_t>(t) * E + e) : -INFINITY;
      mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < ROUTE_REG_PER_LANE; ++i) {
      v[i] = lane + 32 * i < E ? expf(v[i] - mx) : -1.f;   // padding can never win
      sum += fmaxf(v[i], 0.f);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int bi = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < ROUTE_REG_PER_LANE; ++i)
        if (v[i] > best) { best = v[i]; bi = lane + 32 * i; }   // ascending e: the first hit wins ties
      // probabilities are non-negative, so their bit patterns order like unsigned integers: two warp reductions
      // (largest value, then the lowest expert id holding it) replace a ten-shuffle butterfly
      const unsigned best_bits = __reduce_max_sync(0xffffffffu, __float_as_uint(fmaxf(best, 0.f)));
      bi = static_cast<int>(__reduce_min_sync(0xffffffffu, __float_as_uint(fmaxf(best, 0.f)) == best_bits ? static_cast<unsigned>(bi) : 0x7fffffffu));
      best = __uint_as_float(best_bits);
      const float w = best * inv;
      if (lane == j) { my_w = w; my_i = bi; }
      wsum += w;
#pragma unroll
      for (int i = 0; i < ROUTE_REG_PER_LANE; ++i)
        if (bi == lane + 32 * i) v[i] = -2.f;
    }
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) {
      const float v = load_act(logits, dtype, static_cast<int64_t>(t) * E + e);
      p[e] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
      const float v = expf(p[e] - mx);
      p[e] = v;
      sum += v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    __syncwarp();
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float v = p[e];
        if (v > best) { best = v; bi = e; }   // strided scan visits ascending e: first hit wins ties
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      const float w = best * inv;
      if (lane == j) { my_w = w; my_i = bi; }
      wsum += w;
      if (lane == 0) p[bi] = -2.f;
      __syncwarp();
    }
  }
  if (lane < k) {
    float w = renorm ? my_w / wsum : my_w;
    if (weight_round == BM_ROUND_F16) w = __half2float(__float2half_rn(w));
    else if (weight_round == BM_ROUND_BF16) w = __bfloat162float(__float2bfloat16_rn(w));
    idx_out[static_cast<int64_t>(t) * k + lane] = my_i;
    w_out[static_cast<int64_t>(t) * k + lane] = w;
  }
  __syncwarp();
}

// One warp per token; probabilities live in a warp-private shared row.
__global__ void __launch_bounds__(256) route_topk_kernel(const void* __restrict__ logits, int dtype, int T, int E, int k,
                                                        int renorm, int weight_round, int32_t* __restrict__ topk_idx,
                                                        float* __restrict__ topk_w) {
  extern __shared__ float sm_prob[];  // [warps][E]
  const int warp = threadIdx.x >> 5;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  warp_topk_token(logits, dtype, t, E, k, renorm, weight_round, sm_prob + warp * E, topk_idx, topk_w);
}

// ---------------------------------------------------------------- permutation
// Exact per-warp exclusive bases (a block holds up to 1024 assignments of one expert, so
// bases need 16 bits while per-warp counts fit a byte).
__device__ __forceinline__ void block_warp_bases(int E, const uint8_t* warp_cnt, uint16_t* warp_base, int* block_count) {
  for (int x = threadIdx.x; x < E; x += blockDim.x) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < ROUTE_WARPS; ++w) {
      warp_base[w * E + x] = static_cast<uint16_t>(run);
      run += warp_cnt[w * E + x];
    }
    block_count[x] = run;
  }
}

struct RouteSmem {
  // laid out by hand in dynamic shared memory: counts, bases, block_count, scan scratch
  uint8_t* warp_cnt;    // [ROUTE_WARPS][E]
  uint16_t* warp_base;  // [ROUTE_WARPS][E]
  int* block_count;     // [E]
  int* scan;            // [E + 1]
};

__device__ __forceinline__ RouteSmem carve_route_smem(unsigned char* base, int E) {
  RouteSmem s;
  size_t off = 0;
  s.block_count = reinterpret_cast<int*>(base + off); off += sizeof(int) * E;
  s.scan = reinterpret_cast<int*>(base + off); off += sizeof(int) * (E + 1);
  s.warp_base = reinterpret_cast<uint16_t*>(base + off); off += sizeof(uint16_t) * ROUTE_WARPS * E;
  s.warp_cnt = reinterpret_cast<uint8_t*>(base + off);
  return s;
}

__host__ __device__ inline size_t route_smem_bytes_dev(int E) {
  return (sizeof(int) * E + sizeof(int) * (E + 1) + sizeof(uint16_t) * ROUTE_WARPS * E + static_cast<size_t>(ROUTE_WARPS) * E + 15) / 16 * 16;
}
static size_t route_smem_bytes(int E) { return route_smem_bytes_dev(E); }

// Per-block counting shared by the fused and the multi-block paths.  Returns this
// thread's rank inside its warp; warp_base / block_count are valid after the call.
__device__ __forceinline__ int block_count_and_rank(int e, int E, RouteSmem& s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (ROUTE_WARPS * E + 3) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(s.warp_cnt)[i] = 0u;
  __syncthreads();
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_w = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_w == 0) s.warp_cnt[warp * E + e] = static_cast<uint8_t>(__popc(peers));
  __syncthreads();
  block_warp_bases(E, s.warp_cnt, s.warp_base, s.block_count);
  __syncthreads();
  return rank_w;
}

// Exclusive scan of block_count[0..E) into scan[0..E], single block, E <= ROUTE_MAX_E.
__device__ __forceinline__ void block_exclusive_scan(const int* in, int* out, int E) {
  __shared__ int warp_tot[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int x = threadIdx.x;
  int v = (x < E) ? in[x] : 0;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = warp_tot[lane];
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += n;
    }
    warp_tot[lane] = ti - t;
  }
  __syncthreads();
  const int excl = incl - v + warp_tot[warp];
  if (x < E) out[x] = excl;
  if (x == E - 1) out[E] = excl + v;
  __syncthreads();
}

__device__ __forceinline__ void write_tile_table(const int* offsets /*[E+1] shared*/, int E, int tile_rows,
                                                 int32_t* tile_table, int max_tiles, int32_t* counts, int* scratch /*[E+1]*/,
                                                 int* tiles_per /*[E]*/) {
  if (tile_table == nullptr && counts == nullptr) return;
  for (int x = threadIdx.x; x < E; x += blockDim.x) {
    const int n = offsets[x + 1] - offsets[x];
    tiles_per[x] = (n + tile_rows - 1) / tile_rows;
  }
  __syncthreads();
  block_exclusive_scan(tiles_per, scratch, E);
  const int total_tiles = scratch[E];
  if (tile_table) {
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
      const int a0 = offsets[x], n = offsets[x + 1] - offsets[x];
      int slot = scratch[x];
      for (int r = 0; r < n; r += tile_rows, ++slot) {
        tile_table[slot * 3 + 0] = x;
        tile_table[slot * 3 + 1] = a0 + r;
        tile_table[slot * 3 + 2] = min(tile_rows, n - r);
      }
    }
    for (int s = total_tiles + threadIdx.x; s < max_tiles; s += blockDim.x) {
      tile_table[s * 3 + 0] = 0;
      tile_table[s * 3 + 1] = 0;
      tile_table[s * 3 + 2] = 0;
    }
  }
  if (counts && threadIdx.x == 0) {
    counts[0] = offsets[E];
    counts[1] = total_tiles;
  }
}

// Routed expert id of assignment i -> packed id, or -1 (dropped).  Ids outside [0, num_routed) -- a gate that is not
// this library's own can hand in anything -- and map entries outside [0, E) are dropped instead of indexing with them.
__device__ __forceinline__ int local_expert(const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ g2l, int i,
                                            int num_routed, int E) {
  int e = topk_idx[i];
  if (static_cast<unsigned>(e) >= static_cast<unsigned>(num_routed)) return -1;
  if (g2l) e = g2l[e];
  return static_cast<unsigned>(e) < static_cast<unsigned>(E) ? e : -1;
}

// A <= ROUTE_BLOCK: everything in one block.
__global__ void __launch_bounds__(ROUTE_BLOCK) route_build_fused_kernel(
    const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w, const int32_t* __restrict__ g2l, int num_routed,
    int A, int k, int E, int tile_rows, int32_t* __restrict__ token_indices, int32_t* __restrict__ expert_offsets,
    float* __restrict__ route_flat, int32_t* __restrict__ tile_table, int max_tiles, int32_t* __restrict__ counts) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  RouteSmem s = carve_route_smem(sm_raw, E);
  const int i = threadIdx.x;
  int e = -1;
  if (i < A) e = local_expert(topk_idx, g2l, i, num_routed, E);
  const int rank_w = block_count_and_rank(e, E, s);
  block_exclusive_scan(s.block_count, s.scan, E);
  for (int x = threadIdx.x; x <= E; x += blockDim.x) expert_offsets[x] = s.scan[x];
  if (e >= 0) {
    const int pos = s.scan[e] + s.warp_base[(threadIdx.x >> 5) * E + e] + rank_w;
    token_indices[pos] = i / k;
    route_flat[pos] = topk_w[i];
  }
  __syncthreads();
  // reuse block_count / warp_base storage as scratch for the tile table
  write_tile_table(s.scan, E, tile_rows, tile_table, max_tiles, counts, reinterpret_cast<int*>(s.warp_base), s.block_count);
}

// A > ROUTE_BLOCK: count per block, scan across blocks, scatter.
__global__ void __launch_bounds__(ROUTE_BLOCK) route_count_kernel(const int32_t* __restrict__ topk_idx,
                                                                 const int32_t* __restrict__ g2l, int num_routed, int A, int E,
                                                                 int32_t* __restrict__ block_hist /*[nblocks][E]*/) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  RouteSmem s = carve_route_smem(sm_raw, E);
  const int i = blockIdx.x * ROUTE_BLOCK + threadIdx.x;
  int e = -1;
  if (i < A) e = local_expert(topk_idx, g2l, i, num_routed, E);
  block_count_and_rank(e, E, s);
  for (int x = threadIdx.x; x < E; x += blockDim.x) block_hist[static_cast<int64_t>(blockIdx.x) * E + x] = s.block_count[x];
}

__global__ void __launch_bounds__(ROUTE_BLOCK) route_scan_kernel(int32_t* __restrict__ block_hist, int nblocks, int E,
                                                                int tile_rows, int32_t* __restrict__ expert_offsets,
                                                                int32_t* __restrict__ tile_table, int max_tiles,
                                                                int32_t* __restrict__ counts) {
  __shared__ int tot[ROUTE_MAX_E];
  __shared__ int off[ROUTE_MAX_E + 1];
  __shared__ int scratch[ROUTE_MAX_E + 1];
  __shared__ int chunk_tot[ROUTE_BLOCK];
  // The blocks' histograms are cut into `chunks` runs per expert, one thread each: every thread sums its run (independent
  // loads), the runs' totals are combined in shared memory, and a second walk over the run writes the exclusive prefixes.
  // One thread per expert walking all the blocks would serialise nblocks dependent round trips to memory.
  const int chunks = max(1, min(static_cast<int>(blockDim.x) / E, nblocks));
  const int len = (nblocks + chunks - 1) / chunks;
  const int x = threadIdx.x % E, c = threadIdx.x / E;
  const int b0 = c * len, b1 = min(nblocks, b0 + len);
  const bool active = c < chunks;
  if (active) {
    int sum = 0;
#pragma unroll 8
    for (int b = b0; b < b1; ++b) sum += block_hist[static_cast<int64_t>(b) * E + x];
    chunk_tot[c * E + x] = sum;
  }
  __syncthreads();
  if (active) {
    int run = 0;
    for (int cc = 0; cc < c; ++cc) run += chunk_tot[cc * E + x];
    if (c == chunks - 1) tot[x] = run + chunk_tot[c * E + x];
#pragma unroll 8
    for (int b = b0; b < b1; ++b) {
      const int v = block_hist[static_cast<int64_t>(b) * E + x];
      block_hist[static_cast<int64_t>(b) * E + x] = run;
      run += v;
    }
  }
  __syncthreads();
  block_exclusive_scan(tot, off, E);
  for (int i = threadIdx.x; i <= E; i += blockDim.x) expert_offsets[i] = off[i];
  write_tile_table(off, E, tile_rows, tile_table, max_tiles, counts, scratch, tot);
}

__global__ void __launch_bounds__(ROUTE_BLOCK) route_scatter_kernel(
    const int32_t* __restrict__ topk_idx, const float* __restrict__ topk_w, const int32_t* __restrict__ g2l, int num_routed,
    int A, int k, int E, const int32_t* __restrict__ block_hist, const int32_t* __restrict__ expert_offsets,
    int32_t* __restrict__ token_indices, float* __restrict__ route_flat) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  RouteSmem s = carve_route_smem(sm_raw, E);
  const int i = blockIdx.x * ROUTE_BLOCK + threadIdx.x;
  int e = -1;
  if (i < A) e = local_expert(topk_idx, g2l, i, num_routed, E);
  const int rank_w = block_count_and_rank(e, E, s);
  if (e >= 0) {
    const int pos = expert_offsets[e] + block_hist[static_cast<int64_t>(blockIdx.x) * E + e] +
                    s.warp_base[(threadIdx.x >> 5) * E + e] + rank_w;
    token_indices[pos] = i / k;
    route_flat[pos] = topk_w[i];
  }
}

}  // namespace bm

extern "C" int bm_route_topk(const void* logits, int logits_dtype, int32_t T, int32_t E, int32_t k, int32_t renorm,
                             int32_t weight_round, int32_t* topk_idx, float* topk_w, void* stream) {
  bm::NvtxRange nvtx_range("bm_route_topk");
  using namespace bm;
  BM_REQUIRE(T >= 0 && E > 0 && k > 0, BM_ERR_INVALID_ARG, "route_topk: bad sizes T=%d E=%d k=%d", T, E, k);
  BM_REQUIRE(k <= 32 && k <= E, BM_ERR_UNSUPPORTED, "route_topk: top_k=%d must be <= min(32, E=%d)", k, E);
  BM_REQUIRE(E <= ROUTE_MAX_E, BM_ERR_UNSUPPORTED, "route_topk: E=%d exceeds %d", E, ROUTE_MAX_E);
  BM_REQUIRE(logits_dtype >= BM_F16 && logits_dtype <= BM_F32, BM_ERR_INVALID_ARG, "route_topk: bad logits dtype");
  if (T == 0) return BM_OK;
  BM_REQUIRE(logits && topk_idx && topk_w, BM_ERR_INVALID_ARG, "route_topk: null pointer");
  const int warps = 8;
  route_topk_kernel<<<(T + warps - 1) / warps, warps * 32, sizeof(float) * warps * E, static_cast<cudaStream_t>(stream)>>>(
      logits, logits_dtype, T, E, k, renorm, weight_round, topk_idx, topk_w);
  BM_LAUNCH_CHECK("route_topk_kernel");
  return BM_OK;
}

extern "C" int32_t bm_route_max_tiles(int32_t T, int32_t k, int32_t num_local, int32_t tile_rows) {
  if (tile_rows <= 0) return 0;
  const int64_t A = static_cast<int64_t>(T) * k;
  // every expert wastes at most one partial tile
  const int64_t bound = A / tile_rows + num_local;
  const int64_t m = bound < A ? bound : A;  // a tile holds at least one row
  return static_cast<int32_t>(m > 0 ? m : 1);
}

extern "C" size_t bm_route_build_workspace_bytes(int32_t T, int32_t k, int32_t num_local) {
  const int64_t A = static_cast<int64_t>(T) * k;
  if (A <= bm::ROUTE_BLOCK) return 0;
  const int64_t nblocks = (A + bm::ROUTE_BLOCK - 1) / bm::ROUTE_BLOCK;
  return bm::align_up(static_cast<size_t>(nblocks) * num_local * sizeof(int32_t), 256);
}

extern "C" int bm_route_build(const int32_t* topk_idx, const float* topk_w, const int32_t* global_to_local,
                              int32_t num_routed, int32_t T,
                              int32_t k, int32_t num_local, int32_t tile_rows, int32_t* token_indices,
                              int32_t* expert_offsets, float* route_flat, int32_t* tile_table, int32_t* counts,
                              void* workspace, size_t workspace_bytes, void* stream) {
  bm::NvtxRange nvtx_range("bm_route_build");
  using namespace bm;
  BM_REQUIRE(T >= 0 && k > 0 && num_local > 0 && num_routed > 0, BM_ERR_INVALID_ARG, "route_build: bad sizes");
  BM_REQUIRE(global_to_local != nullptr || num_routed == num_local, BM_ERR_INVALID_ARG,
             "route_build: %d routed experts but %d packed and no id map", num_routed, num_local);
  BM_REQUIRE(num_local <= ROUTE_MAX_E, BM_ERR_UNSUPPORTED, "route_build: %d experts exceed %d", num_local, ROUTE_MAX_E);
  BM_REQUIRE(tile_rows > 0, BM_ERR_INVALID_ARG, "route_build: tile_rows must be positive");
  BM_REQUIRE(expert_offsets, BM_ERR_INVALID_ARG, "route_build: null expert_offsets");
  const int64_t A64 = static_cast<int64_t>(T) * k;
  BM_REQUIRE(A64 < (1ll << 30), BM_ERR_UNSUPPORTED, "route_build: too many assignments");
  const int A = static_cast<int>(A64);
  BM_REQUIRE(A == 0 || (topk_idx && topk_w && token_indices && route_flat), BM_ERR_INVALID_ARG, "route_build: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int max_tiles = bm_route_max_tiles(T, k, num_local, tile_rows);
  const size_t smem = route_smem_bytes(num_local);
  static PerDeviceOnce attr_once;
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  if (!attr_once.is_done(dev)) {
    const int big = static_cast<int>(route_smem_bytes(ROUTE_MAX_E));
    BM_CUDA(cudaFuncSetAttribute(route_build_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    BM_CUDA(cudaFuncSetAttribute(route_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    BM_CUDA(cudaFuncSetAttribute(route_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
    attr_once.mark(dev);
  }
  if (A <= ROUTE_BLOCK) {
    route_build_fused_kernel<<<1, ROUTE_BLOCK, smem, st>>>(topk_idx, topk_w, global_to_local, num_routed, A, k, num_local, tile_rows,
                                                           token_indices, expert_offsets, route_flat, tile_table,
                                                           max_tiles, counts);
    BM_LAUNCH_CHECK("route_build_fused_kernel");
    return BM_OK;
  }
  const int nblocks = (A + ROUTE_BLOCK - 1) / ROUTE_BLOCK;
  const size_t need = bm_route_build_workspace_bytes(T, k, num_local);
  BM_REQUIRE(workspace && workspace_bytes >= need, BM_ERR_WORKSPACE, "route_build: workspace of %zu bytes needed, %zu given",
             need, workspace_bytes);
  int32_t* block_hist = static_cast<int32_t*>(workspace);
  route_count_kernel<<<nblocks, ROUTE_BLOCK, smem, st>>>(topk_idx, global_to_local, num_routed, A, num_local, block_hist);
  BM_LAUNCH_CHECK("route_count_kernel");
  route_scan_kernel<<<1, ROUTE_BLOCK, 0, st>>>(block_hist, nblocks, num_local, tile_rows, expert_offsets, tile_table,
                                               max_tiles, counts);
  BM_LAUNCH_CHECK("route_scan_kernel");
  route_scatter_kernel<<<nblocks, ROUTE_BLOCK, smem, st>>>(topk_idx, topk_w, global_to_local, num_routed, A, k, num_local, block_hist,
                                                           expert_offsets, token_indices, route_flat);
  BM_LAUNCH_CHECK("route_scatter_kernel");
  return BM_OK;
}

extern "C" int bm_route(const void* logits, int logits_dtype, int32_t T, int32_t E_routed, int32_t k, int32_t renorm,
                        int32_t weight_round, const int32_t* global_to_local, int32_t num_local, int32_t tile_rows,
                        int32_t* topk_idx, float* topk_w, int32_t* token_indices, int32_t* expert_offsets,
                        float* route_flat, int32_t* tile_table, int32_t* counts, void* workspace, size_t workspace_bytes,
                        void* stream) {
  bm::NvtxRange nvtx_range("bm_route");
  using namespace bm;
  int rc = bm_route_topk(logits, logits_dtype, T, E_routed, k, renorm, weight_round, topk_idx, topk_w, stream);
  if (rc) return rc;
  return bm_route_build(topk_idx, topk_w, global_to_local, E_routed, T, k, num_local, tile_rows, token_indices,
                        expert_offsets, route_flat, tile_table, counts, workspace, workspace_bytes, stream);
}
