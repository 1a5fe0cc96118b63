// Expert-parallel exchange over peer memory (NVLink / NVSwitch, plain peer stores and loads -- no multicast, no
// collective library on the data path).  The reference has no distributed code; experts shard naturally, and because
// the routed experts act in rank space what has to cross the links is small:
//
//   dispatch  every rank writes the rank-space rows [h_gate | h_up] of its tokens straight into the receive buffers of
//             the ranks that own one of the token's experts -- once per (token, destination rank), not per assignment --
//             together with the token's top-k (ids, weights), which every rank gets (80 bytes per token at top-10);
//   combine   after the packed experts ran on each rank, the token's home rank reads the partial rank_accum rows from
//             exactly the ranks that contributed to that token and adds them in ascending rank order (deterministic).
//
// All buffers have fixed sizes (T tokens per rank per wave), so nothing is read back to the host and nothing depends on
// data-dependent split sizes.  The buffers live in memory that every rank has mapped (the caller allocates and
// exchanges the mappings); ranks are separated by stream-ordered barriers that the caller issues between the stages.
//
// Layout of one rank's receive area for a wave of T tokens per rank, G ranks, top-k, rank r (fp16) / r_out (fp32):
//   H     fp16 [2][G][T][r]      gate rows of all ranks' tokens, then up rows: token u = s*T + t is row u of both halves
//   R     int32 [2][G][T][k]     expert ids, then the bit patterns of the fp32 weights
//   PART  fp32 [G*T][r_out]      this rank's partial rank_accum for every token of the wave (written by the expert kernel)
#include "common.cuh"

namespace bm {

constexpr int EP_MAX_WORLD = 16;

struct EpPeers {
  void* p[EP_MAX_WORLD];
};

// One warp per local token.  The token's two rows are staged in shared memory once and then sent by the bulk-copy
// engine, one copy per row and destination rank (512 bytes at r = 256): the engine moves whole rows as large
// transactions, where the lanes' 16-byte stores cross the links as many small ones.  Rows whose size is not a multiple
// of 16 bytes would need the plain path; the launcher requires r % 8 == 0.
__global__ void __launch_bounds__(256) ep_push_kernel(EpPeers H, EpPeers R, int world, int rank, int T, int r, int k,
                                                      int experts_per_rank) {
  extern __shared__ __align__(128) unsigned char push_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  const size_t GT = static_cast<size_t>(world) * T;
  const size_t u = static_cast<size_t>(rank) * T + t;
  const int32_t* my_idx = reinterpret_cast<const int32_t*>(R.p[rank]) + u * k;
  const int32_t* my_w = reinterpret_cast<const int32_t*>(R.p[rank]) + (GT + u) * k;
  const uint32_t row_bytes = static_cast<uint32_t>(r) * 2u;
  unsigned char* stage = push_smem + static_cast<size_t>(warp) * 2 * row_bytes;
  // destinations of this token: owners of its experts
  unsigned need = 0;
  int32_t id = -1, wbits = 0;
  if (lane < k) {
    id = my_idx[lane];
    wbits = my_w[lane];
    const int d = id >= 0 ? id / experts_per_rank : -1;
    if (d >= 0 && d < world) need = 1u << d;
  }
  need = __reduce_or_sync(0xffffffffu, need) & ~(1u << rank);
  const uint4* src_g = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(H.p[rank]) + u * r);
  const uint4* src_u = reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(H.p[rank]) + (GT + u) * r);
  if (need) {
    for (int i = lane; i < r / 8; i += 32) {
      reinterpret_cast<uint4*>(stage)[i] = src_g[i];
      reinterpret_cast<uint4*>(stage + row_bytes)[i] = src_u[i];
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  // routing of every token goes to every rank (its routing build walks all tokens of the wave)
  for (int d = 0; d < world; ++d) {
    if (d == rank || lane >= k) continue;
    reinterpret_cast<int32_t*>(R.p[d])[u * k + lane] = id;
    reinterpret_cast<int32_t*>(R.p[d])[(GT + u) * k + lane] = wbits;
  }
  if (lane < world && ((need >> lane) & 1u)) {
    __half* dst_g = reinterpret_cast<__half*>(H.p[lane]) + u * r;
    __half* dst_u = reinterpret_cast<__half*>(H.p[lane]) + (GT + u) * r;
    const uint32_t s0 = static_cast<uint32_t>(__cvta_generic_to_shared(stage));
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_g), "r"(s0), "r"(row_bytes) : "memory");
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_u), "r"(s0 + row_bytes), "r"(row_bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");      // the copies are complete before the thread exits
  }
}

// One warp per (local token, 128 values of the row): rank_accum[t] = sum over the ranks that own one of its experts of
// their partial row, in ascending rank order.  All peer loads of a warp are issued before the first is used: a load from
// a peer takes microseconds, and one after the other they would add up.
__global__ void __launch_bounds__(256) ep_pull_reduce_kernel(EpPeers PART, const int32_t* __restrict__ my_idx, int world,
                                                             int rank, int T, int r_out, int k, int experts_per_rank,
                                                             float* __restrict__ rank_accum) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pieces = (r_out + 127) / 128;
  const int job = blockIdx.x * (blockDim.x >> 5) + warp;
  const int t = job / pieces, c0 = (job - t * pieces) * 128 + lane * 4;
  if (t >= T) return;
  const size_t u = static_cast<size_t>(rank) * T + t;
  unsigned need = 0;
  if (lane < k) {
    const int id = my_idx[static_cast<size_t>(t) * k + lane];
    const int d = id >= 0 ? id / experts_per_rank : -1;
    if (d >= 0 && d < world) need = 1u << d;
  }
  need = __reduce_or_sync(0xffffffffu, need);
  if (c0 >= r_out) return;
  float4 v[EP_MAX_WORLD];
#pragma unroll
  for (int s = 0; s < EP_MAX_WORLD; ++s) {
    v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (s < world && ((need >> s) & 1u)) v[s] = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(PART.p[s]) + u * r_out + c0);
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int s = 0; s < EP_MAX_WORLD; ++s) {
    // (a rank that did not contribute adds an exact zero: the sum is the same as if it were skipped)
    acc.x += v[s].x; acc.y += v[s].y; acc.z += v[s].z; acc.w += v[s].w;
  }
  *reinterpret_cast<float4*>(rank_accum + static_cast<size_t>(t) * r_out + c0) = acc;
}

// Barrier across the ranks of one box, stream-ordered: one block, thread g talks to rank g.  Every rank keeps, per
// channel, a count of the barriers it has entered (its epoch); it writes the epoch into its slot of every peer's flag
// row and waits until every peer's slot in its own row has reached the same epoch.  The wait is bounded: when it runs
// out the kernel raises the status word and returns, so a rank that never arrives costs a time-out, not a hang.
// Flag area of a rank: uint32 [EP_CHANNELS][32]: entries 0..world-1 = arrivals of rank g, entry 31 = own epoch.
constexpr int EP_CHANNELS = 8;
__global__ void __launch_bounds__(32) ep_barrier_kernel(EpPeers F, int world, int rank, int channel, unsigned long long limit_ns,
                                                        int* __restrict__ status) {
  uint32_t* mine = reinterpret_cast<uint32_t*>(F.p[rank]) + channel * 32;
  uint32_t epoch = 0;
  if (threadIdx.x == 0) {
    epoch = mine[31] + 1u;
    mine[31] = epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int g = threadIdx.x;
  if (g >= world) return;
  __threadfence_system();
  uint32_t* theirs = reinterpret_cast<uint32_t*>(F.p[g]) + channel * 32 + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const uint32_t* slot = mine + g;
  unsigned long long t0 = 0;
  for (uint32_t i = 0;; ++i) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(slot) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if ((i & 63u) == 63u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        atomicExch(status, BM_ERR_TIMEOUT);
        break;
      }
    }
  }
}

}  // namespace bm

extern "C" size_t bm_ep_flag_bytes(void) { return sizeof(uint32_t) * bm::EP_CHANNELS * 32; }

extern "C" int bm_ep_barrier(const bm_layer_t* layer, void* const* flag_bufs, int32_t world, int32_t rank, int32_t channel,
                             int32_t limit_ms, void* stream) {
  bm::NvtxRange nvtx_range("bm_ep_barrier");
  using namespace bm;
  BM_REQUIRE(layer && layer->status_dev && flag_bufs, BM_ERR_INVALID_ARG, "ep_barrier: null pointer");
  BM_REQUIRE(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world && channel >= 0 && channel < EP_CHANNELS,
             BM_ERR_INVALID_ARG, "ep_barrier: bad world / rank / channel");
  BM_REQUIRE(limit_ms > 0, BM_ERR_INVALID_ARG, "ep_barrier: the wait needs a limit");
  EpPeers F{};
  for (int g = 0; g < world; ++g) {
    BM_REQUIRE(flag_bufs[g] != nullptr, BM_ERR_INVALID_ARG, "ep_barrier: flag area of rank %d is null", g);
    F.p[g] = flag_bufs[g];
  }
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(F, world, rank, channel,
                                                                     static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                                                     layer->status_dev);
  BM_LAUNCH_CHECK("ep_barrier_kernel");
  return BM_OK;
}

extern "C" int bm_ep_push(void* const* h_bufs, void* const* route_bufs, int32_t world, int32_t rank, int32_t T, int32_t r,
                          int32_t k, int32_t experts_per_rank, void* stream) {
  bm::NvtxRange nvtx_range("bm_ep_push");
  using namespace bm;
  BM_REQUIRE(h_bufs && route_bufs, BM_ERR_INVALID_ARG, "ep_push: null pointer table");
  BM_REQUIRE(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world, BM_ERR_INVALID_ARG, "ep_push: bad world / rank");
  BM_REQUIRE(T >= 0 && r > 0 && r % 8 == 0 && k > 0 && k <= 32 && experts_per_rank > 0, BM_ERR_INVALID_ARG, "ep_push: bad sizes");
  if (T == 0 || world == 1) return BM_OK;
  EpPeers H{}, R{};
  for (int g = 0; g < world; ++g) {
    BM_REQUIRE(h_bufs[g] && route_bufs[g] && (reinterpret_cast<uintptr_t>(h_bufs[g]) & 15u) == 0, BM_ERR_INVALID_ARG,
               "ep_push: buffer of rank %d is null or misaligned", g);
    H.p[g] = h_bufs[g];
    R.p[g] = route_bufs[g];
  }
  const size_t push_smem = static_cast<size_t>(8) * 2 * r * 2;     // two rows per warp
  BM_REQUIRE(push_smem <= 48 * 1024, BM_ERR_UNSUPPORTED, "ep_push: rank %d too large for the staging buffer", r);
  ep_push_kernel<<<(T + 7) / 8, 256, push_smem, static_cast<cudaStream_t>(stream)>>>(H, R, world, rank, T, r, k, experts_per_rank);
  BM_LAUNCH_CHECK("ep_push_kernel");
  return BM_OK;
}

extern "C" int bm_ep_pull_reduce(void* const* part_bufs, const int32_t* my_topk_idx, int32_t world, int32_t rank, int32_t T,
                                 int32_t r_out, int32_t k, int32_t experts_per_rank, float* rank_accum, void* stream) {
  bm::NvtxRange nvtx_range("bm_ep_pull_reduce");
  using namespace bm;
  BM_REQUIRE(part_bufs && my_topk_idx && rank_accum, BM_ERR_INVALID_ARG, "ep_pull_reduce: null pointer");
  BM_REQUIRE(world >= 1 && world <= EP_MAX_WORLD && rank >= 0 && rank < world, BM_ERR_INVALID_ARG, "ep_pull_reduce: bad world / rank");
  BM_REQUIRE(T >= 0 && r_out > 0 && r_out % 4 == 0 && k > 0 && k <= 32 && experts_per_rank > 0, BM_ERR_INVALID_ARG,
             "ep_pull_reduce: bad sizes");
  if (T == 0) return BM_OK;
  EpPeers P{};
  for (int g = 0; g < world; ++g) {
    BM_REQUIRE(part_bufs[g] && (reinterpret_cast<uintptr_t>(part_bufs[g]) & 15u) == 0, BM_ERR_INVALID_ARG,
               "ep_pull_reduce: buffer of rank %d is null or misaligned", g);
    P.p[g] = part_bufs[g];
  }
  const int64_t jobs = static_cast<int64_t>(T) * ((r_out + 127) / 128);
  ep_pull_reduce_kernel<<<static_cast<unsigned>((jobs + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      P, my_topk_idx, world, rank, T, r_out, k, experts_per_rank, rank_accum);
  BM_LAUNCH_CHECK("ep_pull_reduce_kernel");
  return BM_OK;
}
