// Shared declarations of the bitsmoe_b200 library (host + device).
#pragma once

#include <nvtx3/nvToolsExt.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <vector>

#include "../../include/bitsmoe_b200.h"

namespace bm {

constexpr int K_SLAB = 64;     // rows per slab at most
constexpr int N_TILE = 128;    // columns per scale group
constexpr int K_STAGE = 16;    // rows per payload stage
constexpr int N_MICRO = 32;    // columns per bit-plane word
constexpr int MICROS = N_TILE / N_MICRO;

int set_error(int status, const char* fmt, ...);
void count_launch();   // every kernel launch of the library is counted (bm_launch_count)

#define BM_REQUIRE(cond, status, ...)                       \
  do {                                                      \
    if (!(cond)) return ::bm::set_error((status), __VA_ARGS__); \
  } while (0)

#define BM_CUDA(expr)                                                                   \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::bm::set_error(BM_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define BM_LAUNCH_CHECK(name)                                                              \
  do {                                                                                     \
    ::bm::count_launch();                                                                  \
    cudaError_t _e = cudaGetLastError();                                                   \
    if (_e != cudaSuccess)                                                                 \
      return ::bm::set_error(BM_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
  } while (0)

// Set-up that belongs to a (kernel, device) pair -- cudaFuncSetAttribute, occupancy queries -- runs once per device
// ordinal, not once per process: a second GPU driven from the same process needs its own.  Two host threads may both
// run the set-up for a device (it is idempotent); the flag only publishes that it has been done.
constexpr int MAX_DEVICES = 64;
struct PerDeviceOnce {
  std::atomic<unsigned char> done[MAX_DEVICES] = {};
  bool is_done(int dev) const { return dev >= 0 && dev < MAX_DEVICES && done[dev].load(std::memory_order_acquire) != 0; }
  void mark(int dev) { if (dev >= 0 && dev < MAX_DEVICES) done[dev].store(1, std::memory_order_release); }
};

// One packed matrix as the device sees it (pointers into the caller's buffers).
struct MatDev {
  const uint32_t* payload;
  const int32_t* rank_idx;
  const int32_t* tile_meta;
  const int32_t* slab_meta;
  const __half* scale;
  const __half* s;
  int32_t n_slabs;
  int32_t n_tile_rows;
  int32_t n_rows;
  int32_t pad_;
};

struct ExpertDev {
  MatDev m[3];
};

// Host mirror of one slab (validated at plan time).
struct SlabHost {
  int32_t bits, k_slab, rank_off, tile_off, tile_end;
};

struct MatHost {
  std::vector<SlabHost> slabs;
  std::vector<int32_t> tile_meta;  // [n_tile_rows * 3]
  int64_t bytes = 0;               // as stored by the reference
  int32_t n_rows = 0;
};

constexpr int FAST_MAX_TOK = 8;    // assignments per pass of the decode kernel (one MMA N-block)

struct FastMat {
  int32_t nblk[2];      // 16-slot blocks in the nibble group (3/4-bit rows), in the dense 2-bit group (1/2-bit rows)
  int32_t nslots;       // 16 * (nblk[0] + nblk[1])
  int32_t words;        // uint32 words per tile = 256 nblk[0] + 128 nblk[1]
  int32_t tab_off;      // byte offset (from arena base) of [int16 rank[nslots] | fp16 s[nslots] | int16 row[nslots]]
  int32_t pad_[3];
};

struct FastExpert {
  FastMat m[3];
  int64_t unit_base;    // byte offset of tile 0's unit block from arena base
  int32_t unit_bytes;   // bytes per unit block (multiple of 128)
  int32_t sec_off[6];   // byte offsets inside a unit: [0..2] scales of g,u,d, [3..5] words of g,u,d; sec_off[3+m] == sec_off[m] + 2 * nslots(m)
  int32_t pad_;
};

struct FastPlan {
  bool ok = false;
  std::vector<FastExpert> experts;
  std::vector<int16_t> slot_row;      // concatenated per (expert, matrix): slot -> local row or -1
  std::vector<int32_t> slot_row_off;  // [E*3] element offset into slot_row
  size_t table_off = 0;               // FastExpert table
  size_t tabs_off = 0;                // per-matrix rank/s/row tables
  size_t units_off = 0;
  size_t total = 0;
  int max_unit_bytes = 0, max_slots = 0, max_words = 0;
};

__host__ __device__ inline int words_per_row(int bits) { return bits == 16 ? 16 : bits; }

__host__ __device__ inline int code_offset(int bits) {
  // u = q + offset for bits > 1; the 1-bit case is q = 2u - 1.
  return bits == 1 ? 0 : (1 << (bits - 1));
}

inline bool supported_bits(int b) { return b == 1 || b == 2 || b == 3 || b == 4 || b == 6 || b == 8 || b == 16; }

__device__ __forceinline__ float load_act(const void* p, int dtype, int64_t i) {
  if (dtype == BM_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  if (dtype == BM_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ void store_act(void* p, int dtype, int64_t i, float v) {
  if (dtype == BM_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else if (dtype == BM_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}

// Accumulation into rank_accum: fp32 atomics (as bitsmoe/algorithms/cpp/mlp_forward.cu:2062 does), or -- the
// deterministic mode -- 64-bit fixed-point atomics: integer addition is associative, so the sum does not depend on the
// order in which CTAs arrive and two runs are bit-identical.  2^40 leaves 2^23 of range and 1e-12 of resolution.
constexpr float ACC_FIXED_SCALE = 1099511627776.f;
__device__ __forceinline__ void acc_add(float* __restrict__ acc32, long long* __restrict__ acc64, int64_t idx, float v) {
  if (acc64) atomicAdd(reinterpret_cast<unsigned long long*>(acc64) + idx, static_cast<unsigned long long>(__float2ll_rn(v * ACC_FIXED_SCALE)));
  else atomicAdd(acc32 + idx, v);
}

// C[M,N] = A[M,K] . B[N,K]^T ; up to two problems sharing A's shape in one launch.
struct GemmArgs {
  const void* A[2];
  const __half* B[2];
  void* C[2];
  const void* residual;  // same dtype / shape as C, problem 0 only
  int a_dtype, c_dtype;
  int round_a_f16;       // round an fp32 A through fp16 first (rank_accum.half())
  int M, N, K;
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
__host__ __device__ inline size_t align_up_c(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Arguments of the tensor-core basis products (gemm_tma.cu, gemm_tc.cu): C[z] = X . W[z]^T (+ residual for z = 0).
struct GemmTcArgs {
  const void* X;          // [M, K]
  const __half* W[2];     // [N, K] each
  void* C[2];             // [M, N] each
  const void* residual;   // [M, N] (W[0] only) or null
  int M, N, K;
  int x_dtype, c_dtype;
  int* status;
};
// Tiled-copy kernel first; BM_ERR_UNSUPPORTED (nothing launched) means: use launch_gemm_tc.
int launch_gemm_tma(const GemmTcArgs& a, int problems, cudaStream_t st);
int launch_gemm_tc(const GemmTcArgs& a, int problems, cudaStream_t st);
// Both in order.
inline int launch_gemm_basis(const GemmTcArgs& a, int problems, cudaStream_t st) {
  const int rc = launch_gemm_tma(a, problems, st);
  return rc == BM_ERR_UNSUPPORTED ? launch_gemm_tc(a, problems, st) : rc;
}

// NVTX range around a public entry point (route / projection / experts / combine / exchange show up as named ranges
// in a timeline tool; without a tool attached a push or pop is one null-pointer test).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

}  // namespace bm

struct bm_layer {
  int32_t num_experts = 0, hidden = 0, intermediate = 0, rank_in = 0, rank_out = 0, n_tiles = 0;
  int32_t max_rows = 0;            // largest n_rows over all matrices
  int device = 0;
  const __half* vh_gate = nullptr;
  const __half* vh_up = nullptr;
  const __half* u_down = nullptr;
  std::vector<bm::MatHost> host[3];   // [which][expert]
  std::vector<bm_matrix_t> src[3];    // caller's descriptors (pointers kept)
  bm::ExpertDev* experts_dev = nullptr;  // in the arena
  void* arena = nullptr;
  size_t arena_bytes = 0;
  bool fast_ok = false;            // every slab is 1/2/3/4-bit and shapes fit the decode / tensor paths
  const bm::FastExpert* fast_dev = nullptr;   // in the arena
  std::vector<bm::FastExpert> fast_host;
  int max_unit_bytes = 0, max_slots = 0, max_words = 0;
  // launch geometry of the decode kernel on this layer's device (plan_experts_decode)
  bool dec_ok = false;
  bool deterministic = false;      // rank_accum through 64-bit fixed-point atomics (bm_layer_set_option)
  int dec_ring = 0, dec_sec_bytes = 0, dec_grid = 0, dec_act_bufs = 2, dec_ctas = 0, dec_force_ctas = 0;
  size_t dec_smem = 0;
  int* status_dev = nullptr;       // device flag set by a kernel whose bounded wait gave up
  cudaStream_t side_stream = nullptr;   // routing runs here, beside the basis projection
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};
