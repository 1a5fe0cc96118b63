// Quantise + bit-plane pack + runtime-layout reorder of one slab in one kernel.
//
// Restates, fused, what the reference's packer does per slab in three steps
// (bitsmoe/quant/packer.py:210-306): quantize_symmetric per (rank row, 128-column tile)
// (bitsmoe/quant/quantizer.py:30-84: sign / mean-|x| for 1 bit; 50 rounds of alternating least squares on the scale for
// 2/3/4 bits; absmax for 6/8 bits; round half to even), BitPack.pack into 32-column bit-planes
// (bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu:81-121) and the [tile][stage 16 rows][micro][row][plane] reorder
// (packer.py:169-207).  One warp owns one (row, tile) group: lane l holds columns 32 m + l of the tile (m = 0..3), so
// a plane word is one __ballot_sync and lands at its final payload position directly.
#include "common.cuh"

namespace bm {

constexpr float Q_EPS = 1e-8f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// grid (ceil(k / 8), tiles), 8 warps per block.
__global__ void __launch_bounds__(256) quantize_pack_slab_kernel(const float* __restrict__ rows, int64_t ld, int k, int dim, int bits,
                                                                 uint32_t* __restrict__ payload, __half* __restrict__ scale_out,
                                                                 int8_t* __restrict__ codes_out) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int tile = blockIdx.y;
  if (r >= k) return;
  const int col0 = tile * N_TILE;
  const int n_valid = min(N_TILE, dim - col0);
  float x[MICROS];
  bool live[MICROS];
#pragma unroll
  for (int m = 0; m < MICROS; ++m) {
    const int c = m * N_MICRO + lane;
    live[m] = c < n_valid;
    x[m] = live[m] ? rows[static_cast<int64_t>(r) * ld + col0 + c] : 0.f;
  }
  // means are sums divided by the count, products and sums rounded separately (no fused multiply-add), as the
  // element-wise torch expressions of the reference round them
  const float n_f = static_cast<float>(n_valid);
  float sabs = 0.f;
#pragma unroll
  for (int m = 0; m < MICROS; ++m) sabs = __fadd_rn(sabs, fabsf(x[m]));
  const float mean_abs = fmaxf(__fdiv_rn(warp_sum(sabs), n_f), Q_EPS);
  const int hi = (1 << (bits - 1)) - 1, lo = -hi - 1;
  float q[MICROS];
  float scale;
  if (bits == 1) {
#pragma unroll
    for (int m = 0; m < MICROS; ++m) q[m] = x[m] < 0.f ? -1.f : 1.f;
    scale = mean_abs;
  } else if (bits <= 4) {
    scale = mean_abs;
    for (int it = 0; it < 50; ++it) {
      float xq = 0.f, qq = 0.f;
#pragma unroll
      for (int m = 0; m < MICROS; ++m) {
        q[m] = fminf(fmaxf(rintf(__fdiv_rn(x[m], scale)), static_cast<float>(lo)), static_cast<float>(hi));
        xq = __fadd_rn(xq, __fmul_rn(x[m], q[m]));
        qq = __fadd_rn(qq, __fmul_rn(q[m], q[m]));
      }
      xq = __fdiv_rn(warp_sum(xq), n_f);
      qq = __fdiv_rn(warp_sum(qq), n_f);
      scale = fmaxf(__fdiv_rn(xq, __fadd_rn(qq, Q_EPS)), Q_EPS);
    }
  } else {
    float amax = 0.f;
#pragma unroll
    for (int m = 0; m < MICROS; ++m) amax = fmaxf(amax, fabsf(x[m]));
    scale = fmaxf(__fdiv_rn(warp_max(amax), static_cast<float>(hi)), Q_EPS);
#pragma unroll
    for (int m = 0; m < MICROS; ++m) q[m] = fminf(fmaxf(rintf(__fdiv_rn(x[m], scale)), static_cast<float>(lo)), static_cast<float>(hi));
  }
  if (lane == 0) scale_out[static_cast<int64_t>(tile) * k + r] = __float2half_rn(scale);
  // stored unsigned codes (columns past the matrix hold code 0) and their planes
  const int offset = bits == 1 ? 0 : (1 << (bits - 1));
  const int full = (k / K_STAGE) * K_STAGE;
  const int s0 = r < full ? (r / K_STAGE) * K_STAGE : full;
  const int rows_cur = r < full ? K_STAGE : k - full;
  uint32_t* tile_base = payload + static_cast<int64_t>(tile) * k * MICROS * bits + static_cast<int64_t>(s0) * MICROS * bits;
#pragma unroll
  for (int m = 0; m < MICROS; ++m) {
    const int qi = live[m] ? static_cast<int>(q[m]) : 0;
    const int u = bits == 1 ? ((qi + 1) >> 1) : (qi + offset);
    if (codes_out) codes_out[static_cast<int64_t>(r) * (gridDim.y * N_TILE) + col0 + m * N_MICRO + lane] = static_cast<int8_t>(qi);
    for (int p = 0; p < bits; ++p) {
      const uint32_t word = __ballot_sync(0xffffffffu, (u >> p) & 1);
      if (lane == 0) tile_base[m * rows_cur * bits + (r - s0) * bits + p] = word;
    }
  }
}

}  // namespace bm

extern "C" int bm_quantize_pack_slab(const float* rows, int64_t row_stride, int32_t k, int32_t dim, int32_t bits, uint32_t* payload,
                                     uint16_t* scale, int8_t* codes, void* stream) {
  using namespace bm;
  BM_REQUIRE(k >= 0 && dim > 0 && row_stride >= dim, BM_ERR_INVALID_ARG, "quantize_pack_slab: bad sizes");
  BM_REQUIRE(bits == 1 || bits == 2 || bits == 3 || bits == 4 || bits == 6 || bits == 8, BM_ERR_UNSUPPORTED,
             "Unsupported bits=%d", bits);
  BM_REQUIRE(dim % N_MICRO == 0, BM_ERR_INVALID_ARG, "quantize_pack_slab: dim=%d must be divisible by %d", dim, N_MICRO);
  if (k == 0) return BM_OK;
  BM_REQUIRE(rows && payload && scale, BM_ERR_INVALID_ARG, "quantize_pack_slab: null pointer");
  const int tiles = (dim + N_TILE - 1) / N_TILE;
  dim3 grid((k + 7) / 8, tiles);
  quantize_pack_slab_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(rows, row_stride, k, dim, bits, payload,
                                                                                reinterpret_cast<__half*>(scale), codes);
  BM_LAUNCH_CHECK("quantize_pack_slab_kernel");
  return BM_OK;
}
