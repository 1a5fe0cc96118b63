// Bit-plane codec: int8 codes <-> uint32 planes over groups of 32 columns.
//
// Format (normative, from bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu:81-121 and :157-196):
// word (row, group, plane p) bit l = bit p of u(row, group*32 + l), u = q + 2^(bits-1)
// (1-bit: u = (q + 1) >> 1, q = 2u - 1).  Columns past `cols` pack as u = 0.
//
// One thread owns one (row, group): it reads its 32 codes with two 16-byte loads when the
// row start allows it, builds all planes in registers and writes `bits` consecutive words,
// so a warp touches contiguous memory on both sides and no shuffles are needed.
#include "common.cuh"

namespace bm {

__device__ __forceinline__ uint32_t code_to_unsigned(int q, int bits) {
  return bits == 1 ? static_cast<uint32_t>((q + 1) >> 1) & 1u
                   : static_cast<uint32_t>(q + (1 << (bits - 1))) & ((1u << bits) - 1u);
}

__global__ void __launch_bounds__(256) pack_planes_kernel(const int8_t* __restrict__ q, uint32_t* __restrict__ out,
                                                         int64_t rows, int64_t cols, int64_t groups, int bits) {
  const int64_t total = rows * groups;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = i / groups;
    const int64_t g = i - row * groups;
    const int64_t c0 = g * N_MICRO;
    const int8_t* src = q + row * cols + c0;
    int8_t v[N_MICRO];
    const bool full = c0 + N_MICRO <= cols;
    if (full && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
      const int4 a = reinterpret_cast<const int4*>(src)[0];
      const int4 b = reinterpret_cast<const int4*>(src)[1];
      *reinterpret_cast<int4*>(&v[0]) = a;
      *reinterpret_cast<int4*>(&v[16]) = b;
    } else {
#pragma unroll
      for (int l = 0; l < N_MICRO; ++l) v[l] = (c0 + l < cols) ? src[l] : static_cast<int8_t>(0);
    }
    uint32_t planes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int l = 0; l < N_MICRO; ++l) {
      const uint32_t u = (!full && c0 + l >= cols) ? 0u : code_to_unsigned(v[l], bits);
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < bits) planes[p] |= ((u >> p) & 1u) << l;
    }
    uint32_t* dst = out + i * bits;
#pragma unroll
    for (int p = 0; p < 8; ++p)
      if (p < bits) dst[p] = planes[p];
  }
}

__global__ void __launch_bounds__(256) unpack_planes_kernel(const uint32_t* __restrict__ in, int8_t* __restrict__ q,
                                                           int64_t rows, int64_t groups, int bits) {
  const int64_t total = rows * groups;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    uint32_t planes[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) planes[p] = (p < bits) ? in[i * bits + p] : 0u;
    int8_t v[N_MICRO];
#pragma unroll
    for (int l = 0; l < N_MICRO; ++l) {
      int u = 0;
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < bits) u |= static_cast<int>((planes[p] >> l) & 1u) << p;
      v[l] = static_cast<int8_t>(bits == 1 ? 2 * u - 1 : u - (1 << (bits - 1)));
    }
    int4* dst = reinterpret_cast<int4*>(q + i * N_MICRO);  // rows are groups*32 wide: 16-byte aligned if q is
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      dst[0] = *reinterpret_cast<int4*>(&v[0]);
      dst[1] = *reinterpret_cast<int4*>(&v[16]);
    } else {
      int8_t* d = q + i * N_MICRO;
#pragma unroll
      for (int l = 0; l < N_MICRO; ++l) d[l] = v[l];
    }
  }
}

static bool codec_bits(int b) { return b == 1 || b == 2 || b == 3 || b == 4 || b == 6 || b == 8; }

}  // namespace bm

extern "C" int bm_pack_bitplanes_i8(const int8_t* q, uint32_t* words, int64_t rows, int64_t cols, int bits,
                                    void* stream) {
  using namespace bm;
  BM_REQUIRE(codec_bits(bits), BM_ERR_UNSUPPORTED, "Unsupported bit width: %d", bits);
  BM_REQUIRE(rows >= 0 && cols >= 0, BM_ERR_INVALID_ARG, "pack_bits: invalid input shape");
  const int64_t groups = (cols + 31) / 32;
  if (rows * groups == 0) return BM_OK;
  BM_REQUIRE(q && words, BM_ERR_INVALID_ARG, "pack_bits: null pointer");
  const int64_t blocks = (rows * groups + 255) / 256;
  pack_planes_kernel<<<static_cast<unsigned>(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(q, words, rows, cols, groups, bits);
  BM_LAUNCH_CHECK("pack_planes_kernel");
  return BM_OK;
}

extern "C" int bm_unpack_bitplanes_i8(const uint32_t* words, int8_t* q, int64_t rows, int64_t groups, int bits,
                                      void* stream) {
  using namespace bm;
  BM_REQUIRE(codec_bits(bits), BM_ERR_UNSUPPORTED, "Unsupported bit width: %d", bits);
  BM_REQUIRE(rows >= 0 && groups >= 0, BM_ERR_INVALID_ARG, "unpack_bits: invalid input shape");
  if (rows * groups == 0) return BM_OK;
  BM_REQUIRE(q && words, BM_ERR_INVALID_ARG, "unpack_bits: null pointer");
  const int64_t blocks = (rows * groups + 255) / 256;
  unpack_planes_kernel<<<static_cast<unsigned>(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(words, q, rows, groups, bits);
  BM_LAUNCH_CHECK("unpack_planes_kernel");
  return BM_OK;
}
