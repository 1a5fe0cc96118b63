// Arena ("fast") layout of a layer whose experts use only 1/2/3/4-bit rows.
//
// The reference payload packs bit-planes along the intermediate dimension in a
// [slab][tile][stage][micro][row][plane] order that suits neither tensor-core fragments nor
// one-copy-per-work-item streaming, and turning planes into fp16 operands costs two ALU
// operations per code.  At layer creation every expert is repacked into one contiguous block per
// (expert, 128-column tile):
//
//   unit block = [scale_gate | words_gate | scale_up | words_up | scale_down | words_down]
//
// in which a 32-bit word is the property of ONE thread of an m16n8k16 MMA (lane = 4 g + t) and
// expands into A-fragment registers with one mask (and at most one shift) per register:
//
//   nibble group (3- and 4-bit rows, plus the 1- and 2-bit rows that would only fill padding of the dense
//   group: see plan_fast; stored code u = q + 8, one word = one 16x16 block):
//     nibble i of the lower half-word, i = 0..3 : (row g, k 2t) (row g+8, k 2t) (row g, k 2t+8) (row g+8, k 2t+8)
//     same nibble of the upper half-word        : the neighbour k + 1
//     a0 = w & 0x000F000F, a1 = w & 0x00F000F0, a2 = (w >> 8) & 0x000F000F, a3 = (w >> 8) & 0x00F000F0
//   dense group (1- and 2-bit rows; stored code u = q + 2, one word = two consecutive 16x16 blocks):
//     2-bit field i of the lower half-word, i = 0..7 : block A (row g, 2t) (row g, 2t+8) (row g+8, 2t) (row g+8, 2t+8), block B the same
//     a0 = w & 0x00030003, a1 = w & 0x00300030, a2 = (w >> 2) & 0x00030003, a3 = (w >> 2) & 0x00300030;  block B from w >> 8
//
// Read as fp16 bit patterns these registers are the subnormals u * 2^-24 (rows g) and 16 u * 2^-24
// (rows g + 8); the factor 16 of the upper rows is taken out of the accumulators, the code offset is
// removed with a per-token correction sum (decode path) or an exact fp16 subtract (tensor path).
//
// Rows of a matrix are regrouped (nibble group first) and padded to "slots"; per 32 slots (two
// 16-blocks, "a pair") the token-side operands and the gate/up scales are stored in the order
// pos32(), which puts the eight values one thread needs for a pair next to each other.
//
// gate / up:  operand rows = columns c of the tile (8 blocks x of 16), contraction = row slots
//             nibble words [pair][x][lane][2 blocks], dense words [pair][x][lane]
// down:       operand rows = row slots (blocks of 16), contraction = columns c (4 pairs)
//             nibble words [mblock][pair][lane][2 blocks], dense words [mblock][pair][lane]
// Scales (fp16 per slot per tile) travel with the unit block; logical rank and S per slot live in
// small per-expert tables.
#pragma once

#include "common.cuh"

namespace bm {

constexpr int FAST_NIB_OFFSET = 8;     // stored nibble = q + 8
constexpr int FAST_DENSE_OFFSET = 2;   // stored 2-bit field = q + 2

// position of contraction index i (0..31: block i >> 4, k = i & 15) inside its pair:
// [t = (k & 7) >> 1][block][k >> 3][k & 1]
__host__ __device__ inline int pos32(int i) {
  const int k = i & 15;
  return ((k & 7) >> 1) * 8 + (i >> 4) * 4 + (k >> 3) * 2 + (k & 1);
}
__host__ __device__ inline int pos32_inv(int p) {
  const int t = p >> 3, blk = (p >> 2) & 1, h = (p >> 1) & 1, j = p & 1;
  return blk * 16 + 2 * t + j + 8 * h;
}
__host__ __device__ inline int slot_pos(int slot) { return (slot & ~31) + pos32(slot & 31); }

// bit position of code (row half `hi8`, k) inside the word owned by thread t = (k & 7) >> 1
__host__ __device__ inline int nib_shift(int hi8, int k) { return 16 * (k & 1) + 4 * ((k >> 3) * 2 + hi8); }
__host__ __device__ inline int dense_shift(int blk, int hi8, int k) { return 16 * (k & 1) + 8 * blk + 4 * hi8 + 2 * (k >> 3); }

}  // namespace bm
