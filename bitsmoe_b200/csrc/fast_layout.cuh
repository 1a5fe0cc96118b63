// Arena ("fast") layout of a layer whose experts use only 2/3/4-bit rows.
//
// The reference payload packs bit-planes along the intermediate dimension in a
// [slab][tile][stage][micro][row][plane] order that suits neither tensor-core fragments nor
// one-copy-per-work-item streaming.  At layer creation every expert is repacked, codes
// unchanged, into one contiguous block per (expert, 128-column tile):
//
//   unit block = [scale_gate | scale_up | scale_down | words_gate | words_up | words_down]
//
// Rows of a matrix are regrouped by bit width (4, then 3, then 2 bits; the reference's slabs
// already come in that order) and padded per group to a multiple of 16 "slots".  A word holds,
// for one plane p, 16 consecutive positions along the contraction dimension of two operand
// rows that sit 8 apart in a 16-row MMA block:
//
//   bit i        = bit p of u(row g,     contraction position 16*kb + i)
//   bit 16 + i   = bit p of u(row g + 8, contraction position 16*kb + i)
//
// gate / up:  operand rows = columns c of the tile (8 blocks of 16), contraction = row slots
//             words laid out [kb][mblock][g][plane]
// down:       operand rows = row slots (blocks of 16, uniform width), contraction = columns c
//             words laid out [mblock][kb][g][plane]
// With u = q + 2^(b-1) stored as the fp16 subnormal u * 2^-24 a thread rebuilds its four
// m16n8k16 A-fragment registers from `b` words with 2*b rotate/mask ops and 2 byte permutes per
// 4 codes.  Scales (fp16 per slot per tile) travel with the unit block; logical rank and S per
// slot live in small per-expert tables.
#pragma once

#include "common.cuh"

namespace bm {

__host__ __device__ inline int group_bits(int grp) { return 4 - grp; }

// slot position inside a 16-block so that MMA contraction slots (2t, 2t+1, 2t+8, 2t+9) hold
// positions (t, t+8, t+4, t+12)
__host__ __device__ inline int kperm16(int i) { return 2 * (i & 3) + ((i >> 3) & 1) + 8 * ((i >> 2) & 1); }

}  // namespace bm
