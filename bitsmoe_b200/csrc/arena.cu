// Planning and building of the arena layout (see fast_layout.cuh), and decoding it back to
// integer codes for the bit-exactness tests.
#include "fast_layout.cuh"

namespace bm {


// Decides whether the layer fits the fast layout and lays it out after `base_bytes` of arena.
void plan_fast(const bm_layer* L, size_t base_bytes, FastPlan* P) {
  P->ok = false;
  const int E = L->num_experts;
  if (E == 0 || L->intermediate % N_TILE != 0) return;
  P->experts.assign(E, FastExpert{});
  P->slot_row.clear();
  P->slot_row_off.assign(static_cast<size_t>(E) * 3, 0);
  size_t off = align_up(base_bytes, 256);
  P->table_off = off;
  off += align_up(sizeof(FastExpert) * E, 256);
  P->tabs_off = off;
  // pass 1: slots per matrix, per-expert tables
  for (int e = 0; e < E; ++e) {
    for (int w = 0; w < 3; ++w) {
      const MatHost& mh = L->host[w][e];
      if (mh.n_rows > 32000) return;
      FastMat& fm = P->experts[e].m[w];
      std::vector<int16_t> rows[3];
      for (const SlabHost& s : mh.slabs) {
        if (s.bits < 2 || s.bits > 4) return;
        if (s.tile_end - s.tile_off != L->n_tiles) return;
        for (int r = 0; r < s.k_slab; ++r) rows[4 - s.bits].push_back(static_cast<int16_t>(s.rank_off + r));
      }
      P->slot_row_off[e * 3 + w] = static_cast<int32_t>(P->slot_row.size());
      int total_blk = 0, words = 0;
      for (int g = 0; g < 3; ++g) {
        const int nb = (static_cast<int>(rows[g].size()) + 15) / 16;
        fm.nblk[g] = nb;
        total_blk += nb;
        words += 64 * group_bits(g) * nb;
        for (int i = 0; i < nb * 16; ++i)
          P->slot_row.push_back(i < static_cast<int>(rows[g].size()) ? rows[g][i] : static_cast<int16_t>(-1));
      }
      if (total_blk == 0) return;
      fm.nslots = total_blk * 16;
      fm.words = words;
      fm.tab_off = static_cast<int32_t>(off);
      off += align_up(static_cast<size_t>(fm.nslots) * 6, 16);
      if (fm.nslots > P->max_slots) P->max_slots = fm.nslots;
      if (fm.words > P->max_words) P->max_words = fm.words;
      if (off > (1ull << 31)) return;
    }
  }
  off = align_up(off, 256);
  P->units_off = off;
  for (int e = 0; e < E; ++e) {
    FastExpert& fe = P->experts[e];
    int o = 0;
    for (int w = 0; w < 3; ++w) { fe.sec_off[w] = o; o += fe.m[w].nslots * 2; }       // multiples of 32 bytes
    for (int w = 0; w < 3; ++w) { fe.sec_off[3 + w] = o; o += fe.m[w].words * 4; }   // multiples of 256 bytes
    fe.unit_bytes = static_cast<int32_t>(align_up(o, 128));
    fe.unit_base = static_cast<int64_t>(off);
    off += static_cast<size_t>(fe.unit_bytes) * L->n_tiles;
    if (fe.unit_bytes > P->max_unit_bytes) P->max_unit_bytes = fe.unit_bytes;
  }
  P->total = align_up(off, 256);
  // a unit block plus activation staging has to fit one CTA's shared memory
  P->ok = 2 * (P->max_unit_bytes + 3 * (P->max_slots * 6 + 16) + 2 * FAST_MAX_TOK * L->rank_in * 2) +
              2 * FAST_MAX_TOK * (P->max_slots + 8) * 2 + 8192 <= 200 * 1024 && L->rank_in % 8 == 0;
}

__device__ __forceinline__ int source_bit(const MatDev& md, int row, int col_in_tile, int tile, int plane, int* bits_out) {
  // bit `plane` of u(row, tile*128 + col_in_tile) read from the reference payload
  for (int sl = 0; sl < md.n_slabs; ++sl) {
    const int k_slab = md.slab_meta[sl * 4 + 1], rank_off = md.slab_meta[sl * 4 + 2];
    if (row < rank_off || row >= rank_off + k_slab) continue;
    const int bits = md.slab_meta[sl * 4 + 0];
    *bits_out = bits;
    if (plane >= bits) return 0;
    const int t = md.slab_meta[sl * 4 + 3] + tile;
    const int r = row - rank_off, s0 = (r / K_STAGE) * K_STAGE, rows_cur = min(K_STAGE, k_slab - s0);
    const uint32_t w = md.payload[md.tile_meta[t * 3 + 0] + s0 * MICROS * bits + (col_in_tile / N_MICRO) * rows_cur * bits +
                                  (r - s0) * bits + plane];
    return static_cast<int>((w >> (col_in_tile % N_MICRO)) & 1u);
  }
  *bits_out = 0;
  return 0;
}

__device__ __forceinline__ void slot_group(const FastMat& fm, int blk, int* grp, int* blk_in_grp) {
  if (blk < fm.nblk[0]) { *grp = 0; *blk_in_grp = blk; }
  else if (blk < fm.nblk[0] + fm.nblk[1]) { *grp = 1; *blk_in_grp = blk - fm.nblk[0]; }
  else { *grp = 2; *blk_in_grp = blk - fm.nblk[0] - fm.nblk[1]; }
}

// word offset of slot-block `blk` inside a matrix section (both orientations store 64*b words per block)
__device__ __forceinline__ int block_word_off(const FastMat& fm, int blk) {
  int grp, big;
  slot_group(fm, blk, &grp, &big);
  int off = 0;
  if (grp >= 1) off += fm.nblk[0] * 64 * 4;
  if (grp >= 2) off += fm.nblk[1] * 64 * 3;
  return off + big * 64 * group_bits(grp);
}

// grid (E, n_tiles, 3): fills rank / s / row tables (tile 0 only) and this tile's scales.
__global__ void __launch_bounds__(128) repack_tables_kernel(const ExpertDev* __restrict__ experts,
                                                           const FastExpert* __restrict__ fast,
                                                           const int16_t* __restrict__ slot_row_all,
                                                           const int32_t* __restrict__ slot_row_off,
                                                           unsigned char* __restrict__ arena) {
  const int e = blockIdx.x, tile = blockIdx.y, w = blockIdx.z;
  const MatDev& md = experts[e].m[w];
  const FastExpert& fe = fast[e];
  const FastMat& fm = fe.m[w];
  const int16_t* slot_row = slot_row_all + slot_row_off[e * 3 + w];
  int16_t* t_rank = reinterpret_cast<int16_t*>(arena + fm.tab_off);
  __half* t_s = reinterpret_cast<__half*>(arena + fm.tab_off + fm.nslots * 2);
  int16_t* t_row = reinterpret_cast<int16_t*>(arena + fm.tab_off + fm.nslots * 4);
  __half* scale_out = reinterpret_cast<__half*>(arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes + fe.sec_off[w]);
  for (int slot = threadIdx.x; slot < fm.nslots; slot += blockDim.x) {
    const int row = slot_row[slot];
    __half sc = __float2half(0.f);
    if (row >= 0) {
      for (int sl = 0; sl < md.n_slabs; ++sl) {
        const int k_slab = md.slab_meta[sl * 4 + 1], rank_off = md.slab_meta[sl * 4 + 2];
        if (row < rank_off || row >= rank_off + k_slab) continue;
        const int t = md.slab_meta[sl * 4 + 3] + tile;
        sc = md.scale[md.tile_meta[t * 3 + 1] + row - rank_off];
        break;
      }
    }
    // gate / up scales are stored in the contraction order of the MMA operands (pairs (s, s+8) adjacent)
    scale_out[w < 2 ? (slot & ~15) + kperm16(slot & 15) : slot] = sc;
    if (tile == 0) {
      int rk = row >= 0 ? md.rank_idx[row] : -1;
      if (rk < 0 || rk > 32000) rk = -1;
      t_rank[slot] = static_cast<int16_t>(rk);
      t_s[slot] = row >= 0 ? md.s[row] : __float2half(0.f);
      t_row[slot] = static_cast<int16_t>(row);
    }
  }
}

// grid (E, n_tiles, 3): one thread per output word.
__global__ void __launch_bounds__(256) repack_words_kernel(const ExpertDev* __restrict__ experts,
                                                          const FastExpert* __restrict__ fast,
                                                          const int16_t* __restrict__ slot_row_all,
                                                          const int32_t* __restrict__ slot_row_off,
                                                          unsigned char* __restrict__ arena) {
  const int e = blockIdx.x, tile = blockIdx.y, w = blockIdx.z;
  const MatDev& md = experts[e].m[w];
  const FastExpert& fe = fast[e];
  const FastMat& fm = fe.m[w];
  const int16_t* slot_row = slot_row_all + slot_row_off[e * 3 + w];
  uint32_t* out = reinterpret_cast<uint32_t*>(arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes + fe.sec_off[3 + w]);
  const int nblk = fm.nslots / 16;
  for (int blk = 0; blk < nblk; ++blk) {
    int grp, big;
    slot_group(fm, blk, &grp, &big);
    const int b = group_bits(grp);
    const int base = block_word_off(fm, blk);
    // 64*b words of this slot block: index = ((x * 8) + g) * b + plane, x = the other dimension's block (0..7)
    for (int i = threadIdx.x; i < 64 * b; i += blockDim.x) {
      const int plane = i % b, g = (i / b) % 8, x = i / (8 * b);
      uint32_t word = 0;
      int dummy;
      if (w < 2) {
        // gate / up: operand rows are columns c = 16*x + g (+8); contraction = slots of this block
        for (int k = 0; k < 16; ++k) {
          const int row = slot_row[blk * 16 + k];
          if (row < 0) continue;
          word |= static_cast<uint32_t>(source_bit(md, row, 16 * x + g, tile, plane, &dummy)) << k;
          word |= static_cast<uint32_t>(source_bit(md, row, 16 * x + g + 8, tile, plane, &dummy)) << (16 + k);
        }
      } else {
        // down: operand rows are slots g, g+8 of this block; contraction = columns 16*x .. 16*x+15
        const int r0 = slot_row[blk * 16 + g], r1 = slot_row[blk * 16 + g + 8];
        for (int k = 0; k < 16; ++k) {
          if (r0 >= 0) word |= static_cast<uint32_t>(source_bit(md, r0, 16 * x + k, tile, plane, &dummy)) << k;
          if (r1 >= 0) word |= static_cast<uint32_t>(source_bit(md, r1, 16 * x + k, tile, plane, &dummy)) << (16 + k);
        }
      }
      out[base + i] = word;
    }
  }
}

// int8 codes [n_rows, intermediate] read back from the arena words: one thread per (slot, column).
__global__ void __launch_bounds__(256) arena_decode_kernel(const FastExpert* __restrict__ fast, int e, int w, int n_tiles,
                                                          int intermediate, const unsigned char* __restrict__ arena,
                                                          int8_t* __restrict__ codes) {
  const FastExpert& fe = fast[e];
  const FastMat& fm = fe.m[w];
  const int16_t* t_row = reinterpret_cast<const int16_t*>(arena + fm.tab_off + fm.nslots * 4);
  const int64_t total = static_cast<int64_t>(fm.nslots) * intermediate;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int slot = static_cast<int>(i / intermediate), col = static_cast<int>(i % intermediate);
    const int row = t_row[slot];
    if (row < 0) continue;
    const int tile = col / N_TILE, cc = col % N_TILE;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(arena + fe.unit_base + static_cast<int64_t>(tile) * fe.unit_bytes + fe.sec_off[3 + w]);
    const int blk = slot / 16, k = slot % 16;
    int grp, big;
    slot_group(fm, blk, &grp, &big);
    const int b = group_bits(grp);
    const uint32_t* wb = words + block_word_off(fm, blk);
    int u = 0;
    for (int p = 0; p < b; ++p) {
      uint32_t word;
      int bitpos;
      if (w < 2) {
        const int x = cc / 16, r = cc % 16;
        word = wb[((x * 8) + (r & 7)) * b + p];
        bitpos = (r >= 8 ? 16 : 0) + k;
      } else {
        const int x = cc / 16;
        word = wb[((x * 8) + (k & 7)) * b + p];
        bitpos = (k >= 8 ? 16 : 0) + (cc % 16);
      }
      u |= static_cast<int>((word >> bitpos) & 1u) << p;
    }
    codes[static_cast<int64_t>(row) * intermediate + col] = static_cast<int8_t>(u - (1 << (b - 1)));
  }
}

int build_fast(bm_layer* L, const FastPlan& P, cudaStream_t st) {
  unsigned char* arena = static_cast<unsigned char*>(L->arena);
  // scratch for slot_row tables: placed at the start of the unit region, overwritten afterwards? No --
  // kept in the tables region tail is not possible (kernels read it while writing units), so it is
  // staged in the last unit block area only if it fits; simpler and safe: a dedicated tail.
  const size_t rows_bytes = align_up(P.slot_row.size() * sizeof(int16_t), 256);
  const size_t offs_bytes = align_up(P.slot_row_off.size() * sizeof(int32_t), 256);
  int16_t* d_rows = reinterpret_cast<int16_t*>(arena + P.total);
  int32_t* d_offs = reinterpret_cast<int32_t*>(arena + P.total + rows_bytes);
  (void)offs_bytes;
  BM_CUDA(cudaMemcpyAsync(arena + P.table_off, P.experts.data(), sizeof(FastExpert) * P.experts.size(), cudaMemcpyHostToDevice, st));
  BM_CUDA(cudaMemcpyAsync(d_rows, P.slot_row.data(), P.slot_row.size() * sizeof(int16_t), cudaMemcpyHostToDevice, st));
  BM_CUDA(cudaMemcpyAsync(d_offs, P.slot_row_off.data(), P.slot_row_off.size() * sizeof(int32_t), cudaMemcpyHostToDevice, st));
  const FastExpert* d_fast = reinterpret_cast<const FastExpert*>(arena + P.table_off);
  dim3 grid(L->num_experts, L->n_tiles, 3);
  repack_tables_kernel<<<grid, 128, 0, st>>>(L->experts_dev, d_fast, d_rows, d_offs, arena);
  BM_LAUNCH_CHECK("repack_tables_kernel");
  repack_words_kernel<<<grid, 256, 0, st>>>(L->experts_dev, d_fast, d_rows, d_offs, arena);
  BM_LAUNCH_CHECK("repack_words_kernel");
  BM_CUDA(cudaStreamSynchronize(st));
  return BM_OK;
}

size_t fast_build_scratch_bytes(const FastPlan& P) {
  return align_up(P.slot_row.size() * sizeof(int16_t), 256) + align_up(P.slot_row_off.size() * sizeof(int32_t), 256);
}

int launch_arena_decode(const bm_layer* L, int e, int w, int8_t* codes, cudaStream_t st) {
  const FastMat& fm = L->fast_host[e].m[w];
  const int64_t total = static_cast<int64_t>(fm.nslots) * L->intermediate;
  BM_CUDA(cudaMemsetAsync(codes, 0, static_cast<size_t>(L->host[w][e].n_rows) * L->intermediate, st));
  const int blocks = static_cast<int>((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  arena_decode_kernel<<<blocks, 256, 0, st>>>(L->fast_dev, e, w, L->n_tiles, L->intermediate,
                                             static_cast<const unsigned char*>(L->arena), codes);
  BM_LAUNCH_CHECK("arena_decode_kernel");
  return BM_OK;
}

}  // namespace bm
