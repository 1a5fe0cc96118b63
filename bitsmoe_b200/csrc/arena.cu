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
      std::vector<int16_t> rows[2];
      for (const SlabHost& s : mh.slabs) {
        if (s.bits < 1 || s.bits > 4) return;
        if (s.tile_end - s.tile_off != L->n_tiles) return;
        for (int r = 0; r < s.k_slab; ++r) rows[s.bits >= 3 ? 0 : 1].push_back(static_cast<int16_t>(s.rank_off + r));
      }
      P->slot_row_off[e * 3 + w] = static_cast<int32_t>(P->slot_row.size());
      // gate / up contract over the slots in pairs of 16-blocks; down only needs whole 16-row blocks
      const int gran = w < 2 ? 32 : 16;
      // A 1- or 2-bit row also fits a nibble slot (q + 8 is in [6, 9]).  Moving m of them over can empty padding on
      // both sides: take the m that minimises words (a nibble block is 256 words, a dense one 128) plus 128 per
      // 16-block (= per MMA column block), the smallest such m.
      {
        const int n0 = static_cast<int>(rows[0].size()), n1 = static_cast<int>(rows[1].size());
        long best_cost = -1;
        int best_m = 0;
        for (int m = 0; m <= n1; ++m) {
          const int p0 = (n0 + m + gran - 1) / gran * gran, p1 = (n1 - m + gran - 1) / gran * gran;
          const long cost = 16L * p0 + 8L * p1 + 128L * ((p0 + p1) / 16);
          if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_m = m; }
        }
        for (int i = 0; i < best_m; ++i) {
          rows[0].push_back(rows[1].back());
          rows[1].pop_back();
        }
      }
      int total_blk = 0;
      for (int g = 0; g < 2; ++g) {
        const int padded = (static_cast<int>(rows[g].size()) + gran - 1) / gran * gran;
        fm.nblk[g] = padded / 16;
        total_blk += fm.nblk[g];
        for (int i = 0; i < padded; ++i)
          P->slot_row.push_back(i < static_cast<int>(rows[g].size()) ? rows[g][i] : static_cast<int16_t>(-1));
      }
      if (total_blk == 0) return;
      fm.nslots = total_blk * 16;
      fm.words = 256 * fm.nblk[0] + 128 * fm.nblk[1];
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
    // one section per matrix, scales directly followed by words: a section is one contiguous copy
    for (int w = 0; w < 3; ++w) {
      fe.sec_off[w] = o;     o += fe.m[w].nslots * 2;     // multiples of 32 bytes
      fe.sec_off[3 + w] = o; o += fe.m[w].words * 4;      // multiples of 512 bytes
    }
    fe.unit_bytes = static_cast<int32_t>(align_up(o, 128));
    fe.unit_base = static_cast<int64_t>(off);
    off += static_cast<size_t>(fe.unit_bytes) * L->n_tiles;
    if (fe.unit_bytes > P->max_unit_bytes) P->max_unit_bytes = fe.unit_bytes;
  }
  P->total = align_up(off, 256);
  // whether a kernel's working set fits shared memory is each kernel's own check (plan_experts_decode, experts_tc_fits)
  P->ok = L->rank_in % 8 == 0;
}

// signed code q(row, tile*128 + col_in_tile) read from the reference payload
__device__ __forceinline__ int source_q(const MatDev& md, int row, int col_in_tile, int tile) {
  for (int sl = 0; sl < md.n_slabs; ++sl) {
    const int k_slab = md.slab_meta[sl * 4 + 1], rank_off = md.slab_meta[sl * 4 + 2];
    if (row < rank_off || row >= rank_off + k_slab) continue;
    const int bits = md.slab_meta[sl * 4 + 0];
    const int t = md.slab_meta[sl * 4 + 3] + tile;
    const int r = row - rank_off, s0 = (r / K_STAGE) * K_STAGE, rows_cur = min(K_STAGE, k_slab - s0);
    const uint32_t* w = md.payload + md.tile_meta[t * 3 + 0] + s0 * MICROS * bits + (col_in_tile / N_MICRO) * rows_cur * bits +
                        (r - s0) * bits;
    int u = 0;
    for (int p = 0; p < bits; ++p) u |= static_cast<int>((w[p] >> (col_in_tile % N_MICRO)) & 1u) << p;
    return bits == 1 ? 2 * u - 1 : u - (1 << (bits - 1));
  }
  return 0;
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
    // gate / up scales are stored in the order of the token-side operand (see pos32)
    scale_out[w < 2 ? slot_pos(slot) : slot] = sc;
    if (tile == 0) {
      int rk = row >= 0 ? md.rank_idx[row] : -1;
      if (rk < 0 || rk > 32000) rk = -1;
      t_rank[slot] = static_cast<int16_t>(rk);
      t_s[slot] = row >= 0 ? md.s[row] : __float2half(0.f);
      t_row[slot] = static_cast<int16_t>(row);
    }
  }
}

// Where the codes of word `i` of a matrix section come from.  `first_blk` = the word's first 16-slot (gate/up:
// contraction, down: operand-row) block, `x` = the block of 16 along the tile's columns, `nb` = blocks per word.
struct WordGeom {
  int dense, slot_blk, col_blk, lane, nb;
};
__device__ __forceinline__ WordGeom word_geom(const FastMat& fm, int w, int i) {
  WordGeom q;
  const int nib_words = fm.nblk[0] * 256;
  q.dense = i >= nib_words;
  if (!q.dense) {
    q.nb = 1;
    q.lane = (i >> 1) & 31;
    const int blk = i & 1;
    if (w < 2) { q.slot_blk = (i >> 9) * 2 + blk; q.col_blk = (i >> 6) & 7; }
    else { q.slot_blk = i >> 8; q.col_blk = ((i >> 6) & 3) * 2 + blk; }
  } else {
    const int j = i - nib_words;
    q.nb = 2;
    q.lane = j & 31;
    if (w < 2) { q.slot_blk = fm.nblk[0] + (j >> 8) * 2; q.col_blk = (j >> 5) & 7; }
    else { q.slot_blk = fm.nblk[0] + (j >> 7); q.col_blk = ((j >> 5) & 3) * 2; }
  }
  return q;
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
  for (int i = threadIdx.x; i < fm.words; i += blockDim.x) {
    const WordGeom q = word_geom(fm, w, i);
    const int g = q.lane >> 2, t = q.lane & 3;
    uint32_t word = 0;
    for (int blk = 0; blk < q.nb; ++blk)
      for (int hi8 = 0; hi8 < 2; ++hi8)
        for (int kk = 0; kk < 4; ++kk) {
          const int k = 2 * t + (kk & 1) + 8 * (kk >> 1);
          int slot, col;
          if (w < 2) { slot = (q.slot_blk + blk) * 16 + k; col = q.col_blk * 16 + g + 8 * hi8; }     // contraction = slots
          else { slot = q.slot_blk * 16 + g + 8 * hi8; col = (q.col_blk + blk) * 16 + k; }           // contraction = columns
          const int row = slot_row[slot];
          const int code = row >= 0 ? source_q(md, row, col, tile) : 0;
          if (q.dense) word |= static_cast<uint32_t>((code + FAST_DENSE_OFFSET) & 3) << dense_shift(blk, hi8, k);
          else word |= static_cast<uint32_t>((code + FAST_NIB_OFFSET) & 15) << nib_shift(hi8, k);
        }
    out[i] = word;
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
    const int sblk = slot >> 4, cblk = cc >> 4;
    // operand row / contraction index inside the 16x16 block
    const int m = w < 2 ? (cc & 15) : (slot & 15), k = w < 2 ? (slot & 15) : (cc & 15);
    const int lane = (m & 7) * 4 + ((k & 7) >> 1), hi8 = m >> 3;
    int q;
    if (sblk < fm.nblk[0]) {
      int idx;
      if (w < 2) idx = (((sblk >> 1) * 8 + cblk) * 32 + lane) * 2 + (sblk & 1);
      else idx = ((sblk * 4 + (cblk >> 1)) * 32 + lane) * 2 + (cblk & 1);
      q = static_cast<int>((words[idx] >> nib_shift(hi8, k)) & 15u) - FAST_NIB_OFFSET;
    } else {
      const int db = sblk - fm.nblk[0];
      int idx, blk;
      if (w < 2) { idx = ((db >> 1) * 8 + cblk) * 32 + lane; blk = db & 1; }
      else { idx = (db * 4 + (cblk >> 1)) * 32 + lane; blk = cblk & 1; }
      q = static_cast<int>((words[fm.nblk[0] * 256 + idx] >> dense_shift(blk, hi8, k)) & 3u) - FAST_DENSE_OFFSET;
    }
    codes[static_cast<int64_t>(row) * intermediate + col] = static_cast<int8_t>(q);
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
