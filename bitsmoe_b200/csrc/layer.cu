// C ABI glue: error reporting, layer planning / creation over the reference's buffers,
// stage entry points and the composed layer forward.
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "common.cuh"

namespace bm {

static thread_local char g_err[512] = "";

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// from the other translation units
int launch_gemm_nt(const GemmArgs& g, int problems, cudaStream_t st);
struct SkinnyArgs {
  const __half* W[2];
  void* C[2];
  const void* X;
  const void* residual;
  int rows_per_w, n_w;
  int N, K;
  int x_dtype, c_dtype;
  int round_x_f16;
  int splits;
  int mrows;
  float4* zero;
  int zero_n;
};
int launch_skinny_nt(SkinnyArgs a, cudaStream_t st);
constexpr int SKINNY_MAX_TOKENS = 256;
void plan_fast(const bm_layer* L, size_t base_bytes, FastPlan* P);
int build_fast(bm_layer* L, const FastPlan& P, cudaStream_t st);
size_t fast_build_scratch_bytes(const FastPlan& P);
int launch_arena_decode(const bm_layer* L, int e, int w, int8_t* codes, cudaStream_t st);
int plan_experts_decode(bm_layer* L);
int launch_experts_decode(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                          const int32_t* expert_offsets, const float* route_w, int T, int num_assign, float* rank_accum,
                          long long* acc64, cudaStream_t st);
bool experts_tc_fits(const bm_layer* L);
int launch_experts_tc(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                      const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum, long long* acc64,
                      cudaStream_t st);
int launch_experts_generic(const bm_layer* L, const __half* h_gate, const __half* h_up, const int32_t* token_indices,
                           const int32_t* expert_offsets, const float* route_w, int T, float* rank_accum,
                           long long* acc64, cudaStream_t st);

static const char* which_name(int w) { return w == 0 ? "gate" : (w == 1 ? "up" : "down"); }

// Reads slab/tile meta of one matrix to the host and checks every offset the kernels will use.
static int ingest_matrix(const bm_matrix_t& m, int which, int expert, int intermediate, MatHost* out) {
  const int n_tiles = (intermediate + N_TILE - 1) / N_TILE;
  BM_REQUIRE(m.n_slabs >= 0 && m.n_tile_rows >= 0 && m.n_rows >= 0 && m.payload_words >= 0 && m.n_scales >= 0,
             BM_ERR_INVALID_ARG, "%s[%d]: negative buffer length", which_name(which), expert);
  out->n_rows = m.n_rows;
  out->slabs.clear();
  out->tile_meta.assign(static_cast<size_t>(m.n_tile_rows) * 3, 0);
  std::vector<int32_t> slab(static_cast<size_t>(m.n_slabs) * 4);
  if (m.n_slabs) {
    BM_REQUIRE(m.slab_meta && m.payload && m.rank_idx && m.scale && m.s, BM_ERR_INVALID_ARG, "%s[%d]: null buffer",
               which_name(which), expert);
    BM_CUDA(cudaMemcpy(slab.data(), m.slab_meta, slab.size() * 4, cudaMemcpyDeviceToHost));
  }
  if (m.n_tile_rows) {
    BM_REQUIRE(m.tile_meta, BM_ERR_INVALID_ARG, "%s[%d]: null tile_meta", which_name(which), expert);
    BM_CUDA(cudaMemcpy(out->tile_meta.data(), m.tile_meta, out->tile_meta.size() * 4, cudaMemcpyDeviceToHost));
  }
  for (int i = 0; i < m.n_slabs; ++i) {
    SlabHost s;
    s.bits = slab[i * 4 + 0];
    s.k_slab = slab[i * 4 + 1];
    s.rank_off = slab[i * 4 + 2];
    s.tile_off = slab[i * 4 + 3];
    s.tile_end = (i + 1 < m.n_slabs) ? slab[(i + 1) * 4 + 3] : m.n_tile_rows;
    BM_REQUIRE(supported_bits(s.bits), BM_ERR_UNSUPPORTED, "%s[%d] slab %d: Unsupported bits=%d", which_name(which), expert,
               i, s.bits);
    BM_REQUIRE(s.k_slab >= 1 && s.rank_off >= 0 && s.rank_off + s.k_slab <= m.n_rows, BM_ERR_INVALID_ARG,
               "%s[%d] slab %d: rows [%d, %d) outside rank_idx of %d", which_name(which), expert, i, s.rank_off,
               s.rank_off + s.k_slab, m.n_rows);
    BM_REQUIRE(s.tile_off >= 0 && s.tile_off <= s.tile_end && s.tile_end <= m.n_tile_rows &&
                   s.tile_end - s.tile_off <= n_tiles,
               BM_ERR_INVALID_ARG, "%s[%d] slab %d: tile range [%d, %d) invalid (tile_meta rows %d, tiles per row %d)",
               which_name(which), expert, i, s.tile_off, s.tile_end, m.n_tile_rows, n_tiles);
    const int64_t wpt = static_cast<int64_t>(s.k_slab) * MICROS * words_per_row(s.bits);
    for (int t = s.tile_off; t < s.tile_end; ++t) {
      const int64_t pack_off = out->tile_meta[t * 3 + 0], scale_off = out->tile_meta[t * 3 + 1];
      const int n_valid = out->tile_meta[t * 3 + 2];
      BM_REQUIRE(pack_off >= 0 && pack_off + wpt <= m.payload_words, BM_ERR_INVALID_ARG,
                 "%s[%d] slab %d tile %d: payload [%lld, %lld) outside %lld words", which_name(which), expert, i,
                 t - s.tile_off, (long long)pack_off, (long long)(pack_off + wpt), (long long)m.payload_words);
      BM_REQUIRE(scale_off >= 0 && scale_off + s.k_slab <= m.n_scales, BM_ERR_INVALID_ARG,
                 "%s[%d] slab %d tile %d: scales outside buffer", which_name(which), expert, i, t - s.tile_off);
      BM_REQUIRE(n_valid >= 1 && n_valid <= N_TILE && (t - s.tile_off) * N_TILE + n_valid <= intermediate,
                 BM_ERR_INVALID_ARG, "%s[%d] slab %d tile %d: n_valid=%d does not fit intermediate=%d",
                 which_name(which), expert, i, t - s.tile_off, n_valid, intermediate);
    }
    out->slabs.push_back(s);
  }
  out->bytes = m.payload_words * 4 + m.n_scales * 2 + static_cast<int64_t>(m.n_rows) * (2 + 4) +
               static_cast<int64_t>(m.n_tile_rows) * 12 + static_cast<int64_t>(m.n_slabs) * 16;
  return BM_OK;
}

static int check_desc(const bm_layer_desc_t* d) {
  BM_REQUIRE(d != nullptr, BM_ERR_INVALID_ARG, "null layer descriptor");
  BM_REQUIRE(d->num_experts >= 0, BM_ERR_INVALID_ARG, "num_experts must be >= 0");
  BM_REQUIRE(d->intermediate > 0, BM_ERR_INVALID_ARG, "intermediate_size must be > 0");
  BM_REQUIRE(d->rank_out > 0, BM_ERR_INVALID_ARG, "rank_out must be > 0");
  BM_REQUIRE(d->rank_in > 0, BM_ERR_INVALID_ARG, "rank_in must be > 0");
  BM_REQUIRE(d->intermediate % N_MICRO == 0, BM_ERR_INVALID_ARG, "intermediate_size=%d must be divisible by %d",
             d->intermediate, N_MICRO);
  BM_REQUIRE(d->act_type == 0, BM_ERR_UNSUPPORTED, "only SiLU act_type=0 is currently supported");
  BM_REQUIRE(d->num_experts == 0 || (d->gate && d->up && d->down), BM_ERR_INVALID_ARG, "null matrix tables");
  return BM_OK;
}

// arena = [ExpertDev table][status flag][arena layout ...][build scratch]
static size_t table_bytes(int num_experts) {
  return align_up(sizeof(ExpertDev) * static_cast<size_t>(num_experts > 0 ? num_experts : 1), 256);
}
static size_t base_bytes(int num_experts) { return table_bytes(num_experts) + 256; }

static size_t arena_need(const bm_layer* L, FastPlan* P) {
  plan_fast(L, base_bytes(L->num_experts), P);
  return P->ok ? P->total + fast_build_scratch_bytes(*P) : base_bytes(L->num_experts);
}

static int build_host(const bm_layer_desc_t* d, bm_layer* L) {
  int rc = check_desc(d);
  if (rc) return rc;
  L->num_experts = d->num_experts;
  L->hidden = d->hidden;
  L->intermediate = d->intermediate;
  L->rank_in = d->rank_in;
  L->rank_out = d->rank_out;
  L->n_tiles = (d->intermediate + N_TILE - 1) / N_TILE;
  L->vh_gate = reinterpret_cast<const __half*>(d->vh_gate);
  L->vh_up = reinterpret_cast<const __half*>(d->vh_up);
  L->u_down = reinterpret_cast<const __half*>(d->u_down);
  L->max_rows = 1;
  const bm_matrix_t* tabs[3] = {d->gate, d->up, d->down};
  for (int w = 0; w < 3; ++w) {
    L->host[w].resize(d->num_experts);
    L->src[w].assign(tabs[w], tabs[w] + d->num_experts);
    for (int e = 0; e < d->num_experts; ++e) {
      rc = ingest_matrix(tabs[w][e], w, e, d->intermediate, &L->host[w][e]);
      if (rc) return rc;
      if (tabs[w][e].n_rows > L->max_rows) L->max_rows = tabs[w][e].n_rows;
    }
  }
  return BM_OK;
}

// int8 codes of one matrix, decoded through slab/tile meta: one thread per (row, column).
__global__ void decode_codes_kernel(MatDev md, int intermediate, int8_t* __restrict__ codes) {
  const int64_t total = static_cast<int64_t>(md.n_rows) * intermediate;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(i / intermediate), col = static_cast<int>(i - static_cast<int64_t>(row) * intermediate);
    int8_t q = 0;
    for (int sl = 0; sl < md.n_slabs; ++sl) {
      const int bits = md.slab_meta[sl * 4 + 0], k_slab = md.slab_meta[sl * 4 + 1];
      const int rank_off = md.slab_meta[sl * 4 + 2], tile_off = md.slab_meta[sl * 4 + 3];
      if (row < rank_off || row >= rank_off + k_slab) continue;
      const int tile_end = (sl + 1 < md.n_slabs) ? md.slab_meta[(sl + 1) * 4 + 3] : md.n_tile_rows;
      const int t = tile_off + col / N_TILE;
      if (t >= tile_end || bits == 16) break;
      const int cc = col % N_TILE;
      if (cc >= md.tile_meta[t * 3 + 2]) break;
      const int r = row - rank_off, s0 = (r / K_STAGE) * K_STAGE, rows_cur = min(K_STAGE, k_slab - s0);
      const uint32_t* w = md.payload + md.tile_meta[t * 3 + 0] + s0 * MICROS * bits + (cc / N_MICRO) * rows_cur * bits +
                          (r - s0) * bits;
      int u = 0;
      for (int p = 0; p < bits; ++p) u |= static_cast<int>((w[p] >> (cc % N_MICRO)) & 1u) << p;
      q = static_cast<int8_t>(bits == 1 ? 2 * u - 1 : u - (1 << (bits - 1)));
      break;
    }
    codes[i] = q;
  }
}

static MatDev to_dev(const bm_matrix_t& m) {
  MatDev d;
  d.payload = m.payload;
  d.rank_idx = m.rank_idx;
  d.tile_meta = m.tile_meta;
  d.slab_meta = m.slab_meta;
  d.scale = reinterpret_cast<const __half*>(m.scale);
  d.s = reinterpret_cast<const __half*>(m.s);
  d.n_slabs = m.n_slabs;
  d.n_tile_rows = m.n_tile_rows;
  d.n_rows = m.n_rows;
  d.pad_ = 0;
  return d;
}

struct Carver {
  unsigned char* base;
  size_t off = 0, cap;
  Carver(void* p, size_t c) : base(static_cast<unsigned char*>(p)), cap(c) {}
  template <typename T>
  T* take(size_t n) {
    T* r = reinterpret_cast<T*>(base + off);
    off += align_up(n * sizeof(T), 256);
    return r;
  }
};

struct LayerWs {
  int32_t* topk_idx; float* topk_w; int32_t* token_indices; int32_t* expert_offsets; float* route_flat;
  int32_t* tile_table; int32_t* counts; __half* h_gate; __half* h_up; float* rank_accum;
  void* route_ws; size_t route_ws_bytes; void* experts_ws; size_t experts_ws_bytes; size_t total;
};

constexpr int TILE_ROWS = 128;

static LayerWs carve_layer_ws(const bm_layer* L, void* ws, int T, int k) {
  Carver c(ws, 0);
  LayerWs w;
  const size_t A = static_cast<size_t>(T) * k;
  const int max_tiles = bm_route_max_tiles(T, k, L->num_experts, TILE_ROWS);
  w.topk_idx = c.take<int32_t>(A);
  w.topk_w = c.take<float>(A);
  w.token_indices = c.take<int32_t>(A);
  w.expert_offsets = c.take<int32_t>(L->num_experts + 1);
  w.route_flat = c.take<float>(A);
  w.tile_table = c.take<int32_t>(static_cast<size_t>(max_tiles) * 3);
  w.counts = c.take<int32_t>(2);
  w.h_gate = c.take<__half>(static_cast<size_t>(T) * L->rank_in);
  w.h_up = c.take<__half>(static_cast<size_t>(T) * L->rank_in);
  w.rank_accum = c.take<float>(static_cast<size_t>(T) * L->rank_out);
  w.route_ws_bytes = bm_route_build_workspace_bytes(T, k, L->num_experts);
  w.route_ws = c.take<unsigned char>(w.route_ws_bytes);
  w.experts_ws_bytes = bm_experts_workspace_bytes(L, T, static_cast<int32_t>(A), BM_PATH_AUTO);
  w.experts_ws = c.take<unsigned char>(w.experts_ws_bytes);
  w.total = c.off;
  return w;
}

}  // namespace bm

using namespace bm;

extern "C" int bm_abi_version(void) { return 2; }
extern "C" const char* bm_last_error(void) { return g_err; }
extern "C" uint64_t bm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" int bm_arena_layout_version(void) { return 3; }   // 3: one contiguous [scales | words] section per matrix and tile
extern "C" const char* bm_status_string(int s) {
  switch (s) {
    case BM_OK: return "ok";
    case BM_ERR_INVALID_ARG: return "invalid argument";
    case BM_ERR_UNSUPPORTED: return "unsupported";
    case BM_ERR_CUDA: return "CUDA error";
    case BM_ERR_WORKSPACE: return "workspace too small";
    case BM_ERR_TIMEOUT: return "device wait timed out";
    default: return "unknown status";
  }
}

extern "C" int bm_layer_plan(const bm_layer_desc_t* desc, size_t* arena_bytes) {
  BM_REQUIRE(arena_bytes != nullptr, BM_ERR_INVALID_ARG, "null arena_bytes");
  bm_layer tmp;
  const int rc = build_host(desc, &tmp);
  if (rc) return rc;
  FastPlan P;
  *arena_bytes = arena_need(&tmp, &P);
  return BM_OK;
}

extern "C" int bm_layer_create(const bm_layer_desc_t* desc, void* arena, size_t arena_bytes, void* stream,
                               bm_layer_t** out) {
  BM_REQUIRE(out != nullptr, BM_ERR_INVALID_ARG, "null output handle");
  *out = nullptr;
  bm_layer* L = new (std::nothrow) bm_layer();
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "out of host memory");
  int rc = build_host(desc, L);
  if (rc) { delete L; return rc; }
  FastPlan P;
  const size_t need = arena_need(L, &P);
  if (arena == nullptr || arena_bytes < need || (reinterpret_cast<uintptr_t>(arena) & 255u)) {
    delete L;
    return set_error(BM_ERR_WORKSPACE, "layer arena must be 256-byte aligned and hold %zu bytes (%zu given)", need, arena_bytes);
  }
  cudaGetDevice(&L->device);
  L->arena = arena;
  L->arena_bytes = arena_bytes;
  L->experts_dev = static_cast<ExpertDev*>(arena);
  std::vector<ExpertDev> tab(desc->num_experts);
  for (int e = 0; e < desc->num_experts; ++e) {
    tab[e].m[0] = to_dev(desc->gate[e]);
    tab[e].m[1] = to_dev(desc->up[e]);
    tab[e].m[2] = to_dev(desc->down[e]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  L->status_dev = reinterpret_cast<int*>(static_cast<unsigned char*>(arena) + table_bytes(desc->num_experts));
  cudaError_t ce = cudaMemsetAsync(L->status_dev, 0, 256, st);
  if (ce == cudaSuccess && desc->num_experts)
    ce = cudaMemcpyAsync(L->experts_dev, tab.data(), sizeof(ExpertDev) * tab.size(), cudaMemcpyHostToDevice, st);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
  if (ce != cudaSuccess) {
    delete L;
    return set_error(BM_ERR_CUDA, "uploading the expert table failed: %s", cudaGetErrorString(ce));
  }
  if (P.ok) {
    L->fast_host = P.experts;
    L->fast_dev = reinterpret_cast<const FastExpert*>(static_cast<unsigned char*>(arena) + P.table_off);
    L->max_unit_bytes = P.max_unit_bytes;
    L->max_slots = P.max_slots;
    L->max_words = P.max_words;
    rc = build_fast(L, P, st);
    if (rc) { delete L; return rc; }
    L->fast_ok = true;
    rc = plan_experts_decode(L);
    if (rc) { delete L; return rc; }
  }
  // host-side objects for the fork/join of routing and basis projection (no device memory)
  if (cudaStreamCreateWithFlags(&L->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&L->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&L->ev_join, cudaEventDisableTiming) != cudaSuccess) {
    L->side_stream = nullptr;
    (void)cudaGetLastError();
  }
  *out = L;
  return BM_OK;
}

extern "C" int bm_layer_destroy(bm_layer_t* layer) {
  if (layer) {
    if (layer->ev_fork) cudaEventDestroy(layer->ev_fork);
    if (layer->ev_join) cudaEventDestroy(layer->ev_join);
    if (layer->side_stream) cudaStreamDestroy(layer->side_stream);
  }
  delete layer;
  return BM_OK;
}

extern "C" int64_t bm_layer_expert_bytes(const bm_layer_t* L, int32_t e) {
  if (!L || e < 0 || e >= L->num_experts) return -1;
  return L->host[0][e].bytes + L->host[1][e].bytes + L->host[2][e].bytes;
}

extern "C" int bm_layer_set_option(bm_layer_t* L, int32_t option, int32_t value) {
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "set_option: null layer");
  if (option == BM_OPT_DETERMINISTIC) {
    BM_REQUIRE(value == 0 || value == 1, BM_ERR_INVALID_ARG, "set_option: the deterministic mode is 0 or 1");
    L->deterministic = value != 0;
    return BM_OK;
  }
  BM_REQUIRE(option == BM_OPT_DECODE_CTAS_PER_SM, BM_ERR_INVALID_ARG, "set_option: unknown option %d", option);
  BM_REQUIRE(value >= 0 && value <= 3, BM_ERR_INVALID_ARG, "set_option: CTAs per SM must be 0..3");
  const bm_layer saved = *L;
  L->dec_force_ctas = value;
  const int rc = plan_experts_decode(L);
  if (rc || (saved.dec_ok && !L->dec_ok)) {
    *L = saved;
    return rc ? rc : set_error(BM_ERR_UNSUPPORTED, "set_option: %d CTAs per SM do not fit this layer", value);
  }
  return BM_OK;
}

extern "C" int bm_layer_has_fast_layout(const bm_layer_t* L) { return L && L->fast_ok ? 1 : 0; }

extern "C" int bm_layer_status(const bm_layer_t* L, void* stream) {
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "layer_status: null layer");
  int flag = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BM_CUDA(cudaMemcpyAsync(&flag, L->status_dev, sizeof(int), cudaMemcpyDeviceToHost, st));
  BM_CUDA(cudaStreamSynchronize(st));
  if (flag != 0) {
    BM_CUDA(cudaMemsetAsync(L->status_dev, 0, sizeof(int), st));
    return set_error(BM_ERR_TIMEOUT, "a kernel of this layer gave up a bounded wait; its outputs are undefined");
  }
  return BM_OK;
}

extern "C" int bm_layer_decode_codes(const bm_layer_t* L, int32_t e, int32_t which, int32_t source, int8_t* codes,
                                     void* stream) {
  BM_REQUIRE(L && codes, BM_ERR_INVALID_ARG, "decode_codes: null pointer");
  BM_REQUIRE(e >= 0 && e < L->num_experts && which >= 0 && which < 3, BM_ERR_INVALID_ARG, "decode_codes: bad index");
  if (source == 1) {
    BM_REQUIRE(L->fast_ok, BM_ERR_UNSUPPORTED, "decode_codes: this layer has no arena layout");
    return launch_arena_decode(L, e, which, codes, static_cast<cudaStream_t>(stream));
  }
  const MatDev md = to_dev(L->src[which][e]);
  const int64_t total = static_cast<int64_t>(md.n_rows) * L->intermediate;
  if (total == 0) return BM_OK;
  const int blocks = static_cast<int>((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  decode_codes_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(md, L->intermediate, codes);
  BM_LAUNCH_CHECK("decode_codes_kernel");
  return BM_OK;
}

// `zero` / `zero_bytes`: a buffer (16-byte multiple) the projection kernel clears as a side job; `*zeroed` tells
// the caller whether the path taken did it.
static int basis_project_impl(const bm_layer_t* L, const void* x, int x_dtype, int32_t T, uint16_t* h_gate, uint16_t* h_up,
                              void* zero, size_t zero_bytes, bool* zeroed, void* stream) {
  if (zeroed) *zeroed = false;
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "basis_project: null layer");
  BM_REQUIRE(L->vh_gate && L->vh_up, BM_ERR_INVALID_ARG, "missing shared_vh basis for packed routed experts");
  BM_REQUIRE(T >= 0 && x_dtype >= BM_F16 && x_dtype <= BM_F32, BM_ERR_INVALID_ARG, "basis_project: bad arguments");
  if (T == 0) return BM_OK;
  BM_REQUIRE(x && h_gate && h_up, BM_ERR_INVALID_ARG, "basis_project: null pointer");
  if (T <= SKINNY_MAX_TOKENS && L->hidden % 128 == 0 && L->rank_in % 32 == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    SkinnyArgs a{};
    a.W[0] = L->vh_gate; a.W[1] = L->vh_up;
    a.C[0] = h_gate; a.C[1] = h_up;
    a.X = x; a.residual = nullptr;
    a.rows_per_w = L->rank_in; a.n_w = 2;
    a.N = T; a.K = L->hidden;
    a.x_dtype = x_dtype; a.c_dtype = BM_F16; a.round_x_f16 = 1;
    a.splits = 8; a.mrows = 32;
    if (zero != nullptr && zero_bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(zero) & 15u) == 0 && zero_bytes / 16 < (1u << 30)) {
      a.zero = static_cast<float4*>(zero);
      a.zero_n = static_cast<int>(zero_bytes / 16);
      if (zeroed) *zeroed = true;
    }
    const int rc = launch_skinny_nt(a, static_cast<cudaStream_t>(stream));
    if (rc != BM_ERR_UNSUPPORTED) return rc;
    if (zeroed) *zeroed = false;       // shape does not tile (e.g. a very wide hidden size): the general GEMMs below take it
  }
  if (L->hidden % 64 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    GemmTcArgs t{};
    t.X = x; t.W[0] = L->vh_gate; t.W[1] = L->vh_up; t.C[0] = h_gate; t.C[1] = h_up; t.residual = nullptr;
    t.M = T; t.N = L->rank_in; t.K = L->hidden; t.x_dtype = x_dtype; t.c_dtype = BM_F16; t.status = L->status_dev;
    return launch_gemm_basis(t, 2, static_cast<cudaStream_t>(stream));
  }
  GemmArgs g{};
  g.A[0] = g.A[1] = x;
  g.B[0] = L->vh_gate;
  g.B[1] = L->vh_up;
  g.C[0] = h_gate;
  g.C[1] = h_up;
  g.residual = nullptr;
  g.a_dtype = x_dtype;
  g.c_dtype = BM_F16;
  g.round_a_f16 = 0;
  g.M = T;
  g.N = L->rank_in;
  g.K = L->hidden;
  return launch_gemm_nt(g, 2, static_cast<cudaStream_t>(stream));
}

extern "C" int bm_basis_project(const bm_layer_t* L, const void* x, int x_dtype, int32_t T, uint16_t* h_gate,
                                uint16_t* h_up, void* stream) {
  bm::NvtxRange nvtx_range("bm_basis_project");
  return basis_project_impl(L, x, x_dtype, T, h_gate, h_up, nullptr, 0, nullptr, stream);
}

// fixed-point accumulators -> fp32 rank_accum (deterministic mode)
__global__ void __launch_bounds__(256) acc64_to_f32_kernel(const long long* __restrict__ acc64, float* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    out[i] = static_cast<float>(static_cast<double>(acc64[i]) * (1.0 / static_cast<double>(ACC_FIXED_SCALE)));
}

static size_t experts_ws_need(const bm_layer_t* L, int32_t T) {
  return (L && L->deterministic) ? align_up(sizeof(long long) * static_cast<size_t>(T) * L->rank_out, 256) : 0;
}

extern "C" size_t bm_experts_workspace_bytes(const bm_layer_t* L, int32_t T, int32_t num_assign, int32_t path) {
  (void)num_assign; (void)path;
  return T > 0 ? experts_ws_need(L, T) : 0;
}

static int experts_forward_impl(const bm_layer_t* L, const uint16_t* h_gate, const uint16_t* h_up,
                                const int32_t* token_indices, const int32_t* expert_offsets, const float* route_weights,
                                int32_t T, int32_t num_assign, float* rank_accum, int32_t path, bool already_zero,
                                void* workspace, size_t workspace_bytes, void* stream) {
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "experts_forward: null layer");
  BM_REQUIRE(T >= 0 && num_assign >= 0, BM_ERR_INVALID_ARG, "experts_forward: negative sizes");
  BM_REQUIRE(path >= BM_PATH_AUTO && path <= BM_PATH_TENSOR, BM_ERR_INVALID_ARG, "experts_forward: unknown path %d", path);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (T == 0) return BM_OK;
  BM_REQUIRE(rank_accum, BM_ERR_INVALID_ARG, "experts_forward: null rank_accum");
  long long* acc64 = nullptr;
  const int64_t n_acc = static_cast<int64_t>(T) * L->rank_out;
  if (L->deterministic) {
    const size_t need = experts_ws_need(L, T);
    BM_REQUIRE(workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0, BM_ERR_WORKSPACE,
               "experts_forward: the deterministic mode needs a 16-byte aligned workspace of %zu bytes (%zu given)", need, workspace_bytes);
    acc64 = static_cast<long long*>(workspace);
    BM_CUDA(cudaMemsetAsync(acc64, 0, sizeof(long long) * static_cast<size_t>(n_acc), st));
  } else if (!already_zero) {
    BM_CUDA(cudaMemsetAsync(rank_accum, 0, sizeof(float) * static_cast<size_t>(n_acc), st));
  }
  int rc = BM_OK;
  if (num_assign == 0 || L->num_experts == 0) {
    if (acc64) BM_CUDA(cudaMemsetAsync(rank_accum, 0, sizeof(float) * static_cast<size_t>(n_acc), st));
    return BM_OK;
  }
  BM_REQUIRE(h_gate && h_up && token_indices && expert_offsets && route_weights, BM_ERR_INVALID_ARG,
             "experts_forward: null pointer");
  BM_REQUIRE(path != BM_PATH_TENSOR || L->fast_ok, BM_ERR_UNSUPPORTED,
             "experts_forward: the tensor path needs 1- to 4-bit rows and full tiles; this layer has neither");
  BM_REQUIRE(path != BM_PATH_DECODE || L->fast_ok, BM_ERR_UNSUPPORTED,
             "experts_forward: the decode path needs 1- to 4-bit rows and full tiles; this layer has neither");
  const __half* hg = reinterpret_cast<const __half*>(h_gate);
  const __half* hu = reinterpret_cast<const __half*>(h_up);
  if (L->fast_ok && (path == BM_PATH_TENSOR || (path == BM_PATH_AUTO && num_assign > 16 * L->num_experts && experts_tc_fits(L))))
    rc = launch_experts_tc(L, hg, hu, token_indices, expert_offsets, route_weights, T, rank_accum, acc64, st);
  else if (L->fast_ok && (path == BM_PATH_DECODE || (path != BM_PATH_GENERIC && L->dec_ok && num_assign / 8 + L->num_experts < 60000)))
    rc = launch_experts_decode(L, hg, hu, token_indices, expert_offsets, route_weights, T, num_assign, rank_accum, acc64, st);
  else
    rc = launch_experts_generic(L, hg, hu, token_indices, expert_offsets, route_weights, T, rank_accum, acc64, st);
  if (rc) return rc;
  if (acc64) {
    const int blocks = static_cast<int>((n_acc + 255) / 256 < 148 * 8 ? (n_acc + 255) / 256 : 148 * 8);
    acc64_to_f32_kernel<<<blocks, 256, 0, st>>>(acc64, rank_accum, n_acc);
    BM_LAUNCH_CHECK("acc64_to_f32_kernel");
  }
  return BM_OK;
}

extern "C" int bm_experts_forward(const bm_layer_t* L, const uint16_t* h_gate, const uint16_t* h_up,
                                  const int32_t* token_indices, const int32_t* expert_offsets,
                                  const float* route_weights, int32_t T, int32_t num_assign, float* rank_accum,
                                  int32_t path, void* workspace, size_t workspace_bytes, void* stream) {
  bm::NvtxRange nvtx_range("bm_experts_forward");
  return experts_forward_impl(L, h_gate, h_up, token_indices, expert_offsets, route_weights, T, num_assign, rank_accum, path,
                              false, workspace, workspace_bytes, stream);
}

extern "C" int bm_combine_down_basis(const bm_layer_t* L, const float* rank_accum, int32_t T, const void* residual,
                                     void* y, int y_dtype, void* stream) {
  bm::NvtxRange nvtx_range("bm_combine_down_basis");
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "combine: null layer");
  BM_REQUIRE(L->u_down, BM_ERR_INVALID_ARG, "missing shared_u_down for packed routed experts");
  BM_REQUIRE(T >= 0 && y_dtype >= BM_F16 && y_dtype <= BM_F32, BM_ERR_INVALID_ARG, "combine: bad arguments");
  if (T == 0) return BM_OK;
  BM_REQUIRE(rank_accum && y, BM_ERR_INVALID_ARG, "combine: null pointer");
  if (T <= SKINNY_MAX_TOKENS && L->rank_out % 16 == 0 && L->hidden % 16 == 0 && L->rank_out <= 1024) {
    SkinnyArgs a{};
    a.W[0] = L->u_down; a.W[1] = L->u_down;
    a.C[0] = y; a.C[1] = y;
    a.X = rank_accum; a.residual = residual;
    a.rows_per_w = L->hidden; a.n_w = 1;
    a.N = T; a.K = L->rank_out;
    a.x_dtype = BM_F32; a.c_dtype = y_dtype; a.round_x_f16 = 1;
    a.splits = 1; a.mrows = 16;
    const int rc = launch_skinny_nt(a, static_cast<cudaStream_t>(stream));
    if (rc != BM_ERR_UNSUPPORTED) return rc;
  }
  if (L->rank_out % 64 == 0) {
    GemmTcArgs t{};
    t.X = rank_accum; t.W[0] = t.W[1] = L->u_down; t.C[0] = t.C[1] = y; t.residual = residual;
    t.M = T; t.N = L->hidden; t.K = L->rank_out; t.x_dtype = BM_F32; t.c_dtype = y_dtype; t.status = L->status_dev;
    return launch_gemm_basis(t, 1, static_cast<cudaStream_t>(stream));
  }
  GemmArgs g{};
  g.A[0] = g.A[1] = rank_accum;
  g.B[0] = g.B[1] = L->u_down;
  g.C[0] = g.C[1] = y;
  g.residual = residual;
  g.a_dtype = BM_F32;
  g.c_dtype = y_dtype;
  g.round_a_f16 = 1;
  g.M = T;
  g.N = L->hidden;
  g.K = L->rank_out;
  return launch_gemm_nt(g, 1, static_cast<cudaStream_t>(stream));
}

extern "C" size_t bm_layer_workspace_bytes(const bm_layer_t* L, int32_t T, int32_t k) {
  if (!L || T < 0 || k <= 0) return 0;
  return carve_layer_ws(L, nullptr, T, k).total;
}

extern "C" int bm_layer_forward(const bm_layer_t* L, const void* x, int x_dtype, const void* logits, int logits_dtype,
                                int32_t T, int32_t num_routed, int32_t k, int32_t renorm, int32_t weight_round,
                                const int32_t* global_to_local, const void* residual, void* y, int32_t path,
                                void* workspace, size_t workspace_bytes, void* stream) {
  bm::NvtxRange nvtx_range("bm_layer_forward");
  BM_REQUIRE(L != nullptr, BM_ERR_INVALID_ARG, "layer_forward: null layer");
  BM_REQUIRE(T >= 0 && k > 0 && num_routed > 0, BM_ERR_INVALID_ARG, "layer_forward: bad sizes");
  BM_REQUIRE(global_to_local != nullptr || num_routed == L->num_experts, BM_ERR_INVALID_ARG,
             "layer_forward: %d routed experts but %d packed and no id map", num_routed, L->num_experts);
  if (T == 0) return BM_OK;
  const LayerWs w = carve_layer_ws(L, workspace, T, k);
  BM_REQUIRE(workspace && workspace_bytes >= w.total && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
             BM_ERR_WORKSPACE, "layer_forward: workspace must be 256-byte aligned and hold %zu bytes (%zu given)", w.total,
             workspace_bytes);
  // routing depends only on the logits and the basis projection only on x: run them side by side
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fork = L->side_stream != nullptr && L->ev_fork != nullptr && L->ev_join != nullptr;
  void* route_stream = stream;
  if (fork) {
    BM_CUDA(cudaEventRecord(L->ev_fork, st));
    BM_CUDA(cudaStreamWaitEvent(L->side_stream, L->ev_fork, 0));
    route_stream = L->side_stream;
  }
  int rc = bm_route(logits, logits_dtype, T, num_routed, k, renorm, weight_round, global_to_local, L->num_experts, TILE_ROWS,
                    w.topk_idx, w.topk_w, w.token_indices, w.expert_offsets, w.route_flat, /*tile_table=*/nullptr, /*counts=*/nullptr,
                    w.route_ws, w.route_ws_bytes, route_stream);
  // the accumulator of the expert stage is cleared off the critical path: by the projection kernel when the
  // skinny one runs, else by a memset beside the routing
  bool zeroed = false;
  const size_t acc_bytes = sizeof(float) * static_cast<size_t>(T) * L->rank_out;
  const int rc_basis = basis_project_impl(L, x, x_dtype, T, reinterpret_cast<uint16_t*>(w.h_gate),
                                          reinterpret_cast<uint16_t*>(w.h_up), w.rank_accum, acc_bytes, &zeroed, stream);
  if (!zeroed && cudaMemsetAsync(w.rank_accum, 0, acc_bytes, static_cast<cudaStream_t>(route_stream)) == cudaSuccess) zeroed = true;
  if (fork) {
    // always join, also on error, so that the side stream never stays attached to a capture
    cudaEventRecord(L->ev_join, L->side_stream);
    cudaStreamWaitEvent(st, L->ev_join, 0);
  }
  if (rc) return rc;
  if (rc_basis) return rc_basis;
  // Dropped assignments (experts that are not packed) leave a shorter list; the kernels walk
  // expert_offsets, so passing the upper bound T*k as num_assign is safe.
  rc = experts_forward_impl(L, reinterpret_cast<const uint16_t*>(w.h_gate), reinterpret_cast<const uint16_t*>(w.h_up),
                            w.token_indices, w.expert_offsets, w.route_flat, T, T * k, w.rank_accum, path, zeroed, w.experts_ws,
                            w.experts_ws_bytes, stream);
  if (rc) return rc;
  return bm_combine_down_basis(L, w.rank_accum, T, residual, y, x_dtype == BM_F32 ? BM_F32 : x_dtype, stream);
}
