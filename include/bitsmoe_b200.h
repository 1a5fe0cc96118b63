/*
 * bitsmoe_b200 -- C ABI of the sm_100a quantized-expert forward path.
 *
 * Every entry point returns an int status (BM_OK == 0), takes plain device
 * pointers, element counts and the CUDA stream to enqueue on (passed as
 * void*, i.e. a cudaStream_t), never allocates or frees device memory (the
 * caller owns the arena, the workspace and all tensors), never synchronises
 * the stream unless stated, and never traps: a failed check returns a status
 * and bm_last_error() gives the message for the calling thread.
 *
 * Each declaration names the reference interface it stands in for, by the
 * file's path inside the BitsMoE tree.
 */
#ifndef BITSMOE_B200_H_
#define BITSMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define BM_API __attribute__((visibility("default")))
#else
#define BM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  BM_OK = 0,
  BM_ERR_INVALID_ARG = 1,   /* shape / dtype / null pointer / inconsistent meta (TORCH_CHECK in the reference) */
  BM_ERR_UNSUPPORTED = 2,   /* bit width, activation or size outside what the kernels implement */
  BM_ERR_CUDA = 3,          /* a CUDA runtime call or a launch failed */
  BM_ERR_WORKSPACE = 4,     /* caller-provided arena / workspace too small or misaligned */
  BM_ERR_TIMEOUT = 5        /* a bounded device-side wait gave up; outputs are undefined */
};

enum { BM_F16 = 0, BM_BF16 = 1, BM_F32 = 2 };          /* element types of activations */
enum { BM_ROUND_NONE = 0, BM_ROUND_F16 = 1, BM_ROUND_BF16 = 2 };
enum { BM_PATH_AUTO = 0, BM_PATH_GENERIC = 1, BM_PATH_DECODE = 2, BM_PATH_TENSOR = 3 };
enum { BM_GATE = 0, BM_UP = 1, BM_DOWN = 2 };

BM_API int bm_abi_version(void);
BM_API const char* bm_last_error(void);
/* Kernel launches issued by this library in this process so far (a launch recorded into a CUDA graph during stream
 * capture counts once, when it is captured), and the version of the arena layout that bm_layer_create builds
 * (recorded profiler captures are only comparable within one version). */
BM_API uint64_t bm_launch_count(void);
BM_API int bm_arena_layout_version(void);
BM_API const char* bm_status_string(int status);

/* ---- bit-plane codec ---------------------------------------------------
 * Replaces pack_int8_{1,2,3,4,6,8}bit / unpack_int8_{...}bit of
 * bitsmoe/quant/bitpack/bitpack_cuda_binding.cpp:37-65 (kernels
 * bitsmoe/quant/bitpack/bitpack_cuda_kernel.cu:81-121, :157-196).
 * q: int8 [rows, cols]; words: uint32 [rows, ceil(cols/32) * bits].
 * Unpack writes int8 [rows, groups * 32]. */
BM_API int bm_pack_bitplanes_i8(const int8_t* q, uint32_t* words, int64_t rows, int64_t cols, int bits, void* stream);
BM_API int bm_unpack_bitplanes_i8(const uint32_t* words, int8_t* q, int64_t rows, int64_t groups, int bits, void* stream);

/* Quantise, bit-plane pack and reorder one slab (<= 64 rank rows of one width) in one kernel: the three steps of
 * _pack_lowbit_slab_payload_and_scale (bitsmoe/quant/packer.py:210-306) = quantize_symmetric per (row, 128-column tile)
 * (bitsmoe/quant/quantizer.py:30-84), BitPack.pack, and the [tile][stage][micro][row][plane] reorder (packer.py:169-207).
 * rows fp32 [k, dim] with row_stride elements between rows; payload uint32 [tiles * k * 4 * bits] and scale fp16
 * [tiles, k] are the slab's pieces of payload_buffer / scale_buffer; codes (int8 [k, tiles * 128], may be NULL) receives
 * the signed codes.  bits in {1, 2, 3, 4, 6, 8}. */
BM_API int bm_quantize_pack_slab(const float* rows, int64_t row_stride, int32_t k, int32_t dim, int32_t bits, uint32_t* payload,
                                 uint16_t* scale, int8_t* codes, void* stream);

/* ---- layer state -------------------------------------------------------
 * One packed expert matrix exactly as the reference stores it: the six
 * buffers that bitsmoe/models/base_mlp.py:96-102 registers and
 * bitsmoe/algorithms/cpp/mlp_forward_binding.cpp:58-75 receives. */
typedef struct {
  const uint32_t* payload;     int64_t payload_words;
  const int32_t*  rank_idx;    int32_t n_rows;        /* local row -> logical rank */
  const int32_t*  tile_meta;   int32_t n_tile_rows;   /* [n_tile_rows, 3] = pack_off, scale_off, n_valid */
  const int32_t*  slab_meta;   int32_t n_slabs;       /* [n_slabs, 4] = bits, k_slab, rank_off, tile_off */
  const uint16_t* scale;       int64_t n_scales;      /* fp16 bits */
  const uint16_t* s;                                  /* fp16 bits, n_rows entries */
} bm_matrix_t;

typedef struct {
  int32_t num_experts;         /* packed (local) experts E' */
  int32_t hidden;              /* H */
  int32_t intermediate;        /* I */
  int32_t rank_in;             /* rows of shared_vh_{gate,up}_proj == width of h_gate / h_up */
  int32_t rank_out;            /* columns of shared_u_down == width of rank_accum */
  int32_t act_type;            /* 0 = SiLU; anything else is BM_ERR_UNSUPPORTED (mlp_forward_binding.cpp:126) */
  const bm_matrix_t* gate;     /* host array [num_experts] */
  const bm_matrix_t* up;
  const bm_matrix_t* down;
  const uint16_t* vh_gate;     /* fp16 [rank_in, hidden]  (base_block.py:27), may be NULL for op-only use */
  const uint16_t* vh_up;       /* fp16 [rank_in, hidden]  (base_block.py:28) */
  const uint16_t* u_down;      /* fp16 [hidden, rank_out] (base_block.py:29) */
} bm_layer_desc_t;

typedef struct bm_layer bm_layer_t;

/* Bytes of device arena a layer needs (pointer tables + repacked payload).  Reads the
 * small meta buffers back to the host (synchronous), validates every offset against
 * the buffer lengths, and takes the place of build_packed_meta_cached
 * (bitsmoe/algorithms/cpp/mlp_forward.cu:2529-2697). */
BM_API int bm_layer_plan(const bm_layer_desc_t* desc, size_t* arena_bytes);
/* Builds the layer into caller-owned device memory `arena` (256-byte aligned,
 * >= arena_bytes).  The reference buffers named by desc must stay alive: the generic
 * path reads them in place.  Synchronises `stream` before returning. */
BM_API int bm_layer_create(const bm_layer_desc_t* desc, void* arena, size_t arena_bytes, void* stream, bm_layer_t** out);
BM_API int bm_layer_destroy(bm_layer_t* layer);
/* Bytes the forward path reads for the experts, as stored by the reference
 * (payload + scale + s + rank_idx + meta of the three matrices of expert e). */
BM_API int64_t bm_layer_expert_bytes(const bm_layer_t* layer, int32_t expert);
/* Decoded integer codes of one matrix, int8 [n_rows, intermediate] in stored (local) row order,
 * read either from the reference buffers in place (source 0; the decode of
 * bitsmoe/algorithms/cpp/mlp_forward.cu:203-275) or back out of the repacked arena (source 1;
 * BM_ERR_UNSUPPORTED when the layer has no arena layout).  For the bit-exactness tests. */
BM_API int bm_layer_decode_codes(const bm_layer_t* layer, int32_t expert, int32_t which, int32_t source, int8_t* codes,
                                 void* stream);
/* 1 when the layer was repacked into the arena layout that the decode and tensor paths need
 * (every stored row 1 to 4 bits wide, full tiles), else 0. */
BM_API int bm_layer_has_fast_layout(const bm_layer_t* layer);
/* Synchronises `stream` and reports whether any kernel of this layer gave up a bounded wait since
 * the last call (BM_ERR_TIMEOUT) -- the device-side counterpart of C10_CUDA_KERNEL_LAUNCH_CHECK. */
BM_API int bm_layer_status(const bm_layer_t* layer, void* stream);

/* No counterpart in the reference.  Tuning knobs of a layer; set between forwards, never while one is in flight.
 *   BM_OPT_DECODE_CTAS_PER_SM: resident CTAs per SM of the decode kernel (1, 2 or 3; 0 = the library's choice).
 *   BM_OPT_DETERMINISTIC (0 / 1): the packed-expert kernels add into rank_accum through 64-bit fixed-point atomics
 *     instead of fp32 atomics (bitsmoe/algorithms/cpp/mlp_forward.cu:2062 uses fp32 atomics, whose result depends on
 *     arrival order): two runs on the same inputs are then bit-identical.  bm_experts_workspace_bytes /
 *     bm_layer_workspace_bytes grow by 8 bytes per rank_accum element; ask them again after switching.
 * Returns BM_ERR_UNSUPPORTED when the layer's working set does not fit the requested geometry (nothing changes). */
enum { BM_OPT_DECODE_CTAS_PER_SM = 0, BM_OPT_DETERMINISTIC = 1 };
BM_API int bm_layer_set_option(bm_layer_t* layer, int32_t option, int32_t value);

/* No counterpart in the reference.  Launches a one-warp kernel whose only job is to wait (at most limit_us
 * microseconds, 1..100000) on a barrier that nothing signals: the wait gives up, the kernel returns, and the next
 * bm_layer_status() reports BM_ERR_TIMEOUT.  It is how the time-out path shared by all pipelines of this library
 * is tested on a GPU without faulting or hanging it. */
BM_API int bm_layer_selftest_wait(const bm_layer_t* layer, int32_t limit_us, void* stream);

/* ---- routing -----------------------------------------------------------
 * Router tail of bitsmoe/models/qwen3moe/bitsmoe_block.py:47-51 (softmax in
 * fp32, top-k sorted by descending probability with ties to the lower expert
 * id, optional renormalisation, weights rounded through `weight_round`).
 * logits [T, E] of logits_dtype -> topk_idx int32 [T, k], topk_w fp32 [T, k]. */
BM_API int bm_route_topk(const void* logits, int logits_dtype, int32_t T, int32_t E, int32_t k, int32_t renorm,
                  int32_t weight_round, int32_t* topk_idx, float* topk_w, void* stream);
BM_API size_t bm_route_build_workspace_bytes(int32_t T, int32_t k, int32_t num_local);
/* _build_packed_routing of bitsmoe/models/base_block.py:258-289 plus the task
 * tables of bitsmoe/algorithms/cpp/mlp_forward.cu:331-374, without host syncs:
 *   token_indices int32 [T*k]   expert-contiguous, ascending (token, slot) inside an expert
 *   expert_offsets int32 [num_local+1]
 *   route_flat fp32 [T*k]
 *   tile_table int32 [max_tiles, 3] = (expert, first assignment, rows <= tile_rows), padded
 *              with rows == 0 entries up to max_tiles = bm_route_max_tiles(); may be NULL
 *   counts int32 [2] = {assignments kept, tiles}; may be NULL
 * global_to_local int32 [num_routed] maps a routed expert id to a packed id or -1 (NULL = identity, and then
 * num_routed must equal num_local).  Ids come from the caller's gate: an id outside [0, num_routed), or a map
 * entry outside [0, num_local), is treated as -1 -- the assignment is dropped, nothing is indexed with it. */
BM_API int32_t bm_route_max_tiles(int32_t T, int32_t k, int32_t num_local, int32_t tile_rows);
BM_API int bm_route_build(const int32_t* topk_idx, const float* topk_w, const int32_t* global_to_local, int32_t num_routed,
                   int32_t T, int32_t k, int32_t num_local, int32_t tile_rows,
                   int32_t* token_indices, int32_t* expert_offsets, float* route_flat,
                   int32_t* tile_table, int32_t* counts, void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  Same result as bm_route_build, for hosts that cannot give the
 * library scratch memory (code that must stay off the CUDA allocator while serving, or a plug-in that
 * only ever receives input and output pointers): the per-block histogram table lives in a fixed
 * 1 MiB array inside the library instead of a caller workspace.  Calls nothing that allocates.
 *  - limit: ceil(T*k/1024) * num_local * 4 bytes must fit bm_route_build_static_capacity();
 *    larger problems return BM_ERR_WORKSPACE and should use bm_route_build;
 *  - the first call on each device looks up the array's device address (that device must be
 *    current); make that first call before starting any stream capture;
 *  - all calls on a device share the one array: it still holds the previous call's table on
 *    entry (every entry used is rewritten before it is read, nothing needs to be zero), and two
 *    calls whose kernels overlap on the GPU (different streams) race on it. */
BM_API size_t bm_route_build_static_capacity(void);
BM_API int bm_route_build_static(const int32_t* topk_idx, const float* topk_w, const int32_t* global_to_local,
                                 int32_t num_routed, int32_t T, int32_t k, int32_t num_local, int32_t tile_rows,
                                 int32_t* token_indices, int32_t* expert_offsets, float* route_flat,
                                 int32_t* tile_table, int32_t* counts, void* stream);

/* Router tail and routing build in one call (bm_route_topk then bm_route_build): the sequence
 * bitsmoe/models/qwen3moe/bitsmoe_block.py:47-51 -> bitsmoe/models/base_block.py:258-289. */
BM_API int bm_route(const void* logits, int logits_dtype, int32_t T, int32_t E_routed, int32_t k, int32_t renorm,
                    int32_t weight_round, const int32_t* global_to_local, int32_t num_local, int32_t tile_rows,
                    int32_t* topk_idx, float* topk_w, int32_t* token_indices, int32_t* expert_offsets,
                    float* route_flat, int32_t* tile_table, int32_t* counts, void* workspace, size_t workspace_bytes,
                    void* stream);

/* ---- forward stages ----------------------------------------------------
 * h_gate = x @ Vh_gate^T, h_up = x @ Vh_up^T rounded to fp16
 * (bitsmoe/models/qwen3moe/bitsmoe_block.py:63-64).  x [T, hidden] of x_dtype. */
BM_API int bm_basis_project(const bm_layer_t* layer, const void* x, int x_dtype, int32_t T,
                     uint16_t* h_gate, uint16_t* h_up, void* stream);
/* Scratch bm_experts_forward needs: 0, or the fixed-point accumulators of the deterministic mode. */
BM_API size_t bm_experts_workspace_bytes(const bm_layer_t* layer, int32_t T, int32_t num_assign, int32_t path);
/* The op contract of moe_packed_forward (bitsmoe/algorithms/cpp/mlp_forward_binding.cpp:53-155,
 * bitsmoe/algorithms/cpp/mlp_forward.cu:2701-3074): rank_accum fp32 [T, rank_out] is
 * overwritten with  sum over assignments of  route_w * s_down * (W_down . (silu(g) * u)). */
BM_API int bm_experts_forward(const bm_layer_t* layer, const uint16_t* h_gate, const uint16_t* h_up,
                       const int32_t* token_indices, const int32_t* expert_offsets, const float* route_weights,
                       int32_t T, int32_t num_assign, float* rank_accum, int32_t path,
                       void* workspace, size_t workspace_bytes, void* stream);
/* y = fp16(rank_accum) @ U_down^T (+ residual) in y_dtype (bitsmoe/models/base_block.py:414 and the
 * adds of qwen3moe/bitsmoe_block.py:95, deepseekv2/bitsmoe_block.py:123-124).  residual may be NULL. */
BM_API int bm_combine_down_basis(const bm_layer_t* layer, const float* rank_accum, int32_t T,
                          const void* residual, void* y, int y_dtype, void* stream);

/* Whole block for given router logits: route -> basis -> experts -> down basis, on one
 * stream with no host synchronisation (the forward of
 * bitsmoe/models/qwen3moe/bitsmoe_block.py:39-98 after `router_logits = self.gate(x)`). */
BM_API size_t bm_layer_workspace_bytes(const bm_layer_t* layer, int32_t T, int32_t k);
BM_API int bm_layer_forward(const bm_layer_t* layer, const void* x, int x_dtype, const void* logits, int logits_dtype,
                     int32_t T, int32_t num_routed, int32_t k, int32_t renorm, int32_t weight_round,
                     const int32_t* global_to_local, const void* residual, void* y, int32_t path,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ---- dense products around the packed experts ---------------------------
 * Router logits = x @ W_gate^T (the `self.gate(hidden_states)` of bitsmoe/models/qwen3moe/bitsmoe_block.py:45): x [T, hidden]
 * of x_dtype, gate_w fp16 [num_routed, hidden] -> logits [T, num_routed] of logits_dtype (the reference keeps them in x's type). */
BM_API int bm_gate_logits(const void* x, int x_dtype, const uint16_t* gate_w, int32_t T, int32_t num_routed, int32_t hidden,
                          void* logits, int logits_dtype, void* stream);
/* Dense shared expert(s): y = (silu(x @ Wg^T) * (x @ Wu^T)) @ Wd^T (+ residual), the `shared_experts(identity)` of
 * bitsmoe/models/deepseekv2/bitsmoe_block.py:123-124; with token_gate_w (fp16 [hidden]) every token's result is scaled by
 * sigmoid(x . token_gate_w), the gated shared expert of bitsmoe/models/qwen3next/bitsmoe_block.py:144-147.
 * Weights fp16: w_gate, w_up [intermediate, hidden], w_down [hidden, intermediate].  residual (y_dtype, [T, hidden]) may be
 * NULL; y may be passed on as the residual of bm_layer_forward / bm_combine_down_basis. */
BM_API size_t bm_dense_mlp_workspace_bytes(int32_t T, int32_t intermediate);
BM_API int bm_dense_mlp_forward(const void* x, int x_dtype, const uint16_t* w_gate, const uint16_t* w_up, const uint16_t* w_down,
                                const uint16_t* token_gate_w, int32_t T, int32_t hidden, int32_t intermediate,
                                const void* residual, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* ---- expert parallelism ------------------------------------------------
 * The reference has no distributed code (bitsmoe/models/deepseekv2/bitsmoe_block.py:57-62 copies ep_size / ep_rank and
 * never reads them).  These two kernels are the exchange that sharding the experts over the GPUs of one box needs; they
 * move rank-space rows through memory that every rank has mapped (peer pointers over NVLink), with plain stores and
 * loads.  One wave = T tokens on every one of `world` ranks; rank g owns experts [g * experts_per_rank, (g+1) * ...).
 * Receive area of a rank (all pointer tables are HOST arrays of `world` DEVICE pointers, entry g = rank g's area):
 *   h_bufs      fp16  [2][world][T][r]     gate rows of every rank's tokens, then up rows (token u = s*T + t)
 *   route_bufs  int32 [2][world][T][k]     expert ids, then the bit patterns of the fp32 route weights
 *   part_bufs   fp32  [world*T][r_out]     that rank's partial rank_accum (output of bm_experts_forward over all tokens)
 * The caller separates the stages with barriers across the ranks (stream-ordered): push -> barrier -> routing build and
 * experts on every rank -> barrier -> pull. */
/* Stream-ordered barrier across the ranks: flag_bufs[g] = rank g's flag area (bm_ep_flag_bytes() bytes, zeroed once
 * before the first use, mapped by every rank).  Every rank must enter the barriers of a channel (0..7) in the same
 * order.  The wait is bounded by limit_ms; when it runs out the kernel returns and bm_layer_status(layer) reports
 * BM_ERR_TIMEOUT (a rank that never arrives costs a time-out, not a hang). */
BM_API size_t bm_ep_flag_bytes(void);
BM_API int bm_ep_barrier(const bm_layer_t* layer, void* const* flag_bufs, int32_t world, int32_t rank, int32_t channel,
                         int32_t limit_ms, void* stream);
/* Dispatch: this rank's own slices h_bufs[rank][.][rank] and route_bufs[rank][.][rank] must hold its tokens' rows and
 * top-k.  Every token's top-k is written to every peer; its two rows only to the peers that own one of its experts. */
BM_API int bm_ep_push(void* const* h_bufs, void* const* route_bufs, int32_t world, int32_t rank, int32_t T, int32_t r,
                      int32_t k, int32_t experts_per_rank, void* stream);
/* Combine: rank_accum fp32 [T, r_out] of this rank's tokens = sum, in ascending rank order, of the partial rows of the
 * ranks that own one of the token's experts (my_topk_idx int32 [T, k], this rank's own routing). */
BM_API int bm_ep_pull_reduce(void* const* part_bufs, const int32_t* my_topk_idx, int32_t world, int32_t rank, int32_t T,
                             int32_t r_out, int32_t k, int32_t experts_per_rank, float* rank_accum, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BITSMOE_B200_H_ */
