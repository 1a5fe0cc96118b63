// Routing build for callers that cannot hand the library any scratch memory.
//
// bm_route_build needs a per-block histogram table in global memory once T*k exceeds one block
// (1024 assignments); normally the caller allocates it (bm_route_build_workspace_bytes).  Some hosts
// cannot: a serving loop that must not call the CUDA allocator on its hot path (cudaMalloc stalls
// the whole device), or a plug-in that is handed raw pointers to inputs and outputs by another
// runtime and owns no memory pool of its own.  For them this file keeps the table in a fixed array
// inside the library image.
#include "common.cuh"

namespace bm {

// 1 MiB of block histograms: ceil(T*k / 1024) * num_local int32 entries.  Every GPU that loads the
// library holds this array until the process exits.
constexpr size_t ROUTE_STATIC_SCRATCH_BYTES = 1u << 20;
static __device__ __align__(256) unsigned char g_route_scratch[ROUTE_STATIC_SCRATCH_BYTES];

// Device address of the array, per device ordinal.  Written without a lock: two host threads that race on the first
// call for a device both look the address up and store the same value.
static void* g_route_scratch_ptr[MAX_DEVICES] = {};

// `g_route_scratch` in host code only names the symbol; the address a kernel can use has to be asked for,
// once per device, with that device current.
static int route_scratch_address(void** out) {
  int dev = -1;
  BM_CUDA(cudaGetDevice(&dev));
  BM_REQUIRE(dev >= 0 && dev < MAX_DEVICES, BM_ERR_UNSUPPORTED, "route_build_static: device ordinal %d out of range", dev);
  if (g_route_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    BM_CUDA(cudaGetSymbolAddress(&p, g_route_scratch));
    BM_REQUIRE(p != nullptr, BM_ERR_CUDA, "route_build_static: no device address for the scratch array");
    g_route_scratch_ptr[dev] = p;
  }
  *out = g_route_scratch_ptr[dev];
  return BM_OK;
}

}  // namespace bm

extern "C" size_t bm_route_build_static_capacity(void) { return bm::ROUTE_STATIC_SCRATCH_BYTES; }

extern "C" int bm_route_build_static(const int32_t* topk_idx, const float* topk_w, const int32_t* global_to_local,
                                     int32_t num_routed, int32_t T, int32_t k, int32_t num_local, int32_t tile_rows, int32_t* token_indices,
                                     int32_t* expert_offsets, float* route_flat, int32_t* tile_table, int32_t* counts,
                                     void* stream) {
  using namespace bm;
  const size_t need = bm_route_build_workspace_bytes(T, k, num_local);
  BM_REQUIRE(need <= ROUTE_STATIC_SCRATCH_BYTES, BM_ERR_WORKSPACE,
             "route_build_static: T*k=%lld assignments over %d experts need %zu bytes of scratch, the built-in array holds %zu; "
             "use bm_route_build with a caller-provided workspace",
             static_cast<long long>(T) * k, num_local, need, ROUTE_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int rc = route_scratch_address(&scratch);
  if (rc) return rc;
  return bm_route_build(topk_idx, topk_w, global_to_local, num_routed, T, k, num_local, tile_rows, token_indices, expert_offsets,
                        route_flat, tile_table, counts, scratch, ROUTE_STATIC_SCRATCH_BYTES, stream);
}
