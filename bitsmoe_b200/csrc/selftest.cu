// Self-test of the bounded device-side wait: a kernel that waits on an mbarrier nobody arrives on, with a limit of
// a millisecond or so, gives up, raises the layer's status flag and returns normally.  It exists so that the
// time-out path of every pipeline in this library (the same tc::mbar_wait) can be exercised on a GPU without
// faulting, trapping or hanging it: the context stays usable and bm_layer_status reports BM_ERR_TIMEOUT.
#include "common.cuh"
#include "tc05.cuh"

namespace bm {

__global__ void __launch_bounds__(32) wait_probe_kernel(uint64_t limit_ns, int* __restrict__ status) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    tc::mbar_init_fence();
  }
  __syncwarp();
  const bool ok = tc::mbar_wait(&bar, 0, limit_ns);   // phase 0 never completes
  if (!ok && threadIdx.x == 0) atomicExch(status, BM_ERR_TIMEOUT);
}

}  // namespace bm

extern "C" int bm_layer_selftest_wait(const bm_layer_t* L, int32_t limit_us, void* stream) {
  using namespace bm;
  BM_REQUIRE(L != nullptr && L->status_dev != nullptr, BM_ERR_INVALID_ARG, "selftest_wait: null layer");
  BM_REQUIRE(limit_us > 0 && limit_us <= 100000, BM_ERR_INVALID_ARG, "selftest_wait: limit must be 1..100000 us");
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t>(limit_us) * 1000ull, L->status_dev);
  BM_LAUNCH_CHECK("wait_probe_kernel");
  return BM_OK;
}
