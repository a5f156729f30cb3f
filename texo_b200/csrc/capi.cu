// Library-wide diagnostics of libtexo_b200.so (declared in include/texo_b200.h).  None of
// these has a counterpart in the reference, whose operators expose only `solve`.
#include "host_common.h"
#include "ptx.cuh"

extern "C" long long texo_kernel_launches(void) { return texo::launch_counter(); }

extern "C" void texo_profile_enable(int on) {
  texo::KernelProfile& p = texo::kernel_profile();
  p.enabled = on != 0;
  p.used = 0;
}

extern "C" int texo_profile_read(float* total_ms, int* launches) {
  texo::KernelProfile& p = texo::kernel_profile();
  float total = 0.f;
  int n = 0;
  for (int i = 0; i < p.used; ++i) {
    float ms = 0.f;
    if (cudaEventSynchronize(p.stop[i]) != cudaSuccess ||
        cudaEventElapsedTime(&ms, p.start[i], p.stop[i]) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    total += ms;
    ++n;
  }
  if (total_ms) *total_ms = total;
  if (launches) *launches = n;
  return 0;
}

// Self-test of the bounded-wait failure path (no counterpart in the reference, whose kernels
// have no device-side waits).  One CTA waits on an mbarrier that nothing will ever complete:
// after its clock budget (about a second) the wait gives up, records STATUS_TIMEOUT_FLAG in
// the device status word and the kernel returns normally - the context stays usable.
// Returns the status code read back (5 when the path works), which is also cleared.
namespace texo {
__global__ void wait_timeout_selftest_kernel(int* status, int* reached_end) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(&bar, 0, &abort_flag, status, STATUS_TIMEOUT_FLAG);
  __syncthreads();
  // every other thread sees the abort flag the waiter raised
  if (threadIdx.x == 1) *reached_end = (abort_flag != 0 && ok) ? 1 : 0;
}
}  // namespace texo

extern "C" int texo_selftest_wait_timeout(void) {
  texo::DeviceCtx& ctx = texo::device_ctx();
  if (!ctx.status) return -1;
  int* reached = ctx.status + 32;
  cudaMemset(reached, 0, sizeof(int));
  texo::wait_timeout_selftest_kernel<<<1, 64>>>(ctx.status, reached);
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  int reached_host = 0;
  cudaMemcpy(&reached_host, reached, sizeof(int), cudaMemcpyDeviceToHost);
  const int code = texo::read_and_clear_status();
  return reached_host == 1 ? code : -3;
}

// Hits and misses of the tensor-map cache since the process started (host_common.h); no
// counterpart in the reference, which builds no descriptors on this path.
extern "C" void texo_tensor_map_cache_stats(long long* hits, long long* misses) {
  const texo::TensorMapCache& cache = texo::tensor_map_cache();
  if (hits) *hits = cache.hits;
  if (misses) *misses = cache.misses;
}

// Sets the epoch counter of the current device's sums flags (host_common.h, next_sums_epoch),
// so that a test can drive the counter across its 32-bit wrap.  Diagnostic; no counterpart in
// the reference.
extern "C" void texo_set_sums_epoch(unsigned value) { texo::device_ctx().sums_epoch = value; }
