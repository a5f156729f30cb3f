// Host-memory stand-in for the handful of CUDA runtime calls the reference harnesses make
// (tests/test_utils.h:11-48, tests/mm_int4.cpp:125-135 of frezcirno/Texo): "device" memory
// is plain malloc, copies are memcpy, everything is synchronous.  TEST INFRASTRUCTURE: it
// exists so that the reference's UNCHANGED harness sources - and with them the reference's
// own CPU reference loops - can be compiled with g++ and run on a machine without a GPU,
// with `solve` bound to the CPU oracle (oracle_solve.cpp).  If the harness prints
// ALL PASSED, the reference's own CPU code has accepted the oracle on every default case.
// Never linked into the product.
#include <cuda_runtime.h>

#include <chrono>
#include <cstdlib>
#include <cstring>

extern "C" {

cudaError_t cudaMalloc(void** ptr, size_t bytes) {
  *ptr = std::malloc(bytes ? bytes : 1);
  return *ptr ? cudaSuccess : cudaErrorMemoryAllocation;
}
cudaError_t cudaFree(void* ptr) {
  std::free(ptr);
  return cudaSuccess;
}
cudaError_t cudaMemcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind) {
  if (bytes) std::memcpy(dst, src, bytes);
  return cudaSuccess;
}
cudaError_t cudaGetLastError(void) { return cudaSuccess; }
cudaError_t cudaDeviceSynchronize(void) { return cudaSuccess; }
const char* cudaGetErrorString(cudaError_t) { return "host stand-in: no CUDA errors"; }

// Events carry a host timestamp (only the harness's --bench mode uses them).
struct HostEvent {
  std::chrono::steady_clock::time_point at;
};
cudaError_t cudaEventCreate(cudaEvent_t* event) {
  *event = reinterpret_cast<cudaEvent_t>(new HostEvent);
  return cudaSuccess;
}
cudaError_t cudaEventRecord(cudaEvent_t event, cudaStream_t) {
  reinterpret_cast<HostEvent*>(event)->at = std::chrono::steady_clock::now();
  return cudaSuccess;
}
cudaError_t cudaEventSynchronize(cudaEvent_t) { return cudaSuccess; }
cudaError_t cudaEventElapsedTime(float* ms, cudaEvent_t start, cudaEvent_t stop) {
  *ms = std::chrono::duration<float, std::milli>(reinterpret_cast<HostEvent*>(stop)->at -
                                                 reinterpret_cast<HostEvent*>(start)->at)
            .count();
  return cudaSuccess;
}
}
