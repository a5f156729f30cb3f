// Library-wide diagnostics of libtexo_b200.so (declared in include/texo_b200.h).  None of
// these has a counterpart in the reference, whose operators expose only `solve`.
#include "host_common.h"

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
