// Tile-scale dequantization for B200: Y[m,n] = X[m,n] * S[m / T][n / T], FP32.
//
// Drop-in for frezcirno/Texo src/dequantization.cu:40-51 (same `solve` symbol and argument
// order, device pointers, legacy default stream, no scratch).  The op moves 8 bytes per
// element and does one multiply, so it is bound by HBM bandwidth: the kernel keeps four
// independent 16-byte streaming loads in flight per thread and writes with streaming stores
// so neither stream pollutes L2.
#include <algorithm>
#include <cstdint>
#include <cuda_runtime.h>

#include "host_common.h"

namespace texo {
namespace dq {

constexpr int THREADS = 256;
constexpr int UNROLL = 4;  // float4 per thread

// One block = one row segment of THREADS * UNROLL float4.  n4 = N / 4.
__global__ void __launch_bounds__(THREADS)
    rows_vec4_kernel(const float4* __restrict__ X, const float* __restrict__ S,
                     float4* __restrict__ Y, int n4, int T, int nt, int m0) {
  const int m = m0 + blockIdx.y;
  const float* s_row = S + size_t(m / T) * nt;
  const float4* x_row = X + size_t(m) * n4;
  float4* y_row = Y + size_t(m) * n4;
  const int base = blockIdx.x * (THREADS * UNROLL) + threadIdx.x;
  float4 v[UNROLL];
#pragma unroll
  for (int j = 0; j < UNROLL; ++j) {
    const int c = base + j * THREADS;
    if (c < n4) v[j] = __ldcs(x_row + c);
  }
#pragma unroll
  for (int j = 0; j < UNROLL; ++j) {
    const int c = base + j * THREADS;
    if (c < n4) {
      const float s = __ldg(s_row + (c * 4) / T);  // T % 4 == 0: one scale per float4
      v[j].x *= s;
      v[j].y *= s;
      v[j].z *= s;
      v[j].w *= s;
      __stcs(y_row + c, v[j]);
    }
  }
}

__global__ void __launch_bounds__(THREADS)
    rows_scalar_kernel(const float* __restrict__ X, const float* __restrict__ S,
                       float* __restrict__ Y, int N, int T, int nt, int m0) {
  const int m = m0 + blockIdx.y;
  const float* s_row = S + size_t(m / T) * nt;
  const float* x_row = X + size_t(m) * N;
  float* y_row = Y + size_t(m) * N;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < N; c += gridDim.x * blockDim.x)
    y_row[c] = x_row[c] * __ldg(s_row + c / T);
}

}  // namespace dq
}  // namespace texo

// X, S, Y are device pointers: X, Y [M,N]; S [ceil(M/T), ceil(N/T)], row-major FP32.
extern "C" void solve(const float* X, const float* S, float* Y, int M, int N, int T) {
  using namespace texo;
  using namespace texo::dq;
  if (M <= 0 || N <= 0 || T <= 0 || !X || !S || !Y) return;
  const int nt = (N + T - 1) / T;
  const bool vec = N % 4 == 0 && T % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(Y)) & 15) == 0;
  // gridDim.y is limited to 65535 rows per launch.
  const int slot = profile_start();
  for (int m0 = 0; m0 < M; m0 += 65535) {
    ++launch_counter();
    const int rows = M - m0 < 65535 ? M - m0 : 65535;
    if (vec) {
      const int n4 = N / 4;
      dim3 grid((n4 + THREADS * UNROLL - 1) / (THREADS * UNROLL), rows);
      rows_vec4_kernel<<<grid, THREADS>>>(reinterpret_cast<const float4*>(X), S,
                                          reinterpret_cast<float4*>(Y), n4, T, nt, m0);
    } else {
      dim3 grid(std::min((N + THREADS - 1) / THREADS, 64), rows);
      rows_scalar_kernel<<<grid, THREADS>>>(X, S, Y, N, T, nt, m0);
    }
  }
  profile_stop(slot);
}
