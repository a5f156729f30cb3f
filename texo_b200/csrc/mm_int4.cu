// W4A16 weight-only quantized matmul for B200 (sm_100a).
//
//   y[m,n] = fp16( sum_k x[m,k] * (q[n,k] - 8) * scales[n, k / G] )
//   q[n,2i] = w_q[n,i] >> 4,  q[n,2i+1] = w_q[n,i] & 15
//
// Drop-in for the operator of frezcirno/Texo src/mm_int4.cu:386-414: same
// `extern "C" void solve(x, w_q, scales, y, M, N, K, group_size)` symbol, FP16 x / scales /
// y, packed uint8 weights [N, K/2], device pointers, legacy default stream.  Results are
// accepted within atol = rtol = 0.01 of a double-precision reference (tests/mm_int4.cpp:10-11).
#include <algorithm>
#include <cstdint>
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"

namespace texo {
namespace w4 {

// -------------------------------------------------------------- generic path
// Any M, N, even K, any group size dividing K, any 2-byte aligned y.  FP32 SIMT tiles: the
// weight tile is expanded to (q - 8) * scale in shared memory, x to FP32.
constexpr int GT = 64, GK = 32, G_THREADS = 256;

__global__ void __launch_bounds__(G_THREADS)
    generic_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ w_q,
                   const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K,
                   int G) {
  __shared__ float xs[GK][GT + 1];
  __shared__ float ws[GK][GT + 1];
  const int t = threadIdx.x;
  const int row0 = blockIdx.y * GT, col0 = blockIdx.x * GT;
  const int ty = t / 16, tx = t % 16;
  const int groups = K / G;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += GK) {
    {
      // x: thread -> row t/4, eight k starting at (t%4)*8
      const int r = t / 4, kb = (t % 4) * 8;
      const int m = row0 + r;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int k = k0 + kb + e;
        xs[kb + e][r] = (m < M && k < K) ? __half2float(x[size_t(m) * K + k]) : 0.f;
      }
    }
    {
      // w: thread -> column t/4, four bytes (eight k) starting at byte (t%4)*4
      const int c = t / 4, bb = (t % 4) * 4;
      const int n = col0 + c;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = k0 + (bb + e) * 2;
        float hi = 0.f, lo = 0.f;
        if (n < N && k < K) {
          const int byte = w_q[size_t(n) * (K / 2) + k / 2];
          hi = float((byte >> 4) - 8) * __half2float(scales[size_t(n) * groups + k / G]);
          lo = float((byte & 15) - 8) * __half2float(scales[size_t(n) * groups + (k + 1) / G]);
        }
        ws[(bb + e) * 2][c] = hi;
        ws[(bb + e) * 2 + 1][c] = lo;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = row0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = col0 + tx * 4 + j;
      if (n < N) y[size_t(m) * N + n] = __float2half_rn(acc[i][j]);
    }
  }
}

inline int& last_path() {
  static int path = 0;
  return path;
}

}  // namespace w4
}  // namespace texo

// x, w_q, scales, y are device pointers: x [M,K] fp16, w_q [N,K/2] u8, scales [N,K/G] fp16,
// y [M,N] fp16.
extern "C" void solve(const __half* x, const uint8_t* w_q, const __half* scales, __half* y, int M,
                      int N, int K, int group_size) {
  using namespace texo;
  using namespace texo::w4;
  if (M <= 0 || N <= 0) return;
  if (K < 0 || (K & 1) || group_size <= 0 || (K % group_size) != 0 || !y ||
      (K > 0 && (!x || !w_q || !scales))) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  const int slot = profile_start();
  generic_kernel<<<grid, G_THREADS>>>(x, w_q, scales, y, M, N, K, group_size);
  profile_stop(slot);
  ++launch_counter();
  last_path() = 1;
}

extern "C" int texo_mm_int4_last_path(void) { return texo::w4::last_path(); }
extern "C" int texo_mm_int4_status(void) { return texo::read_and_clear_status(); }
