// Host-buffer entry point for mm_int8 (libtexo_b200.so only).
//
// The reference harness wraps `solve` in synchronous uploads and a download
// (tests/mm_int8.cpp:56-79 of frezcirno/Texo).  This call does the same job for a caller
// whose operands live in host memory, but as a pipeline: B is uploaded once, A in row
// chunks; the kernel for chunk i runs as soon as its rows have landed, and its rows of C
// stream back while chunk i+1 is being uploaded and computed.  With pinned host buffers the
// call is bound by the slower PCIe direction instead of the sum of both plus the compute.
// No counterpart in the reference.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "host_common.h"

extern "C" void texo_mm_int8_solve(const int8_t*, const int8_t*, int8_t*, int, int, int, float, float,
                                   float, int, int, int);

namespace texo {
namespace hostapi {

constexpr int MAX_CHUNKS = 16;

struct Pipeline {
  bool ready = false;
  cudaStream_t up = nullptr, down = nullptr;  // non-blocking copy streams
  cudaEvent_t entry = nullptr, done = nullptr, landed[MAX_CHUNKS] = {}, computed[MAX_CHUNKS] = {};
  void* staging = nullptr;
  size_t staging_bytes = 0;
};

static Pipeline* pipeline() {
  static Pipeline table[MAX_DEVICES];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return nullptr;
  Pipeline& p = table[device];
  if (!p.ready) {
    bool ok = cudaStreamCreateWithFlags(&p.up, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p.down, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&p.entry, cudaEventDisableTiming) == cudaSuccess &&
              cudaEventCreateWithFlags(&p.done, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok && i < MAX_CHUNKS; ++i)
      ok = cudaEventCreateWithFlags(&p.landed[i], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&p.computed[i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
      cudaGetLastError();
      return nullptr;
    }
    p.ready = true;
  }
  return &p;
}

}  // namespace hostapi
}  // namespace texo

// A [M,K], B [K,N], C [M,N] are HOST pointers (pinned memory for full speed; pageable memory
// works but serialises).  Same arithmetic and arguments as texo_mm_int8_solve.  Asynchronous:
// returns once everything is enqueued; C_host is valid after cudaDeviceSynchronize() (or after
// any later default-stream work has completed: the default stream is made to wait for the
// last download).  Returns 0, -1 for invalid arguments, -3 for a CUDA failure.
extern "C" int texo_mm_int8_solve_host(const int8_t* A_host, const int8_t* B_host, int8_t* C_host,
                                       int M, int N, int K, float scale_A, float scale_B,
                                       float scale_C, int zero_point_A, int zero_point_B,
                                       int zero_point_C) {
  using namespace texo;
  using namespace texo::hostapi;
  if (M <= 0 || N <= 0 || K < 0 || !C_host || (K > 0 && (!A_host || !B_host))) return -1;
  Pipeline* p = pipeline();
  if (!p) return -3;
  const size_t a_bytes = (size_t(M) * K + 255) & ~size_t(255);
  const size_t b_bytes = (size_t(K) * N + 255) & ~size_t(255);
  const size_t c_bytes = size_t(M) * N;
  const size_t need = a_bytes + b_bytes + c_bytes;
  if (need > p->staging_bytes) {
    cudaDeviceSynchronize();  // earlier calls may still be using the old staging buffer
    if (p->staging) cudaFree(p->staging);
    p->staging = nullptr;
    p->staging_bytes = 0;
    if (cudaMalloc(&p->staging, need) != cudaSuccess) {
      cudaGetLastError();
      return -3;
    }
    p->staging_bytes = need;
  }
  int8_t* dA = static_cast<int8_t*>(p->staging);
  int8_t* dB = dA + a_bytes;
  int8_t* dC = dB + b_bytes;

  // Row chunks: multiples of 256 rows (whole pair tiles), at most MAX_CHUNKS, about eight.
  int rows = std::max(256, ((M + 7) / 8 + 255) / 256 * 256);
  while ((M + rows - 1) / rows > MAX_CHUNKS) rows += 256;
  const int chunks = (M + rows - 1) / rows;

  // The staging buffers may still be read by kernels of an earlier call on the default stream.
  cudaEventRecord(p->entry, 0);
  cudaStreamWaitEvent(p->up, p->entry, 0);
  if (K > 0) cudaMemcpyAsync(dB, B_host, size_t(K) * N, cudaMemcpyHostToDevice, p->up);
  for (int i = 0; i < chunks; ++i) {
    const int r0 = i * rows, nr = std::min(rows, M - r0);
    if (K > 0)
      cudaMemcpyAsync(dA + size_t(r0) * K, A_host + size_t(r0) * K, size_t(nr) * K,
                      cudaMemcpyHostToDevice, p->up);
    cudaEventRecord(p->landed[i], p->up);
  }
  for (int i = 0; i < chunks; ++i) {
    const int r0 = i * rows, nr = std::min(rows, M - r0);
    cudaStreamWaitEvent(0, p->landed[i], 0);
    texo_mm_int8_solve(K > 0 ? dA + size_t(r0) * K : nullptr, K > 0 ? dB : nullptr,
                       dC + size_t(r0) * N, nr, N, K, scale_A, scale_B, scale_C, zero_point_A,
                       zero_point_B, zero_point_C);
    cudaEventRecord(p->computed[i], 0);
    cudaStreamWaitEvent(p->down, p->computed[i], 0);
    cudaMemcpyAsync(C_host + size_t(r0) * N, dC + size_t(r0) * N, size_t(nr) * N,
                    cudaMemcpyDeviceToHost, p->down);
  }
  cudaEventRecord(p->done, p->down);
  cudaStreamWaitEvent(0, p->done, 0);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
