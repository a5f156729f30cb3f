// Packed-weight stream shared by the two decode kernels (w4_decode.cuh: FP16 activations,
// w4a8_decode.cuh: INT8 activations).
//
// Both kernels are bound by how fast the packed INT4 weights w_q [N, K/2] arrive from HBM, and
// an SM needs on the order of 100 KiB in flight to cover the memory latency at its share of the
// bandwidth.  Registers cannot hold that much, so the weights take one hop through shared
// memory - in their PACKED form, half a byte per weight, written once by TMA and read once
// into registers by the lanes that own them: a producer warp keeps a ring of W_RING_BYTES
// filled with 2-D TMA boxes (32 weight rows x 64 bytes = one row group's 128 k), a stage per
// (128-k block, k part of the CTA); the consumer warps of that k part wait on the stage's
// barrier, copy their 16-byte pieces to registers (row-major 64-byte rows: the four lanes of a
// quad read 64 consecutive bytes, a quarter-warp 128: no bank conflicts) and release the
// stage at once, before they compute.  Rows past N are zero-filled by TMA.  Waits are bounded.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace texo {
namespace w4s {

constexpr int W_CONSUMER_WARPS = 16;
constexpr int W_THREADS = (W_CONSUMER_WARPS + 1) * 32;  // + the producer warp
constexpr int W_RING_BYTES = 128 * 1024;
constexpr int W_MAX_STAGES = 16;
constexpr int W_GROUP_BYTES = 32 * 64;  // one row group's 128 k, packed

struct StreamBarriers {
  uint64_t full[W_MAX_STAGES];
  uint64_t empty[W_MAX_STAGES];
  int abort_flag;
};

__host__ __device__ inline int stream_stages(int rowgroups) {
  const int n = W_RING_BYTES / (rowgroups * W_GROUP_BYTES);
  return n < W_MAX_STAGES ? n : W_MAX_STAGES;
}

// Consumers only (the producer warp never joins): barrier 1 over the 512 consumer threads.
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

__device__ __forceinline__ void stream_init(StreamBarriers* bars, int stages, int rowgroups) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], rowgroups);  // one arrival per consumer warp of the stage's k part
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
}

// The producer warp's whole job.  Stage s = (128-k block s / ksplit, k part s % ksplit).
__device__ __forceinline__ void stream_produce(const CUtensorMap* map_w, uint8_t* ring, StreamBarriers* bars,
                                               int stages, int rowgroups, int ksplit, int iters,
                                               int part_k, int n_cta, int* status) {
  if (threadIdx.x % 32 != 0) return;
  volatile int* abort_flag = &bars->abort_flag;
  const int total = iters * ksplit;
  const int stage_bytes = rowgroups * W_GROUP_BYTES;
  for (int s = 0; s < total; ++s) {
    const int slot = s % stages;
    if (s >= stages &&
        !mbar_wait(&bars->empty[slot], ((s / stages) - 1) & 1, abort_flag, status, STATUS_TIMEOUT_EMPTY))
      return;
    const int it = s / ksplit, part = s % ksplit;
    mbar_arrive_expect_tx(&bars->full[slot], uint32_t(stage_bytes));
    uint8_t* dst = ring + slot * stage_bytes;
    const int x = part * (part_k / 2) + it * 64;  // byte offset in the packed rows (a multiple of 16)
    for (int g = 0; g < rowgroups; ++g)
      tma_load_2d(dst + g * W_GROUP_BYTES, map_w, &bars->full[slot], x, n_cta + g * 32);
  }
}

// A consumer warp's view of one stage: waits for it, copies this lane's four 16-byte pieces
// (tile t: row 8t + r of the warp's row group, bytes 16j..16j+15) and releases the stage.
// Returns false if the wait gave up.
__device__ __forceinline__ bool stream_take(uint8_t* ring, StreamBarriers* bars, int stages, int rowgroups,
                                            int ksplit, int it, int part, int rg, int r, int j,
                                            uint4 (&w)[4], int* status) {
  const int s = it * ksplit + part;
  const int slot = s % stages;
  bool ok = mbar_wait(&bars->full[slot], (s / stages) & 1, &bars->abort_flag, status, STATUS_TIMEOUT_FULL);
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) return false;
  const uint8_t* base = ring + slot * (rowgroups * W_GROUP_BYTES) + rg * W_GROUP_BYTES + r * 64 + j * 16;
#pragma unroll
  for (int t = 0; t < 4; ++t) w[t] = *reinterpret_cast<const uint4*>(base + t * 8 * 64);
  __syncwarp();
  if (threadIdx.x % 32 == 0) mbar_arrive(&bars->empty[slot]);
  return true;
}

}  // namespace w4s
}  // namespace texo
