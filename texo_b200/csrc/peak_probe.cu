// INT8 tensor-pipe ceiling probe for B200: how fast does tcgen05.mma kind::i8 retire when
// nothing else limits it?  Operands stay resident in shared memory (filled once with
// pseudo-random bytes, so the data toggles like real inputs), no TMA, no epilogue: one
// thread per SM (or per SM pair) issues 128x256x32 (or 256x256x32 pair) MMAs back to back.
// The measured rate - under the same power cap as the real kernels - is the denominator
// the benchmark quotes next to the nominal figure.  No counterpart in the reference.
#include <algorithm>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace texo {
namespace probe {

constexpr int A_BYTES = 128 * 128;        // 128 rows x 128 k-bytes (four k=32 slices)
constexpr int B_BYTES_SINGLE = 128 * 256; // 128 k-rows x 256 columns
constexpr int B_BYTES_PAIR = 128 * 128;   // this CTA's half of the columns
constexpr int BATCH = 64;                 // MMAs per commit
constexpr int THREADS = 128;

struct ProbeBarriers {
  uint64_t done[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int CTAS, bool F16>
__global__ void __launch_bounds__(THREADS, 1) issue_kernel(int batches, int per_commit, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int B_BYTES = CTAS == 2 ? B_BYTES_PAIR : B_BYTES_SINGLE;
  ProbeBarriers* bars = reinterpret_cast<ProbeBarriers*>(smem + A_BYTES + B_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = CTAS == 2 ? cluster_ctarank() : 0;

  // pseudo-random operand bytes
  uint32_t* words = reinterpret_cast<uint32_t*>(smem);
  for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 4; i += THREADS) {
    uint32_t x = (blockIdx.x * 2654435761u) ^ (i * 0x9E3779B9u);
    x ^= x >> 15;
    x *= 0x85EBCA6Bu;
    x ^= x >> 13;
    words[i] = x;
  }
  if (threadIdx.x == 0) {
    mbar_init(&bars->done[0], 1);
    mbar_init(&bars->done[1], 1);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    if (CTAS == 2) {
      tmem_alloc_pair(&bars->tmem_base, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&bars->tmem_base, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0 && rank == 0) {
    // int8: A K-major, B N-major (as the INT8 kernels); f16: both K-major (as the W4A16 kernel)
    constexpr uint32_t IDESC = F16 ? umma_idesc(1, 0, 0, 0, 0, CTAS == 2 ? 256 : 128, 256)
                                   : umma_idesc(2, 1, 1, 0, 1, CTAS == 2 ? 256 : 128, 256);
    const uint32_t sa = smem_u32(smem), sb = sa + A_BYTES;
    bool ok = true;
    for (int b = 0; b < batches && ok; ++b) {
      if (lane == 0) {
        // keep at most two batches in flight
        if (b >= 2)
          ok = mbar_wait(&bars->done[b & 1], ((b >> 1) - 1) & 1, abort_flag, status,
                         STATUS_TIMEOUT_FULL);
        if (ok) {
          tc_fence_after_sync();
#pragma unroll 4
          for (int i = 0; i < per_commit; ++i) {
            const int j = i & 3;
            const uint64_t da = smem_desc(sa + j * 32, 16, 1024, SMEM_SWIZZLE_128B);
            const uint64_t db = F16 ? smem_desc(sb + j * 32, 16, 1024, SMEM_SWIZZLE_128B)
                                    : smem_desc(sb + j * 32 * 128, 128 * 128, 1024, SMEM_SWIZZLE_128B);
            const uint32_t d = tmem_base + ((i >> 2) & 1) * 256;
            if (F16) {
              if (CTAS == 2)
                umma_f16_pair(d, da, db, IDESC, 1);
              else
                umma_f16(d, da, db, IDESC, 1);
            } else if (CTAS == 2) {
              umma_i8_pair(d, da, db, IDESC, 1);
            } else {
              umma_i8(d, da, db, IDESC, 1);
            }
          }
          if (CTAS == 2)
            umma_commit_pair(&bars->done[b & 1], 1);
          else
            umma_commit(&bars->done[b & 1]);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    // drain: wait for the last two batches
    if (lane == 0 && ok) {
      for (int b = max(0, batches - 2); b < batches && ok; ++b)
        ok = mbar_wait(&bars->done[b & 1], (b >> 1) & 1, abort_flag, status, STATUS_TIMEOUT_FULL);
    }
    __syncwarp();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();
  if (warp == 0) {
    tc_fence_after_sync();
    if (CTAS == 2)
      tmem_dealloc_pair(tmem_base, 512);
    else
      tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- operand feed probe
// Streams the operand boxes of a 256 x 256-pair-tile INT8 GEMM through a shared-memory ring
// with TMA and throws them away: the rate at which L2 can feed all SMs with exactly the
// access pattern of the tensor kernel (A box 128 rows x 128 B, B box 128 k-rows x 128 B per
// CTA and k block; CTA 2i and 2i+1 share a pair tile).  mode bit 0 = load A, bit 1 = load B.
constexpr int F_BOX = 128 * 128;
struct FeedBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  int abort_flag;
};
__global__ void __launch_bounds__(64, 1)
    feed_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                int tiles_m, int tiles_n, int num_kb, int stages, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  FeedBarriers* bars = reinterpret_cast<FeedBarriers*>(smem + stages * 2 * F_BOX);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const int pair = blockIdx.x / 2, rank = blockIdx.x % 2, num_pairs = gridDim.x / 2;
  const int num_tiles = tiles_m * tiles_n;
  const uint32_t bytes = ((mode & 1) ? F_BOX : 0) + ((mode & 2) ? F_BOX : 0);
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  if (lane == 0) {
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
      const int group_tiles = 8 * tiles_n;
      const int first_m = tile / group_tiles * 8;
      const int group_m = min(tiles_m - first_m, 8);
      const int tm = first_m + (tile % group_tiles) % group_m, tn = (tile % group_tiles) / group_m;
      const int m0 = tm * 256 + rank * 128, n0 = tn * 256 + rank * 128;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (warp == 0) {
          ok = mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY);
          if (ok) {
            uint8_t* sa = smem + stage * 2 * F_BOX;
            mbar_arrive_expect_tx(&bars->full[stage], bytes);
            if (mode & 1) tma_load_2d(sa, &map_a, &bars->full[stage], kb * 128, m0);
            if (mode & 2) tma_load_2d(sa + F_BOX, &map_b, &bars->full[stage], n0, kb * 128);
          }
        } else {
          ok = mbar_wait(&bars->full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
          if (ok) mbar_arrive(&bars->empty[stage]);
        }
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  }
  __syncthreads();
}

}  // namespace probe
}  // namespace texo

#include "host_common.h"
// Streams A [M,K] and B [K,N] (device pointers, 16-byte aligned rows) once per pair tile as
// the tensor kernel would; returns the aggregate operand bytes per second in TB/s
// (negative on error).  stages in 1..7, mode bit 0 = A, bit 1 = B.  Synchronises.
extern "C" double texo_int8_feed_rate_tbs(const void* A, const void* B, int M, int N, int K,
                                          int stages, int mode) {
  using namespace texo;
  using namespace texo::probe;
  if (stages < 1 || stages > 7 || !(mode & 3)) return -1.0;
  int device = 0, sms = 0;
  cudaGetDevice(&device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  CUtensorMap map_a, map_b;
  if (!make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, K, 128, 128,
                          CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, K, N, N, 128, 128,
                          CU_TENSOR_MAP_SWIZZLE_128B))
    return -2.0;
  int* status = nullptr;
  if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) return -1.0;
  cudaMemset(status, 0, sizeof(int));
  const int smem = stages * 2 * F_BOX + 1024 + 256;
  cudaFuncSetAttribute(feed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256, num_kb = (K + 127) / 128;
  const int grid = std::min(2 * tiles_m * tiles_n, sms / 2 * 2);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0, 0);
  feed_kernel<<<grid, 64, smem>>>(map_a, map_b, tiles_m, tiles_n, num_kb, stages, mode, status);
  cudaEventRecord(e1, 0);
  double result = -1.0;
  if (cudaGetLastError() == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess) {
    float ms = 0.f;
    int code = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost);
    const double bytes = double(tiles_m) * tiles_n * num_kb * 2.0 *
                         (((mode & 1) ? F_BOX : 0) + ((mode & 2) ? F_BOX : 0));
    result = code ? -double(code) : bytes / (ms * 1e-3) / 1e12;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(status);
  return result;
}

// Runs the probe for `batches` x 64 MMAs per SM (pairs = 0) or per SM pair (pairs = 1) on the
// current device's default stream and returns the achieved rate in tera-ops per second
// (2 x MACs), or a negative value on error.  Synchronises.
extern "C" double texo_int8_issue_rate_tops(int pairs, int batches, int per_commit);
extern "C" double texo_int8_issue_ceiling_tops(int pairs, int batches) {
  return texo_int8_issue_rate_tops(pairs, batches, texo::probe::BATCH);
}
// Same measurement with `per_commit` MMAs between completion signals.  On B200 the rate
// falls off below eight MMAs per tcgen05.commit (four per commit: ~80 %), which is why the
// tensor kernel releases its stages two k blocks at a time.
static double issue_rate(int pairs, int batches, int per_commit, bool f16);
extern "C" double texo_int8_issue_rate_tops(int pairs, int batches, int per_commit) {
  return issue_rate(pairs, batches, per_commit, false);
}
// The same probe with kind::f16 MMAs (x16 k per instruction): tera-flops per second.
extern "C" double texo_f16_issue_rate_tflops(int pairs, int batches, int per_commit) {
  return issue_rate(pairs, batches, per_commit, true);
}
static double issue_rate(int pairs, int batches, int per_commit, bool f16) {
  using namespace texo;
  using namespace texo::probe;
  if (per_commit < 1 || per_commit > 1024 || batches < 1) return -1.0;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
    return -1.0;
  int* status = nullptr;
  if (cudaMalloc(&status, sizeof(int)) != cudaSuccess) return -1.0;
  cudaMemset(status, 0, sizeof(int));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  const int smem = A_BYTES + (pairs ? B_BYTES_PAIR : B_BYTES_SINGLE) + 1024 + 64;
  cudaError_t err;
  int grid = sms;
  if (pairs) {
    cudaFuncSetAttribute(issue_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(issue_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaLaunchConfig_t cfg = {};
    grid = sms / 2 * 2;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaEventRecord(e0, 0);
    err = f16 ? cudaLaunchKernelEx(&cfg, issue_kernel<2, true>, batches, per_commit, status)
              : cudaLaunchKernelEx(&cfg, issue_kernel<2, false>, batches, per_commit, status);
  } else {
    cudaFuncSetAttribute(issue_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaFuncSetAttribute(issue_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    cudaEventRecord(e0, 0);
    if (f16)
      issue_kernel<1, true><<<grid, THREADS, smem>>>(batches, per_commit, status);
    else
      issue_kernel<1, false><<<grid, THREADS, smem>>>(batches, per_commit, status);
    err = cudaGetLastError();
  }
  cudaEventRecord(e1, 0);
  double result = -1.0;
  if (err == cudaSuccess && cudaEventSynchronize(e1) == cudaSuccess) {
    float ms = 0.f;
    int code = 0;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaMemcpy(&code, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (code == 0 && ms > 0.f) {
      // every SM retires 128 x 256 x 32 (int8) or x 16 (f16) MACs per instruction in both modes
      const double macs = double(sms / (pairs ? 2 : 1) * (pairs ? 2 : 1)) * batches * double(per_commit) * 128.0 *
                          256.0 * (f16 ? 16.0 : 32.0);
      result = 2.0 * macs / (ms * 1e-3) / 1e12;
    } else if (code != 0) {
      result = -double(code);
    }
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(status);
  return result;
}
