// INT8 zero-point/scale quantized matmul for B200 (sm_100a).
//
//   C[m,n] = clamp(rint(float(sum_k (A[m,k]-zA)(B[k,n]-zB)) * sA * sB / sC) + zC, -128, 127)
//
// Drop-in for the operator of frezcirno/Texo src/mm_int8.cu:530-592: same
// `extern "C" void solve(...)` symbol, argument order (M, N, K), device pointers, legacy
// default stream, asynchronous, output fully overwritten.  The FP32 epilogue keeps the
// operation order of src/mm_int8.cu:12-25, which is what makes results bit-identical.
//
// Three device paths, chosen per call:
//   * tensor path  - persistent, warp-specialised tcgen05 kernel: TMA loads A (K-major) and B
//                    straight from its row-major [K,N] layout (an N-major UMMA operand, so no
//                    transposed copy of B is ever made), kind::i8 MMAs accumulate int32 in
//                    TMEM (two 128x256 accumulators, so the drain of tile i overlaps the
//                    MMAs of tile i+1), eight epilogue warps apply the zero-point identity
//                       sum (a-zA)(b-zB) = sum ab - zB*rowsum(A) - zA*colsum(B) + K*zA*zB
//                    and requantise.  Needs 16-byte aligned A/B and K % 16 == N % 16 == 0.
//   * skinny path  - M <= 128 (decode, small batches): HBM-bound; weights stream through the same TMA/UMMA
//                    machinery with the roles of the operands swapped (weights are the
//                    128-row operand, activations the narrow one) and the K range split over
//                    CTAs so all SMs pull on HBM; colsum(B) falls out of an extra all-ones
//                    activation row, so B is read exactly once.
//   * generic path - any shape, any byte alignment, K = 0, K >= 2^17: SIMT dp4a tiles with
//                    int64 totals.
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <type_traits>
#include <cuda.h>
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"
#include "requant.cuh"
#include "skinny.cuh"

namespace texo {
namespace i8 {

// -------------------------------------------------------------- generic path
constexpr int GT = 64;        // output tile edge
constexpr int GK = 64;        // k bytes per smem tile
constexpr int GKW = GK / 4;   // packed words per row
constexpr int G_THREADS = 256;
constexpr int G_FLUSH_TILES = 512;  // 512 * 64 = 2^15 k per int32 accumulation window

__global__ void __launch_bounds__(G_THREADS)
    generic_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B,
                   int8_t* __restrict__ C, int M, int N, int K, Quant q) {
  __shared__ int As[GT][GKW + 1];  // As[m][kw]: four consecutive k of row m
  __shared__ int Bs[GT][GKW + 1];  // Bs[n][kw]: four consecutive k of column n
  const int t = threadIdx.x;
  const int row0 = blockIdx.y * GT, col0 = blockIdx.x * GT;
  const int ty = t / 16, tx = t % 16;

  int acc[4][4] = {}, ra[4] = {}, cb[4] = {};
  long long tot[4][4] = {}, tra[4] = {}, tcb[4] = {};
  const int tiles_k = (K + GK - 1) / GK;
  int since_flush = 0;

  for (int kt = 0; kt < tiles_k; ++kt) {
    const int k0 = kt * GK;
    {
      // A: thread -> row t/4, sixteen k bytes starting at (t%4)*16
      const int r = t / 4, kb = (t % 4) * 16;
      const int m = row0 + r;
      const int8_t* src = A + size_t(m) * K + k0 + kb;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        unsigned word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int k = k0 + kb + w * 4 + e;
          const unsigned v = (m < M && k < K) ? uint8_t(src[w * 4 + e]) : 0u;
          word |= v << (8 * e);
        }
        As[r][kb / 4 + w] = int(word);
      }
    }
    {
      // B: thread -> four k rows (t/16)*4.., four columns (t%16)*4..
      const int kw = t / 16, nb = (t % 16) * 4;
      unsigned word[4] = {0, 0, 0, 0};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int k = k0 + kw * 4 + e;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = col0 + nb + j;
          const unsigned v = (k < K && n < N) ? uint8_t(B[size_t(k) * N + n]) : 0u;
          word[j] |= v << (8 * e);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) Bs[nb + j][kw] = int(word[j]);
    }
    __syncthreads();
#pragma unroll
    for (int kw = 0; kw < GKW; ++kw) {
      int a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[ty * 4 + i][kw];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[tx * 4 + j][kw];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ra[i] = __dp4a(a[i], 0x01010101, ra[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(a[i], b[j], acc[i][j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) cb[j] = __dp4a(b[j], 0x01010101, cb[j]);
    }
    __syncthreads();
    if (++since_flush == G_FLUSH_TILES || kt + 1 == tiles_k) {
      since_flush = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        tra[i] += ra[i];
        ra[i] = 0;
        tcb[i] += cb[i];
        cb[i] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tot[i][j] += acc[i][j];
          acc[i][j] = 0;
        }
      }
    }
  }

  const long long kza = (long long)K * q.za;
  const float zc = float(q.zc);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = row0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = col0 + tx * 4 + j;
      if (n >= N) continue;
      const float sb = q.sb_vec ? q.sb_vec[n] : q.sb;
      const long long zb = q.sb_vec ? (q.zb_vec ? q.zb_vec[n] : 0) + q.zb_bias : q.zb;
      const long long dot = tot[i][j] - zb * tra[i] - (long long)q.za * tcb[j] + kza * zb;
      const int8_t value = int8_t(requantize(float(dot), q.sa, sb, q.sc, zc));
      if (q.n_peers > 0) {
        for (int p = 0; p < q.n_peers; ++p) q.peers[p][size_t(m) * q.ldc + q.n_off + n] = value;
      } else {
        C[size_t(m) * N + n] = value;
      }
    }
  }
}

// ------------------------------------------------------------ sums pre-pass
// row_sum[m] = sum_k A[m,k] and col_sum[n] = sum_k B[k,n] for the zero-point identity, in ONE
// launch with plain stores (no atomics, nothing to clear beforehand).  One persistent block
// per SM walks a list of work items: first the column items (64 columns of B over the whole K
// range: 4 threads across x 128 k lanes, eight independent 16-byte loads in flight per
// thread, per-byte dp4a selectors, shuffles + a shared-memory tree over the k lanes), then the
// row items (16 rows of A, one warp per row).  The block is small enough (512 threads, 4 KiB
// of shared memory) to share an SM with a CTA of the tensor kernel: it signals
// launch_dependents at once, so a tensor kernel launched behind it with programmatic stream
// serialisation starts immediately and its first tile's MMAs run while the sums are still
// being computed; the tensor kernel's epilogue waits (griddepcontrol.wait) for this grid
// before it reads them.  Needs 16-byte aligned A / B and K % 16 == N % 16 == 0 (the tensor
// path's own preconditions).
constexpr int SUM_THREADS = 512;
constexpr int SUM_COLS = 64;
constexpr int SUM_TX = SUM_COLS / 16;             // threads across the columns
constexpr int SUM_KLANES = SUM_THREADS / SUM_TX;  // k lanes per block
constexpr int SUM_ROWS = SUM_THREADS / 32;        // rows per row item

__device__ __forceinline__ void add_bytes(int (&acc)[16], const int4& v) {
  const int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[i * 4 + 0] = __dp4a(w[i], 0x00000001, acc[i * 4 + 0]);
    acc[i * 4 + 1] = __dp4a(w[i], 0x00000100, acc[i * 4 + 1]);
    acc[i * 4 + 2] = __dp4a(w[i], 0x00010000, acc[i * 4 + 2]);
    acc[i * 4 + 3] = __dp4a(w[i], 0x01000000, acc[i * 4 + 3]);
  }
}

__global__ void __launch_bounds__(SUM_THREADS)
    sums_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B,
                int* __restrict__ row_sum, int* __restrict__ col_sum, int M, int N, int K,
                int col_items, int row_items) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ int part[SUM_THREADS / 32][SUM_COLS + 1];
  for (int item = blockIdx.x; item < col_items + row_items; item += gridDim.x) {
    if (item < col_items) {
      const int tx = threadIdx.x % SUM_TX, ty = threadIdx.x / SUM_TX;
      const int n = item * SUM_COLS + tx * 16;
      int acc[16] = {};
      if (n < N) {
        const int8_t* col = B + n;
        int k = ty;
        for (; k + 7 * SUM_KLANES < K; k += 8 * SUM_KLANES) {
          int4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            v[u] = __ldg(reinterpret_cast<const int4*>(col + size_t(k + u * SUM_KLANES) * N));
#pragma unroll
          for (int u = 0; u < 8; ++u) add_bytes(acc, v[u]);
        }
        for (; k < K; k += SUM_KLANES)
          add_bytes(acc, __ldg(reinterpret_cast<const int4*>(col + size_t(k) * N)));
      }
      // a warp holds 32 / SUM_TX k lanes of the same column chunks: fold them with shuffles
#pragma unroll
      for (int i = 0; i < 16; ++i) {
#pragma unroll
        for (int o = SUM_TX; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
      }
      __syncthreads();  // previous item's readers are done with `part`
      if (threadIdx.x % 32 < SUM_TX) {
#pragma unroll
        for (int i = 0; i < 16; ++i) part[threadIdx.x / 32][tx * 16 + i] = acc[i];
      }
      __syncthreads();
      if (threadIdx.x < SUM_COLS) {
        int total = 0;
#pragma unroll
        for (int r = 0; r < SUM_THREADS / 32; ++r) total += part[r][threadIdx.x];
        const int out = item * SUM_COLS + threadIdx.x;
        if (out < N) col_sum[out] = total;
      }
    } else {
      const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
      const int m = (item - col_items) * SUM_ROWS + warp;
      if (m < M) {
        const int4* a = reinterpret_cast<const int4*>(A + size_t(m) * K);
        const int chunks = K / 16;
        int acc = 0;
        int i = lane;
        for (; i + 7 * 32 < chunks; i += 8 * 32) {  // eight independent loads in flight
          int4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = __ldg(a + i + u * 32);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            acc = __dp4a(v[u].x, 0x01010101, acc);
            acc = __dp4a(v[u].y, 0x01010101, acc);
            acc = __dp4a(v[u].z, 0x01010101, acc);
            acc = __dp4a(v[u].w, 0x01010101, acc);
          }
        }
        for (; i < chunks; i += 32) {
          const int4 v = __ldg(a + i);
          acc = __dp4a(v.x, 0x01010101, acc);
          acc = __dp4a(v.y, 0x01010101, acc);
          acc = __dp4a(v.z, 0x01010101, acc);
          acc = __dp4a(v.w, 0x01010101, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) row_sum[m] = acc;
      }
    }
  }
}

// Launches the pre-pass for whichever sums the zero points require; returns whether a kernel
// was launched.  col_sum entries past N (the accumulator tile is 256 wide) are never written;
// the epilogue may read them for columns it then discards.
// `max_blocks` = number of SMs when the tensor kernel is going to run beside it (one
// persistent block per SM), 0 for one block per work item when it runs on its own.
static bool launch_sums(const int8_t* A, const int8_t* B, int* row_sum, int* col_sum, int M, int N,
                        int K, const Quant& q, int max_blocks) {
  const int col_items = q.za != 0 ? (N + SUM_COLS - 1) / SUM_COLS : 0;
  const int row_items = q.zb != 0 ? (M + SUM_ROWS - 1) / SUM_ROWS : 0;
  if (col_items + row_items == 0) return false;
  // Ask for the largest shared-memory carve-out although the kernel needs little: an SM can
  // only host a tensor-kernel CTA next to this block if it is already configured that way.
  // (function attributes are per device)
  static bool configured[MAX_DEVICES] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device >= 0 && device < MAX_DEVICES && !configured[device]) {
    cudaFuncSetAttribute(sums_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured[device] = true;
  }
  const int grid = max_blocks > 0 ? std::min(col_items + row_items, max_blocks) : col_items + row_items;
  sums_kernel<<<grid, SUM_THREADS>>>(A, B, row_sum, col_sum, M, N, K, col_items, row_items);
  if (cudaPeekAtLastError() != cudaSuccess) {
    cudaGetLastError();
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;
  }
  ++launch_counter();
  return true;
}

// --------------------------------------------------------------- tensor path
constexpr int BM = 128, BN = 256, BK = 128;  // CTA tile; BK bytes = one 128-byte swizzle row of A
constexpr int UMMA_K = 32;                   // K per kind::i8 instruction
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK;          // 16 KiB: 128 rows x 128 k-bytes
constexpr int B_BOX_BYTES = BK * 128;           // 16 KiB: 128 k-rows x 128 n-bytes
constexpr int B_STAGE_BYTES = B_BOX_BYTES * 2;  // two boxes side by side cover BN = 256
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int ACC_COLS = BN;  // TMEM columns per accumulator (int32 per column per lane)
constexpr int TMEM_COLS = 2 * ACC_COLS;
constexpr int EPI_WARPS = 8;
constexpr int MMA_THREADS = 64 + EPI_WARPS * 32;
constexpr int GROUP_M = 8;  // tile-row group walked column by column (L2 reuse)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct Barriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group_tiles = GROUP_M * tiles_n;
  const int first_m = tile / group_tiles * GROUP_M;
  const int group_m = min(tiles_m - first_m, GROUP_M);
  const int in_group = tile % group_tiles;
  tm = first_m + in_group % group_m;
  tn = in_group / group_m;
}

// WIDE = false: |dot| < 2^31 (K <= 33025), zero-point identity in wrapping 32-bit;
// WIDE = true: 64-bit.
template <bool WIDE>
__global__ void __launch_bounds__(MMA_THREADS, 1)
    umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                int8_t* __restrict__ C, const int* __restrict__ row_sum,
                const int* __restrict__ col_sum, int M, int N, int K, Quant q, int tiles_m,
                int tiles_n, int c_vector_ok, int* status) {
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B tiles want 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], EPI_WARPS);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY);
          if (ok) {
            uint8_t* sa = smem + stage * STAGE_BYTES;
            uint8_t* sb = sa + A_STAGE_BYTES;
            mbar_arrive_expect_tx(&bars->full[stage], STAGE_BYTES);
            tma_load_2d(sa, &map_a, &bars->full[stage], kb * BK, tm * BM);
            tma_load_2d(sb, &map_b, &bars->full[stage], tn * BN, kb * BK);
            tma_load_2d(sb + B_BOX_BYTES, &map_b, &bars->full[stage], tn * BN + 128, kb * BK);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // A: K-major, 128-byte swizzle: rows 128 B apart, 8-row groups 1024 B apart (SBO).
    // B: N-major, 128-byte swizzle: k rows 128 B apart, 8-row k groups 1024 B apart (SBO),
    //    the second 128-column box B_BOX_BYTES further on (LBO).
    constexpr uint32_t IDESC = umma_idesc(/*D=s32*/ 2, /*A=s8*/ 1, /*B=s8*/ 1, /*A K-major*/ 0,
                                          /*B N-major*/ 1, BM, BN);
    int stage = 0;
    uint32_t phase = 0;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      if (lane == 0) {
        ok = mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, status,
                       STATUS_TIMEOUT_TMEM_EMPTY);
        tc_fence_after_sync();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(&bars->full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
          if (ok) {
            tc_fence_after_sync();
            const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
            const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
            for (int j = 0; j < BK / UMMA_K; ++j) {
              const uint64_t da = smem_desc(sa + j * UMMA_K, 16, 1024, SMEM_SWIZZLE_128B);
              const uint64_t db =
                  smem_desc(sb + j * UMMA_K * 128, B_BOX_BYTES, 1024, SMEM_SWIZZLE_128B);
              umma_i8(tmem_d, da, db, IDESC, (kb | j) != 0);
            }
            umma_commit(&bars->empty[stage]);  // stage reusable once these MMAs have read it
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (lane == 0 && ok) umma_commit(&bars->acc_full[acc]);
      __syncwarp();
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int quarter = warp % 4;  // TMEM lanes this warp may read: 32*quarter .. +31
    const int half = ew / 4;       // which 128 of the 256 accumulator columns
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      ok = mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, status,
                     STATUS_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int m = tm * BM + quarter * 32 + lane;
      drain_half<WIDE>(tmem_base + acc * ACC_COLS + (uint32_t(quarter * 32) << 16), half * 128,
                       tn * BN, m, m < M, C, row_sum, col_sum, N, K, q, c_vector_ok);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------- sums inside the CTA-pair kernel
// The CTA-pair kernel needs no pre-pass: its eight epilogue warps compute rowsum(A) /
// colsum(B) themselves, in the time they would otherwise spend waiting for accumulators.  The
// work is cut into items (128 columns of B over all K, or 16 rows of A: the access pattern of
// sums_kernel; the bytes are the ones the TMA producer is pulling through L2 anyway), put in
// the order in which the tiles need them - the rows of the first raster group of tile rows, then
// the column items from left to right (the raster walks a group's tile rows column by column), then
// the remaining rows - and dealt round robin over all CTAs of the grid (position blockIdx.x,
// += gridDim.x).  Every finished item is published by storing the call's epoch number into
// its flag (the flags are never cleared: an epoch is used once).  Before it drains a tile an
// epilogue waits for exactly the flags of that tile's rows and columns - and while it waits,
// for them or for the accumulator, it keeps working through its own items, so a CTA only ever
// blocks when it has none left: no cycle of CTAs waiting for one another can form, and since
// all CTAs of the grid are resident at once (the grid never exceeds what the device holds)
// every item's owner is running.  The items the first wave of tiles needs are finished
// within the first few microseconds, long before the first accumulators are.
constexpr int ES_THREADS = EPI_WARPS * 32;                        // 256 epilogue threads
// Columns of a column item: 128, i.e. whole 128-byte lines of B per k row.  Measured on the
// stateless 8192^3 call (same box): 32 columns 406 us, 64 columns 400 us, 128 columns 394 us,
// 256 columns 396 us (items of 256 columns are few and long).  For K > 12288 the host asks for
// 64 columns: an item must stay shorter than the MMAs of a tile, or the drain behind it is late.
constexpr int ES_COLS = 128;                                      // widest column item
constexpr int ES_PART_BYTES = EPI_WARPS * (ES_COLS + 1) * 4;      // partials of a column item
// Shared memory of the epilogue warps behind the ring and the barriers: 64 bytes of decision
// words (aliased with nothing: warps read them while others have already gone on), then
//   plain call:   128 column sums per epilogue warp (4 KiB) | partials of a column item
//   fused gather: one 4 KiB staging tile per epilogue warp, whose first bytes double as the
//                 partials of a column item (inside an item all eight warps are between the
//                 same barriers, none of them drains)
constexpr int P_DECISION_BYTES = 64;
constexpr int P_COLSUM_SMEM_BYTES = EPI_WARPS * 512;
constexpr int P_AUX_SMEM_BYTES = P_DECISION_BYTES + P_COLSUM_SMEM_BYTES + ((ES_PART_BYTES + 127) & ~127);
constexpr int ES_FIRST_ROW_ITEMS = P_GROUP_M * 256 / SUM_ROWS;    // row items of the first raster group

constexpr int ES_ROW_THREADS = ES_THREADS / SUM_ROWS;             // threads per row of a row item
static_assert(ES_ROW_THREADS == 16, "a row item is sixteen rows by sixteen threads");

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }



// Position of a row / column item in the processing order described above.
__device__ __forceinline__ int pos_of_row_item(int i, int row_items, int col_items) {
  const int first = min(row_items, ES_FIRST_ROW_ITEMS);
  return i < first ? i : i + col_items;
}
__device__ __forceinline__ int pos_of_col_item(int c, int row_items) {
  return min(row_items, ES_FIRST_ROW_ITEMS) + c;
}

// One column item: colsum(B) of COLS columns over all K, by the 256 epilogue threads (COLS / 16
// threads across the columns, the rest along k; partials of the eight warps meet in `part`).
template <int COLS>
__device__ __forceinline__ void column_sum_item(int item, const int8_t* __restrict__ B, int* __restrict__ col_sum,
                                                int N, int K, int (*part)[ES_COLS + 1], int et) {
  constexpr int TX = COLS / 16, KLANES = ES_THREADS / TX;
  const int warp = et / 32, lane = et % 32;
  const int tx = et % TX, ty = et / TX;
  const int n = item * COLS + tx * 16;
  int acc[16] = {};
  if (n < N) {
    // (sixteen 16-byte loads in flight per thread: an item is bound by load latency under
    // the tensor kernel's own L2 traffic, not by the additions)
    const int8_t* col = B + n;
    int k = ty;
    for (; k + 15 * KLANES < K; k += 16 * KLANES) {
      int4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = __ldcs(reinterpret_cast<const int4*>(col + size_t(k + u * KLANES) * N));
#pragma unroll
      for (int u = 0; u < 16; ++u) add_bytes(acc, v[u]);
    }
    for (; k + 3 * KLANES < K; k += 4 * KLANES) {
      int4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(reinterpret_cast<const int4*>(col + size_t(k + u * KLANES) * N));
#pragma unroll
      for (int u = 0; u < 4; ++u) add_bytes(acc, v[u]);
    }
    for (; k < K; k += KLANES) add_bytes(acc, __ldcs(reinterpret_cast<const int4*>(col + size_t(k) * N)));
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
#pragma unroll
    for (int o = TX; o < 32; o <<= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  epilogue_bar();  // the previous item's readers are done with `part`
  if (lane < TX) {
#pragma unroll
    for (int i = 0; i < 16; ++i) part[warp][tx * 16 + i] = acc[i];
  }
  epilogue_bar();
  if (et < COLS) {
    int total = 0;
#pragma unroll
    for (int r = 0; r < EPI_WARPS; ++r) total += part[r][et];
    const int out = item * COLS + et;
    if (out < N) col_sum[out] = total;
  }
}

// Computes the item at position `pos` with the 256 epilogue threads of this CTA (`et` = index
// among them) and publishes it.  `col_cols` = columns per column item (64 or 128).
__device__ __forceinline__ void epilogue_sum_item(int pos, const int8_t* __restrict__ A,
                                                  const int8_t* __restrict__ B, int* __restrict__ row_sum,
                                                  int* __restrict__ col_sum, int M, int N, int K,
                                                  int col_items, int row_items, int col_cols,
                                                  int (*part)[ES_COLS + 1], int et, unsigned* flags,
                                                  unsigned epoch) {
  const int first_rows = min(row_items, ES_FIRST_ROW_ITEMS);
  const bool is_col = pos >= first_rows && pos < first_rows + col_items;
  if (is_col) {
    if (col_cols == 128)
      column_sum_item<128>(pos - first_rows, B, col_sum, N, K, part, et);
    else
      column_sum_item<64>(pos - first_rows, B, col_sum, N, K, part, et);
  } else {
    // sixteen threads per row, all sixteen rows at once: every load of a short row is in
    // flight before the first is used (a row of 1024 bytes is four loads per thread)
    const int item = pos < first_rows ? pos : pos - col_items;
    const int sub = et % ES_ROW_THREADS;
    const int m = item * SUM_ROWS + et / ES_ROW_THREADS;
    int acc = 0;
    if (m < M) {
      const int4* a = reinterpret_cast<const int4*>(A + size_t(m) * K);
      const int chunks = K / 16;
      int i = sub;
      for (; i + 15 * ES_ROW_THREADS < chunks; i += 16 * ES_ROW_THREADS) {
        int4 v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldcs(a + i + u * ES_ROW_THREADS);
#pragma unroll
        for (int u = 0; u < 16; ++u) acc = sum_bytes(v[u], acc);
      }
      for (; i + 3 * ES_ROW_THREADS < chunks; i += 4 * ES_ROW_THREADS) {
        int4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcs(a + i + u * ES_ROW_THREADS);
#pragma unroll
        for (int u = 0; u < 4; ++u) acc = sum_bytes(v[u], acc);
      }
      for (; i < chunks; i += ES_ROW_THREADS) acc = sum_bytes(__ldcs(a + i), acc);
    }
#pragma unroll
    for (int o = ES_ROW_THREADS / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (sub == 0 && m < M) row_sum[m] = acc;
  }
  // (the barrier orders every thread's stores before the release of the first thread, which is
  // cumulative over them: no fence per thread)
  epilogue_bar();
  if (et == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + pos), "r"(epoch) : "memory");
}

// Whether the sums this CTA's part of tile (tm, tn) needs are published: its 128 rows (eight
// row items) and the tile's 256 columns (two or four column items).  Called by one full warp.
__device__ __forceinline__ bool tile_sums_ready(int tm, int tn, int rank, int row_items, int col_items,
                                                int col_cols, const unsigned* flags, unsigned epoch, int lane) {
  int pos = -1;
  if (lane < 8) {
    const int i = (tm * 256 + rank * 128) / SUM_ROWS + lane;
    if (i < row_items) pos = pos_of_row_item(i, row_items, col_items);
  } else if (lane < 8 + 256 / col_cols) {
    const int c = tn * (256 / col_cols) + (lane - 8);
    if (c < col_items) pos = pos_of_col_item(c, row_items);
  }
  bool ready = true;
  if (pos >= 0) {
    unsigned seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + pos) : "memory");
    ready = seen == epoch;
  }
  return __all_sync(0xffffffffu, ready);
}

// ---------------------------------------------------- tensor path, CTA pairs
// Same pipeline with the MMA spanning two CTAs of a cluster (cta_group::2): pair tile
// 256 x 256, each CTA stages only its own 128 rows of A and its own 128 columns of B per
// k block (32 KiB instead of 48 KiB for the same 128 x 256 outputs per SM), which cuts the
// L2 -> SM operand stream and the shared-memory operand reads by a third and leaves room for
// a deeper ring.  The even CTA of the pair issues the MMAs; both CTAs drain their own 128
// accumulator rows from their own TMEM.
//
// Stage release: a tcgen05.commit costs the tensor pipe about as much time as five MMAs of
// this shape (measured: four MMAs per commit run at 80 % of the rate of eight per commit),
// so stages are not released one by one.  K blocks are numbered globally across the tiles a
// pair works through; one commit is issued after every even-numbered block and covers that
// block and its predecessor.  Commit number c arrives on ring[c % 4]; the producer, before it
// refills the stage of block g - P_STAGES, waits for the commit that covers that block.  The
// consumer can never be four commits ahead of what the producer has observed (the ring is
// six blocks deep), so the phase parity of ring[c % 4] is unambiguous.
constexpr int P_STAGES = 6;
constexpr int P_RING = 4;
constexpr int P_A_BYTES = BM * BK;   // 128 rows x 128 k-bytes
constexpr int P_B_BYTES = BK * 128;  // 128 k-rows x 128 n-bytes (this CTA's half of the columns)
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_GATHER_SMEM_BYTES = P_DECISION_BYTES + EPI_WARPS * 4096;  // staging tiles of the fused all-gather
static_assert(ES_PART_BYTES <= EPI_WARPS * 4096, "the partials of a column item must fit the staging tiles");
static_assert(P_SMEM_BYTES + P_GATHER_SMEM_BYTES <= 232448, "CTA-pair kernel: shared memory over the limit");

struct PairBarriers {
  uint64_t full[P_STAGES];  // used in the even CTA: bytes of both CTAs' loads
  uint64_t ring[P_RING];    // one set per CTA, signalled by the even CTA's MMA commits
  uint64_t acc_full[2];     // one per CTA, signalled by the even CTA's MMA commits
  uint64_t acc_empty[2];    // used in the even CTA: epilogue warps of both CTAs arrive
  uint32_t tmem_base;
  int abort_flag;
};

template <bool WIDE>
__global__ void __launch_bounds__(MMA_THREADS, 1)
    umma_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b, int8_t* __restrict__ C,
                     const int* __restrict__ row_sum, const int* __restrict__ col_sum, int M, int N,
                     int K, Quant q, int tiles_m, int tiles_n, int c_vector_ok, int* status,
                     const int8_t* __restrict__ A_raw, const int8_t* __restrict__ B_raw,
                     int* row_sum_w, int* col_sum_w, int col_items, int row_items,
                     unsigned* item_flags, unsigned epoch, int raster_rows, int col_cols) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + P_STAGES * P_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs)
  const int cluster_id = blockIdx.x / 2, num_clusters = gridDim.x / 2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;

  // The next grid in the stream may be scheduled from now on (it matters when that grid was
  // launched with programmatic stream serialisation, as this one is): its CTAs take the SMs
  // this grid's CTAs leave, set up their barriers and tensor memory, and wait in
  // griddepcontrol.wait until this grid has completed and its writes are visible.
  asm volatile("griddepcontrol.launch_dependents;");

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) mbar_init(&bars->full[s], 1);
    for (int r = 0; r < P_RING; ++r) mbar_init(&bars->ring[r], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2 * EPI_WARPS);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    int g = 0;          // global k-block number of the next load
    int observed = -1;  // highest commit number seen complete
    bool ok = true;
    // the operands may have been written by the grid ahead of this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tm, tn;
      pair_tile_coords(tile, tiles_m, tiles_n, raster_rows, tm, tn);
      const int m0 = tm * 256 + int(rank) * 128;
      const int n0 = tn * 256 + int(rank) * 128;
      for (int kb = 0; kb < num_kb && ok; ++kb, ++g) {
        if (lane == 0) {
          if (g >= P_STAGES) {
            const int c = (g - P_STAGES + 1) >> 1;  // commit covering block g - P_STAGES
            if (c > observed) {
              ok = mbar_wait(&bars->ring[c & (P_RING - 1)], (c >> 2) & 1, abort_flag, status,
                             STATUS_TIMEOUT_EMPTY);
              observed = c;
            }
          }
          if (ok) {
            uint8_t* sa = smem + stage * P_STAGE_BYTES;
            uint8_t* sb = sa + P_A_BYTES;
            const uint32_t full_even = map_to_cta(smem_u32(&bars->full[stage]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&bars->full[stage], 2 * P_STAGE_BYTES);
            tma_load_2d_pair(sa, &map_a, full_even, kb * BK, m0);
            tma_load_2d_pair(sb, &map_b, full_even, n0, kb * BK);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == P_STAGES) stage = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (even CTA only)
    if (rank == 0) {
      constexpr uint32_t IDESC = umma_idesc(/*D=s32*/ 2, /*A=s8*/ 1, /*B=s8*/ 1, /*A K-major*/ 0,
                                            /*B N-major*/ 1, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
      int g = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (lane == 0) {
          ok = mbar_wait_cluster(&bars->acc_empty[acc], acc_phase ^ 1, abort_flag, status,
                                 STATUS_TIMEOUT_TMEM_EMPTY);
          tc_fence_after_sync();
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++g) {
          if (lane == 0) {
            ok = mbar_wait(&bars->full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
            if (ok) {
              tc_fence_after_sync();
              const uint32_t sa = smem_u32(smem + stage * P_STAGE_BYTES);
              const uint32_t sb = sa + P_A_BYTES;
#pragma unroll
              for (int j = 0; j < BK / UMMA_K; ++j) {
                const uint64_t da = smem_desc(sa + j * UMMA_K, 16, 1024, SMEM_SWIZZLE_128B);
                const uint64_t db = smem_desc(sb + j * UMMA_K * 128, 16, 1024, SMEM_SWIZZLE_128B);
                umma_i8_pair(tmem_d, da, db, IDESC, (kb | j) != 0);
              }
              // releases this block's stage and its predecessor's, in both CTAs
              if ((g & 1) == 0) umma_commit_pair(&bars->ring[(g >> 1) & (P_RING - 1)], 3);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (++stage == P_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (lane == 0 && ok) umma_commit_pair(&bars->acc_full[acc], 3);
        __syncwarp();
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int quarter = warp % 4;
    const int half = ew / 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // Everything this kernel reads or writes may be in use by the grid ahead of it in the
    // stream until that grid has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Row / column sums: computed by the epilogue warps of all CTAs in the gaps of their own
    // work (see epilogue_sum_item above).  Decisions that steer all eight warps (they meet at
    // named barriers inside an item) are taken by the first of them and passed through shared
    // memory.
    const int et = threadIdx.x - 64;
    const int total_items = col_items + row_items;
    int next_item = blockIdx.x;  // this CTA's next position in the processing order
    uint8_t* const aux = smem + P_STAGES * P_STAGE_BYTES + 256;
    volatile int* decision = reinterpret_cast<volatile int*>(aux);
    const bool gathering = q.n_peers > 0;
    int(*part)[ES_COLS + 1] = reinterpret_cast<int(*)[ES_COLS + 1]>(
        aux + P_DECISION_BYTES + (gathering ? 0 : P_COLSUM_SMEM_BYTES));
    // 128 column sums per epilogue warp (plain calls), or a 4 KiB staging tile per warp (fused
    // all-gather; the host sizes the launch accordingly)
    int4* colsum_stage = gathering ? nullptr : reinterpret_cast<int4*>(aux + P_DECISION_BYTES) + ew * 32;
    uint8_t* gather_stage = gathering ? aux + P_DECISION_BYTES + ew * 4096 : nullptr;
    int round = 0;  // alternates the two decision words, so that one barrier per decision suffices
    int items_done = 0;
    if (next_item < total_items) {  // the first item needs no decision: nothing else can be ready yet
      epilogue_sum_item(next_item, A_raw, B_raw, row_sum_w, col_sum_w, M, N, K, col_items, row_items, col_cols,
                        part, et, item_flags, epoch);
      next_item += gridDim.x;
      ++items_done;
    }
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tm, tn;
      pair_tile_coords(tile, tiles_m, tiles_n, raster_rows, tm, tn);
      if (total_items > 0) {
        // Until the accumulator is complete AND this tile's sums are published.  The first two
        // items of a CTA (what the first waves of tiles need) are done at once; after that one
        // item per tile keeps ahead of the need (the order of the items is the order of need)
        // and spreads the extra memory traffic over the run instead of piling it onto the
        // first wave's own loads - except when this tile's sums are missing: then the CTA
        // works through its items without pause (it must never sit idle on a flag while it
        // still owes items to others).
        const long long start = clock64();
        bool item_this_tile = false;
        while (true) {
          if (ew == 0) {
            int d = 0;  // 0 = wait, 1 = go on to the drain, 2 = do an item, 3 = give up
            const bool acc_ready = mbar_try_wait(&bars->acc_full[acc], acc_phase);
            const bool sums_ready = tile_sums_ready(tm, tn, int(rank), row_items, col_items, col_cols, item_flags, epoch, lane);
            if (acc_ready && sums_ready) d = 1;
            else if (next_item < total_items && (items_done < 2 || !sums_ready || !item_this_tile)) d = 2;
            else if (*abort_flag) d = 3;
            else if (clock64() - start > WAIT_BUDGET_CLOCKS) {
              d = 3;
              *abort_flag = 1;
              if (status) atomicCAS(status, 0, acc_ready ? STATUS_TIMEOUT_FLAG : STATUS_TIMEOUT_TMEM_FULL);
            }
            if (lane == 0) decision[round & 1] = d;
          }
          epilogue_bar();
          const int d = decision[round & 1];
          ++round;
          if (d == 1) break;
          if (d == 3) {
            ok = false;
            break;
          }
          if (d == 2) {
            epilogue_sum_item(next_item, A_raw, B_raw, row_sum_w, col_sum_w, M, N, K, col_items, row_items,
                              col_cols, part, et, item_flags, epoch);
            next_item += gridDim.x;
            ++items_done;
            item_this_tile = true;
          } else {
            __nanosleep(100);
          }
        }
        if (!ok) break;
        __threadfence();
      }
      ok = mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int m = tm * 256 + int(rank) * 128 + quarter * 32 + lane;
      drain_half<WIDE>(tmem_base + acc * ACC_COLS + (uint32_t(quarter * 32) << 16), half * 128,
                       tn * 256, m, m < M, C, row_sum, col_sum, N, K, q, c_vector_ok, gather_stage,
                       colsum_stage);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->acc_empty[acc]), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // whatever is left of this CTA's share of the sums (other CTAs' later tiles wait for it; a
    // pair that owns no tile does all of its share here)
    while (ok && next_item < total_items) {
      epilogue_sum_item(next_item, A_raw, B_raw, row_sum_w, col_sum_w, M, N, K, col_items, row_items, col_cols,
                        part, et, item_flags, epoch);
      next_item += gridDim.x;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its partner may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ dispatch
// PATH_TENSOR = one-CTA tensor kernel, PATH_TENSOR_PAIR = CTA-pair tensor kernel (the
// automatic choice for M > 128).  Forcing PATH_TENSOR keeps the one-CTA kernel for any M.
enum Path { PATH_AUTO = 0, PATH_GENERIC = 1, PATH_TENSOR = 2, PATH_SKINNY = 3, PATH_TENSOR_PAIR = 4 };

inline int& forced_path() {
  static int path = [] {
    const char* env = std::getenv("TEXO_MM_INT8_PATH");
    return env ? std::atoi(env) : 0;
  }();
  return path;
}

inline int& last_path() {
  static int path = 0;
  return path;
}

static void launch_generic(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                           const Quant& q) {
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  const int slot = profile_start();
  generic_kernel<<<grid, G_THREADS>>>(A, B, C, M, N, K, q);
  profile_stop(slot);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}

static bool tensor_path_ok(const int8_t* A, const int8_t* B, int M, int N, int K) {
  (void)M;
  return K > 0 && K < (1 << 17) && K % 16 == 0 && N % 16 == 0 &&
         (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(B) & 15) == 0;
}

// Largest number of CTA pairs that can be resident at once (0 if pairs cannot be launched).
static int max_active_pairs(DeviceCtx& ctx) {
  static int cached[MAX_DEVICES] = {};
  static bool known[MAX_DEVICES] = {};
  if (!known[ctx.device]) {
    known[ctx.device] = true;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * ctx.sm_count);
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = P_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, umma_pair_kernel<false>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cached[ctx.device] = n;
  }
  return cached[ctx.device];
}

// Skinny (decode) path: M <= 128.
// The skinny path for this operator: runs the rowsum(A) pre-pass the kernel needs beyond 32
// rows (unless the caller already has the sums) and records the path.
static bool launch_skinny_i8(DeviceCtx& ctx, const int8_t* A, const int8_t* B, int8_t* C, int M, int N,
                             int K, const Quant& q, int weights_stable = 0,
                             const int* cached_row_sum = nullptr) {
  const int* row_sum = cached_row_sum;
  if (M > 32 && !row_sum && (q.zb != 0 || q.zb_vec != nullptr || (q.swiglu && q.z_up != 0))) {
    int* sums = static_cast<int*>(device_scratch(ctx, size_t(M) * sizeof(int) + 256));
    if (!sums) return false;
    Quant rows_only = q;
    rows_only.za = 0;
    rows_only.zb = 1;
    launch_sums(A, B, sums, nullptr, M, N, K, rows_only, 0);
    row_sum = sums;
  }
  if (!launch_skinny(ctx, A, B, C, M, N, K, q, weights_stable, row_sum)) return false;
  last_path() = PATH_SKINNY;
  return true;
}

// `cached_col_sum` (may be null): colsum(B) computed earlier for these weights, padded to a
// multiple of the 256-column tile; the pre-pass then only sums the rows of A.
static bool launch_tensor(DeviceCtx& ctx, const int8_t* A, const int8_t* B, int8_t* C, int M, int N,
                          int K, const Quant& q, int force, const int* cached_col_sum = nullptr,
                          const int* cached_row_sum = nullptr) {
  static bool configured[MAX_DEVICES] = {};
  if (!configured[ctx.device]) {
    cudaFuncSetAttribute(umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaFuncSetAttribute(umma_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         P_SMEM_BYTES + P_GATHER_SMEM_BYTES);
    cudaFuncSetAttribute(umma_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         P_SMEM_BYTES + P_GATHER_SMEM_BYTES);
    configured[ctx.device] = true;
  }
  // One TMA box shape serves both kernels: A 128 rows x 128 k-bytes, B 128 k-rows x 128 columns.
  CUtensorMap map_a, map_b;
  if (!make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, K, BM, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, K, N, N, BK, 128,
                          CU_TENSOR_MAP_SWIZZLE_128B)) {
    note_host_error(STATUS_TENSORMAP_FAILED);
    return false;
  }
  const int tiles_n = (N + BN - 1) / BN;
  const int np = tiles_n * BN;
  // Scratch: row_sum[M] | col_sum[np] (int32); one flag per sum item in an array of its own.
  const size_t row_bytes = (size_t(M) * 4 + 255) & ~size_t(255);
  int* row_sum = static_cast<int*>(device_scratch(ctx, row_bytes + size_t(np) * 4));
  if (!row_sum) return false;
  int* col_sum = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(row_sum) + row_bytes);
  unsigned* item_flags = device_item_flags(
      ctx, size_t((M + SUM_ROWS - 1) / SUM_ROWS + (N + 63) / 64) * sizeof(unsigned));
  if (!item_flags) return false;
  // 16-byte row stores need aligned rows of the output (H [M, N/2] in the SwiGLU form, FP16
  // [M, N] in the dequantising form)
  int c_vector_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
                    (q.swiglu ? (N / 2) % 16 == 0 : q.out_f16 ? N % 8 == 0 : N % 16 == 0);
  if (q.n_peers > 0) {
    c_vector_ok = q.ldc % 16 == 0 && q.n_off % 16 == 0;
    for (int p = 0; p < q.n_peers; ++p)
      c_vector_ok = c_vector_ok && (reinterpret_cast<uintptr_t>(q.peers[p]) & 15) == 0;
  }
  const int pairs = (force == PATH_TENSOR || (force != PATH_TENSOR_PAIR && M <= BM))
                        ? 0 : max_active_pairs(ctx);
  Quant sums_q = q;
  if (q.zb_vec || (q.swiglu && q.z_up != 0)) sums_q.zb = 1;  // the row sums are needed
  if (cached_col_sum) {
    sums_q.za = 0;  // nothing to do for the columns
    col_sum = const_cast<int*>(cached_col_sum);
  }
  if (cached_row_sum) {
    sums_q.zb = 0;  // rowsum(A) came with the activations (their producer computed it)
    row_sum = const_cast<int*>(cached_row_sum);
  }
  // The CTA-pair kernel computes the sums itself (its epilogue warps, during the first tile's
  // MMAs); the one-CTA kernel takes them from the pre-pass.
  if (pairs <= 0) launch_sums(A, B, row_sum, col_sum, M, N, K, sums_q, 0);
  const int slot = profile_start();
  if (pairs > 0) {
    const int tiles_m = (M + 255) / 256;
    // column items of 128 columns, unless K makes such an item longer than a tile's MMAs take
    const int col_cols = K <= 12288 ? 128 : 64;
    const int col_items = sums_q.za != 0 ? (N + col_cols - 1) / col_cols : 0;
    const int row_items = sums_q.zb != 0 ? (M + SUM_ROWS - 1) / SUM_ROWS : 0;
    // a finished item is marked with this call's epoch number: never zero, never used twice
    const unsigned epoch = next_sums_epoch(ctx);
    cudaLaunchConfig_t cfg = {};
    // One pair per tile up to what the device holds; a small problem gets extra pairs that own
    // no tile and only help with the sums (one item per CTA: an item is one memory round trip),
    // so that e.g. four tiles' worth of CTAs do not have to add up the whole of A and B by
    // themselves, one item after the other.
    const int helper_pairs = (col_items + row_items + 1) / 2;
    cfg.gridDim = dim3(2 * std::min(std::max(tiles_m * tiles_n, helper_pairs), pairs));
    cfg.blockDim = dim3(MMA_THREADS);
    cfg.dynamicSmemBytes = P_SMEM_BYTES + (q.n_peers > 0 ? P_GATHER_SMEM_BYTES : P_AUX_SMEM_BYTES);
    cfg.stream = 0;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 2;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    // may be scheduled while the grid ahead of it drains (the kernel waits in
    // griddepcontrol.wait before it touches memory)
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    const int* rs = row_sum;
    const int* cs = col_sum;
    const cudaError_t err =
        K <= 33025 ? cudaLaunchKernelEx(&cfg, umma_pair_kernel<false>, map_a, map_b, C, rs, cs, M, N, K, q,
                                        tiles_m, tiles_n, c_vector_ok, ctx.status, A, B, row_sum, col_sum,
                                        col_items, row_items, item_flags, epoch, raster_group_rows(K), col_cols)
                   : cudaLaunchKernelEx(&cfg, umma_pair_kernel<true>, map_a, map_b, C, rs, cs, M, N, K, q,
                                        tiles_m, tiles_n, c_vector_ok, ctx.status, A, B, row_sum, col_sum,
                                        col_items, row_items, item_flags, epoch, raster_group_rows(K), col_cols);
    if (err != cudaSuccess) {
      cudaGetLastError();
      profile_stop(slot);
      note_host_error(STATUS_LAUNCH_FAILED);
      return false;  // the caller falls back to the generic kernel
    }
    last_path() = PATH_TENSOR_PAIR;
  } else {
    const int tiles_m = (M + BM - 1) / BM;
    const int grid = std::min(tiles_m * tiles_n, ctx.sm_count);
    if (K <= 33025)
      umma_kernel<false><<<grid, MMA_THREADS, SMEM_BYTES>>>(map_a, map_b, C, row_sum, col_sum, M, N,
                                                           K, q, tiles_m, tiles_n, c_vector_ok,
                                                           ctx.status);
    else
      umma_kernel<true><<<grid, MMA_THREADS, SMEM_BYTES>>>(map_a, map_b, C, row_sum, col_sum, M, N,
                                                          K, q, tiles_m, tiles_n, c_vector_ok,
                                                          ctx.status);
    if (cudaPeekAtLastError() != cudaSuccess) {
      cudaGetLastError();
      profile_stop(slot);
      note_host_error(STATUS_LAUNCH_FAILED);
      return false;
    }
    last_path() = PATH_TENSOR;
  }
  profile_stop(slot);
  ++launch_counter();
  return true;
}

}  // namespace i8
}  // namespace texo

namespace texo {
namespace i8 {
// Dispatch shared by the per-tensor and the per-channel entry points.
static void solve_with(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                       const Quant& q) {
  if (M <= 0 || N <= 0) return;
  if (K < 0 || !C || (K > 0 && (!A || !B))) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  DeviceCtx& ctx = device_ctx();
  const int force = forced_path();
  const bool vectors_ok = (reinterpret_cast<uintptr_t>(q.sb_vec) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(q.zb_vec) & 15) == 0;
  if (force != PATH_GENERIC && ctx.cc_major >= 10 && vectors_ok && tensor_path_ok(A, B, M, N, K)) {
    // (with neither sum needed and more than 64 rows the one-CTA tensor kernel, which then
    // runs without a pre-pass, measured a little faster: 45 against 52 us at M = 128)
    const bool no_sums = q.za == 0 && q.zb == 0 && q.zb_vec == nullptr;
    if (M <= S_MAX_ROWS && (force == PATH_SKINNY || (force == PATH_AUTO && !(no_sums && M > 64))) &&
        launch_skinny_i8(ctx, A, B, C, M, N, K, q))
      return;
    if (launch_tensor(ctx, A, B, C, M, N, K, q, force)) return;
  }
  launch_generic(A, B, C, M, N, K, q);
}
}  // namespace i8
}  // namespace texo

// A, B, C are device pointers: A [M,K], B [K,N], C [M,N], row-major int8.
extern "C" void solve(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                      float scale_A, float scale_B, float scale_C, int zero_point_A,
                      int zero_point_B, int zero_point_C) {
  using namespace texo::i8;
  solve_with(A, B, C, M, N, K,
             make_quant(scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C, K));
}

namespace texo {
namespace i8 {
// Any shape / alignment for the fused SwiGLU form: one output per thread, int64 dots.
__global__ void __launch_bounds__(256)
    swiglu_generic_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B,
                          int8_t* __restrict__ H, int M, int F, int K, Quant q) {
  const int f = blockIdx.x * 16 + threadIdx.x % 16, m = blockIdx.y * 16 + threadIdx.x / 16;
  if (m >= M || f >= F) return;
  const int N = 2 * F;
  long long dg = 0, du = 0;
  for (int k = 0; k < K; ++k) {
    const int a = int(A[size_t(m) * K + k]) - q.za;
    dg += (long long)a * (int(B[size_t(k) * N + 2 * f]) - q.zb);
    du += (long long)a * (int(B[size_t(k) * N + 2 * f + 1]) - q.z_up);
  }
  const float gate = __fmul_rn(__fmul_rn(float(dg), q.sa), q.sb);
  const float up = __fmul_rn(__fmul_rn(float(du), q.sa), q.s_up);
  H[size_t(m) * F + f] = int8_t(swiglu_requantize(gate, up, q));
}
}  // namespace i8
}  // namespace texo

// Gate/up projection with the SwiGLU consumer fused into the TMEM drain.  B_gu [K, 2F] holds
// the gate and up weight columns interleaved (column 2j = gate j, column 2j+1 = up j), each
// with its own per-tensor scale and zero point; H [M, F] int8 =
//   clamp(rint(up * gate / (1 + exp(-gate)) / scale_H) + zero_point_H, -128, 127),
//   gate = float(dot_gate) * scale_A * scale_gate,  up = float(dot_up) * scale_A * scale_up.
// The [M, 2F] intermediate never exists in memory.
extern "C" void texo_mm_int8_swiglu_solve(const int8_t* A, const int8_t* B_gu, int8_t* H, int M, int F,
                                          int K, float scale_A, float scale_gate, float scale_up,
                                          float scale_H, int zero_point_A, int zero_point_gate,
                                          int zero_point_up, int zero_point_H) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || F <= 0) return;
  if (K < 0 || F > (1 << 30) || !H || (K > 0 && (!A || !B_gu))) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  Quant q = make_quant(scale_A, scale_gate, 1.0f, zero_point_A, zero_point_gate, 0, K);
  q.swiglu = 1;
  q.s_up = scale_up;
  q.s_out = scale_H;
  q.z_up = zero_point_up;
  q.z_out = zero_point_H;
  DeviceCtx& ctx = device_ctx();
  const int force = forced_path();
  const int N = 2 * F;
  if (force != PATH_GENERIC && ctx.cc_major >= 10 && tensor_path_ok(A, B_gu, M, N, K)) {
    // few activation rows: the streaming kernel (weights read once, gate/up pairs combined
    // between neighbouring lanes of its drain)
    if (M <= S_MAX_ROWS && (force == PATH_AUTO || force == PATH_SKINNY) &&
        launch_skinny_i8(ctx, A, B_gu, H, M, N, K, q))
      return;
    if (launch_tensor(ctx, A, B_gu, H, M, N, K, q, force == PATH_SKINNY ? PATH_AUTO : force)) return;
  }
  swiglu_generic_kernel<<<dim3((F + 15) / 16, (M + 15) / 16), 256>>>(A, B_gu, H, M, F, K, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}

namespace texo {
namespace i8 {
// Any shape / alignment for the dequantising form: one output per thread, int64 dot.
__global__ void __launch_bounds__(256)
    dequant_generic_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B,
                           __half* __restrict__ Y, int M, int N, int K, Quant q) {
  const int n = blockIdx.x * 16 + threadIdx.x % 16, m = blockIdx.y * 16 + threadIdx.x / 16;
  if (m >= M || n >= N) return;
  long long dot = 0;
  for (int k = 0; k < K; ++k)
    dot += (long long)(int(A[size_t(m) * K + k]) - q.za) * (int(B[size_t(k) * N + n]) - q.zb);
  Y[size_t(m) * N + n] = __float2half_rn(__fmul_rn(__fmul_rn(float(dot), q.sa), q.sb));
}
}  // namespace i8
}  // namespace texo

// INT8 matmul with a dequantising drain: Y [M,N] FP16 = half(float(dot) * scale_A * scale_B),
// dot = sum_k (A - zA)(B - zB) exact, FP32 multiplies in this order, one rounding to FP16.
// The int8 C and the separate dequantisation pass over it never exist.
extern "C" void texo_mm_int8_dequant_solve(const int8_t* A, const int8_t* B, void* Y, int M, int N,
                                           int K, float scale_A, float scale_B, int zero_point_A,
                                           int zero_point_B) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || N <= 0) return;
  if (K < 0 || !Y || (K > 0 && (!A || !B))) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  Quant q = make_quant(scale_A, scale_B, 1.0f, zero_point_A, zero_point_B, 0, K);
  q.out_f16 = 1;
  DeviceCtx& ctx = device_ctx();
  const int force = forced_path();
  if (force != PATH_GENERIC && ctx.cc_major >= 10 && tensor_path_ok(A, B, M, N, K)) {
    if (M <= S_MAX_ROWS && (force == PATH_AUTO || force == PATH_SKINNY) &&
        launch_skinny_i8(ctx, A, B, static_cast<int8_t*>(Y), M, N, K, q))
      return;
    if (launch_tensor(ctx, A, B, static_cast<int8_t*>(Y), M, N, K, q,
                      force == PATH_SKINNY ? PATH_AUTO : force))
      return;
  }
  dequant_generic_kernel<<<dim3((N + 15) / 16, (M + 15) / 16), 256>>>(A, B, static_cast<__half*>(Y),
                                                                    M, N, K, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}

// mm_int8 on this GPU's column slab of the weights with the all-gather of C fused into the
// drain.  C_all: HOST array of n_gpus DEVICE pointers, entry r = GPU r's copy of the full
// output [M, ld_c] (this process's own copy included; the others are peer mappings of the
// same allocation, e.g. from torch symmetric memory or CUDA IPC).  The call computes
// C[:, col_offset : col_offset + N_slab] = requantised A x B_slab and writes every finished
// piece into all n_gpus copies with plain stores, so when every GPU's call has completed (the
// caller synchronises them, e.g. with a barrier on the symmetric-memory handle) each copy holds
// the whole row-major C.  The kernel never waits for another GPU.
//
// texo_mm_int8_solve_allgather_multicast: the same with C_multicast, the NVLink multicast
// (NVLS) mapping of that allocation (torch symmetric memory: handle.multicast_ptr; cuMem:
// the address a multicast object is mapped at), or null.  With it, whole 128-byte row
// segments of the CTA-pair kernel's drain are written with ONE multimem.st that NVSwitch
// replicates into every copy; without it (and for ragged edges and the other kernels) every
// copy is written with its own store.  C_multicast must be 16-byte aligned and cover the same
// [M, ld_c] matrix as the entries of C_all.
extern "C" int texo_mm_int8_solve_allgather_multicast(
    const int8_t* A, const int8_t* B_slab, int8_t* const* C_all, int8_t* C_multicast, int n_gpus,
    int M, int N_slab, int K, int ld_c, int col_offset, float scale_A, float scale_B, float scale_C,
    int zero_point_A, int zero_point_B, int zero_point_C) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || N_slab <= 0) return 0;
  if (!C_all || n_gpus < 1 || n_gpus > MAX_PEERS || col_offset < 0 || ld_c < col_offset + N_slab ||
      (reinterpret_cast<uintptr_t>(C_multicast) & 15) != 0) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return -1;
  }
  Quant q = make_quant(scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C, K);
  q.n_peers = n_gpus;
  q.ldc = ld_c;
  q.n_off = col_offset;
  q.mc = C_multicast;
  for (int r = 0; r < n_gpus; ++r) {
    if (!C_all[r]) {
      note_host_error(STATUS_BAD_ARGUMENT);
      return -1;
    }
    q.peers[r] = C_all[r];
  }
  solve_with(A, B_slab, C_all[0], M, N_slab, K, q);
  return 0;
}

extern "C" int texo_mm_int8_solve_allgather(const int8_t* A, const int8_t* B_slab,
                                            int8_t* const* C_all, int n_gpus, int M, int N_slab,
                                            int K, int ld_c, int col_offset, float scale_A,
                                            float scale_B, float scale_C, int zero_point_A,
                                            int zero_point_B, int zero_point_C) {
  return texo_mm_int8_solve_allgather_multicast(A, B_slab, C_all, nullptr, n_gpus, M, N_slab, K, ld_c,
                                                col_offset, scale_A, scale_B, scale_C, zero_point_A,
                                                zero_point_B, zero_point_C);
}

// The same operator with one weight scale (and optionally one weight zero point) per output
// column: scale_B [N] FP32 and zero_point_B [N] int32 are DEVICE arrays; zero_point_B may be
// null (all zero).  Column n is requantised as float(dot) * scale_A * scale_B[n] / scale_C
// with dot = sum_k (A[m,k] - zA)(B[k,n] - zero_point_B[n]), in the same FP32 operation order.
extern "C" void texo_mm_int8_solve_per_channel(const int8_t* A, const int8_t* B, int8_t* C, int M,
                                               int N, int K, float scale_A, const float* scale_B,
                                               float scale_C, int zero_point_A,
                                               const int* zero_point_B, int zero_point_C) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || N <= 0) return;
  if (!scale_B) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  // The scalar fields stand for "a column inside the fast range"; the kernels check every
  // column's own scale and zero point before they take the branch-free division.
  Quant q = make_quant(scale_A, 1.0f, scale_C, zero_point_A, 0, zero_point_C, K);
  q.sb_vec = scale_B;
  q.zb_vec = zero_point_B;
  solve_with(A, B, C, M, N, K, q);
}

// --------------------------------------------------- per-group weight scales
// One weight scale per (scale group of `group_size` consecutive k, output column):
// scale_B [K / group_size, N] FP32 on the device (row g holds the scales of k in
// [g * group_size, (g + 1) * group_size)).  With dot_g the exact integer dot of group g,
//   acc = 0;  for g = 0, 1, ...:  acc = fma(RN(float(dot_g) * scale_A), scale_B[g, n], acc)
//   C[m, n] = clamp(rint(acc / scale_C) + zC, -128, 127)
// all in FP32, groups in ascending order.  With a single group (group_size == K) this is
// exactly the per-channel form ((float(dot) * sA) * sB[n]) / sC.  No counterpart in the
// reference (its mm_int8 is per-tensor, src/mm_int8.cu:533-535; its per-group handling is the
// FP16 path of src/mm_int4.cu:309-317).  This form runs on a SIMT kernel for every shape: a
// tensor-core path would have to drain the accumulator once per group, which tensor-memory
// bandwidth makes two to three times as expensive as the MMAs themselves at group_size = 128
// (measured on the W4A16 kernel), so it is left out rather than shipped slow and complex.
namespace texo {
namespace i8 {
__global__ void __launch_bounds__(256)
    per_group_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ B, int8_t* __restrict__ C,
                     int M, int N, int K, int G, const float* __restrict__ scale_B, Quant q) {
  __shared__ int8_t As[16][64 + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int n = blockIdx.x * 16 + tx, m = blockIdx.y * 16 + ty;
  float acc = 0.f;
  long long dot = 0;
  for (int k0 = 0; k0 < K; k0 += 64) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int r = i / 64, c = i % 64;
      const int mm = blockIdx.y * 16 + r, k = k0 + c;
      As[r][c] = (mm < M && k < K) ? A[size_t(mm) * K + k] : int8_t(0);
    }
    __syncthreads();
    if (n < N) {
      const int kend = min(64, K - k0);
      for (int c = 0; c < kend; ++c) {
        const int k = k0 + c;
        dot += (long long)(int(As[ty][c]) - q.za) * (int(B[size_t(k) * N + n]) - q.zb);
        if ((k + 1) % G == 0) {  // the group ends here
          const float t = __fmul_rn(float(dot), q.sa);
          acc = __fmaf_rn(t, scale_B[size_t(k / G) * N + n], acc);
          dot = 0;
        }
      }
    }
    __syncthreads();
  }
  if (m < M && n < N) {
    float v = __fdiv_rn(acc, q.sc);
    v = __fadd_rn(rintf(v), float(q.zc));
    C[size_t(m) * N + n] = int8_t(__float2int_rn(fminf(fmaxf(v, -128.f), 127.f)));
  }
}
}  // namespace i8
}  // namespace texo

extern "C" void texo_mm_int8_solve_per_group(const int8_t* A, const int8_t* B, int8_t* C, int M, int N,
                                             int K, int group_size, float scale_A, const float* scale_B,
                                             float scale_C, int zero_point_A, int zero_point_B,
                                             int zero_point_C) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || N <= 0) return;
  if (K <= 0 || group_size <= 0 || K % group_size != 0 || !A || !B || !C || !scale_B) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  const Quant q = make_quant(scale_A, 1.0f, scale_C, zero_point_A, zero_point_B, zero_point_C, K);
  per_group_kernel<<<dim3((N + 15) / 16, (M + 15) / 16), 256>>>(A, B, C, M, N, K, group_size, scale_B, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}

// ------------------------------------------------------------ prepared weights
// Inference calls the same weights with new activations again and again; colsum(B) depends
// on the weights only.  The reference recomputes it (together with a transposed copy of B)
// on every call (src/mm_int8.cu:559-561 of frezcirno/Texo).  These entry points compute it
// once per weight matrix and keep it with the handle, so a call only has to sum the rows of
// the new activations.  B must stay alive and unchanged while the handle is in use.
struct texo_int8_weights {
  const int8_t* B;
  int K, N, device;
  int* col_sum;  // [ceil(N/256)*256] on `device`, or null when the tensor path cannot take B
};

extern "C" texo_int8_weights* texo_mm_int8_prepare_weights(const int8_t* B, int K, int N) {
  using namespace texo;
  using namespace texo::i8;
  if (!B || K <= 0 || N <= 0) return nullptr;
  DeviceCtx& ctx = device_ctx();
  texo_int8_weights* w = new texo_int8_weights{B, K, N, ctx.device, nullptr};
  const bool aligned = K < (1 << 17) && K % 16 == 0 && N % 16 == 0 &&
                       (reinterpret_cast<uintptr_t>(B) & 15) == 0;
  if (ctx.cc_major >= 10 && aligned) {
    const size_t np = size_t((N + BN - 1) / BN) * BN;
    if (cudaMalloc(&w->col_sum, np * sizeof(int)) != cudaSuccess) {
      cudaGetLastError();
      w->col_sum = nullptr;
      return w;  // still usable: calls fall back to the stateless path
    }
    cudaMemsetAsync(w->col_sum, 0, np * sizeof(int), 0);
    Quant only_cols = {1.f, 1.f, 1.f, 1, 0, 0};
    launch_sums(nullptr, B, nullptr, w->col_sum, 0, N, K, only_cols, 0);
  }
  return w;
}

extern "C" void texo_mm_int8_release_weights(texo_int8_weights* w) {
  if (!w) return;
  if (w->col_sum) {
    cudaDeviceSynchronize();  // calls that still read the sums must finish first
    cudaFree(w->col_sum);
  }
  delete w;
}

static void solve_prepared_with(const int8_t* A, const int* row_sum_A, const texo_int8_weights* w,
                                int8_t* C, int M, float scale_A, float scale_B, float scale_C,
                                int zero_point_A, int zero_point_B, int zero_point_C);

// Same operation as `solve` with B, K, N taken from the handle.
extern "C" void texo_mm_int8_solve_prepared(const int8_t* A, const texo_int8_weights* w, int8_t* C,
                                            int M, float scale_A, float scale_B, float scale_C,
                                            int zero_point_A, int zero_point_B, int zero_point_C) {
  solve_prepared_with(A, nullptr, w, C, M, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                      zero_point_C);
}

// The same with rowsum(A) supplied by the caller: row_sum_A [M] int32 (device), row m holding
// sum_k A[m,k] - what texo_rms_norm_quant_solve writes next to the activations it produces.
// With both sums known beforehand a call is the tensor kernel alone, no pre-pass.  A null
// row_sum_A is texo_mm_int8_solve_prepared.
extern "C" void texo_mm_int8_solve_presummed(const int8_t* A, const int* row_sum_A,
                                             const texo_int8_weights* w, int8_t* C, int M,
                                             float scale_A, float scale_B, float scale_C,
                                             int zero_point_A, int zero_point_B, int zero_point_C) {
  solve_prepared_with(A, row_sum_A, w, C, M, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                      zero_point_C);
}

static void solve_prepared_with(const int8_t* A, const int* row_sum_A, const texo_int8_weights* w,
                                int8_t* C, int M, float scale_A, float scale_B, float scale_C,
                                int zero_point_A, int zero_point_B, int zero_point_C) {
  using namespace texo;
  using namespace texo::i8;
  if (!w || M <= 0) {
    if (!w) note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  DeviceCtx& ctx = device_ctx();
  const Quant q =
      make_quant(scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C, w->K);
  const int force = forced_path();
  if (w->col_sum && ctx.device == w->device && A && C && M > S_MAX_ROWS && force != PATH_GENERIC &&
      force != PATH_SKINNY && tensor_path_ok(A, w->B, M, w->N, w->K)) {
    if (launch_tensor(ctx, A, w->B, C, M, w->N, w->K, q, force, w->col_sum, row_sum_A)) return;
  }
  // Decode shapes get colsum(B) for free inside the skinny kernel; what the handle adds
  // there is the promise that B is unchanged, so the kernel may load weights before the
  // previous call on the stream has completed.
  if (ctx.device == w->device && A && C && M <= S_MAX_ROWS && ctx.cc_major >= 10 &&
      (force == PATH_AUTO || force == PATH_SKINNY) && tensor_path_ok(A, w->B, M, w->N, w->K) &&
      launch_skinny_i8(ctx, A, w->B, C, M, w->N, w->K, q, /*weights_stable=*/1, row_sum_A))
    return;
  // everything else is the stateless path
  solve(A, w->B, C, M, w->N, w->K, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
        zero_point_C);
}

// Diagnostics (declared in include/texo_b200.h).
extern "C" int texo_mm_int8_last_path(void) { return texo::i8::last_path(); }
extern "C" void texo_mm_int8_force_path(int path) { texo::i8::forced_path() = path; }
extern "C" int texo_mm_int8_status(void) { return texo::read_and_clear_status(); }

// ------------------------------------------------------- allocation-free entry
// Some callers must not trigger a device allocation once they are running: a serving
// process that has already handed all of HBM to its own pools (a late cudaMalloc from a
// library then simply fails), or a latency-critical loop that cannot accept the
// device-wide synchronisation cudaMalloc / cudaFree imply.  For them the tensor path is
// also offered with its scratch (row sums, column sums, status word) in a fixed array that
// is part of the loaded module instead of the grow-only cudaMalloc'd buffer `solve` uses.
// The price is a fixed ceiling on M and N and 256 KiB of device memory held by every GPU
// that loads the library, until the process exits.
namespace texo {
namespace i8 {

constexpr int NOALLOC_MAX_M = 32768;  // rows of A / C
constexpr int NOALLOC_MAX_N = 32768;  // columns of B / C (a multiple of the 256-column tile)
constexpr int NOALLOC_STATUS_WORDS = 64;
// Layout: row_sum[NOALLOC_MAX_M] | col_sum[NOALLOC_MAX_N] | status[64].  262,400 bytes.
static __device__ __align__(256) int noalloc_scratch[NOALLOC_MAX_M + NOALLOC_MAX_N +
                                                     NOALLOC_STATUS_WORDS];

struct NoAllocDevice {
  bool ready = false;
  int* scratch = nullptr;  // device address of noalloc_scratch on this device
  int sm_count = 0;
  int cc_major = 0;
};

// Once per device, with that device current: resolve the device address of the array (the
// name `noalloc_scratch` in host code is only a handle, never a device pointer), opt the
// kernels into their shared-memory sizes, and make the driver load the code of every kernel
// the entry point can launch.  With lazy module loading a kernel's code is brought onto the
// device at its first launch, which may take device memory; asking for each kernel's
// attributes here moves that cost into the set-up, so that later calls - whichever path
// their shapes and zero points select - find everything resident.  Returns nullptr on a
// CUDA error.
static NoAllocDevice* noalloc_device() {
  static NoAllocDevice table[MAX_DEVICES];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= MAX_DEVICES) return nullptr;
  NoAllocDevice& d = table[device];
  if (!d.ready) {
    void* address = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&address, noalloc_scratch);
    if (err != cudaSuccess || !address) {
      std::fprintf(stderr, "texo_b200: cudaGetSymbolAddress(noalloc_scratch) failed: %s\n",
                   cudaGetErrorString(err));
      cudaGetLastError();
      return nullptr;
    }
    d.scratch = static_cast<int*>(address);
    cudaFuncAttributes attr;
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess ||
        cudaFuncSetAttribute(umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(sums_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared) != cudaSuccess ||
        cudaFuncGetAttributes(&attr, sums_kernel) != cudaSuccess ||
        cudaFuncGetAttributes(&attr, generic_kernel) != cudaSuccess ||
        cudaFuncGetAttributes(&attr, umma_kernel<false>) != cudaSuccess ||
        cudaFuncGetAttributes(&attr, umma_kernel<true>) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    tensor_map_encoder();  // resolve the driver entry point now, not at the first tensor call
    d.ready = true;
  }
  return &d;
}

}  // namespace i8
}  // namespace texo

// Same operation and arguments as `solve`, but guaranteed to allocate nothing: no cudaMalloc,
// cudaFree or allocating library routine is called, on any call.  Returns 0 on success,
// -1 for invalid arguments, -2 when M or N exceeds the fixed scratch (M <= 32768,
// N <= 32768), -3 when the one-time device set-up failed.  Output is bit-identical to
// `solve`.  The first call on each device performs the set-up above, so make that call
// outside of any stream capture.  All calls share the one scratch array, which still holds
// the previous call's sums when the next one starts; nothing in it has to start at zero
// (every entry a call reads is first rewritten by that call's own pre-pass with plain
// stores, and the status word is only ever set, by a kernel that gave up, and cleared by
// texo_mm_int8_noalloc_status).  Two calls whose kernels overlap on the GPU (different host
// threads or streams) would race on the array - issue them one after another, as `solve`
// requires anyway.
extern "C" int texo_mm_int8_solve_noalloc(const int8_t* A, const int8_t* B, int8_t* C, int M, int N,
                                          int K, float scale_A, float scale_B, float scale_C,
                                          int zero_point_A, int zero_point_B, int zero_point_C) {
  using namespace texo;
  using namespace texo::i8;
  if (M <= 0 || N <= 0 || K < 0 || !C || (K > 0 && (!A || !B))) {
    std::fprintf(stderr, "texo_mm_int8_solve_noalloc: invalid arguments (M=%d N=%d K=%d)\n", M, N, K);
    return -1;
  }
  if (M > NOALLOC_MAX_M || N > NOALLOC_MAX_N) {
    std::fprintf(stderr,
                 "texo_mm_int8_solve_noalloc: M=%d N=%d exceeds the fixed scratch (M <= %d, N <= %d); "
                 "use solve() instead\n", M, N, NOALLOC_MAX_M, NOALLOC_MAX_N);
    return -2;
  }
  NoAllocDevice* dev = noalloc_device();
  if (!dev) return -3;
  const Quant q = make_quant(scale_A, scale_B, scale_C, zero_point_A, zero_point_B, zero_point_C, K);
  if (dev->cc_major >= 10 && tensor_path_ok(A, B, M, N, K)) {
    CUtensorMap map_a, map_b;
    if (make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, K, BM, BK,
                           CU_TENSOR_MAP_SWIZZLE_128B) &&
        make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, K, N, N, BK, 128,
                           CU_TENSOR_MAP_SWIZZLE_128B)) {
      const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
      int* row_sum = dev->scratch;
      int* col_sum = dev->scratch + NOALLOC_MAX_M;
      int* status = dev->scratch + NOALLOC_MAX_M + NOALLOC_MAX_N;
      // Every entry the main kernel uses is rewritten by plain stores here, so nothing in the
      // shared array has to be cleared first.
      launch_sums(A, B, row_sum, col_sum, M, N, K, q, 0);
      const int grid = std::min(tiles_m * tiles_n, dev->sm_count);
      const int c_vector_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && N % 16 == 0;
      if (K <= 33025)
        umma_kernel<false><<<grid, MMA_THREADS, SMEM_BYTES>>>(map_a, map_b, C, row_sum, col_sum, M,
                                                             N, K, q, tiles_m, tiles_n,
                                                             c_vector_ok, status);
      else
        umma_kernel<true><<<grid, MMA_THREADS, SMEM_BYTES>>>(map_a, map_b, C, row_sum, col_sum, M,
                                                            N, K, q, tiles_m, tiles_n,
                                                            c_vector_ok, status);
      ++launch_counter();
      last_path() = PATH_TENSOR;
      return 0;
    }
  }
  // Shapes the tensor path does not take need no scratch at all.
  generic_kernel<<<dim3((N + GT - 1) / GT, (M + GT - 1) / GT), G_THREADS>>>(A, B, C, M, N, K, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
  return 0;
}

// Error state of the allocation-free entry point on the current device, read without
// allocating anything (texo_mm_int8_status goes through the library's cudaMalloc'd status
// block and is therefore not for these callers).  The tensor kernel's waits are bounded; one
// that runs out records a code (1-5, see ptx.cuh) in the status word that lives at the end of
// the fixed scratch array and the kernel returns early, leaving C incomplete - the call
// itself had long returned 0.  This copies the word out (a blocking 4-byte copy: it waits for
// the calls issued so far), clears it if it was set, and returns it: 0 = every
// texo_mm_int8_solve_noalloc call since the last query ran to completion.  -3 when the
// device set-up failed.
extern "C" int texo_mm_int8_noalloc_status(void) {
  using namespace texo::i8;
  NoAllocDevice* dev = noalloc_device();
  if (!dev) return -3;
  int* word = dev->scratch + NOALLOC_MAX_M + NOALLOC_MAX_N;
  int code = 0;
  if (cudaMemcpy(&code, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
    cudaGetLastError();
    return -3;
  }
  if (code != 0) {
    const int zero = 0;
    cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice);
  }
  return code;
}
