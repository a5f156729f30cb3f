// Packed-INT4-weight x INT8-activation quantized matmul (W4A8) for B200 (sm_100a).
//
//   C[m,n] = clamp(rint(float(sum_k (A[m,k]-zA)(q[n,k]-zB)) * sA * sB / sC) + zC, -128, 127)
//   q[n,k] = (k even ? w_q[n,k/2] >> 4 : w_q[n,k/2] & 15) - 8
//
// A [M,K] int8 row-major, w_q [N,K/2] bytes in the nibble order of frezcirno/Texo
// src/mm_int4.cu:5-6,25-26 (high nibble = even k), C [M,N] int8 row-major; scales and zero
// points, rounding and clamping exactly as the INT8 operator (src/mm_int8.cu:12-25).  The
// reference has no such operator (its mm_int4 takes FP16 activations): this one combines
// the reference's INT4 weight format with its INT8 arithmetic, and is checked against an
// oracle built from those two pinned pieces.
//
// Tensor path: CTA pairs, 256 x 256 output tile, 128 k per stage.  Per stage and CTA: TMA
// brings 128 rows of A (16 KiB, K-major, 128-byte swizzle) and this CTA's 128 weight rows as
// packed nibbles (8 KiB); eight unpack warps expand the nibbles to bytes 0..15 directly into
// a K-major, 128-byte-swizzled operand tile (16 KiB); the even CTA issues
// tcgen05.mma.cta_group::2.kind::i8 with A signed and B UNSIGNED, accumulating int32 in TMEM.
// Keeping the nibbles unsigned makes the unpack five integer instructions per eight
// weights; the offset moves into the zero point:
//   sum (a-zA)(q-zB) = sum a*u - (zB+8)*rowsum(A) - zA*rowsum(u) + K*zA*(zB+8),   u = q + 8.
// The epilogue is the INT8 operator's TMEM drain (zero-point identity, requantisation,
// 32-byte row stores).  rowsum(A) and the nibble sums are computed inside the same kernel by
// its epilogue warps (one launch per call).
//
// Decode paths: M <= 16 (K a multiple of 128): a register-streaming mma.sync kernel
// (w4a8_decode.cuh); M <= 32: the INT8 operator's streaming kernel (skinny.cuh) in its
// packed-weight form - w_q crosses HBM once, four extra warps unpack it next to the tensor core.
// Generic path: any shape with even K, any alignment, K = 0: SIMT tiles with int64 totals.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"
#include "requant.cuh"
#include "skinny.cuh"
#include "w4a8_decode.cuh"

namespace texo {
namespace w4a8 {

using i8::Quant;

// -------------------------------------------------------------- generic path
constexpr int GT = 16;   // output tile edge, one output per thread
constexpr int GKB = 32;  // packed bytes (64 k) per shared-memory tile

__global__ void __launch_bounds__(GT * GT)
    generic_kernel(const int8_t* __restrict__ A, const uint8_t* __restrict__ W,
                   int8_t* __restrict__ C, int M, int N, int K, Quant q) {
  __shared__ int8_t As[GT][2 * GKB + 4];
  __shared__ uint8_t Ws[GT][GKB + 4];
  const int tx = threadIdx.x % GT, ty = threadIdx.x / GT;
  const int m = blockIdx.y * GT + ty, n = blockIdx.x * GT + tx;
  const int kbytes = K / 2;
  long long raw = 0, sum_a = 0, sum_u = 0;
  for (int j0 = 0; j0 < kbytes; j0 += GKB) {
    for (int i = threadIdx.x; i < GT * 2 * GKB; i += GT * GT) {
      const int r = i / (2 * GKB), c = i % (2 * GKB);
      const int mm = blockIdx.y * GT + r, k = 2 * j0 + c;
      As[r][c] = (mm < M && k < K) ? A[size_t(mm) * K + k] : int8_t(0);
    }
    for (int i = threadIdx.x; i < GT * GKB; i += GT * GT) {
      const int r = i / GKB, c = i % GKB;
      const int nn = blockIdx.x * GT + r, j = j0 + c;
      Ws[r][c] = (nn < N && j < kbytes) ? W[size_t(nn) * kbytes + j] : uint8_t(0);
    }
    __syncthreads();
    int acc = 0, sa = 0, su = 0;
#pragma unroll 8
    for (int c = 0; c < GKB; ++c) {
      const int hi = Ws[tx][c] >> 4, lo = Ws[tx][c] & 15;
      const int a0 = As[ty][2 * c], a1 = As[ty][2 * c + 1];
      acc += a0 * hi + a1 * lo;
      sa += a0 + a1;
      su += hi + lo;
    }
    // beyond K both tiles hold zeros except that a zero byte still counts as u = 0: fine
    raw += acc;
    sum_a += sa;
    sum_u += su;
    __syncthreads();
  }
  if (m < M && n < N) {
    // per-channel: column n has its own weight scale and zero point (+8: unsigned nibbles)
    const float sb = q.sb_vec ? q.sb_vec[n] : q.sb;
    const long long zb = q.sb_vec ? (long long)(q.zb_vec ? q.zb_vec[n] : 0) + q.zb_bias : (long long)q.zb;
    const long long dot = raw - zb * sum_a - (long long)q.za * sum_u + (long long)K * q.za * zb;
    C[size_t(m) * N + n] = int8_t(i8::requantize(float(dot), q.sa, sb, q.sc, float(q.zc)));
  }
}

// --------------------------------------------------------------- tensor path
constexpr int BK = 128;    // k per stage = one 128-byte swizzle row of int8
constexpr int UMMA_K = 32;  // k per kind::i8 instruction
constexpr int Q_STAGES = 5;
constexpr int Q_RING = 4;
constexpr int Q_A_BYTES = 128 * BK;          // this CTA's 128 rows of A
constexpr int Q_B_BYTES = 128 * BK;          // this CTA's 128 weight rows as bytes 0..15
constexpr int Q_RAW_BYTES = 128 * (BK / 2);  // the same rows as packed nibbles
constexpr int Q_STAGE_BYTES = Q_A_BYTES + Q_B_BYTES + Q_RAW_BYTES;
constexpr int Q_SMEM_BYTES = Q_STAGES * Q_STAGE_BYTES + 1024 + 256;
constexpr int Q_UNPACK_WARPS = 8, Q_UNPACK_WARP0 = 2;  // measured: 8 warps 2.52 POP/s, 4 warps 2.32, 2 warps 1.77
constexpr int Q_EPI_WARPS = 8, Q_EPI_WARP0 = Q_UNPACK_WARP0 + Q_UNPACK_WARPS;
constexpr int Q_THREADS = (Q_EPI_WARP0 + Q_EPI_WARPS) * 32;
constexpr int Q_ACC_COLS = 256, Q_TMEM_COLS = 512;

struct PairBarriers {
  uint64_t ready[Q_STAGES];     // even CTA: A bytes of both CTAs landed AND all unpack warps arrived
  uint64_t raw_full[Q_STAGES];  // per CTA: packed nibbles landed
  uint64_t ring[Q_RING];        // per CTA: MMA commits that free stages (see the producer)
  uint64_t acc_full[2];         // per CTA
  uint64_t acc_empty[2];        // even CTA: epilogue warps of both CTAs arrive
  uint32_t tmem_base;
  int abort_flag;
};

// Sixteen packed bytes (32 weights, k ascending, high nibble first) -> 32 bytes 0..15.
__device__ __forceinline__ void unpack32(const uint4& packed, uint4& first, uint4& second) {
  const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
  uint32_t out[8];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t hi = (words[w] >> 4) & 0x0f0f0f0fu, lo = words[w] & 0x0f0f0f0fu;
    out[2 * w] = __byte_perm(hi, lo, 0x5140);      // hi.b0 lo.b0 hi.b1 lo.b1
    out[2 * w + 1] = __byte_perm(hi, lo, 0x7362);  // hi.b2 lo.b2 hi.b3 lo.b3
  }
  first = make_uint4(out[0], out[1], out[2], out[3]);
  second = make_uint4(out[4], out[5], out[6], out[7]);
}

// ----------------------------------------------- sums inside the pair kernel
// rowsum(A) (signed bytes, needed when the effective weight zero point zB + 8 is non-zero) and
// the per-row sums of the unsigned nibbles of W (needed when zA is non-zero) are computed by
// the epilogue warps of this kernel, exactly as the INT8 CTA-pair kernel computes its sums
// (mm_int8.cu, "sums inside the CTA-pair kernel"): items of sixteen rows (sixteen threads per
// row), ordered as the raster needs them - the A rows of the first raster group of tile rows, all weight
// rows, the remaining A rows -, dealt round robin over the CTAs of the grid, each published by
// a release store of the call's epoch number into the item's flag; a tile is drained when the
// flags of its 8 + 16 items carry the epoch.  A CTA blocks on a flag only when it has no item
// left to do, and every wait is bounded.
constexpr int QS_ROWS = 16;                          // rows per item
constexpr int QS_FIRST_A_ITEMS = i8::P_GROUP_M * 256 / QS_ROWS;  // A items of the first raster group
constexpr int Q_DECISION_BYTES = 64;
constexpr int Q_AUX_SMEM_BYTES = Q_DECISION_BYTES + Q_EPI_WARPS * 512;  // + 128 nibble sums per epilogue warp
static_assert(Q_SMEM_BYTES + Q_AUX_SMEM_BYTES <= 232448, "W4A8 pair kernel: shared memory over the limit");

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// Sum of the 32 unsigned nibbles of v, added to acc.
__device__ __forceinline__ int sum_nibbles(const int4& v, int acc) {
  const uint32_t words[4] = {uint32_t(v.x), uint32_t(v.y), uint32_t(v.z), uint32_t(v.w)};
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t both = (words[w] & 0x0f0f0f0fu) + ((words[w] >> 4) & 0x0f0f0f0fu);  // bytes <= 30
    acc = int(__dp4a(both, 0x01010101u, unsigned(acc)));
  }
  return acc;
}

// Sixteen rows of `row_bytes` bytes each (a multiple of 16), sixteen threads per row, up to
// sixteen 16-byte streaming loads in flight per thread; out[row] = sum of the signed bytes
// (NIBBLES = false) or of the unsigned nibbles (true).  `et` = index among the 256 epilogue
// threads.
template <bool NIBBLES>
__device__ __forceinline__ void sum_sixteen_rows(const uint8_t* __restrict__ base, int row_bytes, int rows_total,
                                                 int item, int* __restrict__ out, int et) {
  const int sub = et % 16, r = item * QS_ROWS + et / 16;
  int acc = 0;
  if (r < rows_total) {
    const int4* src = reinterpret_cast<const int4*>(base + size_t(r) * row_bytes);
    const int chunks = row_bytes / 16;
    auto add = [](const int4& v, int a) { return NIBBLES ? sum_nibbles(v, a) : i8::sum_bytes(v, a); };
    int i = sub;
    for (; i + 15 * 16 < chunks; i += 16 * 16) {
      int4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = __ldcs(src + i + u * 16);
#pragma unroll
      for (int u = 0; u < 16; ++u) acc = add(v[u], acc);
    }
    for (; i + 3 * 16 < chunks; i += 4 * 16) {
      int4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcs(src + i + u * 16);
#pragma unroll
      for (int u = 0; u < 4; ++u) acc = add(v[u], acc);
    }
    for (; i < chunks; i += 16) acc = add(__ldcs(src + i), acc);
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (sub == 0 && r < rows_total) out[r] = acc;
}

// Computes the item at position `pos` of the processing order and publishes it.
__device__ __forceinline__ void epilogue_sum_item(int pos, const int8_t* __restrict__ A,
                                                  const uint8_t* __restrict__ W, int* __restrict__ row_sum,
                                                  int* __restrict__ w_sum, int M, int N, int K, int a_items,
                                                  int w_items, int et, unsigned* flags, unsigned epoch) {
  const int first_a = min(a_items, QS_FIRST_A_ITEMS);
  if (pos >= first_a && pos < first_a + w_items)
    sum_sixteen_rows<true>(W, K / 2, N, pos - first_a, w_sum, et);
  else
    sum_sixteen_rows<false>(reinterpret_cast<const uint8_t*>(A), K, M, pos < first_a ? pos : pos - w_items,
                            row_sum, et);
  epilogue_bar();  // orders every thread's stores before the first thread's (cumulative) release
  if (et == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + pos), "r"(epoch) : "memory");
}

// Whether the sums this CTA's part of tile (tm, tn) needs are published: its 128 rows of A
// (eight items) and the tile's 256 weight rows (sixteen items).  Called by one full warp.
__device__ __forceinline__ bool tile_sums_ready(int tm, int tn, int rank, int a_items, int w_items,
                                                const unsigned* flags, unsigned epoch, int lane) {
  const int first_a = min(a_items, QS_FIRST_A_ITEMS);
  int pos = -1;
  if (lane < 8) {
    const int i = (tm * 256 + rank * 128) / QS_ROWS + lane;
    if (i < a_items) pos = i < first_a ? i : i + w_items;
  } else if (lane < 24) {
    const int j = tn * (256 / QS_ROWS) + (lane - 8);
    if (j < w_items) pos = first_a + j;
  }
  bool ready = true;
  if (pos >= 0) {
    unsigned seen;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + pos) : "memory");
    ready = seen == epoch;
  }
  return __all_sync(0xffffffffu, ready);
}

template <bool WIDE>
__global__ void __launch_bounds__(Q_THREADS, 1)
    pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_raw,
                int8_t* __restrict__ C, int* row_sum, int* w_sum, int M, int N, int K, Quant q,
                int tiles_m, int tiles_n, int c_vector_ok, int* status, const int8_t* __restrict__ A_raw,
                const uint8_t* __restrict__ W_raw, int a_items, int w_items, unsigned* item_flags,
                unsigned epoch, int raster_rows) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  PairBarriers* bars = reinterpret_cast<PairBarriers*>(smem + Q_STAGES * Q_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA (issues the MMAs)
  const int cluster_id = blockIdx.x / 2, num_clusters = gridDim.x / 2;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  grid_dependency_trigger();  // the next grid may set itself up while this one runs

  if (threadIdx.x == 0) {
    for (int s = 0; s < Q_STAGES; ++s) {
      mbar_init(&bars->ready[s], 1 + 2 * Q_UNPACK_WARPS);  // producer's expect_tx + unpack warps
      mbar_init(&bars->raw_full[s], 1);
    }
    for (int r = 0; r < Q_RING; ++r) mbar_init(&bars->ring[r], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2 * Q_EPI_WARPS);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_raw);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, Q_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  // Stage release: k blocks are numbered globally over the tiles a pair works through; the
  // MMA warp commits after every even-numbered block (a commit costs the tensor pipe about
  // as much as five MMAs of this shape), covering that block and its predecessor.  Commit c
  // arrives on ring[c % 4] of both CTAs.
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    int g = 0;          // global k-block number of the next load
    int observed = -1;  // highest commit number seen complete
    bool ok = true;
    grid_dependency_wait();  // the operands may have been written by the grid ahead of this one
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tm, tn;
      i8::pair_tile_coords(tile, tiles_m, tiles_n, raster_rows, tm, tn);
      const int m0 = tm * 256 + int(rank) * 128;
      const int n0 = tn * 256 + int(rank) * 128;
      for (int kb = 0; kb < num_kb && ok; ++kb, ++g) {
        if (lane == 0) {
          if (g >= Q_STAGES) {
            const int c = (g - Q_STAGES + 1) >> 1;  // commit covering block g - Q_STAGES
            if (c > observed) {
              ok = mbar_wait(&bars->ring[c & (Q_RING - 1)], (c >> 2) & 1, abort_flag, status,
                             STATUS_TIMEOUT_EMPTY);
              observed = c;
            }
          }
          if (ok) {
            uint8_t* sa = smem + stage * Q_STAGE_BYTES;
            uint8_t* sraw = sa + Q_A_BYTES + Q_B_BYTES;
            const uint32_t ready_even = map_to_cta(smem_u32(&bars->ready[stage]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&bars->ready[stage], 2 * Q_A_BYTES);
            tma_load_2d_pair(sa, &map_a, ready_even, kb * BK, m0);
            mbar_arrive_expect_tx(&bars->raw_full[stage], Q_RAW_BYTES);
            tma_load_2d(sraw, &map_raw, &bars->raw_full[stage], kb * (BK / 2), n0);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == Q_STAGES) stage = 0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (even CTA only)
    if (rank == 0) {
      constexpr uint32_t IDESC = umma_idesc(/*D=s32*/ 2, /*A=s8*/ 1, /*B=u8*/ 0, /*A K-major*/ 0,
                                            /*B K-major*/ 0, 256, 256);
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
        const uint32_t tmem_d = tmem_base + acc * Q_ACC_COLS;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++g) {
          if (lane == 0) {
            ok = mbar_wait(&bars->ready[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
            if (ok) {
              tc_fence_after_sync();
              const uint32_t sa = smem_u32(smem + stage * Q_STAGE_BYTES);
              const uint32_t sb = sa + Q_A_BYTES;
#pragma unroll
              for (int j = 0; j < BK / UMMA_K; ++j) {
                const uint64_t da = smem_desc(sa + j * UMMA_K, 16, 1024, SMEM_SWIZZLE_128B);
                const uint64_t db = smem_desc(sb + j * UMMA_K, 16, 1024, SMEM_SWIZZLE_128B);
                umma_i8_pair(tmem_d, da, db, IDESC, (kb | j) != 0);
              }
              // releases this block's stage and its predecessor's, in both CTAs
              if ((g & 1) == 0) umma_commit_pair(&bars->ring[(g >> 1) & (Q_RING - 1)], 3);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (++stage == Q_STAGES) {
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
  } else if (warp < Q_EPI_WARP0) {
    // ------------------------------------------------------- nibble unpacking
    const int t = (warp - Q_UNPACK_WARP0) * 32 + lane;  // 0 .. 32 * Q_UNPACK_WARPS - 1
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        ok = mbar_wait(&bars->raw_full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* sb = smem + stage * Q_STAGE_BYTES + Q_A_BYTES;
        const uint8_t* sraw = sb + Q_B_BYTES;
        // 512 sixteen-byte pieces (128 rows x 4): consecutive threads take consecutive pieces,
        // so loads are contiguous; the two 16-byte chunks a piece expands to go to the
        // 128-byte-swizzled positions 2p and 2p+1 of its row (bank-conflict free: the eight
        // threads of a store phase cover two rows of opposite parity).
#pragma unroll
        for (int i = 0; i < 512 / (32 * Q_UNPACK_WARPS); ++i) {
          const int piece = t + 32 * Q_UNPACK_WARPS * i;
          const int row = piece >> 2, p = piece & 3;
          const uint4 packed = *reinterpret_cast<const uint4*>(sraw + piece * 16);
          uint4 first, second;
          unpack32(packed, first, second);
          uint8_t* dst = sb + row * 128;
          *reinterpret_cast<uint4*>(dst + (((2 * p) ^ (row & 7)) << 4)) = first;
          *reinterpret_cast<uint4*>(dst + (((2 * p + 1) ^ (row & 7)) << 4)) = second;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->ready[stage]), 0));
        if (++stage == Q_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - Q_EPI_WARP0;
    const int quarter = warp % 4;  // TMEM lanes this warp may read: 32*quarter .. +31
    const int half = ew / 4;       // which 128 of the 256 accumulator columns
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // Everything this kernel reads or writes may be in use by the grid ahead of it in the
    // stream until that grid has completed.
    grid_dependency_wait();
    const int et = threadIdx.x - Q_EPI_WARP0 * 32;
    const int total_items = a_items + w_items;
    int next_item = blockIdx.x;  // this CTA's next position in the processing order
    uint8_t* const aux = smem + Q_STAGES * Q_STAGE_BYTES + 256;
    volatile int* decision = reinterpret_cast<volatile int*>(aux);
    int4* colsum_stage = reinterpret_cast<int4*>(aux + Q_DECISION_BYTES) + ew * 32;
    int round = 0;  // alternates the two decision words, so that one barrier per decision suffices
    int items_done = 0;
    if (next_item < total_items) {  // the first item needs no decision: nothing else can be ready yet
      epilogue_sum_item(next_item, A_raw, W_raw, row_sum, w_sum, M, N, K, a_items, w_items, et, item_flags, epoch);
      next_item += gridDim.x;
      ++items_done;
    }
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tm, tn;
      i8::pair_tile_coords(tile, tiles_m, tiles_n, raster_rows, tm, tn);
      if (total_items > 0) {
        // Until the accumulator is complete AND this tile's sums are published: the second item
        // at once, then one item per tile, all remaining ones without pause if this tile's
        // sums are missing (a CTA never sits idle on a flag while it still owes items).
        const long long start = clock64();
        bool item_this_tile = false;
        while (true) {
          if (ew == 0) {
            int d = 0;  // 0 = wait, 1 = go on to the drain, 2 = do an item, 3 = give up
            const bool acc_ready = mbar_try_wait(&bars->acc_full[acc], acc_phase);
            const bool sums_ready = tile_sums_ready(tm, tn, int(rank), a_items, w_items, item_flags, epoch, lane);
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
            epilogue_sum_item(next_item, A_raw, W_raw, row_sum, w_sum, M, N, K, a_items, w_items, et, item_flags,
                              epoch);
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
      i8::drain_half<WIDE>(tmem_base + acc * Q_ACC_COLS + (uint32_t(quarter * 32) << 16), half * 128,
                           tn * 256, m, m < M, C, row_sum, w_sum, N, K, q, c_vector_ok, nullptr, colsum_stage);
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
      epilogue_sum_item(next_item, A_raw, W_raw, row_sum, w_sum, M, N, K, a_items, w_items, et, item_flags, epoch);
      next_item += gridDim.x;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees TMEM) while its partner may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, Q_TMEM_COLS);
  }
}

// ------------------------------------------------------------------ dispatch
enum Path { PATH_AUTO = 0, PATH_GENERIC = 1, PATH_TENSOR = 2, PATH_SKINNY = 3, PATH_DECODE = 4 };

inline int& forced_path() {
  static int path = [] {
    const char* env = std::getenv("TEXO_MM_INT4A8_PATH");
    return env ? std::atoi(env) : 0;
  }();
  return path;
}

inline int& last_path() {
  static int path = 0;
  return path;
}

static bool tensor_path_ok(const int8_t* A, const uint8_t* W, int K) {
  return K > 0 && K < (1 << 17) && K % 32 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
         (reinterpret_cast<uintptr_t>(W) & 15) == 0;
}

// Largest number of CTA pairs that can be resident at once (0 if pairs cannot be launched).
static int max_active_pairs(DeviceCtx& ctx) {
  static int cached[MAX_DEVICES] = {};
  static bool known[MAX_DEVICES] = {};
  if (!known[ctx.device]) {
    known[ctx.device] = true;
    cudaFuncSetAttribute(pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Q_SMEM_BYTES + Q_AUX_SMEM_BYTES);
    cudaFuncSetAttribute(pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         Q_SMEM_BYTES + Q_AUX_SMEM_BYTES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * ctx.sm_count);
    cfg.blockDim = dim3(Q_THREADS);
    cfg.dynamicSmemBytes = Q_SMEM_BYTES + Q_AUX_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, pair_kernel<false>, &cfg) != cudaSuccess) n = 0;
    cudaGetLastError();
    cached[ctx.device] = n;
  }
  return cached[ctx.device];
}

static bool launch_tensor(DeviceCtx& ctx, const int8_t* A, const uint8_t* W, int8_t* C, int M, int N,
                          int K, const Quant& q, bool wide) {
  const int pairs = max_active_pairs(ctx);
  if (pairs <= 0) return false;
  CUtensorMap map_a, map_raw;
  if (!make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, K, 128, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tensor_map_2d(&map_raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, N, K / 2, K / 2, 128, BK / 2,
                          CU_TENSOR_MAP_SWIZZLE_NONE)) {
    note_host_error(STATUS_TENSORMAP_FAILED);
    return false;
  }
  const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
  // scratch: rowsum(A) [M] | nibble sums [tiles_n * 256] (padded: the drain reads whole tiles)
  const size_t m_pad = (size_t(M) + 63) & ~size_t(63);
  int* scratch = static_cast<int*>(device_scratch(ctx, (m_pad + size_t(tiles_n) * 256) * sizeof(int)));
  if (!scratch) return false;
  int* row_sum = scratch;
  int* w_sum = scratch + m_pad;
  // rows of A are needed when the effective weight zero point (zB + 8) is non-zero, the
  // nibble sums when zA is; the kernel's epilogue warps compute both (no pre-pass)
  const bool need_rows = q.zb != 0 || q.sb_vec != nullptr;  // per-channel zero points: unknown here
  const int a_items = need_rows ? (M + QS_ROWS - 1) / QS_ROWS : 0;
  const int w_items = q.za != 0 ? (N + QS_ROWS - 1) / QS_ROWS : 0;
  unsigned* item_flags = device_item_flags(ctx, size_t(std::max(a_items + w_items, 1)) * sizeof(unsigned));
  if (!item_flags) return false;
  // a finished item is marked with this call's epoch number: never zero, never used twice
  const unsigned epoch = next_sums_epoch(ctx);
  const int slot = profile_start();
  cudaLaunchConfig_t cfg = {};
  // one pair per tile up to what the device holds; a small problem gets extra pairs that own
  // no tile and only help with the sums
  const int helper_pairs = (a_items + w_items + 1) / 2;
  cfg.gridDim = dim3(2 * std::min(std::max(tiles_m * tiles_n, helper_pairs), pairs));
  cfg.blockDim = dim3(Q_THREADS);
  cfg.dynamicSmemBytes = Q_SMEM_BYTES + Q_AUX_SMEM_BYTES;
  cfg.stream = 0;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  // may be scheduled while the grid ahead of it drains (the kernel waits before it touches memory)
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  const int c_vector_ok = (reinterpret_cast<uintptr_t>(C) & 15) == 0 && N % 16 == 0;
  const cudaError_t err =
      wide ? cudaLaunchKernelEx(&cfg, pair_kernel<true>, map_a, map_raw, C, row_sum, w_sum, M, N, K, q, tiles_m,
                                tiles_n, c_vector_ok, ctx.status, A, W, a_items, w_items, item_flags, epoch,
                                i8::raster_group_rows(K))
           : cudaLaunchKernelEx(&cfg, pair_kernel<false>, map_a, map_raw, C, row_sum, w_sum, M, N, K, q, tiles_m,
                                tiles_n, c_vector_ok, ctx.status, A, W, a_items, w_items, item_flags, epoch,
                                i8::raster_group_rows(K));
  if (err != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;  // the caller falls back to the generic kernel
  }
  profile_stop(slot);
  ++launch_counter();
  last_path() = PATH_TENSOR;
  return true;
}

}  // namespace w4a8
}  // namespace texo

namespace texo {
namespace w4a8 {
// Decode kernel (w4a8_decode.cuh): up to 16 activation rows, weights straight from HBM into
// registers.  Picks how many 32-row groups a CTA owns (the rest of its 16 warps split K): as
// many as still give about three quarters of the SMs a CTA.
static bool decode_path_ok(const int8_t* A, const uint8_t* w_q, int M, int N, int K) {
  return M <= 16 && K >= 128 && K % 128 == 0 && K < (1 << 17) && (long long)N * (K / 2) < (1LL << 31) &&
         (reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_q) & 15) == 0;
}

static bool launch_decode(DeviceCtx& ctx, const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N,
                          int K, const i8::Quant& q) {
  static bool configured[MAX_DEVICES] = {};
  if (!configured[ctx.device]) {
    if (cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, E_SMEM_BYTES) !=
        cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    configured[ctx.device] = true;
  }
  int rowgroups = 0;
  for (int rg = E_WARPS; rg >= 1; rg /= 2) {
    if (K % (128 * (E_WARPS / rg)) != 0) continue;
    rowgroups = rg;  // the smallest valid one is kept if none fills the SMs
    if ((N + 32 * rg - 1) / (32 * rg) >= ctx.sm_count * 3 / 4) break;
  }
  if (rowgroups == 0) return false;
  const int grid = (N + 32 * rowgroups - 1) / (32 * rowgroups);
  const int slot = profile_start();
  if (launch_overlapping_predecessor(decode_kernel, dim3(grid), dim3(E_THREADS), E_SMEM_BYTES, A, w_q, C, M, N, K,
                                     q, rowgroups) != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;
  }
  profile_stop(slot);
  ++launch_counter();
  last_path() = PATH_DECODE;
  return true;
}

// Dispatch shared by the per-tensor and the per-channel entry points.  scale_B_vec /
// zero_point_B_vec: per-output-channel weight quantisation (device arrays [N], see
// texo_mm_int4a8_solve_per_channel), both null for per-tensor.
static void solve_with(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N, int K, float scale_A,
                       float scale_B, float scale_C, int zero_point_A, int zero_point_B,
                       int zero_point_C, const float* scale_B_vec, const int* zero_point_B_vec) {
  if (M <= 0 || N <= 0) return;
  if (K < 0 || K % 2 != 0 || !C || (K > 0 && (!A || !w_q))) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  DeviceCtx& ctx = device_ctx();
  // unsigned nibbles u = q + 8 against the zero point zB + 8
  const long long zb_eff = (long long)zero_point_B + 8;
  if (zb_eff > 0x7fffffffLL) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  i8::Quant q = i8::make_quant(scale_A, scale_B, scale_C, zero_point_A, int(zb_eff), zero_point_C, K);
  q.sb_vec = scale_B_vec;
  q.zb_vec = zero_point_B_vec;
  q.zb_bias = 8;
  const bool vectors_ok = (reinterpret_cast<uintptr_t>(scale_B_vec) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(zero_point_B_vec) & 15) == 0 &&
                          (scale_B_vec == nullptr || N % 4 == 0);
  const int force = forced_path();
  if ((force == PATH_AUTO || force == PATH_DECODE) && ctx.cc_major >= 8 && K > 0 &&
      decode_path_ok(A, w_q, M, N, K) && launch_decode(ctx, A, w_q, C, M, N, K, q))
    return;
  if (force != PATH_GENERIC && ctx.cc_major >= 10 && vectors_ok && tensor_path_ok(A, w_q, K)) {
    // the 32-bit (mod 2^32) correction is exact while |dot| < 2^31; per-channel zero points
    // live on the device, so the bound assumes the int8 range for them
    const double zb_bound = scale_B_vec ? 136.0 : std::abs(double(zb_eff));
    const double bound = double(K) * (128.0 + std::abs(double(zero_point_A))) * (15.0 + zb_bound);
    // decode shapes: the streaming kernel shared with mm_int8, unpacking on the fly
    if (M <= 32 && (force == PATH_AUTO || force == PATH_SKINNY) &&
        i8::launch_skinny<true>(ctx, A, w_q, C, M, N, K, q)) {
      last_path() = PATH_SKINNY;
      return;
    }
    if (launch_tensor(ctx, A, w_q, C, M, N, K, q, bound >= 2147483648.0)) return;
  }
  generic_kernel<<<dim3((N + GT - 1) / GT, (M + GT - 1) / GT), GT * GT>>>(A, w_q, C, M, N, K, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}
}  // namespace w4a8
}  // namespace texo

// A [M,K] int8, w_q [N,K/2] packed nibbles, C [M,N] int8: device pointers.  K must be even.
extern "C" void solve(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N, int K,
                      float scale_A, float scale_B, float scale_C, int zero_point_A,
                      int zero_point_B, int zero_point_C) {
  texo::w4a8::solve_with(A, w_q, C, M, N, K, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                         zero_point_C, nullptr, nullptr);
}

// The same operator with one weight scale (and optionally one weight zero point) per output
// column, i.e. per row of w_q: scale_B [N] FP32 and zero_point_B [N] int32 are DEVICE arrays,
// zero_point_B may be null (all zero); zero points within [-128, 127].  Column n is
// requantised as float(dot) * scale_A * scale_B[n] / scale_C with
// dot = sum_k (A[m,k] - zA)(q[n,k] - zero_point_B[n]), in the FP32 operation order of the
// per-tensor form.  On every device path (CTA-pair tensor kernel, streaming kernel, generic).
extern "C" void texo_mm_int4a8_solve_per_channel(const int8_t* A, const uint8_t* w_q, int8_t* C, int M,
                                                 int N, int K, float scale_A, const float* scale_B,
                                                 float scale_C, int zero_point_A,
                                                 const int* zero_point_B, int zero_point_C) {
  if (M <= 0 || N <= 0) return;
  if (!scale_B) {
    texo::note_host_error(texo::STATUS_BAD_ARGUMENT);
    return;
  }
  texo::w4a8::solve_with(A, w_q, C, M, N, K, scale_A, 1.0f, scale_C, zero_point_A, 0, zero_point_C,
                         scale_B, zero_point_B);
}

// W4A8 with one weight scale per (output column, scale group): scale_B [N, K / group_size] FP32
// on the device - the layout of the reference's W4A16 scales (src/mm_int4.cu:5-6 of
// frezcirno/Texo), in FP32.  Arithmetic as texo_mm_int8_solve_per_group (mm_int8.cu):
//   acc = fma(RN(float(dot_g) * scale_A), scale_B[n, g], acc) over the groups in order, then
//   C[m, n] = clamp(rint(acc / scale_C) + zC, -128, 127).
// SIMT kernel for every shape (see there for why no tensor-core path is offered).
namespace texo {
namespace w4a8 {
__global__ void __launch_bounds__(256)
    per_group_kernel(const int8_t* __restrict__ A, const uint8_t* __restrict__ W, int8_t* __restrict__ C,
                     int M, int N, int K, int G, const float* __restrict__ scale_B, Quant q) {
  __shared__ int8_t As[16][64 + 4];
  __shared__ uint8_t Ws[16][32 + 4];
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int n = blockIdx.x * 16 + tx, m = blockIdx.y * 16 + ty;
  const int groups = K / G;
  float acc = 0.f;
  long long dot = 0;
  for (int k0 = 0; k0 < K; k0 += 64) {
    for (int i = threadIdx.x; i < 16 * 64; i += 256) {
      const int r = i / 64, c = i % 64;
      const int mm = blockIdx.y * 16 + r, k = k0 + c;
      As[r][c] = (mm < M && k < K) ? A[size_t(mm) * K + k] : int8_t(0);
    }
    for (int i = threadIdx.x; i < 16 * 32; i += 256) {
      const int r = i / 32, c = i % 32;
      const int nn = blockIdx.x * 16 + r, k = k0 + 2 * c;
      Ws[r][c] = (nn < N && k < K) ? W[size_t(nn) * (K / 2) + k / 2] : uint8_t(0);
    }
    __syncthreads();
    if (n < N) {
      const int kend = min(64, K - k0);
      for (int c = 0; c < kend; ++c) {
        const int k = k0 + c;
        const int byte = Ws[tx][c / 2];
        const int wq = ((c & 1) == 0 ? byte >> 4 : byte & 15) - 8;  // high nibble = even k
        dot += (long long)(int(As[ty][c]) - q.za) * (wq - q.zb);
        if ((k + 1) % G == 0) {
          const float t = __fmul_rn(float(dot), q.sa);
          acc = __fmaf_rn(t, scale_B[size_t(n) * groups + k / G], acc);
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
}  // namespace w4a8
}  // namespace texo

extern "C" void texo_mm_int4a8_solve_per_group(const int8_t* A, const uint8_t* w_q, int8_t* C, int M, int N,
                                               int K, int group_size, float scale_A, const float* scale_B,
                                               float scale_C, int zero_point_A, int zero_point_B,
                                               int zero_point_C) {
  using namespace texo;
  using namespace texo::w4a8;
  if (M <= 0 || N <= 0) return;
  if (K <= 0 || K % 2 != 0 || group_size <= 0 || K % group_size != 0 || !A || !w_q || !C || !scale_B) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  const i8::Quant q = i8::make_quant(scale_A, 1.0f, scale_C, zero_point_A, zero_point_B, zero_point_C, K);
  per_group_kernel<<<dim3((N + 15) / 16, (M + 15) / 16), 256>>>(A, w_q, C, M, N, K, group_size, scale_B, q);
  ++launch_counter();
  last_path() = PATH_GENERIC;
}

extern "C" int texo_mm_int4a8_last_path() { return texo::w4a8::last_path(); }
extern "C" void texo_mm_int4a8_force_path(int path) { texo::w4a8::forced_path() = path; }
extern "C" int texo_mm_int4a8_status() { return texo::read_and_clear_status(); }
