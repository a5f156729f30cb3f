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

// --------------------------------------------------------------- tensor path
// CTA-pair tcgen05 kernel, kind::f16 with FP32 accumulation in TMEM.
//
// The product is computed transposed, D[n, m] = sum_k W[n,k] x[m,k]: the dequantised
// weights are the 256-row operand (each CTA of the pair unpacks only its own 128 rows), x is
// the 256-column operand (each CTA loads its own 128 rows of x by TMA).  With the weights on
// the accumulator ROWS, the per-group scale s[n, g] is one scalar per TMEM lane, i.e. per
// epilogue thread: every group's MMAs start a fresh accumulator (two 256-column buffers
// alternate), the epilogue drains it with tcgen05.ld and does acc += s * partial in FP32
// registers.  Weights enter the MMA as the exact integers q - 8 in FP16, so the only
// roundings are the FP32 accumulations - the property the reference kernel relies on
// (src/mm_int4.cu:31-38), without its s_g / s_{g+1} rescaling trick.
//
// Per CTA: warp 0 TMA (x tile + packed nibbles), warp 1 MMA issue (even CTA), warps 4-7
// unpack nibbles -> FP16 into the swizzled operand tile, warps 8-15 epilogue.
constexpr int T_BK = 64;  // k per stage: 64 halves = one 128-byte swizzle row
constexpr int T_STAGES = 6;
constexpr int T_X_BYTES = 128 * 128;   // this CTA's 128 rows of x, 64 halves each
constexpr int T_W_BYTES = 128 * 128;   // this CTA's 128 weight rows, unpacked to FP16
constexpr int T_RAW_BYTES = 128 * 32;  // the same rows as packed nibbles
constexpr int T_STAGE_BYTES = T_X_BYTES + T_W_BYTES + T_RAW_BYTES;
constexpr int T_RING = 32;  // group-completion barriers (see the commit numbering below)
// 16 warps in four warpgroups: {TMA, MMA, 2 idle} | 4 unpack warps | 8 epilogue warps.  The
// kernel starts with 128 registers per thread; the first two groups hand registers back
// (setmaxnreg) so that each epilogue thread can keep its 128 FP32 accumulators live.
constexpr int T_CONV_WARPS = 4;
constexpr int T_CONV_WARP0 = 4;
constexpr int T_EPI_WARPS = 8;
constexpr int T_EPI_WARP0 = 8;
constexpr int T_THREADS = 512;
// 128 * (32 + 64) + 256 * 208 = 65536, the SM's register file.
constexpr int T_REGS_CONTROL = 32, T_REGS_UNPACK = 64, T_REGS_EPILOGUE = 208;
constexpr int T_SMEM_BYTES = T_STAGES * T_STAGE_BYTES + 1024 + 512;


struct TensorBarriers {
  uint64_t ready[T_STAGES];     // even CTA: x bytes of both CTAs landed AND all unpack warps arrived
  uint64_t raw_full[T_STAGES];  // per CTA: packed nibbles landed
  uint64_t group_done[T_RING];   // per CTA: MMAs of a scale group complete
  uint64_t acc_empty[2];         // even CTA: epilogue warps of both CTAs arrived
  uint32_t tmem_base;
  int abort_flag;
};

// Four packed bytes (eight nibbles, k ascending: high nibble first) -> eight FP16 values
// q - 8.  0x6400 is 1024.0: OR-ing a nibble into mantissa bits 0-3 gives 1024 + v, into bits
// 4-7 gives 1024 + 16 v; one HFMA2 per byte removes the offsets exactly.  This is the
// byte-permute + one-HFMA2 conversion of the reference's dequant() (frezcirno/Texo
// src/mm_int4.cu:141-148; same magic constant, mask, multipliers (1/16, 1) and addends
// (-72, -1032)), applied here to a whole word on its way into the swizzled operand tile.
__device__ __forceinline__ uint4 unpack8(uint32_t word) {
  const __half2 mul = __halves2half2(__float2half(0.0625f), __float2half(1.0f));
  const __half2 add = __halves2half2(__float2half(-72.0f), __float2half(-1032.0f));
  uint32_t out[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bytes [b, 0x64, b, 0x64]: low half 0x64:(b & 0xf0), high half 0x64:(b & 0x0f)
    uint32_t pair = __byte_perm(word, 0x64646464u, 0x4040u + 0x0101u * i) & 0xff0ffff0u;
    const __half2 v = __hfma2(*reinterpret_cast<const __half2*>(&pair), mul, add);
    out[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

// acc[first .. first+15] += s * v[0 .. 31], two FP32 lanes per instruction (sm_100 packed FMA).
}  // namespace w4
}  // namespace texo
#include "w4_decode.cuh"
namespace texo {
namespace w4 {

__device__ __forceinline__ void fold32(unsigned long long* acc, int first, const uint32_t (&v)[32],
                                       unsigned long long s2) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    unsigned long long pair;
    asm("mov.b64 %0, {%1, %2};" : "=l"(pair) : "r"(v[2 * j]), "r"(v[2 * j + 1]));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc[first + j]) : "l"(pair), "l"(s2));
  }
}

// Weight-row tiles per raster group for K weights per row: 32 while a group's packed rows stay
// within 48 MB, else 16 or 8 (measured at 4096 x 8192 x 8192, G = 128: 502 / 491 / 487 / 486 us
// for groups of 4 / 8 / 16 / 32).
inline int w4_raster_group(int K) {
  for (int g = 32; g > 8; g /= 2)
    if ((long long)g * 256 * (K / 2) <= (48LL << 20)) return g;
  return 8;
}

__device__ __forceinline__ void w4_tile_coords(int tile, int tiles_n, int tiles_m, int group, int& tn, int& tm) {
  // groups of `group` weight-row tiles walked along m, so that a wave shares x rows and a
  // group's weights in L2
  const int group_tiles = group * tiles_m;
  const int first_n = tile / group_tiles * group;
  const int group_n = min(tiles_n - first_n, group);
  const int in_group = tile % group_tiles;
  tn = first_n + in_group % group_n;
  tm = in_group / group_n;
}

// -DW4_STALL_PROBE: the first CTA's warps accumulate the clock cycles they spend waiting on
// each kind of barrier and in their own work, and store them behind the status word
// (status[16..]) when they finish - a way to see which role bounds the pipeline.
#ifdef W4_STALL_PROBE
#define PROBE_DECL long long probe_t0 = 0, probe_wait_a = 0, probe_wait_b = 0, probe_work = 0
#define PROBE_BEGIN() probe_t0 = clock64()
#define PROBE_END(var) var += clock64() - probe_t0
#define PROBE_STORE(slot, value) \
  if (blockIdx.x == 0 && lane == 0) status[16 + (slot)] = int((value) >> 10)
#else
#define PROBE_DECL
#define PROBE_BEGIN()
#define PROBE_END(var)
#define PROBE_STORE(slot, value)
#endif

__global__ void __launch_bounds__(T_THREADS, 1)
    tensor_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_raw,
                  const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K,
                  int G, int tiles_n, int tiles_m, int* status, int raster_group) {
  extern __shared__ uint8_t smem_raw[];
  grid_dependency_trigger();  // the next grid may set itself up while this one runs
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  TensorBarriers* bars = reinterpret_cast<TensorBarriers*>(smem + T_STAGES * T_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x / 2, num_clusters = gridDim.x / 2;
  const int num_tiles = tiles_n * tiles_m;
  const int num_kb = K / T_BK;
  const int steps_per_group = G / 16;  // MMA k-steps (16 k each) per scale group: 1, 2, 4 or 8
  const int groups = K / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T_STAGES; ++s) {
      mbar_init(&bars->ready[s], 1 + 2 * T_CONV_WARPS);  // producer's expect_tx + unpack warps
      mbar_init(&bars->raw_full[s], 1);
    }
    for (int r = 0; r < T_RING; ++r) mbar_init(&bars->group_done[r], 1);
    for (int b = 0; b < 2; ++b) mbar_init(&bars->acc_empty[b], 2 * T_EPI_WARPS);
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_raw);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // set-up done while the grid ahead of this one may still be running; nothing below touches
  // global memory before that grid has completed
  grid_dependency_wait();

  // Commit numbering: scale groups are numbered globally over the tiles this pair processes;
  // the MMA warp issues one tcgen05.commit per group, number c, onto group_done[c % T_RING].
  // It tells the epilogue that accumulator c % 2 is complete and the producer that the
  // group's stages may be refilled.  Nobody lags T_RING commits behind, so parities are safe.
  if (warp < T_CONV_WARP0) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T_REGS_CONTROL));
   if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    int kbg = 0;        // global k-block number of the next load
    int observed = -1;  // highest commit seen
    bool ok = true;
    PROBE_DECL;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tn, tm;
      w4_tile_coords(tile, tiles_n, tiles_m, raster_group, tn, tm);
      const int n0 = tn * 256 + int(rank) * 128;
      const int m0 = tm * 256 + int(rank) * 128;
      for (int kb = 0; kb < num_kb && ok; ++kb, ++kbg) {
        if (lane == 0) {
          if (kbg >= T_STAGES) {
            // the commit of the last scale group that touches block kbg - T_STAGES
            const int c = ((kbg - T_STAGES + 1) * T_BK - 1) / G;
            if (c > observed) {
              PROBE_BEGIN();
              ok = mbar_wait(&bars->group_done[c % T_RING], (c / T_RING) & 1, abort_flag, status,
                             STATUS_TIMEOUT_EMPTY);
              PROBE_END(probe_wait_a);
              observed = c;
            }
          }
          if (ok) {
            uint8_t* sx = smem + stage * T_STAGE_BYTES;
            uint8_t* sraw = sx + T_X_BYTES + T_W_BYTES;
            const uint32_t ready_even = map_to_cta(smem_u32(&bars->ready[stage]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&bars->ready[stage], 2 * T_X_BYTES);
            tma_load_2d_pair(sx, &map_x, ready_even, kb * T_BK, m0);
            mbar_arrive_expect_tx(&bars->raw_full[stage], T_RAW_BYTES);
            tma_load_2d(sraw, &map_raw, &bars->raw_full[stage], kb * (T_BK / 2), n0);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == T_STAGES) stage = 0;
      }
    }
    PROBE_STORE(0, probe_wait_a);  // producer: waiting for a stage to be released
  } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (even CTA only)
    if (rank == 0) {
      constexpr uint32_t IDESC = umma_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, 0, 0, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
      int step = 0;  // k-step inside the current stage (T_BK / 16 of them)
      int gc = 0;    // global group (= commit) number
      bool ok = true;
      PROBE_DECL;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        for (int g = 0; g < groups && ok; ++g, ++gc) {
          const int buf = gc & 1;
          if (lane == 0) {
            PROBE_BEGIN();
            ok = mbar_wait(&bars->acc_empty[buf], ((gc >> 1) & 1) ^ 1, abort_flag, status,
                           STATUS_TIMEOUT_TMEM_EMPTY);
            PROBE_END(probe_wait_a);
            tc_fence_after_sync();
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          const uint32_t tmem_d = tmem_base + buf * 256;
          // A group is steps_per_group k-steps: two stages, one stage, half or a quarter of one.
          // Lane 0 issues them; the issue code is unrolled per case with compile-time
          // descriptor offsets - a generic loop with run-time offsets fed the tensor pipe at
          // little more than half the rate (0.90 against 0.51 ms for G = 128).
          if (lane == 0) {
            if (steps_per_group >= 4) {
              for (int kk = 0; kk < steps_per_group / 4 && ok; ++kk) {
                PROBE_BEGIN();
                ok = mbar_wait(&bars->ready[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
                PROBE_END(probe_wait_b);
                if (ok) {
                  tc_fence_after_sync();
                  const uint32_t sx = smem_u32(smem + stage * T_STAGE_BYTES);
                  const uint32_t sw = sx + T_X_BYTES;
#pragma unroll
                  for (int j = 0; j < T_BK / 16; ++j) {
                    const uint64_t da = smem_desc(sw + j * 32, 16, 1024, SMEM_SWIZZLE_128B);
                    const uint64_t db = smem_desc(sx + j * 32, 16, 1024, SMEM_SWIZZLE_128B);
                    umma_f16_pair(tmem_d, da, db, IDESC, (kk | j) != 0);
                  }
                }
                if (++stage == T_STAGES) {
                  stage = 0;
                  phase ^= 1;
                }
              }
            } else {
              // part of a stage: `step` is the first k-step of this group inside the stage
              if (step == 0) {
                PROBE_BEGIN();
                ok = mbar_wait(&bars->ready[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
                PROBE_END(probe_wait_b);
                tc_fence_after_sync();
              }
              if (ok) {
                const uint32_t sx = smem_u32(smem + stage * T_STAGE_BYTES) + step * 32;
                const uint32_t sw = sx + T_X_BYTES;
                umma_f16_pair(tmem_d, smem_desc(sw, 16, 1024, SMEM_SWIZZLE_128B),
                              smem_desc(sx, 16, 1024, SMEM_SWIZZLE_128B), IDESC, false);
                if (steps_per_group == 2)
                  umma_f16_pair(tmem_d, smem_desc(sw + 32, 16, 1024, SMEM_SWIZZLE_128B),
                                smem_desc(sx + 32, 16, 1024, SMEM_SWIZZLE_128B), IDESC, true);
              }
              step += steps_per_group;
              if (step == T_BK / 16) {
                step = 0;
                if (++stage == T_STAGES) {
                  stage = 0;
                  phase ^= 1;
                }
              }
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (lane == 0 && ok) umma_commit_pair(&bars->group_done[gc % T_RING], 3);
          __syncwarp();
        }
      }
      PROBE_STORE(1, probe_wait_a);  // MMA warp: waiting for an accumulator to be drained
      PROBE_STORE(2, probe_wait_b);  // MMA warp: waiting for a stage's operands
    }
   }
  } else if (warp < T_EPI_WARP0) {
    // ------------------------------------------------------- nibble unpacking
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(T_REGS_UNPACK));
    const int cw = warp - T_CONV_WARP0;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    PROBE_DECL;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        PROBE_BEGIN();
        ok = mbar_wait(&bars->raw_full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        PROBE_END(probe_wait_a);
        if (!ok) break;
        PROBE_BEGIN();
        uint8_t* sw = smem + stage * T_STAGE_BYTES + T_X_BYTES;
        const uint8_t* sraw = sw + T_W_BYTES;
#pragma unroll
        for (int i = 0; i < 128 / (T_CONV_WARPS * 32); ++i) {
          const int row = cw * (128 / T_CONV_WARPS) + i * 32 + lane;
          const uint4 lo = *reinterpret_cast<const uint4*>(sraw + row * 32);
          const uint4 hi = *reinterpret_cast<const uint4*>(sraw + row * 32 + 16);
          const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
          for (int c = 0; c < 8; ++c)  // chunk c = k 8c .. 8c+7, stored 128-byte swizzled
            *reinterpret_cast<uint4*>(sw + row * 128 + ((c ^ (row & 7)) << 4)) = unpack8(words[c]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->ready[stage]), 0));
        PROBE_END(probe_work);
        if (++stage == T_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (cw == 0) {
      PROBE_STORE(3, probe_wait_a);  // unpack warp: waiting for packed rows to land
      PROBE_STORE(4, probe_work);    // unpack warp: unpacking
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(T_REGS_EPILOGUE));
    const int ew = warp - T_EPI_WARP0;
    const int quarter = warp % 4;  // TMEM lanes 32*quarter .. +31
    const int half = ew / 4;       // which 128 of the 256 accumulator columns (m)
    int gc = 0;
    bool ok = true;
    PROBE_DECL;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tn, tm;
      w4_tile_coords(tile, tiles_n, tiles_m, raster_group, tn, tm);
      const int n = tn * 256 + int(rank) * 128 + quarter * 32 + lane;
      const bool n_ok = n < N;
      const __half* s_row = scales + size_t(n_ok ? n : 0) * groups;
      // 128 FP32 accumulators per thread, kept as 64 two-float pairs: the fold below is the
      // packed fma.rn.f32x2 (two independent IEEE FP32 FMAs per instruction), which halves the
      // issue slots the per-group fold costs next to the unpack warps.
      unsigned long long acc[64];
#pragma unroll
      for (int j = 0; j < 64; ++j) acc[j] = 0ull;
      float s_next = n_ok ? __half2float(s_row[0]) : 0.f;
      for (int g = 0; g < groups && ok; ++g, ++gc) {
        const float s = s_next;
        if (g + 1 < groups && n_ok) s_next = __half2float(s_row[g + 1]);
        unsigned long long s2;
        asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(s));
        PROBE_BEGIN();
        ok = mbar_wait(&bars->group_done[gc % T_RING], (gc / T_RING) & 1, abort_flag, status,
                       STATUS_TIMEOUT_TMEM_FULL);
        ok = __all_sync(0xffffffffu, ok);
        PROBE_END(probe_wait_a);
        if (!ok) break;
        PROBE_BEGIN();
        tc_fence_after_sync();
        const uint32_t taddr = tmem_base + (gc & 1) * 256 + half * 128 + (uint32_t(quarter * 32) << 16);
        // A TMEM load takes a few hundred cycles to return, and tcgen05.wait::ld waits for every
        // load in flight: the 128 columns come in as four 32-column loads, two in flight at a
        // time (two latency exposures per group instead of one per 16 columns); the buffer goes
        // back to the MMA warp as soon as the last load has landed, before the last folds.
        uint32_t va[32], vb[32];
        tmem_ld_32x32(taddr, va);
        tmem_ld_32x32(taddr + 32, vb);
        tmem_ld_wait();
        fold32(acc, 0, va, s2);
        tmem_ld_32x32(taddr + 64, va);
        fold32(acc, 16, vb, s2);
        tmem_ld_32x32(taddr + 96, vb);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->acc_empty[gc & 1]), 0));
        fold32(acc, 32, va, s2);
        fold32(acc, 48, vb, s2);
        PROBE_END(probe_work);
      }
      if (ok && n_ok) {
        const int m_base = tm * 256 + half * 128;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          float lo, hi;
          asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[j]));
          const int m = m_base + 2 * j;
          if (m < M) y[size_t(m) * N + n] = __float2half_rn(lo);
          if (m + 1 < M) y[size_t(m + 1) * N + n] = __float2half_rn(hi);
        }
      }
    }
    if (ew == 0) {
      PROBE_STORE(5, probe_wait_a);  // epilogue warp: waiting for a group's MMAs
      PROBE_STORE(6, probe_work);    // epilogue warp: draining (incl. the TMEM load latency)
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// ------------------------------- tensor path for small scale groups (G <= 64)
// With a drain per scale group the kernel above is bound by tensor-memory traffic: every group
// moves the whole 128 x 256 FP32 accumulator out through tcgen05.ld (about as long as a
// 128-k group's MMAs take, and the two do not overlap), so at G = 32 / 16 the drains cost 4x /
// 8x the MMAs.  For small groups the scale goes INTO the weight operand instead - exactly:
// w * s (a 4-bit integer times an 11-bit significand) does not fit FP16, but it is the exact
// sum of two FP16 numbers, hi = RN(w * s) and lo = fma(w, s, -hi) (the rounding error of a
// product is representable), so each k step issues two MMAs, x * hi and x * lo, into ONE
// accumulator that runs over the whole K range and is drained once per tile.  Twice the MMA
// work, no per-group drains: the time no longer depends on the group size (about 0.7 ms for
// 4096 x 8192 x 8192 against 1.05 / 1.93 ms at G = 32 / 16).  The roundings are those of the
// FP32 accumulation plus 2^-22 relative from hi + lo - well inside the reference tolerance,
// unlike a single FP16 product (which the reference found breaks it, src/mm_int4.cu:36-38 of
// frezcirno/Texo).
constexpr int W4_SPLIT_MAX_GROUP = 64;  // largest group size routed to this kernel by default
constexpr int S_STAGES = 4;
constexpr int S_STAGE_BYTES = T_X_BYTES + 2 * T_W_BYTES + T_RAW_BYTES;  // x | hi | lo | packed
constexpr int S_SMEM_BYTES = S_STAGES * S_STAGE_BYTES + 1024 + 512;
constexpr int S_REGS_CONTROL = 40, S_REGS_UNPACK = 88, S_REGS_EPILOGUE = 192;  // 128*(40+88) + 256*192 = 65536

struct SplitBarriers {
  uint64_t ready[S_STAGES];      // even CTA: x bytes of both CTAs landed AND all unpack warps arrived
  uint64_t raw_full[S_STAGES];   // per CTA: packed nibbles landed
  uint64_t stage_free[S_STAGES]; // per CTA: the MMAs that read the stage are complete
  uint64_t acc_full[2];          // per CTA: a tile's MMAs are complete
  uint64_t acc_empty[2];         // even CTA: epilogue warps of both CTAs arrived
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(T_THREADS, 1)
    tensor_split_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_raw,
                        const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K,
                        int G, int tiles_n, int tiles_m, int* status, int raster_group) {
  extern __shared__ uint8_t smem_raw[];
  grid_dependency_trigger();  // the next grid may set itself up while this one runs
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  SplitBarriers* bars = reinterpret_cast<SplitBarriers*>(smem + S_STAGES * S_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x / 2, num_clusters = gridDim.x / 2;
  const int num_tiles = tiles_n * tiles_m;
  const int num_kb = K / T_BK;
  const int groups = K / G;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S_STAGES; ++s) {
      mbar_init(&bars->ready[s], 1 + 2 * T_CONV_WARPS);
      mbar_init(&bars->raw_full[s], 1);
      mbar_init(&bars->stage_free[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 2 * T_EPI_WARPS);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map_x);
    tma_prefetch_desc(&map_raw);
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // set-up done while the grid ahead of this one may still be running; nothing below touches
  // global memory before that grid has completed
  grid_dependency_wait();

  if (warp < T_CONV_WARP0) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S_REGS_CONTROL));
   if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tn, tm;
      w4_tile_coords(tile, tiles_n, tiles_m, raster_group, tn, tm);
      const int n0 = tn * 256 + int(rank) * 128;
      const int m0 = tm * 256 + int(rank) * 128;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(&bars->stage_free[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY);
          if (ok) {
            uint8_t* sx = smem + stage * S_STAGE_BYTES;
            uint8_t* sraw = sx + T_X_BYTES + 2 * T_W_BYTES;
            const uint32_t ready_even = map_to_cta(smem_u32(&bars->ready[stage]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&bars->ready[stage], 2 * T_X_BYTES);
            tma_load_2d_pair(sx, &map_x, ready_even, kb * T_BK, m0);
            mbar_arrive_expect_tx(&bars->raw_full[stage], T_RAW_BYTES);
            tma_load_2d(sraw, &map_raw, &bars->raw_full[stage], kb * (T_BK / 2), n0);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == S_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
   } else if (warp == 1) {
    // ------------------------------------------- MMA issuer (even CTA only)
    if (rank == 0) {
      constexpr uint32_t IDESC = umma_idesc(/*D=f32*/ 1, /*A=f16*/ 0, /*B=f16*/ 0, 0, 0, 256, 256);
      int stage = 0;
      uint32_t phase = 0;
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
        const uint32_t tmem_d = tmem_base + acc * 256;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (lane == 0) {
            ok = mbar_wait(&bars->ready[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
            if (ok) {
              tc_fence_after_sync();
              const uint32_t sx = smem_u32(smem + stage * S_STAGE_BYTES);
              const uint32_t shi = sx + T_X_BYTES, slo = shi + T_W_BYTES;
#pragma unroll
              for (int j = 0; j < T_BK / 16; ++j) {
                const uint64_t db = smem_desc(sx + j * 32, 16, 1024, SMEM_SWIZZLE_128B);
                umma_f16_pair(tmem_d, smem_desc(shi + j * 32, 16, 1024, SMEM_SWIZZLE_128B), db, IDESC,
                              (kb | j) != 0);
                umma_f16_pair(tmem_d, smem_desc(slo + j * 32, 16, 1024, SMEM_SWIZZLE_128B), db, IDESC, 1);
              }
              umma_commit_pair(&bars->stage_free[stage], 3);  // both CTAs' stages reusable
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (++stage == S_STAGES) {
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
   }
  } else if (warp < T_EPI_WARP0) {
    // ------------------------- nibble unpacking + exact scaling into hi / lo
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S_REGS_UNPACK));
    const int cw = warp - T_CONV_WARP0;
    const int row = cw * 32 + lane;  // this thread's weight row within the CTA's 128
    const int gps = T_BK / G;        // scale groups per 64-k stage: 1 (G = 64), 2 (G = 32) or 4 (G = 16)
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tn, tm;
      w4_tile_coords(tile, tiles_n, tiles_m, raster_group, tn, tm);
      const int n = min(tn * 256 + int(rank) * 128 + row, N - 1);
      const __half* s_row = scales + size_t(n) * groups;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        // this stage's scales (2 or 4 consecutive halves), fetched before the wait
        __half sc[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) sc[g] = g < gps ? s_row[kb * gps + g] : __float2half(0.f);
        ok = mbar_wait(&bars->raw_full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* shi = smem + stage * S_STAGE_BYTES + T_X_BYTES;
        uint8_t* slo = shi + T_W_BYTES;
        const uint8_t* sraw = slo + T_W_BYTES;
        const uint4 lo16 = *reinterpret_cast<const uint4*>(sraw + row * 32);
        const uint4 hi16 = *reinterpret_cast<const uint4*>(sraw + row * 32 + 16);
        const uint32_t words[8] = {lo16.x, lo16.y, lo16.z, lo16.w, hi16.x, hi16.y, hi16.z, hi16.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {  // chunk c = k 8c .. 8c+7 of the stage
          // the scale group of k 8c..8c+7 within the stage
          const __half sg = G == 16 ? sc[c >> 1] : G == 32 ? sc[c >> 2] : sc[0];
          const __half2 s2 = __half2half2(sg);
          const uint4 w = unpack8(words[c]);
          const uint32_t win[4] = {w.x, w.y, w.z, w.w};
          uint32_t h[4], l[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __half2 wv = *reinterpret_cast<const __half2*>(&win[i]);
            const __half2 hv = __hmul2(wv, s2);            // RN(w * s)
            const __half2 lv = __hfma2(wv, s2, __hneg2(hv));  // w * s - hi, exact
            h[i] = *reinterpret_cast<const uint32_t*>(&hv);
            l[i] = *reinterpret_cast<const uint32_t*>(&lv);
          }
          const int at = row * 128 + ((c ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(shi + at) = make_uint4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<uint4*>(slo + at) = make_uint4(l[0], l[1], l[2], l[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&bars->ready[stage]), 0));
        if (++stage == S_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(S_REGS_EPILOGUE));
    const int ew = warp - T_EPI_WARP0;
    const int quarter = warp % 4;
    const int half = ew / 4;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int tn, tm;
      w4_tile_coords(tile, tiles_n, tiles_m, raster_group, tn, tm);
      const int n = tn * 256 + int(rank) * 128 + quarter * 32 + lane;
      ok = mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * 256 + half * 128 + (uint32_t(quarter * 32) << 16);
      const int m_base = tm * 256 + half * 128;
#pragma unroll 1
      for (int chunk = 0; chunk < 4; ++chunk) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + chunk * 32, v);
        tmem_ld_wait();
        if (chunk == 3) {  // everything is in registers: hand the accumulator back
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars->acc_empty[acc]), 0));
        }
        if (n < N) {
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) {
            const int m = m_base + chunk * 32 + jj;
            if (m < M) y[size_t(m) * N + n] = __float2half_rn(__uint_as_float(v[jj]));
          }
        }
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

inline int& last_path() {
  static int path = 0;
  return path;
}

inline int& forced_path() {
  static int path = 0;
  return path;
}


// TMA needs 16-byte aligned rows: x rows of K halves, packed rows of K/2 bytes; the kernel
// works in 64-wide k blocks and whole scale groups per accumulator.
static bool tensor_path_ok(const __half* x, const uint8_t* w_q, int K, int G) {
  return K > 0 && K % T_BK == 0 && (G == 16 || G == 32 || G == 64 || G == 128) &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_q) & 15) == 0;
}

// The split-scale kernel for small groups (see tensor_split_kernel): same operands and tensor maps.
static bool launch_tensor_split(DeviceCtx& ctx, const __half* x, const uint8_t* w_q, const __half* scales,
                                __half* y, int M, int N, int K, int G) {
  static bool configured[MAX_DEVICES] = {};
  static int pairs[MAX_DEVICES] = {};
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(T_THREADS);
  cfg.dynamicSmemBytes = S_SMEM_BYTES;
  cfg.stream = 0;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait in the kernel
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  if (!configured[ctx.device]) {
    configured[ctx.device] = true;
    cudaFuncSetAttribute(tensor_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S_SMEM_BYTES);
    cfg.gridDim = dim3(2 * ctx.sm_count);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, tensor_split_kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    pairs[ctx.device] = n;
  }
  if (pairs[ctx.device] <= 0) return false;
  CUtensorMap map_x, map_raw;
  if (!make_tensor_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, M, K, size_t(K) * 2, 128,
                          T_BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tensor_map_2d(&map_raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_q, N, K / 2, K / 2, 128,
                          T_BK / 2, CU_TENSOR_MAP_SWIZZLE_NONE)) {
    note_host_error(STATUS_TENSORMAP_FAILED);
    return false;
  }
  const int tiles_n = (N + 255) / 256, tiles_m = (M + 255) / 256;
  cfg.gridDim = dim3(2 * std::min(tiles_n * tiles_m, pairs[ctx.device]));
  const int slot = profile_start();
  if (cudaLaunchKernelEx(&cfg, tensor_split_kernel, map_x, map_raw, scales, y, M, N, K, G, tiles_n, tiles_m,
                         ctx.status, w4_raster_group(K)) != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;
  }
  profile_stop(slot);
  ++launch_counter();
  last_path() = 4;
  return true;
}

static bool launch_tensor(DeviceCtx& ctx, const __half* x, const uint8_t* w_q, const __half* scales,
                          __half* y, int M, int N, int K, int G) {
  static bool configured[MAX_DEVICES] = {};
  static int pairs[MAX_DEVICES] = {};
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(T_THREADS);
  cfg.dynamicSmemBytes = T_SMEM_BYTES;
  cfg.stream = 0;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // see grid_dependency_wait in the kernel
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 2;
  if (!configured[ctx.device]) {
    configured[ctx.device] = true;
    cudaFuncSetAttribute(tensor_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T_SMEM_BYTES);
    cfg.gridDim = dim3(2 * ctx.sm_count);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, tensor_kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    pairs[ctx.device] = n;
  }
  if (pairs[ctx.device] <= 0) return false;
  CUtensorMap map_x, map_raw;
  if (!make_tensor_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, M, K, size_t(K) * 2, 128,
                          T_BK, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tensor_map_2d(&map_raw, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w_q, N, K / 2, K / 2, 128,
                          T_BK / 2, CU_TENSOR_MAP_SWIZZLE_NONE)) {
    note_host_error(STATUS_TENSORMAP_FAILED);
    return false;
  }
  const int tiles_n = (N + 255) / 256, tiles_m = (M + 255) / 256;
  cfg.gridDim = dim3(2 * std::min(tiles_n * tiles_m, pairs[ctx.device]));
  const int slot = profile_start();
  if (cudaLaunchKernelEx(&cfg, tensor_kernel, map_x, map_raw, scales, y, M, N, K, G, tiles_n, tiles_m,
                         ctx.status, w4_raster_group(K)) != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;  // the caller falls back to the generic kernel
  }
  profile_stop(slot);
  ++launch_counter();
  last_path() = 2;
  return true;
}

// Decode path (w4_decode.cuh): M <= 16, one scale group per 128-k iteration.  Picks how many
// 32-row groups a CTA owns (the rest of its 16 warps split K): as many as still give about
// three quarters of the SMs a CTA, since more rows per CTA means fewer re-reads of x.
static bool decode_path_ok(const __half* x, const uint8_t* w_q, int M, int N, int K, int G) {
  return M <= 16 && G == 128 && K >= 128 && K % 128 == 0 && (long long)N * (K / 2) < (1LL << 31) &&
         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_q) & 15) == 0;
}

static bool launch_decode(DeviceCtx& ctx, const __half* x, const uint8_t* w_q, const __half* scales,
                          __half* y, int M, int N, int K) {
  static bool configured[MAX_DEVICES] = {};
  if (!configured[ctx.device]) {
    if (cudaFuncSetAttribute(decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, D_SMEM_BYTES) !=
        cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    configured[ctx.device] = true;
  }
  int rowgroups = 0;
  for (int rg = D_WARPS; rg >= 1; rg /= 2) {
    if (K % (128 * (D_WARPS / rg)) != 0) continue;
    rowgroups = rg;  // the smallest valid one is kept if none fills the SMs
    if ((N + 32 * rg - 1) / (32 * rg) >= ctx.sm_count * 3 / 4) break;
  }
  if (rowgroups == 0) return false;
  const int grid = (N + 32 * rowgroups - 1) / (32 * rowgroups);
  const int slot = profile_start();
  if (launch_overlapping_predecessor(decode_kernel, dim3(grid), dim3(D_THREADS), D_SMEM_BYTES, x, w_q, scales, y,
                                     M, N, K, rowgroups) != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;
  }
  profile_stop(slot);
  ++launch_counter();
  last_path() = 3;
  return true;
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
  DeviceCtx& ctx = device_ctx();
  if ((forced_path() == 0 || forced_path() == 3) && ctx.cc_major >= 8 &&
      decode_path_ok(x, w_q, M, N, K, group_size) && launch_decode(ctx, x, w_q, scales, y, M, N, K))
    return;
  if (forced_path() != 1 && ctx.cc_major >= 10 && tensor_path_ok(x, w_q, K, group_size)) {
    // small groups: the scale goes into the weight operand (path 4), no per-group drain
    if (group_size <= W4_SPLIT_MAX_GROUP && forced_path() != 2 &&
        launch_tensor_split(ctx, x, w_q, scales, y, M, N, K, group_size))
      return;
    if (forced_path() != 4 && launch_tensor(ctx, x, w_q, scales, y, M, N, K, group_size)) return;
  }
  dim3 grid((N + GT - 1) / GT, (M + GT - 1) / GT);
  const int slot = profile_start();
  generic_kernel<<<grid, G_THREADS>>>(x, w_q, scales, y, M, N, K, group_size);
  profile_stop(slot);
  ++launch_counter();
  last_path() = 1;
}

extern "C" int texo_mm_int4_last_path(void) { return texo::w4::last_path(); }
extern "C" void texo_mm_int4_force_path(int path) { texo::w4::forced_path() = path; }
extern "C" int texo_mm_int4_status(void) { return texo::read_and_clear_status(); }

#ifdef W4_STALL_PROBE
// Probe builds only: copies the seven stall counters (units of 1024 clock cycles) out of the
// status block and clears them.
extern "C" void texo_w4_probe_read(int* out7) {
  texo::DeviceCtx& ctx = texo::device_ctx();
  cudaMemcpy(out7, ctx.status + 16, 7 * sizeof(int), cudaMemcpyDeviceToHost);
  cudaMemset(ctx.status + 16, 0, 7 * sizeof(int));
}
#endif
