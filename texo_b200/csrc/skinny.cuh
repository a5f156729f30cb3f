// The decode ("skinny") path of the INT8 operators: kernel, schedule and launch.  Kept in a
// header because two operators instantiate it: INT8 weights (mm_int8) and packed INT4 weights
// unpacked on the fly (mm_int4a8).
#pragma once
#include <algorithm>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"
#include "requant.cuh"

namespace texo {
namespace i8 {

constexpr int S_BK = 128;     // k per ring stage = one 128-byte swizzle row of int8
constexpr int S_UMMA_K = 32;  // k per kind::i8 instruction

// --------------------------------------------------------------- skinny path
// M <= 128 (decode and small batches): the job is to stream B [K,N] from HBM exactly once.  Operand roles are
// swapped: a 128-column box of B is the 128-row MMA operand (N-major in memory = M-major
// operand, again no transposed copy), the activations are the narrow operand.  The
// activation tile carries one extra all-ones row (written once into every ring slot at
// kernel start), so column R of the accumulator is colsum(B) for free and B is never read a
// second time.
//
// A column tile is 256 columns = two 128-column boxes side by side, loaded back to back for
// the same 128 k rows (ring slot i takes the left box, slot i+1 the right one, each with its
// own accumulator half): HBM then sees 256 contiguous bytes per row instead of 128, which
// measured 6.0 TB/s against 4.3 TB/s for the same bytes fetched as lone 128-byte rows.
//
// Schedule (one CTA per SM, T = ceil(N/256) column tiles, G CTAs): every CTA owns
// P = T / G whole tiles (tile p*G + c, so neighbouring CTAs stream neighbouring columns) and
// the remaining S = T - P*G tiles are cut stream-K style into equal contiguous ranges of
// (tile, k block) units, so every SM pulls the same number of bytes.  The shared ranges are
// processed FIRST: a CTA adds its int32 partials into a zero-initialised workspace with
// integer reductions (order-independent, hence still bit-exact); whoever arrives last at
// the half tile's counter reads the sums, requantises, and puts workspace and counter back to
// zero - all while its producer and MMA warps are already streaming the next tile.  The
// owned tiles come LAST and need no reduction, so the kernel's tail is a plain drain.
// Nobody ever waits for another CTA.
// Nearly all of an SM's shared memory goes to the ring (M <= 16: 6 stages of 32 KiB weights +
// 4 KiB activations; M <= 32 / 64: 5 stages of 32 KiB + 6 / 10 KiB; M <= 128: 4 stages of
// 32 + 18 KiB): each SM has to keep about
// 100 KiB in flight to cover HBM latency at its share of the bandwidth, and a ring that deep
// measured faster than a shallow one that would let two CTAs share an SM.  The kernel is
// launched with programmatic stream serialisation all the same: the next call's CTA starts on
// an SM as soon as this call's CTA there has exited (at once on SMs the grid left idle) and
// does its set-up while the slowest CTAs of this call finish.
// When the tiles divide evenly over at least three quarters of the SMs the grid is shrunk to
// that count, so nothing is shared and no reduction runs at all: 112 CTAs streaming one
// 256-column tile each reach the same HBM rate as 148 and finish without a flush.
constexpr int S_MAX_STAGES = 6;
constexpr int S_MAX_ROWS = 128;  // activation rows this path takes
constexpr int S_BOX_BYTES = 128 * 128;     // one 128 k-row x 128 column box of B
constexpr int S_W_BYTES = 2 * S_BOX_BYTES;  // the two boxes of a 256-column tile
// R = activation rows per MMA (16, 32, 64 or 128; M <= R).  TMEM: one accumulator per
// 128-column half, R + 16 columns wide (rows + the ones row + padding), two halves per tile,
// double buffered except for R = 128, whose two 144-column halves leave no room for a second
// set.
__host__ __device__ constexpr int skinny_acc_cols(int R) { return R <= 32 ? 64 : (R == 64 ? 128 : 144); }
__host__ __device__ constexpr int skinny_acc_buffers(int R) { return R == 128 ? 1 : 2; }
__host__ __device__ constexpr int skinny_tmem_cols(int R) { return R <= 32 ? 256 : 512; }
__host__ __device__ constexpr int skinny_act_bytes(int R) { return (R + 16) * 128; }
__host__ __device__ constexpr int skinny_stages(int R) { return R == 16 ? 6 : (R == 128 ? 4 : 5); }
__host__ __device__ constexpr int skinny_smem_bytes(int R) {
  return skinny_stages(R) * (S_W_BYTES + skinny_act_bytes(R)) + 1024 /*alignment*/ +
         1024 /*SkinnyBarriers*/;
}
constexpr int S_TILE_N = 256;  // two 128-column boxes side by side, see above
constexpr int S_EPI_WARPS = 4;
constexpr int S_THREADS = 64 + S_EPI_WARPS * 32;
// Packed-INT4 weights (W4 = true): w_q [N, K/2] bytes, two nibbles per byte (high nibble =
// even k, value - 8).  A stage then holds the TMA-loaded packed rows of the tile (256 rows x
// 64 bytes), the operand tile eight extra warps unpack them into (256 rows x 128 bytes of
// u = nibble, K-major, 128-byte swizzle; the -8 lives in the zero point, see mm_int4a8.cu),
// and the activations.  Half the weight bytes cross HBM, but shared memory carries 16 + 16 +
// 32 + 32 KiB of weights per k block (packed in, packed out, operand in, operand out) plus the
// activations, about 104 KiB at 128 bytes per clock: that, not HBM, bounds this form (measured:
// the unpack step alone takes ~900 clocks per k block; M=16, N=28672, K=8192 in 48 us against
// 92 us on the CTA-pair kernel and 40 us for the same shape with INT8 weights).  Deeper packed
// rings, a separate activation ring and 8 or 16 unpack warps were tried and changed nothing.
constexpr int S_W4_UNPACK_WARPS = 4;  // (320 threads: the epilogue keeps its ~170 registers)
constexpr int S_W4_THREADS = S_THREADS + S_W4_UNPACK_WARPS * 32;
constexpr int S_W4_PACKED_BYTES = 256 * (S_BK / 2);
constexpr int S_W4_STAGES = 4;
__host__ __device__ constexpr int skinny_w4_stage_bytes(int R) {
  return S_W_BYTES + skinny_act_bytes(R) + S_W4_PACKED_BYTES;
}
__host__ __device__ constexpr int skinny_w4_smem_bytes(int R) {
  return S_W4_STAGES * skinny_w4_stage_bytes(R) + 1024 + 1024;
}

struct SkinnyBarriers {  // at most 1024 bytes, see skinny_smem_bytes
  uint64_t full[S_MAX_STAGES];
  uint64_t empty[S_MAX_STAGES];
  uint64_t raw_full[S_MAX_STAGES];  // W4 only: packed rows landed
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int last_flag;
  int row_sum[128];
};

static_assert(sizeof(SkinnyBarriers) <= 1024, "SkinnyBarriers outgrew its shared-memory reserve");

// First unit of CTA `c` when `units` are dealt to `ctas` CTAs as evenly as possible.
__host__ __device__ __forceinline__ long long skinny_first_unit(long long units, int ctas, int c) {
  const long long q = units / ctas, r = units % ctas;
  return c * q + (c < r ? c : r);
}
// The CTA that owns unit `u` under the same deal.
__device__ __forceinline__ int skinny_owner(long long units, int ctas, long long u) {
  const long long q = units / ctas, r = units % ctas;
  if (u < r * (q + 1)) return int(u / (q + 1));
  return int(r + (u - r * (q + 1)) / q);
}

// The segments (tile, k-block range) of one CTA, in processing order; every warp role walks
// an identical copy.
struct SkinnySchedule {
  int num_kb, ctas, owned, shared_tiles;
  long long shared_units, su, su_end;
  int next_owned, cta;
  // whole_tiles: no tile is split between CTAs (CTA c takes tiles c, c + G, ...), for the
  // row counts whose epilogue has no reduction path.
  __device__ SkinnySchedule(int tiles, int num_kb_, int ctas_, int cta_, bool whole_tiles = false)
      : num_kb(num_kb_), ctas(ctas_), cta(cta_) {
    owned = whole_tiles ? (tiles - cta_ + ctas_ - 1) / ctas_ : tiles / ctas;
    shared_tiles = whole_tiles ? 0 : tiles - owned * ctas;
    shared_units = (long long)shared_tiles * num_kb;
    su = skinny_first_unit(shared_units, ctas, cta);
    su_end = skinny_first_unit(shared_units, ctas, cta + 1);
    next_owned = 0;
  }
  // Returns false when the CTA has no more work.  `shared_index` >= 0 marks a segment
  // that covers only part of its tile's K range (index of the tile among the shared ones).
  __device__ bool next(int& tile, int& kb0, int& kb1, int& shared_index) {
    if (su < su_end) {
      const int t = int(su / num_kb);
      const long long seg_end = min(su_end, (long long)(t + 1) * num_kb);
      kb0 = int(su - (long long)t * num_kb);
      kb1 = int(seg_end - (long long)t * num_kb);
      tile = owned * ctas + t;
      shared_index = (kb0 == 0 && kb1 == num_kb) ? -1 : t;
      su = seg_end;
      return true;
    }
    if (next_owned < owned) {
      tile = next_owned * ctas + cta;
      kb0 = 0;
      kb1 = num_kb;
      shared_index = -1;
      ++next_owned;
      return true;
    }
    return false;
  }
  __device__ int contributors(int t) const {
    return skinny_owner(shared_units, ctas, (long long)(t + 1) * num_kb - 1) -
           skinny_owner(shared_units, ctas, (long long)t * num_kb) + 1;
  }
};

// Requantises ROWS accumulator rows of one output column and stores the first M of them.  All
// rows are computed without a branch (rows past M hold zeros), so their dependent chains
// (64-bit correction, int-to-float, two multiplies, an IEEE division, round, saturate)
// interleave; with one warp per scheduler a per-row branch would run them back to back.
// `kza` = K * zA, `col_term` = zA * colsum(B)[n], `sb_n` / `zb_n` the weight scale and zero
// point of this thread's column: dot = raw + zB * (K*zA - rowsum(A)[m]) - zA * colsum(B)[n].
// Where element [row0, n] of the output lives and its row stride in elements, by output form:
// int8 C [M, N]; SwiGLU H [M, N/2] (column n / 2); FP16 Y [M, N] (byte pointer to the half).
__device__ __forceinline__ int8_t* skinny_out_at(int8_t* C, const Quant& q, int row0, int n, int N,
                                                 size_t& stride) {
  if (q.swiglu) {
    stride = size_t(N / 2);
    return C + size_t(row0) * stride + n / 2;
  }
  stride = size_t(N);
  if (q.out_f16) return C + 2 * (size_t(row0) * N + n);
  return C + size_t(row0) * N + n;
}

template <int ROWS, bool FAST>
__device__ __forceinline__ void skinny_store_rows(const uint32_t (&v)[32], const int* row_sum,
                                                  long long kza, long long col_term, float sb_n,
                                                  int zb_n, const Quant& q, float zc, int M,
                                                  int8_t* out, size_t stride, int col,
                                                  int row0 = 0) {
  if (q.out_f16) {
    // dequantising form: y[m, n] = half(float(dot) * sA * sB), FP16 output with row stride
    // `stride` elements (`out` points at element [row0, n] counted in bytes of int8: redo it)
    __half* y = reinterpret_cast<__half*>(out);
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      const long long dot = (long long)int(v[m]) + (long long)zb_n * (kza - row_sum[m]) - col_term;
      if (m < M) y[m * stride] = __float2half_rn(__fmul_rn(__fmul_rn(float(dot), q.sa), sb_n));
    }
    return;
  }
  if (q.swiglu) {
    // fused SwiGLU form: this lane's column is a gate column (even n) or an up column (odd n)
    // of the interleaved weights; the neighbouring lane holds the other one.  Both lanes of a
    // pair compute every h (same inputs, same arithmetic); the even lane stores the even
    // rows, the odd lane the odd rows.  `out` points at H[row0, n / 2], row stride `stride`.
    // (N is a multiple of 16 here, so a warp's active lanes always hold whole pairs)
    const unsigned lanes = __activemask();
    const bool is_up = (col & 1) != 0;
    const float s_col = is_up ? q.s_up : q.sb;
    const long long z_col = is_up ? q.z_up : q.zb;
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      const long long dot = (long long)int(v[m]) + z_col * (kza - row_sum[m]) - col_term;
      const float mine = __fmul_rn(__fmul_rn(float(dot), q.sa), s_col);
      const float other = __shfl_xor_sync(lanes, mine, 1);
      const float gate = is_up ? other : mine, up = is_up ? mine : other;
      const int h = swiglu_requantize(gate, up, q);
      if (m < M && ((m & 1) != 0) == is_up) out[m * stride] = int8_t(h);
    }
    return;
  }
  int r[ROWS];
#pragma unroll
  for (int m = 0; m < ROWS; ++m) {
    const long long dot = (long long)int(v[m]) + (long long)zb_n * (kza - row_sum[m]) - col_term;
    if (FAST) {
      const float acc = div_rn_inrange(__fmul_rn(__fmul_rn(float(dot), q.sa), sb_n), q.sc, q.rsc);
      r[m] = min(max(add_zero_point(__float2int_rn(acc), q.zc), -128), 127);
    } else {
      r[m] = requantize(float(dot), q.sa, sb_n, q.sc, zc);
    }
  }
  if (q.n_peers > 0) {
    // `out` is C + n of a private result; the gathered form stores at column n_off + n of
    // every peer's [M, ldc] matrix instead (n recovered from the pointer difference)
    for (int p = 0; p < q.n_peers; ++p) {
      int8_t* dst = q.peers[p] + size_t(row0) * q.ldc + q.n_off + col;
#pragma unroll
      for (int m = 0; m < ROWS; ++m)
        if (m < M) dst[size_t(m) * q.ldc] = int8_t(r[m]);
    }
    return;
  }
#pragma unroll
  for (int m = 0; m < ROWS; ++m)
    if (m < M) out[m * stride] = int8_t(r[m]);
}

// Sixteen packed bytes (32 weights, k ascending, high nibble first) -> 32 bytes 0..15.
__device__ __forceinline__ void skinny_unpack32(const uint4& packed, uint4& first, uint4& second) {
  const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
  uint32_t out[8];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const uint32_t hi = (words[w] >> 4) & 0x0f0f0f0fu, lo = words[w] & 0x0f0f0f0fu;
    out[2 * w] = __byte_perm(hi, lo, 0x5140);
    out[2 * w + 1] = __byte_perm(hi, lo, 0x7362);
  }
  first = make_uint4(out[0], out[1], out[2], out[3]);
  second = make_uint4(out[4], out[5], out[6], out[7]);
}

template <bool W4>
__global__ void __launch_bounds__(W4 ? S_W4_THREADS : S_THREADS, 1)
    skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_act,
                  const int8_t* __restrict__ A, int8_t* __restrict__ C, int* __restrict__ workspace,
                  int* __restrict__ counters, const int* __restrict__ row_sum_g, int M, int N, int K,
                  Quant q, int R, int weights_stable, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // A later call's kernel may start its set-up now (it waits for this grid before it touches
  // global memory, see griddepcontrol.wait below).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int S_STAGES = W4 ? S_W4_STAGES : skinny_stages(R);
  const int S_STAGE_BYTES = W4 ? skinny_w4_stage_bytes(R) : S_W_BYTES + skinny_act_bytes(R);
  const int S_PACKED_AT = S_W_BYTES + skinny_act_bytes(R);  // W4: packed rows behind the activations
  SkinnyBarriers* bars = reinterpret_cast<SkinnyBarriers*>(smem + S_STAGES * S_STAGE_BYTES);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int num_kb = (K + S_BK - 1) / S_BK;
  const int tiles = (N + S_TILE_N - 1) / S_TILE_N;
  const int n_mma = R + 16;  // activation rows + the ones row + zero padding
  const int acc_cols = skinny_acc_cols(R), acc_buffers = skinny_acc_buffers(R);

  // Producer state lives outside the role branch: the first ring fill is issued before the
  // CTA-wide set-up barrier, so HBM latency overlaps TMEM allocation and the fills below.
  SkinnySchedule prod_sched(tiles, num_kb, gridDim.x, blockIdx.x, R > 32);
  int p_stage = 0, p_tile = 0, p_kb = 0, p_kb1 = 0, p_shared = -1;
  uint32_t p_phase = 0;
  bool p_ok = true;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S_STAGES; ++s) {
      // W4: the producer's expect_tx for the activations + one arrival per unpack warp
      mbar_init(&bars->full[s], W4 ? 1 + S_W4_UNPACK_WARPS : 1);
      mbar_init(&bars->empty[s], 1);
      mbar_init(&bars->raw_full[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], S_EPI_WARPS);
    }
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    __syncwarp();
    // The grid ahead of this one in the stream is still finishing (its slowest SMs end several
    // microseconds after its fastest, and its completion takes a couple more to reach this
    // grid).  Use that time for the first ring fill of weights.  With prepared weights the
    // caller has promised that B does not change, so the boxes are loaded into shared memory
    // right away and only the activations wait.  Otherwise B might be the output of that
    // grid, and all that is safe is a hint: an L2 prefetch brings nothing into the SM, and L2
    // is the point of coherence for every SM's global accesses, so it is harmless even if B
    // were still being written; the loads proper then start after griddepcontrol.wait and
    // find their data in L2.
    if (lane == 0) {
      SkinnySchedule early(tiles, num_kb, gridDim.x, blockIdx.x, R > 32);
      int e_tile = 0, e_kb = 0, e_kb1 = 0, e_shared = -1;
      for (int i = 0; i < S_STAGES; ++i) {
        if (e_kb == e_kb1 && !early.next(e_tile, e_kb, e_kb1, e_shared)) break;
        uint8_t* sw = smem + i * S_STAGE_BYTES;
        if (W4) {
          // w_q is [N, K/2]: x = packed byte offset of the k block, y = weight row
          if (weights_stable) {
            mbar_arrive_expect_tx(&bars->raw_full[i], S_W4_PACKED_BYTES);
            tma_load_2d(sw + S_PACKED_AT, &map_w, &bars->raw_full[i], e_kb * (S_BK / 2),
                        e_tile * S_TILE_N);
            tma_load_2d(sw + S_PACKED_AT + S_W4_PACKED_BYTES / 2, &map_w, &bars->raw_full[i],
                        e_kb * (S_BK / 2), e_tile * S_TILE_N + 128);
          } else {
            tma_prefetch_l2_2d(&map_w, e_kb * (S_BK / 2), e_tile * S_TILE_N);
            tma_prefetch_l2_2d(&map_w, e_kb * (S_BK / 2), e_tile * S_TILE_N + 128);
          }
        } else if (weights_stable) {
          mbar_arrive_expect_tx(&bars->full[i], S_W_BYTES + R * 128);
          tma_load_2d(sw, &map_w, &bars->full[i], e_tile * S_TILE_N, e_kb * S_BK);
          tma_load_2d(sw + S_BOX_BYTES, &map_w, &bars->full[i], e_tile * S_TILE_N + 128, e_kb * S_BK);
        } else {
          tma_prefetch_l2_2d(&map_w, e_tile * S_TILE_N, e_kb * S_BK);
          tma_prefetch_l2_2d(&map_w, e_tile * S_TILE_N + 128, e_kb * S_BK);
        }
        ++e_kb;
      }
    }
    __syncwarp();
    // From here on memory that the grids ahead may have written is read: wait for them (no-op
    // without such a dependency).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = 0; i < S_STAGES; ++i) {
      if (p_kb == p_kb1 && !prod_sched.next(p_tile, p_kb, p_kb1, p_shared)) break;
      if (lane == 0) {
        uint8_t* sw = smem + p_stage * S_STAGE_BYTES;
        if (W4) {
          if (!weights_stable) {
            mbar_arrive_expect_tx(&bars->raw_full[p_stage], S_W4_PACKED_BYTES);
            tma_load_2d(sw + S_PACKED_AT, &map_w, &bars->raw_full[p_stage], p_kb * (S_BK / 2),
                        p_tile * S_TILE_N);
            tma_load_2d(sw + S_PACKED_AT + S_W4_PACKED_BYTES / 2, &map_w, &bars->raw_full[p_stage],
                        p_kb * (S_BK / 2), p_tile * S_TILE_N + 128);
          }
          mbar_arrive_expect_tx(&bars->full[p_stage], R * 128);
        } else if (!weights_stable) {
          mbar_arrive_expect_tx(&bars->full[p_stage], S_W_BYTES + R * 128);
          tma_load_2d(sw, &map_w, &bars->full[p_stage], p_tile * S_TILE_N, p_kb * S_BK);
          tma_load_2d(sw + S_BOX_BYTES, &map_w, &bars->full[p_stage], p_tile * S_TILE_N + 128, p_kb * S_BK);
        }
        tma_load_2d(sw + S_W_BYTES, &map_act, &bars->full[p_stage], p_kb * S_BK, 0);
      }
      ++p_kb;
      if (++p_stage == S_STAGES) {
        p_stage = 0;
        p_phase ^= 1;
      }
    }
  } else {
    // Rows R .. R+15 of every ring slot's activation tile are never touched by TMA (its box
    // has R rows): row R is all ones when colsum(B) is needed, the rest zero.  A constant
    // row is the same under any swizzle.
    for (int i = threadIdx.x - 32; i < S_STAGES * 16 * 8; i += int(blockDim.x) - 32) {
      const int stage = i / (16 * 8), row = (i / 8) % 16, chunk = i % 8;
      const uint32_t fill = (row == 0 && q.za != 0) ? 0x01010101u : 0u;
      uint4* dst = reinterpret_cast<uint4*>(smem + stage * S_STAGE_BYTES + S_W_BYTES +
                                            (R + row) * 128 + chunk * 16);
      *dst = make_uint4(fill, fill, fill, fill);
    }
    if (threadIdx.x >= 32 && threadIdx.x < 64) bars->row_sum[threadIdx.x - 32] = 0;
    fence_proxy_async_smem();
    if (warp == 1) {
      tmem_alloc(&bars->tmem_base, skinny_tmem_cols(R));
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------- TMA producer (rest)
    while (p_ok) {
      if (p_kb == p_kb1 && !prod_sched.next(p_tile, p_kb, p_kb1, p_shared)) break;
      if (lane == 0) {
        p_ok = mbar_wait(&bars->empty[p_stage], p_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY);
        if (p_ok) {
          uint8_t* sw = smem + p_stage * S_STAGE_BYTES;
          if (W4) {
            mbar_arrive_expect_tx(&bars->raw_full[p_stage], S_W4_PACKED_BYTES);
            tma_load_2d(sw + S_PACKED_AT, &map_w, &bars->raw_full[p_stage], p_kb * (S_BK / 2),
                        p_tile * S_TILE_N);
            tma_load_2d(sw + S_PACKED_AT + S_W4_PACKED_BYTES / 2, &map_w, &bars->raw_full[p_stage],
                        p_kb * (S_BK / 2), p_tile * S_TILE_N + 128);
            mbar_arrive_expect_tx(&bars->full[p_stage], R * 128);
          } else {
            mbar_arrive_expect_tx(&bars->full[p_stage], S_W_BYTES + R * 128);
            tma_load_2d(sw, &map_w, &bars->full[p_stage], p_tile * S_TILE_N, p_kb * S_BK);
            tma_load_2d(sw + S_BOX_BYTES, &map_w, &bars->full[p_stage], p_tile * S_TILE_N + 128, p_kb * S_BK);
          }
          tma_load_2d(sw + S_W_BYTES, &map_act, &bars->full[p_stage], p_kb * S_BK, 0);
        }
      }
      p_ok = __shfl_sync(0xffffffffu, p_ok, 0);
      ++p_kb;
      if (++p_stage == S_STAGES) {
        p_stage = 0;
        p_phase ^= 1;
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    // D[n, m] += W[n, k] * act[m, k]: the W box is M-major (128 columns contiguous), the
    // activations K-major.
    // (W4: the unpacked weights are unsigned bytes in a K-major tile)
    const uint32_t idesc = umma_idesc(/*D=s32*/ 2, /*A=s8 or u8*/ W4 ? 0 : 1, /*B=s8*/ 1,
                                      /*A M-major, W4: K-major*/ W4 ? 0 : 1, /*B K-major*/ 0, 128,
                                      uint32_t(n_mma));
    SkinnySchedule sched(tiles, num_kb, gridDim.x, blockIdx.x, R > 32);
    int stage = 0;
    uint32_t phase = 0;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    int tile, kb0, kb1, shared_index;
    while (ok && sched.next(tile, kb0, kb1, shared_index)) {
      if (lane == 0) {
        ok = mbar_wait(&bars->acc_empty[buf], buf_phase ^ 1, abort_flag, status,
                       STATUS_TIMEOUT_TMEM_EMPTY);
        tc_fence_after_sync();
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(&bars->full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
          if (ok) {
            tc_fence_after_sync();
            const uint32_t sw = smem_u32(smem + stage * S_STAGE_BYTES);
            const uint32_t sact = sw + S_W_BYTES;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint32_t tmem_d = tmem_base + (buf * 2 + half) * acc_cols;
#pragma unroll
              for (int j = 0; j < S_BK / S_UMMA_K; ++j) {
                const uint64_t da =
                    smem_desc(sw + half * S_BOX_BYTES + j * (W4 ? S_UMMA_K : S_UMMA_K * 128), 16, 1024,
                              SMEM_SWIZZLE_128B);
                const uint64_t db = smem_desc(sact + j * S_UMMA_K, 16, 1024, SMEM_SWIZZLE_128B);
                umma_i8(tmem_d, da, db, idesc, (kb == kb0 && j == 0) ? 0u : 1u);
              }
            }
            umma_commit(&bars->empty[stage]);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (++stage == S_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (lane == 0 && ok) umma_commit(&bars->acc_full[buf]);
      __syncwarp();
      if (++buf == acc_buffers) {
        buf = 0;
        buf_phase ^= 1;
      }
    }
  } else if (W4 && warp >= 2 + S_EPI_WARPS) {
    // ------------------------------------------------- nibble unpacking (W4 only)
    // 1024 sixteen-byte pieces per stage (256 rows x 4), eight per thread: consecutive threads
    // take consecutive pieces (contiguous loads); the two 16-byte chunks a piece expands to
    // go to the swizzled positions 2p and 2p+1 of its row (conflict free: the eight threads
    // of a store phase cover two rows of opposite parity).
    const int t = (warp - 2 - S_EPI_WARPS) * 32 + lane;  // 0 .. 127
    SkinnySchedule sched(tiles, num_kb, gridDim.x, blockIdx.x, R > 32);
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int tile, kb0, kb1, shared_index;
    while (ok && sched.next(tile, kb0, kb1, shared_index)) {
      for (int kb = kb0; kb < kb1 && ok; ++kb) {
        ok = mbar_wait(&bars->raw_full[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* su = smem + stage * S_STAGE_BYTES;
        const uint8_t* sraw = su + S_PACKED_AT;
#pragma unroll
        for (int i = 0; i < 1024 / (32 * S_W4_UNPACK_WARPS); ++i) {
          const int piece = t + 32 * S_W4_UNPACK_WARPS * i;
          const int row = piece >> 2, p = piece & 3;  // row 0..255: half = row / 128
          const uint4 packed = *reinterpret_cast<const uint4*>(sraw + piece * 16);
          uint4 first, second;
          skinny_unpack32(packed, first, second);
          uint8_t* dst = su + row * 128;  // the two 128-row halves are contiguous
          *reinterpret_cast<uint4*>(dst + (((2 * p) ^ (row & 7)) << 4)) = first;
          *reinterpret_cast<uint4*>(dst + (((2 * p + 1) ^ (row & 7)) << 4)) = second;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->full[stage]);
        if (++stage == S_STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp - 2;
    const int quarter = warp % 4;     // TMEM lanes 32*quarter .. +31
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    asm volatile("griddepcontrol.wait;" ::: "memory");  // before reading A / touching C, workspace
    // rowsum(A) for the zero-point identity.  Up to 32 rows the activations are tiny and every
    // CTA sums them itself; beyond that a pre-pass has done it once (row_sum_g).
    if ((q.zb != 0 || q.zb_vec != nullptr || (q.swiglu && q.z_up != 0)) && R > 32) {
      for (int m = et; m < M; m += S_EPI_WARPS * 32) bars->row_sum[m] = __ldcg(row_sum_g + m);
    } else if (q.zb != 0 || q.zb_vec != nullptr || (q.swiglu && q.z_up != 0)) {
      for (int m = ew; m < M; m += S_EPI_WARPS) {
        const int4* a = reinterpret_cast<const int4*>(A + size_t(m) * K);
        int acc = 0;
        for (int i = lane; i < K / 16; i += 32) {
          const int4 v = __ldg(a + i);
          acc = __dp4a(v.x, 0x01010101, acc);
          acc = __dp4a(v.y, 0x01010101, acc);
          acc = __dp4a(v.z, 0x01010101, acc);
          acc = __dp4a(v.w, 0x01010101, acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) bars->row_sum[m] = acc;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const long long kza = (long long)K * q.za;
    const float zc = float(q.zc);
    const int ws_rows = M + 1;  // workspace rows per shared tile: M dot rows + the colsum row
    SkinnySchedule sched(tiles, num_kb, gridDim.x, blockIdx.x, R > 32);
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    int tile, kb0, kb1, shared_index;
    while (sched.next(tile, kb0, kb1, shared_index)) {
      ok = mbar_wait(&bars->acc_full[buf], buf_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL);
      // All four epilogue warps go on or give up together (they meet at named barriers below).
      {
        uint32_t all_ok;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ok)
            : "r"(uint32_t(ok))
            : "memory");
        ok = all_ok != 0;
      }
      if (!ok) break;
      tc_fence_after_sync();
      const int cur = buf;
      if (++buf == acc_buffers) {
        buf = 0;
        buf_phase ^= 1;
      }
      if (!W4 && R > 32) {
        // 64 or 128 activation rows: whole tiles only (no partial sums to flush); each thread
        // requantises its column 32 rows at a time.
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const uint32_t taddr = tmem_base + (cur * 2 + half) * acc_cols + (uint32_t(quarter * 32) << 16);
          const int n_local = quarter * 32 + lane;
          const int n = tile * S_TILE_N + half * 128 + n_local;
          uint32_t ones[16];  // accumulator column R: colsum(B) of this thread's column
          tmem_ld_32x16(taddr + R, ones);
          tmem_ld_wait();
          const long long col_term = (long long)q.za * int(ones[0]);
          float sb_n = q.sb;
          int zb_n = q.zb;
          if (q.sb_vec && n < N) {
            sb_n = __ldg(q.sb_vec + n);
            zb_n = (q.zb_vec ? __ldg(q.zb_vec + n) : 0) + q.zb_bias;
          }
          const bool fast = q.fast_div && (!q.sb_vec || channel_in_fast_range(sb_n, zb_n));
#pragma unroll 1
          for (int r0 = 0; r0 < R; r0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + r0, v);
            tmem_ld_wait();
            if (half == 1 && r0 + 32 >= R) {
              // everything is in registers or stored: hand the TMEM buffer back
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->acc_empty[cur]);
            }
            if (n < N && r0 < M) {
              size_t stride;
              int8_t* at = skinny_out_at(C, q, r0, n, N, stride);
              if (fast)
                skinny_store_rows<32, true>(v, bars->row_sum + r0, kza, col_term, sb_n, zb_n, q, zc,
                                            M - r0, at, stride, n, r0);
              else
                skinny_store_rows<32, false>(v, bars->row_sum + r0, kza, col_term, sb_n, zb_n, q, zc,
                                             M - r0, at, stride, n, r0);
            }
          }
        }
        continue;
      }
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
        uint32_t v[32];   // accumulator columns 0..31: dot rows m (and colsum at column 16 when R = 16)
        uint32_t cs_raw;  // colsum(B) for this thread's column
        {
          const uint32_t taddr =
              tmem_base + (cur * 2 + half) * acc_cols + (uint32_t(quarter * 32) << 16);
          tmem_ld_32x32(taddr, v);
          uint32_t hi[16];
          if (R == 32) tmem_ld_32x16(taddr + 32, hi);
          tmem_ld_wait();
          cs_raw = (R == 32) ? hi[0] : v[16];
        }
        if (half == 1) {
          // both halves are in registers or already flushed: hand the TMEM buffer back
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->acc_empty[cur]);
        }
        const int n_local = quarter * 32 + lane;  // column within the 128-column half
        const int n = tile * S_TILE_N + half * 128 + n_local;
        bool finalize = shared_index < 0;
        if (shared_index >= 0) {
          const int slot = shared_index * 2 + half;
          int* ws = workspace + size_t(slot) * ws_rows * 128;
#pragma unroll
          for (int m = 0; m < 32; ++m)
            if (m < M) atomicAdd(ws + m * 128 + n_local, int(v[m]));
          if (q.za != 0) atomicAdd(ws + M * 128 + n_local, int(cs_raw));
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            const int contributors = sched.contributors(shared_index);
            const int before = atomicAdd(&counters[slot], 1);
            bars->last_flag = (before == contributors - 1);
            if (before == contributors - 1) counters[slot] = 0;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          finalize = bars->last_flag != 0;
          if (finalize) {
            __threadfence();
#pragma unroll
            for (int m = 0; m < 32; ++m)
              if (m < M) {
                v[m] = uint32_t(__ldcg(ws + m * 128 + n_local));
                __stcg(ws + m * 128 + n_local, 0);
              }
            if (q.za != 0) {
              cs_raw = uint32_t(__ldcg(ws + M * 128 + n_local));
              __stcg(ws + M * 128 + n_local, 0);
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");  // last_flag is rewritten by the next half
        }
        if (finalize && n < N) {
          const long long col_term = (long long)q.za * int(cs_raw);
          const float sb_n = q.sb_vec ? __ldg(q.sb_vec + n) : q.sb;
          const int zb_n = q.sb_vec ? (q.zb_vec ? __ldg(q.zb_vec + n) : 0) + q.zb_bias : q.zb;
          const bool fast = q.fast_div && (!q.sb_vec || channel_in_fast_range(sb_n, zb_n));
          size_t stride;
          int8_t* at = skinny_out_at(C, q, 0, n, N, stride);
          if (R == 16) {
            if (fast)
              skinny_store_rows<16, true>(v, bars->row_sum, kza, col_term, sb_n, zb_n, q, zc, M, at, stride, n);
            else
              skinny_store_rows<16, false>(v, bars->row_sum, kza, col_term, sb_n, zb_n, q, zc, M, at, stride, n);
          } else {
            if (fast)
              skinny_store_rows<32, true>(v, bars->row_sum, kza, col_term, sb_n, zb_n, q, zc, M, at, stride, n);
            else
              skinny_store_rows<32, false>(v, bars->row_sum, kza, col_term, sb_n, zb_n, q, zc, M, at, stride, n);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, skinny_tmem_cols(R));
  }
}

// `weights_stable`: the caller guarantees that B has not been written since before the
// previous call on this stream started (prepared weights), see the kernel's first ring fill.
// `cached_row_sum`: rowsum(A) [M] on the device.  Up to 32 rows it may be null (every CTA sums
// the few rows itself); beyond that the caller has to supply it whenever a weight zero point
// can be non-zero (from a pre-pass, or from the producer of the activations).
// W4: `B` is w_q [N, K/2] (packed nibbles; q.zb must already be the zero point + 8), at most
// 32 rows.
template <bool W4 = false>
static bool launch_skinny(DeviceCtx& ctx, const int8_t* A, const void* B, int8_t* C, int M, int N,
                          int K, const Quant& q, int weights_stable = 0,
                          const int* cached_row_sum = nullptr) {
  static bool configured[MAX_DEVICES] = {};
  if (!configured[ctx.device]) {
    cudaFuncSetAttribute(skinny_kernel<W4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         W4 ? skinny_w4_smem_bytes(32) : skinny_smem_bytes(16));
    configured[ctx.device] = true;
  }
  if (W4 && M > 32) return false;
  const int R = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  CUtensorMap map_w, map_act;
  const bool weights_ok =
      W4 ? make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, N, K / 2, K / 2, 128, S_BK / 2,
                              CU_TENSOR_MAP_SWIZZLE_NONE)
         : make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, K, N, N, S_BK, 128,
                              CU_TENSOR_MAP_SWIZZLE_128B);
  if (!weights_ok ||
      !make_tensor_map_2d(&map_act, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, M, K, K, R, S_BK,
                          CU_TENSOR_MAP_SWIZZLE_128B)) {
    note_host_error(STATUS_TENSORMAP_FAILED);
    return false;
  }
  const int tiles = (N + S_TILE_N - 1) / S_TILE_N;
  const int num_kb = (K + S_BK - 1) / S_BK;
  const long long units = (long long)tiles * num_kb;
  int grid = int(std::min<long long>(units, ctx.sm_count));
  {
    // p whole tiles per CTA and nothing shared, if that keeps >= 3/4 of the SMs streaming.
    const int per_cta = (tiles + ctx.sm_count - 1) / ctx.sm_count;
    if (tiles % per_cta == 0 && (tiles / per_cta) * 4 >= ctx.sm_count * 3) grid = tiles / per_cta;
  }
  // More than 32 rows: whole tiles only (CTA c takes tiles c, c + grid, ...), and rowsum(A)
  // comes from a pre-pass instead of being recomputed by every CTA.
  const int* row_sum_g = nullptr;
  if (R > 32) {
    const int per_cta = (tiles + ctx.sm_count - 1) / ctx.sm_count;
    grid = (tiles + per_cta - 1) / per_cta;
    row_sum_g = cached_row_sum;
    if (!row_sum_g && (q.zb != 0 || q.zb_vec != nullptr || (q.swiglu && q.z_up != 0))) return false;
  }
  // Tiles that are split between CTAs (see the schedule above) need the workspace:
  // counters[shared][2] (padded) | partial sums [shared][2][M+1][128] int32, one slot per
  // 128-column half.
  const int shared_tiles = R > 32 ? 0 : tiles - tiles / grid * grid;
  const size_t counter_bytes = (size_t(shared_tiles) * 2 * 4 + 255) & ~size_t(255);
  const size_t ws_bytes = size_t(shared_tiles) * 2 * (M + 1) * 128 * 4;
  uint8_t* base = static_cast<uint8_t*>(device_workspace(ctx, counter_bytes + ws_bytes + 256));
  if (!base) return false;
  const int slot = profile_start();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(W4 ? S_W4_THREADS : S_THREADS);
  cfg.dynamicSmemBytes = W4 ? skinny_w4_smem_bytes(R) : skinny_smem_bytes(R);
  cfg.stream = 0;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  int* ws = reinterpret_cast<int*>(base + counter_bytes);
  int* counters = reinterpret_cast<int*>(base);
  static bool overlap_ok = true;
  cudaError_t err = cudaSuccess;
  for (int attempt = 0; attempt < 2; ++attempt) {
    cfg.numAttrs = (overlap_ok && attempt == 0) ? 1 : 0;
    err = cudaLaunchKernelEx(&cfg, skinny_kernel<W4>, map_w, map_act, A, C, ws, counters, row_sum_g, M, N,
                             K, q, R, weights_stable, ctx.status);
    if (err == cudaSuccess || cfg.numAttrs == 0) break;
    cudaGetLastError();  // attribute refused: launch again, fully serialised
    overlap_ok = false;
  }
  if (err != cudaSuccess) {
    cudaGetLastError();
    profile_stop(slot);
    note_host_error(STATUS_LAUNCH_FAILED);
    return false;  // the caller falls back to another kernel
  }
  profile_stop(slot);
  ++launch_counter();
  return true;
}

}  // namespace i8
}  // namespace texo
