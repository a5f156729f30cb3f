// W4A8 for few activation rows (decode): C [M,N] int8 = requantised A [M,K] (int8) times the
// packed INT4 weights w_q [N,K/2], M <= 16.  Same plan as the W4A16 decode kernel
// (w4_decode.cuh): the packed weights - the only large operand - are read from HBM exactly
// once, by 16-byte loads straight into registers (four lanes of a quad cover 64 consecutive
// bytes = 128 k of one weight row, several such loads in flight per thread), expanded to
// unsigned bytes 0..15 in registers (two masks and two byte permutes per eight weights) and
// multiplied on the tensor cores by mma.sync.m16n8k32 (s8 x u8 -> s32).  Nothing of the
// weights ever crosses shared memory, which is what bounded the TMA + unpack-warps form of
// this path.  The k slots of an MMA are a free permutation as long as both operands agree:
// lane j of a quad supplies, in step s, its own nibbles 8s..8s+7, i.e.
// k = k0 + 32j + 8s + {0..7}; the matching activations are 8 consecutive bytes of a row of A,
// read from a shared-memory copy of A in its natural order (rows padded by 16 bytes, which
// makes the quad's 16-byte reads bank-conflict free).
//
// The sums of the zero-point identity come from the same registers: the nibble sums of a
// weight row from the words a lane loads (dp4a), rowsum(A) from the A fragments of the
// warps that own row group 0.  K is split over the warps of a CTA; partial dots and sums
// are added in a fixed order through shared memory (integers: exact either way).
//   dot = sum a*u - (zB+8) rowsum(A) - zA rowsum(u) + K zA (zB+8),  u = q + 8.
//
// Preconditions (otherwise the caller uses another kernel): M <= 16, K % 128 == 0, K < 2^17,
// A and w_q 16-byte aligned, N * K / 2 < 2^31.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "requant.cuh"

namespace texo {
namespace w4a8 {

constexpr int E_WARPS = 16;
constexpr int E_THREADS = E_WARPS * 32;
constexpr int E_TILES = 4;   // n8 tiles (32 weight rows) per warp
constexpr int E_DEPTH = 3;   // 128-k loads in flight per thread and tile
constexpr int E_ROW_BYTES = 128 + 16;           // one 128-k block of one activation row + pad
constexpr int E_ABLK_BYTES = 16 * E_ROW_BYTES;  // one 128-k block of A (16 rows)
constexpr int E_CHUNK_K = 4096;                 // k of A staged per buffer, over all k parts of the CTA
constexpr int E_A_BYTES = (E_CHUNK_K / 128) * E_ABLK_BYTES;
// reduction area: per warp 4 tiles x 4 accumulators + 4 nibble sums + 2 row sums, x 32 lanes
constexpr int E_RED_WORDS = E_TILES * 4 + E_TILES + 2;
constexpr int E_RED_BYTES = E_WARPS * E_RED_WORDS * 32 * 4;
constexpr int E_SMEM_BYTES = 2 * E_A_BYTES + 128;
static_assert(E_RED_BYTES <= 2 * E_A_BYTES, "the final reduction reuses the activation buffers");

__device__ __forceinline__ void mma_s8u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void e_cp_async_16(void* smem_dst, const void* src, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 16 : 0;  // zero-fill: rows past M, k past the part
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// Stages A[:, p * part_k + k_first + [0, span)) for every k part p of the CTA into `buf`; part
// p's i-th 128-k block lands at block p * (span/128) + i, rows in natural byte order.
__device__ __forceinline__ void stage_a(uint8_t* buf, const int8_t* __restrict__ A, int M, int K,
                                        int k_first, int part_k, int ksplit, int span) {
  // A staged chunk is E_CHUNK_K bytes = E_THREADS / 2 sixteen-byte pieces per row, whatever
  // the k split: a thread owns one piece position and the rows of one parity (consecutive
  // lanes copy consecutive pieces of a row).  ksplit and span are powers of two.
  static_assert(E_CHUNK_K / 16 == E_THREADS / 2, "one piece position per thread pair");
  const int pieces_per_part = span / 16;
  const int part_log = 31 - __clz(pieces_per_part);
  const int piece = threadIdx.x & (E_THREADS / 2 - 1), parity = threadIdx.x / (E_THREADS / 2);
  const int p = piece >> part_log, within = (piece & (pieces_per_part - 1)) * 16;
  const int k_in_part = k_first + within;
  const int kk = p * span + within;
  uint8_t* const dst0 = buf + (kk >> 7) * E_ABLK_BYTES + (kk & 127);
  const bool k_valid = k_in_part < part_k;
  const int8_t* const src0 = A + (k_valid ? size_t(p) * part_k + k_in_part : 0);
  // rows at and beyond M rounded up to even were zeroed once, when the kernel started
#pragma unroll
  for (int pair = 0; pair < 8; ++pair) {
    const int m = 2 * pair + parity;
    if (2 * pair >= M) break;
    const bool valid = k_valid && m < M;
    e_cp_async_16(dst0 + m * E_ROW_BYTES, src0 + (valid ? size_t(m) * K : 0), valid);
  }
}

// grid.x CTAs, each owning 32 * rowgroups weight rows; ksplit = E_WARPS / rowgroups warps share
// a row group, each taking K / ksplit of the k range.  q.zb already includes the +8 of the
// unsigned nibbles (per-channel: q.zb_bias = 8 is added to zb_vec[n]).
__global__ void __launch_bounds__(E_THREADS, 1)
    decode_kernel(const int8_t* __restrict__ A, const uint8_t* __restrict__ w_q, int8_t* __restrict__ C,
                  int M, int N, int K, i8::Quant q, int rowgroups) {
  extern __shared__ uint8_t smem_raw[];
  // scheduled while the grid ahead of it drains; nothing is read before that grid is complete
  grid_dependency_trigger();
  grid_dependency_wait();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int r = lane / 4, j = lane % 4;
  const int ksplit = E_WARPS / rowgroups;
  const int rg = warp % rowgroups, part = warp / rowgroups;
  const int part_k = K / ksplit;        // a multiple of 128
  const int span = E_CHUNK_K / ksplit;  // k per part per staged chunk, a multiple of 128
  const int ipc = span / 128;           // iterations per chunk (a power of two)
  const int ipc_log = 31 - __clz(ipc);
  const int iters = part_k / 128;
  const int chunks = (iters + ipc - 1) >> ipc_log;
  const int n_base = (blockIdx.x * rowgroups + rg) * 32;

  uint32_t w_off[E_TILES];
#pragma unroll
  for (int t = 0; t < E_TILES; ++t)
    w_off[t] = uint32_t(min(n_base + t * 8 + r, N - 1)) * uint32_t(K / 2) + uint32_t(part) * uint32_t(part_k / 2) +
               uint32_t(j * 16);

  int acc[E_TILES][4];
  int usum[E_TILES];      // sum of this lane's nibbles of weight row n_base + 8t + r
  int asum[2] = {0, 0};   // sum of this lane's bytes of activation rows r and r + 8 (row group 0 only)
#pragma unroll
  for (int t = 0; t < E_TILES; ++t) {
    usum[t] = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[t][e] = 0;
  }

  uint4 ring[E_DEPTH][E_TILES];
#pragma unroll
  for (int d = 0; d < E_DEPTH; ++d)
#pragma unroll
    for (int t = 0; t < E_TILES; ++t)
      ring[d][t] = d < iters ? __ldcs(reinterpret_cast<const uint4*>(w_q + w_off[t] + d * 64))
                             : make_uint4(0, 0, 0, 0);

  if (M < 15) {  // rows that are never staged must read as zero in both buffers
    for (int i = threadIdx.x; i < 2 * E_A_BYTES / 16; i += E_THREADS)
      reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }
  stage_a(smem, A, M, K, 0, part_k, ksplit, span);
  asm volatile("cp.async.commit_group;" ::: "memory");

#pragma unroll 1
  for (int it0 = 0; it0 < iters; it0 += E_DEPTH) {
#pragma unroll
    for (int d = 0; d < E_DEPTH; ++d) {
      const int it = it0 + d;
      if (it >= iters) break;  // uniform over the CTA
      const int c = it >> ipc_log;
      if ((it & (ipc - 1)) == 0) {  // entering chunk c (uniform over the CTA)
        __syncthreads();    // everyone is done with chunk c - 1, whose buffer is refilled now
        if (c + 1 < chunks)
          stage_a(smem + ((c + 1) & 1) * E_A_BYTES, A, M, K, (c + 1) * span, part_k, ksplit, span);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // chunk c has landed for every thread
      }
      // this lane's 32 bytes of activation rows r and r + 8 in this 128-k block
      const uint8_t* ab = smem + (c & 1) * E_A_BYTES + (part * ipc + (it & (ipc - 1))) * E_ABLK_BYTES + j * 32;
      const uint4* a_lo = reinterpret_cast<const uint4*>(ab + r * E_ROW_BYTES);
      const uint4* a_hi = reinterpret_cast<const uint4*>(ab + (r + 8) * E_ROW_BYTES);
#pragma unroll
      for (int h = 0; h < 2; ++h) {  // 16 bytes of A per row = two MMA steps
        const uint4 lo = a_lo[h], hi = a_hi[h];
        if (rg == 0) {  // warp-uniform
          asum[0] = __dp4a(int(lo.x), 0x01010101, asum[0]);
          asum[0] = __dp4a(int(lo.y), 0x01010101, asum[0]);
          asum[0] = __dp4a(int(lo.z), 0x01010101, asum[0]);
          asum[0] = __dp4a(int(lo.w), 0x01010101, asum[0]);
          asum[1] = __dp4a(int(hi.x), 0x01010101, asum[1]);
          asum[1] = __dp4a(int(hi.y), 0x01010101, asum[1]);
          asum[1] = __dp4a(int(hi.z), 0x01010101, asum[1]);
          asum[1] = __dp4a(int(hi.w), 0x01010101, asum[1]);
        }
#pragma unroll
        for (int t = 0; t < E_TILES; ++t) {
          // two packed words = 16 nibbles = this lane's k of steps 2h and 2h + 1
          const uint32_t w0 = h == 0 ? ring[d][t].x : ring[d][t].z;
          const uint32_t w1 = h == 0 ? ring[d][t].y : ring[d][t].w;
          const uint32_t e0 = (w0 >> 4) & 0x0f0f0f0fu, o0 = w0 & 0x0f0f0f0fu;  // even / odd k
          const uint32_t e1 = (w1 >> 4) & 0x0f0f0f0fu, o1 = w1 & 0x0f0f0f0fu;
          usum[t] = int(__dp4a(e0 + o0, 0x01010101u, unsigned(usum[t])));
          usum[t] = int(__dp4a(e1 + o1, 0x01010101u, unsigned(usum[t])));
          mma_s8u8(acc[t], lo.x, hi.x, lo.y, hi.y, __byte_perm(e0, o0, 0x5140), __byte_perm(e0, o0, 0x7362));
          mma_s8u8(acc[t], lo.z, hi.z, lo.w, hi.w, __byte_perm(e1, o1, 0x5140), __byte_perm(e1, o1, 0x7362));
        }
      }
      if (it + E_DEPTH < iters) {
#pragma unroll
        for (int t = 0; t < E_TILES; ++t)
          ring[d][t] = __ldcs(reinterpret_cast<const uint4*>(w_q + w_off[t] + (it + E_DEPTH) * 64));
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // the four lanes of a quad hold disjoint k of the same weight row / activation rows
#pragma unroll
  for (int t = 0; t < E_TILES; ++t) {
    usum[t] += __shfl_xor_sync(0xffffffffu, usum[t], 1);
    usum[t] += __shfl_xor_sync(0xffffffffu, usum[t], 2);
  }
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    asum[e] += __shfl_xor_sync(0xffffffffu, asum[e], 1);
    asum[e] += __shfl_xor_sync(0xffffffffu, asum[e], 2);
  }

  // add the k parts through shared memory (the activation buffers are free now)
  int* red = reinterpret_cast<int*>(smem);
  __syncthreads();
  {
    int* mine = red + warp * E_RED_WORDS * 32 + lane;
#pragma unroll
    for (int t = 0; t < E_TILES; ++t) {
#pragma unroll
      for (int e = 0; e < 4; ++e) mine[(t * 4 + e) * 32] = acc[t][e];
      mine[(E_TILES * 4 + t) * 32] = usum[t];
    }
    mine[(E_TILES * 5 + 0) * 32] = asum[0];
    mine[(E_TILES * 5 + 1) * 32] = asum[1];
  }
  __syncthreads();
  if (part == 0) {
    // rowsum(A) of rows r and r + 8: parts of row group 0 (warps p * rowgroups)
    long long row_sum[2] = {0, 0};
    for (int p = 0; p < ksplit; ++p) {
      const int* w0 = red + (p * rowgroups) * E_RED_WORDS * 32 + lane;
      row_sum[0] += w0[(E_TILES * 5 + 0) * 32];
      row_sum[1] += w0[(E_TILES * 5 + 1) * 32];
    }
    const long long kza = (long long)K * q.za;
    const float zc = float(q.zc);
#pragma unroll
    for (int t = 0; t < E_TILES; ++t) {
      long long raw[4] = {0, 0, 0, 0};
      int us = 0;
      for (int p = 0; p < ksplit; ++p) {
        const int* w = red + (p * rowgroups + rg) * E_RED_WORDS * 32 + lane;
#pragma unroll
        for (int e = 0; e < 4; ++e) raw[e] += w[(t * 4 + e) * 32];
        us += w[(E_TILES * 4 + t) * 32];
      }
      // C fragment columns are weight rows 2j and 2j + 1 of the tile: their nibble sums live in
      // the lanes whose r is that row
      const int us_col[2] = {__shfl_sync(0xffffffffu, us, (2 * j) * 4), __shfl_sync(0xffffffffu, us, (2 * j + 1) * 4)};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = r + (e >= 2 ? 8 : 0);
        const int n = n_base + t * 8 + 2 * j + (e & 1);
        if (m >= M || n >= N) continue;
        const float sb_n = q.sb_vec ? __ldg(q.sb_vec + n) : q.sb;
        const long long zb_n = q.sb_vec ? (long long)(q.zb_vec ? __ldg(q.zb_vec + n) : 0) + q.zb_bias : (long long)q.zb;
        const long long dot = raw[e] - zb_n * row_sum[e >= 2 ? 1 : 0] - (long long)q.za * us_col[e & 1] + kza * zb_n;
        C[size_t(m) * N + n] = int8_t(i8::requantize(float(dot), q.sa, sb_n, q.sc, zc));
      }
    }
  }
}

}  // namespace w4a8
}  // namespace texo
