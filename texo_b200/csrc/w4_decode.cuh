// W4A16 for few activation rows (decode): y [M,N] = x [M,K] @ dequant(w_q [N,K/2])^T with
// M <= 16.  The job is to stream the packed weights from HBM exactly once; at 16 rows the
// 256-row CTA-pair tensor kernel would spend 15/16 of its MMA work on padding and take several
// times the HBM time.
//
// Each warp owns 32 weight rows (four n8 tiles of mma.sync.m16n8k16, f16 x f16 -> f32) over a
// contiguous part of K.  The four lanes of a quad read 4 x 16 = 64 consecutive bytes (128 k)
// of one weight row straight from global memory into registers (no shared-memory round trip
// for the weights), D_DEPTH such loads in flight per thread and tile.  The MMA's k slots are a
// free permutation as long as both operands agree on it: lane j of a quad supplies, in MMA
// step s, its own nibbles 4s..4s+3, i.e. k = k0 + 32j + 4s + {0,1,2,3}; the matching x values
// are 4 consecutive halves of rows r and r + 8 of x, kept in shared memory in exactly the
// order of the MMA's A operand (see stage_x): one 16-byte load per step is the operand, and
// it feeds the MMAs of all four tiles.  Nibbles become the exact FP16 integers q - 8 by the byte-permute + one
// HFMA2 conversion of mm_int4.cu (unpack8); per scale group (= one 128-k iteration) each
// tile's 16x8 FP32 partial is folded into the running result with the group's scale,
// acc += s[n,g] * partial, so the only roundings are FP32 accumulations (the property the
// reference kernel keeps, src/mm_int4.cu:31-38 of frezcirno/Texo).  K is split over the warps
// of a CTA (and summed in a fixed order through shared memory at the end: deterministic) so
// that narrow problems still fill the SMs with loads in flight.
//
// Preconditions (otherwise the caller uses another kernel): M <= 16, group_size == 128,
// K % (128 * ksplit) == 0, x and w_q 16-byte aligned, N * K / 2 < 2^31.
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace texo {
namespace w4 {

constexpr int D_WARPS = 16;
constexpr int D_THREADS = D_WARPS * 32;
constexpr int D_TILES = 4;   // n8 tiles (32 weight rows) per warp
constexpr int D_DEPTH = 2;   // 128-k loads in flight per thread and tile
constexpr int D_GROUP_BYTES = 32 * 16;            // one 16-byte x fragment of every lane
constexpr int D_XBLK_BYTES = 8 * D_GROUP_BYTES;   // one 128-k block of x (16 rows) = eight fragments per lane
constexpr int D_CHUNK_K = 2048;                   // k of x staged per buffer, over all k parts of the CTA
constexpr int D_X_BYTES = (D_CHUNK_K / 128) * D_XBLK_BYTES;
constexpr int D_RED_BYTES = D_WARPS * D_TILES * 4 * 32 * 4;  // FP32 partial results of every warp
constexpr int D_SMEM_BYTES = 2 * D_X_BYTES + 128;
static_assert(D_RED_BYTES <= 2 * D_X_BYTES, "the final reduction reuses the x buffers");

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* src, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int bytes = valid ? 4 : 0;  // zero-fill: rows past M, k past K
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// Stages x[:, p * part_k + k_first + [0, span)) for every k part p of the CTA into `buf`; part
// p's i-th 128-k block lands at block p * (span/128) + i.  Inside a block the halves are laid
// out as the MMA wants them: lane (r, j) uses, in MMA step s = 0..7, the A fragment
// {row r: its k 4s, 4s+1 | row r + 8: the same k | row r: k 4s+2, 4s+3 | row r + 8: the same}
// (its k = 32 j + ...), one 16-byte piece at [step s][lane][16 bytes]: a conflict-free
// 16-byte shared load yields the operand's four registers in order, with no register
// shuffling in front of the MMA.
__device__ __forceinline__ void stage_x(uint8_t* buf, const __half* __restrict__ x, int M, int K,
                                        int k_first, int part_k, int ksplit, int span) {
  // A staged chunk is D_CHUNK_K halves = D_THREADS / 2 sixteen-byte pieces per row, whatever
  // the k split: a thread owns one piece position and the rows of one parity.  (A warp so
  // copies sixteen consecutive pieces of two neighbouring rows per step: contiguous global
  // reads, and the 4-byte shared-memory writes of one instruction spread over eight banks,
  // the most this layout allows.)  ksplit and span are powers of two.
  static_assert(D_CHUNK_K / 8 == D_THREADS / 2, "one piece position per thread pair");
  const int pieces_per_part = span / 8;  // 16-byte pieces (8 halves) per row and part
  const int part_log = 31 - __clz(pieces_per_part);
  const int piece = threadIdx.x >> 1, parity = threadIdx.x & 1;
  const int p = piece >> part_log, within = (piece & (pieces_per_part - 1)) * 8;
  const int k_in_part = k_first + within;
  const int kk = p * span + within;  // k index inside the staged chunk, a multiple of 8
  // 8 halves of a row = two steps' worth of one lane: k = 32 j + 8 q + (0..7)
  const int j = (kk >> 5) & 3, q = (kk >> 3) & 3;
  uint8_t* const dst0 = buf + (kk >> 7) * D_XBLK_BYTES + (2 * q) * D_GROUP_BYTES + j * 16;
  const bool k_valid = k_in_part < part_k;
  const __half* const src0 = x + (k_valid ? size_t(p) * part_k + k_in_part : 0);
  // rows at and beyond M rounded up to even were zeroed once, when the kernel started
#pragma unroll
  for (int pair = 0; pair < 8; ++pair) {
    const int m = 2 * pair + parity;
    if (2 * pair >= M) break;
    uint8_t* dst = dst0 + (m & 7) * 64 + (m >> 3) * 4;
    const bool valid = k_valid && m < M;
    const __half* src = src0 + (valid ? size_t(m) * K : 0);
    cp_async_4(dst, src, valid);                          // k 0, 1 -> step 2q, slot of this row
    cp_async_4(dst + 8, src + 2, valid);                  // k 2, 3 -> step 2q, second pair
    cp_async_4(dst + D_GROUP_BYTES, src + 4, valid);      // k 4, 5 -> step 2q + 1
    cp_async_4(dst + D_GROUP_BYTES + 8, src + 6, valid);  // k 6, 7
  }
}

// grid.x CTAs, each owning 32 * rowgroups weight rows; ksplit = D_WARPS / rowgroups warps share
// a row group, each taking K / ksplit of the k range.
__global__ void __launch_bounds__(D_THREADS, 1)
    decode_kernel(const __half* __restrict__ x, const uint8_t* __restrict__ w_q,
                  const __half* __restrict__ scales, __half* __restrict__ y, int M, int N, int K,
                  int rowgroups) {
  extern __shared__ uint8_t smem_raw[];
  // scheduled while the grid ahead of it drains; nothing is read before that grid is complete
  grid_dependency_trigger();
  grid_dependency_wait();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int r = lane / 4, j = lane % 4;
  const int ksplit = D_WARPS / rowgroups;
  const int rg = warp % rowgroups, part = warp / rowgroups;
  const int part_k = K / ksplit;        // a multiple of 128
  const int span = D_CHUNK_K / ksplit;  // k per part per staged chunk, a multiple of 128
  const int ipc = span / 128;           // iterations per chunk (a power of two)
  const int ipc_log = 31 - __clz(ipc);
  const int iters = part_k / 128;       // 128-k iterations (= scale groups) of this warp
  const int chunks = (iters + ipc - 1) >> ipc_log;
  const int groups = K / 128;
  const int n_base = (blockIdx.x * rowgroups + rg) * 32;

  // byte offset of this lane's first 16 bytes in each tile's weight row (rows clamped so that
  // loads of a ragged last block stay inside the matrix), and the element offsets of the
  // scales of the two output columns this thread holds per tile (C fragment: columns 2j, 2j+1)
  uint32_t w_off[D_TILES], s_off[D_TILES][2];
#pragma unroll
  for (int t = 0; t < D_TILES; ++t) {
    w_off[t] = uint32_t(min(n_base + t * 8 + r, N - 1)) * uint32_t(K / 2) + uint32_t(part) * uint32_t(part_k / 2) +
               uint32_t(j * 16);
#pragma unroll
    for (int e = 0; e < 2; ++e)
      s_off[t][e] = uint32_t(min(n_base + t * 8 + 2 * j + e, N - 1)) * uint32_t(groups) + uint32_t(part * iters);
  }

  float total[D_TILES][4];
#pragma unroll
  for (int t = 0; t < D_TILES; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) total[t][e] = 0.f;

  // weight ring: D_DEPTH iterations of 128 k in flight
  uint4 ring[D_DEPTH][D_TILES];
#pragma unroll
  for (int d = 0; d < D_DEPTH; ++d)
#pragma unroll
    for (int t = 0; t < D_TILES; ++t)
      ring[d][t] = d < iters ? __ldcs(reinterpret_cast<const uint4*>(w_q + w_off[t] + d * 64))
                             : make_uint4(0, 0, 0, 0);

  if (M < 15) {  // rows that are never staged must read as zero in both buffers
    for (int i = threadIdx.x; i < 2 * D_X_BYTES / 16; i += D_THREADS)
      reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
  }
  stage_x(smem, x, M, K, 0, part_k, ksplit, span);
  asm volatile("cp.async.commit_group;" ::: "memory");

#pragma unroll 1
  for (int it0 = 0; it0 < iters; it0 += D_DEPTH) {
#pragma unroll
    for (int d = 0; d < D_DEPTH; ++d) {
      const int it = it0 + d;
      if (it >= iters) break;  // uniform over the CTA
      const int c = it >> ipc_log;
      if ((it & (ipc - 1)) == 0) {  // entering chunk c (uniform over the CTA)
        __syncthreads();    // everyone is done with chunk c - 1, whose buffer is refilled now
        if (c + 1 < chunks)
          stage_x(smem + ((c + 1) & 1) * D_X_BYTES, x, M, K, (c + 1) * span, part_k, ksplit, span);
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 1;" ::: "memory");
        __syncthreads();  // chunk c has landed for every thread
      }
      // this lane's eight x fragments of this 128-k block (see stage_x)
      const uint8_t* xb = smem + (c & 1) * D_X_BYTES + (part * ipc + (it & (ipc - 1))) * D_XBLK_BYTES + lane * 16;
      float acc[D_TILES][4];
#pragma unroll
      for (int t = 0; t < D_TILES; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {  // one packed word per tile = two MMA steps
        const uint4 f0 = *reinterpret_cast<const uint4*>(xb + (2 * q4) * D_GROUP_BYTES);
        const uint4 f1 = *reinterpret_cast<const uint4*>(xb + (2 * q4 + 1) * D_GROUP_BYTES);
#pragma unroll
        for (int t = 0; t < D_TILES; ++t) {
          const uint32_t word = q4 == 0 ? ring[d][t].x : q4 == 1 ? ring[d][t].y : q4 == 2 ? ring[d][t].z : ring[d][t].w;
          const uint4 b = unpack8(word);  // 8 nibbles -> halves (k0,k1) (k2,k3) (k4,k5) (k6,k7)
          mma_16816(acc[t], f0.x, f0.y, f0.z, f0.w, b.x, b.y);
          mma_16816(acc[t], f1.x, f1.y, f1.z, f1.w, b.z, b.w);
        }
      }
      // this slot's next load: D_DEPTH iterations ahead
      if (it + D_DEPTH < iters) {
#pragma unroll
        for (int t = 0; t < D_TILES; ++t)
          ring[d][t] = __ldcs(reinterpret_cast<const uint4*>(w_q + w_off[t] + (it + D_DEPTH) * 64));
      }
      // fold the group's partial in with its scale
#pragma unroll
      for (int t = 0; t < D_TILES; ++t) {
        const float s0 = __half2float(__ldg(scales + s_off[t][0] + it));
        const float s1 = __half2float(__ldg(scales + s_off[t][1] + it));
        total[t][0] = fmaf(s0, acc[t][0], total[t][0]);
        total[t][1] = fmaf(s1, acc[t][1], total[t][1]);
        total[t][2] = fmaf(s0, acc[t][2], total[t][2]);
        total[t][3] = fmaf(s1, acc[t][3], total[t][3]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  // sum the k parts in a fixed order through shared memory (the x buffers are free now)
  float* red = reinterpret_cast<float*>(smem);
  __syncthreads();
#pragma unroll
  for (int t = 0; t < D_TILES; ++t)
#pragma unroll
    for (int e = 0; e < 4; ++e) red[((warp * D_TILES + t) * 4 + e) * 32 + lane] = total[t][e];
  __syncthreads();
  if (part == 0) {
#pragma unroll
    for (int t = 0; t < D_TILES; ++t) {
      float out[4] = {0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < ksplit; ++p) {
        const int w = p * rowgroups + rg;
#pragma unroll
        for (int e = 0; e < 4; ++e) out[e] += red[((w * D_TILES + t) * 4 + e) * 32 + lane];
      }
      // C fragment: (row r, columns 2j, 2j+1), (row r + 8, same columns)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = r + (e >= 2 ? 8 : 0);
        const int n = n_base + t * 8 + 2 * j + (e & 1);
        if (m < M && n < N) y[size_t(m) * N + n] = __float2half_rn(out[e]);
      }
    }
  }
}

}  // namespace w4
}  // namespace texo
