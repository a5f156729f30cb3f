// INT8 requantisation shared by the tensor-core kernels that end in an int8 output (the
// INT8 operator and the packed-INT4-weight x INT8-activation operator): the FP32 epilogue of
// frezcirno/Texo src/mm_int8.cu:12-25 and the zero-point identity of :127-129, as a TMEM
// drain.
#pragma once
#include <cstdint>
#include <type_traits>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace texo {
namespace i8 {

// ------------------------------------------------------------------ epilogue
// FP32 requantisation; the operation order is contractual (no reassociation, no
// reciprocal, IEEE division, ties-to-even rounding).
__device__ __forceinline__ int requantize(float dot, float sa, float sb, float sc, float zc) {
  float acc = __fdiv_rn(__fmul_rn(__fmul_rn(dot, sa), sb), sc);
  acc = __fadd_rn(rintf(acc), zc);
  acc = fminf(fmaxf(acc, -128.f), 127.f);
  return __float2int_rn(acc);
}

struct Quant {
  float sa, sb, sc;
  int za, zb, zc;
  float rsc;     // RN(1 / sc), for the branch-free division below
  int fast_div;  // 1 when every quotient of this call is inside that division's safe range
  // Per-output-channel weight quantisation (both null for per-tensor): device arrays [N],
  // 16-byte aligned; column n then uses sb_vec[n] instead of sb and, if zb_vec is not null,
  // zb_vec[n] instead of zb (zb_vec null with sb_vec set means zero point 0 everywhere).
  const float* sb_vec;
  const int* zb_vec;
  // Added to every per-channel zero point read from zb_vec (and standing for it when zb_vec is
  // null): 0 for the INT8 operator, 8 for packed-INT4 weights, whose nibbles the kernels keep
  // unsigned (u = q + 8), so a column's effective zero point is zb_vec[n] + 8.
  int zb_bias;
  // Fused SwiGLU consumer (swiglu != 0): B holds gate and up columns interleaved (column 2j =
  // gate j, 2j+1 = up j); sb / zb describe the gate columns, s_up / z_up the up columns, and
  // the output is H [M, N/2] = requantised up * silu(gate) with scale s_out, zero point z_out.
  int swiglu;
  float s_up, s_out;
  int z_up, z_out;
  // Dequantising drain (out_f16 != 0): no requantisation, the output is FP16 [M, N],
  // y = half(float(dot) * sa * sb).
  int out_f16;
  // Fused all-gather (n_peers > 0): the [M, N] result is a column slab of a wider matrix
  // [M, ldc] that every GPU of the node holds; each finished piece is stored at column
  // n_off + n of ALL of them (plain stores into peer-mapped memory over NVLink), so the
  // gather rides under the main loop and no collective follows.  The C argument is unused.
  int n_peers, ldc, n_off;
  int8_t* peers[8];
  // Optional NVLink multicast mapping of the same [M, ldc] matrix (null = none): one
  // multimem.st to mc + offset is replicated by the switch into every GPU's copy, so a slab
  // leaves this GPU once instead of once per peer.  Used by the staged (whole 128-byte row
  // segment) stores of the CTA-pair drain; everything else keeps the per-peer stores.
  int8_t* mc;
};
constexpr int MAX_PEERS = 8;

// Host side: fills the derived fields.  The branch-free division is exact only while no
// intermediate leaves the normal range, so it is enabled when the scales bound every
// possible numerator: a non-zero |dot| lies in [1, 2^49] (K < 2^17 terms of at most 2^32
// with |zA|, |zB| <= 2^15), hence |dot * sA * sB| in [2^-60, 2^59] for |sA|, |sB| in
// [2^-30, 2^5]; and |sC| in [2^-60, 2^60] keeps quotient and residuals normal.  |zC| <= 2^22
// lets the tail run in integers (see requantize_fast).  Anything else (including NaN or
// infinite scales) takes the plain IEEE division, element by element.
inline Quant make_quant(float sa, float sb, float sc, int za, int zb, int zc, int K) {
  Quant q = {sa, sb, sc, za, zb, zc, 0.f, 0, nullptr, nullptr, 0, 0, 0.f, 0.f, 0, 0, 0, 0, 0, 0, {}, nullptr};
  auto within = [](float v, float lo, float hi) {
    const float a = v < 0 ? -v : v;
    return a >= lo && a <= hi;  // false for NaN
  };
  const bool ok = within(sa, 0x1p-30f, 0x1p5f) && within(sb, 0x1p-30f, 0x1p5f) &&
                  within(sc, 0x1p-60f, 0x1p60f) && za >= -32768 && za <= 32768 && zb >= -32768 &&
                  zb <= 32768 && zc >= -(1 << 22) && zc <= (1 << 22) && K < (1 << 17);
  if (ok) {
    q.rsc = 1.0f / sc;  // correctly rounded on the host
    q.fast_div = 1;
  }
  return q;
}

// x / sc, correctly rounded (identical to __fdiv_rn), for x and sc in the range make_quant
// admits: two Newton corrections of x * RN(1/sc) with exact FMA residuals.  Unlike the IEEE
// division sequence it has no slow-path branch, so the divisions of neighbouring outputs
// interleave instead of running one dependent chain after the other.
__device__ __forceinline__ float div_rn_inrange(float x, float sc, float rsc) {
  const float q0 = __fmul_rn(x, rsc);
  const float r0 = __fmaf_rn(-sc, q0, x);
  const float q1 = __fmaf_rn(r0, rsc, q0);
  const float r1 = __fmaf_rn(-sc, q1, x);
  return __fmaf_rn(r1, rsc, q1);
}

// rint(acc) + zC in integers, for |zC| <= 2^22: `rounded` is cvt.rni.s32 of acc (saturating).
// Clamped to +-2^24 first, so that the sum cannot wrap; the caller saturates to int8.
// Identical to the FP32 tail: if |rint(acc)| <= 2^24 the float add is exact (or lands far
// outside [-128, 127] on the same side); beyond that both forms saturate to the same end.
__device__ __forceinline__ int add_zero_point(int rounded, int zc) {
  return max(-(1 << 24), min(rounded, 1 << 24)) + zc;
}

// Requantisation with that division and the tail done in integers.
__device__ __forceinline__ int requantize_fast(float dot, const Quant& q) {
  const float acc = div_rn_inrange(__fmul_rn(__fmul_rn(dot, q.sa), q.sb), q.sc, q.rsc);
  return add_zero_point(__float2int_rn(acc), q.zc);
}
__device__ __forceinline__ uint32_t pack_sat_s8(int r0, int r1, int r2, int r3) {
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(r3), "r"(r2), "r"(0));
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(r1), "r"(r0), "r"(hi));
  return out;
}

// The scalar checks of make_quant applied to one column's weight scale and zero point.
__device__ __forceinline__ bool channel_in_fast_range(float sb, int zb) {
  const float a = fabsf(sb);
  return a >= 0x1p-30f && a <= 0x1p5f && zb >= -32768 && zb <= 32768;
}

// One thread's 32 consecutive accumulator columns -> 32 int8 in eight words: zero-point
// identity, then requantisation.  `col_sums` holds colsum(B) of the 32 columns (zeros when
// the activation zero point is zero), `rt_row`
// is K*zA - rowsum(A)[m] for this thread's row, so that
//   dot = raw + zB * rt_row - zA * colsum(B)[n].
// PC: per-channel weight scale / zero point, read from q.sb_vec / q.zb_vec at column n0 + ...
// (N is a multiple of 4 on the tensor paths, so a group of four columns is inside or outside
// the matrix as a whole).
template <bool WIDE, bool FAST, bool PC>
__device__ __forceinline__ void requantize_chunk(
    const uint32_t (&v)[32], const int4 (&col_sums)[8],
    typename std::conditional<WIDE, long long, unsigned>::type rt_row, const Quant& q, int n0, int N,
    uint32_t (&packed)[8]) {
  using Wide = typename std::conditional<WIDE, long long, unsigned>::type;
  using Signed = typename std::conditional<WIDE, long long, int>::type;
  const float zc = float(q.zc);
  const Wide tensor_term = Wide(Signed(q.zb)) * rt_row;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    const int csv[4] = {col_sums[g].x, col_sums[g].y, col_sums[g].z, col_sums[g].w};
    float sbv[4] = {q.sb, q.sb, q.sb, q.sb};
    int zbv[4] = {q.zb_bias, q.zb_bias, q.zb_bias, q.zb_bias};
    if (PC && n0 + g * 4 < N) {
      const float4 s4 = __ldg(reinterpret_cast<const float4*>(q.sb_vec + n0 + g * 4));
      sbv[0] = s4.x, sbv[1] = s4.y, sbv[2] = s4.z, sbv[3] = s4.w;
      if (q.zb_vec) {
        const int4 z4 = __ldg(reinterpret_cast<const int4*>(q.zb_vec + n0 + g * 4));
        zbv[0] += z4.x, zbv[1] += z4.y, zbv[2] += z4.z, zbv[3] += z4.w;
      }
    }
    int r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const Wide zb_term = PC ? Wide(Signed(zbv[e])) * rt_row : tensor_term;
      const Wide dot = Wide(Signed(int(v[g * 4 + e]))) + zb_term - Wide(Signed(q.za)) * Wide(Signed(csv[e]));
      const float x = float(Signed(dot));
      if (FAST) {
        const float acc = div_rn_inrange(__fmul_rn(__fmul_rn(x, q.sa), sbv[e]), q.sc, q.rsc);
        r[e] = add_zero_point(__float2int_rn(acc), q.zc);
      } else {
        r[e] = requantize(x, q.sa, sbv[e], q.sc, zc);
      }
    }
    packed[g] = pack_sat_s8(r[0], r[1], r[2], r[3]);
  }
}

// Whether all per-channel parameters of the 32 columns starting at n0 allow the branch-free
// division (warp-uniform: every lane of an epilogue warp looks at the same columns).
__device__ __forceinline__ bool chunk_channels_fast(const Quant& q, int n0, int N) {
  bool ok = true;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (n0 + g * 4 >= N) continue;
    const float4 s4 = __ldg(reinterpret_cast<const float4*>(q.sb_vec + n0 + g * 4));
    int4 z4 = make_int4(0, 0, 0, 0);
    if (q.zb_vec) z4 = __ldg(reinterpret_cast<const int4*>(q.zb_vec + n0 + g * 4));
    ok = ok && channel_in_fast_range(s4.x, z4.x + q.zb_bias) && channel_in_fast_range(s4.y, z4.y + q.zb_bias) &&
         channel_in_fast_range(s4.z, z4.z + q.zb_bias) && channel_in_fast_range(s4.w, z4.w + q.zb_bias);
  }
  return ok;
}

// Picks the form of requantize_chunk for one chunk.
template <bool WIDE>
__device__ __forceinline__ void requantize_chunk_auto(
    const uint32_t (&v)[32], const int4 (&col_sums)[8],
    typename std::conditional<WIDE, long long, unsigned>::type rt_row, const Quant& q, int n0, int N,
    uint32_t (&packed)[8]) {
  if (q.sb_vec == nullptr) {
    if (q.fast_div)
      requantize_chunk<WIDE, true, false>(v, col_sums, rt_row, q, n0, N, packed);
    else
      requantize_chunk<WIDE, false, false>(v, col_sums, rt_row, q, n0, N, packed);
  } else {
    if (q.fast_div && chunk_channels_fast(q, n0, N))
      requantize_chunk<WIDE, true, true>(v, col_sums, rt_row, q, n0, N, packed);
    else
      requantize_chunk<WIDE, false, true>(v, col_sums, rt_row, q, n0, N, packed);
  }
}

// K*zA - rowsum(A)[m]: the per-row factor of the zero-point identity.  The row sums exist
// only when some weight zero point can be non-zero.
template <bool WIDE>
__device__ __forceinline__ typename std::conditional<WIDE, long long, unsigned>::type row_factor(
    const int* __restrict__ row_sum, int m, bool row_ok, int K, const Quant& q) {
  using Wide = typename std::conditional<WIDE, long long, unsigned>::type;
  using Signed = typename std::conditional<WIDE, long long, int>::type;
  Wide rt = Wide(Signed(K)) * Wide(Signed(q.za));
  if (row_ok && (q.zb != 0 || q.zb_vec != nullptr || (q.swiglu && q.z_up != 0)))
    rt -= Wide(Signed(__ldcg(row_sum + m)));
  return rt;
}

// 16 bytes to a multicast address: the switch replicates the store into every GPU bound to
// the multicast object (the bits are not interpreted; .v4.f32 is just the 16-byte form).
__device__ __forceinline__ void multimem_st_16(void* mc_addr, const int4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__int_as_float(v.x)), "f"(__int_as_float(v.y)), "f"(__int_as_float(v.z)),
               "f"(__int_as_float(v.w))
               : "memory");
}

// Raster of the CTA-pair kernels: tile rows are taken in groups, a group's tiles are walked
// column by column, so the CTAs running at one time share a group's rows of A and a few
// columns of B in L2.  Measured on B200 (stateless INT8 call): 8192^3 409 / 402 / 395 / 411 us
// and 4096^3 65 / 74 / 65 / 65 us for groups of 4 / 8 / 16 / 32 tile rows; with K = 28672 a
// group of 16 (117 MB of A) no longer fits L2 and 8 is faster again.  The host picks the
// group size (raster_group_rows) and passes it to the kernel.
constexpr int P_GROUP_M = 16;  // largest group; also orders the sums' items (any order is correct)

// Tile rows per raster group for rows of `row_bytes` bytes of A: sixteen while a group's rows
// of A stay within 48 MB, else eight.
inline int raster_group_rows(long long row_bytes) {
  return 16LL * 256 * row_bytes <= (48LL << 20) ? 16 : 8;
}

__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int group_rows, int& tm,
                                                 int& tn) {
  const int group_tiles = group_rows * tiles_n;
  const int first_m = tile / group_tiles * group_rows;
  const int group_m = min(tiles_m - first_m, group_rows);
  const int in_group = tile % group_tiles;
  tm = first_m + in_group % group_m;
  tn = in_group / group_m;
}

// Sum of the sixteen signed bytes of v, added to acc.
__device__ __forceinline__ int sum_bytes(const int4& v, int acc) {
  acc = __dp4a(v.x, 0x01010101, acc);
  acc = __dp4a(v.y, 0x01010101, acc);
  acc = __dp4a(v.z, 0x01010101, acc);
  return __dp4a(v.w, 0x01010101, acc);
}


// up * silu(gate), requantised: the arithmetic of the reference's src/swiglu.cu:15-18
// (x2 * x1 / (1 + __expf(-x1)), FP32, same operation order) on the dequantised gate and up
// values, then clamp(rint(h / s_out) + z_out).
__device__ __forceinline__ int swiglu_requantize(float gate, float up, const Quant& q) {
  const float h = __fdiv_rn(__fmul_rn(up, gate), __fadd_rn(1.f, __expf(-gate)));
  float r = __fadd_rn(rintf(__fdiv_rn(h, q.s_out)), float(q.z_out));
  r = fminf(fmaxf(r, -128.f), 127.f);
  return __float2int_rn(r);
}

// The SwiGLU form of drain_half (below): this thread's row, 128 accumulator columns = 64
// (gate, up) pairs -> 64 int8 of H, sixteen per 32-column chunk.  N counts accumulator
// columns (2F); H has row stride N / 2.
template <bool WIDE>
__device__ __forceinline__ void drain_half_swiglu(uint32_t tmem_row_addr, int col0, int n_tile0,
                                                  int m, bool row_ok, int8_t* __restrict__ H,
                                                  const int* __restrict__ row_sum,
                                                  const int* __restrict__ col_sum, int N, int K,
                                                  const Quant& q, int h_vector_ok) {
  using Wide = typename std::conditional<WIDE, long long, unsigned>::type;
  using Signed = typename std::conditional<WIDE, long long, int>::type;
  const Wide rt_row = row_factor<WIDE>(row_sum, m, row_ok, K, q);
  const Wide gate_term = Wide(Signed(q.zb)) * rt_row, up_term = Wide(Signed(q.z_up)) * rt_row;
  int8_t* h_row = H + size_t(row_ok ? m : 0) * (N / 2);
#pragma unroll 1
  for (int chunk = 0; chunk < 4; ++chunk) {
    const int col = col0 + chunk * 32;
    const int n0 = n_tile0 + col;
    uint32_t v[32];
    tmem_ld_32x32(tmem_row_addr + col, v);
    tmem_ld_wait();
    if (n0 >= N) continue;  // warp-uniform
    uint32_t packed[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) {  // eight accumulator columns -> four outputs
      int4 c0 = make_int4(0, 0, 0, 0), c1 = c0;
      if (q.za != 0) {
        c0 = __ldcg(reinterpret_cast<const int4*>(col_sum + n0 + g * 8));
        c1 = __ldcg(reinterpret_cast<const int4*>(col_sum + n0 + g * 8 + 4));
      }
      const int csv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      int r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const Wide dg = Wide(Signed(int(v[g * 8 + 2 * e]))) + gate_term -
                        Wide(Signed(q.za)) * Wide(Signed(csv[2 * e]));
        const Wide du = Wide(Signed(int(v[g * 8 + 2 * e + 1]))) + up_term -
                        Wide(Signed(q.za)) * Wide(Signed(csv[2 * e + 1]));
        const float gate = __fmul_rn(__fmul_rn(float(Signed(dg)), q.sa), q.sb);
        const float up = __fmul_rn(__fmul_rn(float(Signed(du)), q.sa), q.s_up);
        r[e] = swiglu_requantize(gate, up, q);
      }
      packed[g] = pack_sat_s8(r[0], r[1], r[2], r[3]);
    }
    if (row_ok) {
      const int f0 = n0 / 2;  // first output column of this chunk
      if (h_vector_ok && f0 + 16 <= N / 2) {
        *reinterpret_cast<int4*>(h_row + f0) = make_int4(packed[0], packed[1], packed[2], packed[3]);
      } else {
        for (int e = 0; e < 16 && f0 + e < N / 2; ++e)
          h_row[f0 + e] = int8_t((packed[e / 4] >> (8 * (e % 4))) & 0xff);
      }
    }
  }
}

// The dequantising form of drain_half (below): y = half(float(dot) * sA * sB), 32 halves per
// 32-column chunk.  Y is FP16 [M, N].
template <bool WIDE>
__device__ __forceinline__ void drain_half_f16(uint32_t tmem_row_addr, int col0, int n_tile0, int m,
                                               bool row_ok, __half* __restrict__ Y,
                                               const int* __restrict__ row_sum,
                                               const int* __restrict__ col_sum, int N, int K,
                                               const Quant& q, int y_vector_ok) {
  using Wide = typename std::conditional<WIDE, long long, unsigned>::type;
  using Signed = typename std::conditional<WIDE, long long, int>::type;
  const Wide rt_row = row_factor<WIDE>(row_sum, m, row_ok, K, q);
  const Wide zb_term = Wide(Signed(q.zb)) * rt_row;
  __half* y_row = Y + size_t(row_ok ? m : 0) * N;
#pragma unroll 1
  for (int chunk = 0; chunk < 4; ++chunk) {
    const int col = col0 + chunk * 32;
    const int n0 = n_tile0 + col;
    uint32_t v[32];
    tmem_ld_32x32(tmem_row_addr + col, v);
    tmem_ld_wait();
    if (n0 >= N) continue;  // warp-uniform
    uint32_t packed[16];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      int4 cs = make_int4(0, 0, 0, 0);
      if (q.za != 0) cs = __ldcg(reinterpret_cast<const int4*>(col_sum + n0 + g * 4));
      const int csv[4] = {cs.x, cs.y, cs.z, cs.w};
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const Wide dot = Wide(Signed(int(v[g * 4 + e]))) + zb_term - Wide(Signed(q.za)) * Wide(Signed(csv[e]));
        y[e] = __fmul_rn(__fmul_rn(float(Signed(dot)), q.sa), q.sb);
      }
      const __half2 lo = __floats2half2_rn(y[0], y[1]), hi = __floats2half2_rn(y[2], y[3]);
      packed[2 * g] = *reinterpret_cast<const uint32_t*>(&lo);
      packed[2 * g + 1] = *reinterpret_cast<const uint32_t*>(&hi);
    }
    if (row_ok) {
      if (y_vector_ok && n0 + 32 <= N) {
        int4* dst = reinterpret_cast<int4*>(y_row + n0);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          dst[i] = make_int4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
      } else {
        for (int e = 0; e < 32 && n0 + e < N; ++e) {
          const uint32_t word = packed[e / 2];
          const unsigned short bits = (e & 1) ? (unsigned short)(word >> 16) : (unsigned short)(word & 0xffff);
          reinterpret_cast<unsigned short*>(y_row)[n0 + e] = bits;
        }
      }
    }
  }
}

// Drains 128 columns [col0, col0+128) of one accumulator for this thread's row: zero-point
// identity, FP32 requantisation, 32 int8 per 32-column chunk, vector stores when possible.
template <bool WIDE>
__device__ __forceinline__ void drain_half(uint32_t tmem_row_addr, int col0, int n_tile0, int m,
                                           bool row_ok, int8_t* __restrict__ C,
                                           const int* __restrict__ row_sum,
                                           const int* __restrict__ col_sum, int N, int K,
                                           const Quant& q, int c_vector_ok,
                                           uint8_t* gather_stage = nullptr,
                                           int4* colsum_stage = nullptr) {
  if (q.swiglu) {
    drain_half_swiglu<WIDE>(tmem_row_addr, col0, n_tile0, m, row_ok, C, row_sum, col_sum, N, K, q,
                            c_vector_ok);
    return;
  }
  if (q.out_f16) {
    drain_half_f16<WIDE>(tmem_row_addr, col0, n_tile0, m, row_ok, reinterpret_cast<__half*>(C),
                         row_sum, col_sum, N, K, q, c_vector_ok);
    return;
  }
  const auto rt_row = row_factor<WIDE>(row_sum, m, row_ok, K, q);
  int8_t* c_row = C + size_t(row_ok ? m : 0) * N;
  // Fused all-gather, whole 128-column half inside the matrix: the warp's 32 rows x 128 bytes
  // go through a 4 KiB shared-memory tile so that every store instruction writes four
  // complete 128-byte row segments.  Stores into a peer's memory travel over NVLink as they
  // are issued; 16-byte pieces scattered over 32 rows used a fifth of the link rate.
  const bool staged = q.n_peers > 0 && gather_stage != nullptr && c_vector_ok &&
                      n_tile0 + col0 + 128 <= N;  // warp-uniform
  const int lane = threadIdx.x % 32;
  // Column sums (col_sum is padded to a multiple of the tile width: never out of bounds; read
  // through L2: other CTAs of this grid may have produced them).  With a staging area the warp
  // fetches the 128 sums of its half in one load, four per lane, and every chunk reads its 32
  // from shared memory: one trip to L2 per drain instead of one per chunk.
  const bool staged_sums = colsum_stage != nullptr && q.za != 0;
  if (staged_sums) {
    __syncwarp();  // the previous drain's readers are done
    colsum_stage[lane] = __ldcg(reinterpret_cast<const int4*>(col_sum + n_tile0 + col0) + lane);
    __syncwarp();
  }
#pragma unroll 1
  for (int chunk = 0; chunk < 4; ++chunk) {
    const int col = col0 + chunk * 32;
    const int n0 = n_tile0 + col;
    uint32_t v[32];
    tmem_ld_32x32(tmem_row_addr + col, v);
    // the chunk's column sums travel while the accumulator columns do
    int4 col_sums[8];
#pragma unroll
    for (int g = 0; g < 8; ++g)
      col_sums[g] = staged_sums ? colsum_stage[chunk * 8 + g]
                    : q.za != 0 ? __ldcg(reinterpret_cast<const int4*>(col_sum + n0 + g * 4))
                                : make_int4(0, 0, 0, 0);
    tmem_ld_wait();
    if (n0 >= N) continue;  // warp-uniform
    uint32_t packed[8];
    requantize_chunk_auto<WIDE>(v, col_sums, rt_row, q, n0, N, packed);
    if (staged) {
      // row `lane` of the tile, 16-byte pieces 2*chunk and 2*chunk+1, XOR-swizzled by the row
      uint8_t* row = gather_stage + lane * 128;
      *reinterpret_cast<int4*>(row + (((2 * chunk) ^ (lane & 7)) << 4)) =
          make_int4(packed[0], packed[1], packed[2], packed[3]);
      *reinterpret_cast<int4*>(row + (((2 * chunk + 1) ^ (lane & 7)) << 4)) =
          make_int4(packed[4], packed[5], packed[6], packed[7]);
    } else if (row_ok && q.n_peers > 0) {
      const size_t at = size_t(m) * q.ldc + q.n_off + n0;
      for (int p = 0; p < q.n_peers; ++p) {
        int8_t* dst_row = q.peers[p] + at;
        if (c_vector_ok && n0 + 32 <= N) {
          int4* dst = reinterpret_cast<int4*>(dst_row);
          dst[0] = make_int4(packed[0], packed[1], packed[2], packed[3]);
          dst[1] = make_int4(packed[4], packed[5], packed[6], packed[7]);
        } else {
          for (int e = 0; e < 32 && n0 + e < N; ++e)
            dst_row[e] = int8_t((packed[e / 4] >> (8 * (e % 4))) & 0xff);
        }
      }
    } else if (row_ok) {
      if (c_vector_ok && n0 + 32 <= N) {
        int4* dst = reinterpret_cast<int4*>(c_row + n0);
        dst[0] = make_int4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_int4(packed[4], packed[5], packed[6], packed[7]);
      } else {
        for (int e = 0; e < 32 && n0 + e < N; ++e)
          c_row[n0 + e] = int8_t((packed[e / 4] >> (8 * (e % 4))) & 0xff);
      }
    }
  }
  if (staged) {
    __syncwarp();
    const unsigned rows_ok = __ballot_sync(0xffffffffu, row_ok);  // bit r: row r is inside M
    const int m_base = m - lane;  // first row of this warp's 32
    const int piece = lane & 7;
    if (q.mc != nullptr) {
      // one store per piece into the multicast mapping: NVSwitch writes all copies
      int8_t* dst = q.mc + q.n_off + n_tile0 + col0 + piece * 16;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        if ((rows_ok >> r) & 1u) {
          const int4 value =
              *reinterpret_cast<const int4*>(gather_stage + r * 128 + ((piece ^ (r & 7)) << 4));
          multimem_st_16(dst + size_t(m_base + r) * q.ldc, value);
        }
      }
    } else
    for (int p = 0; p < q.n_peers; ++p) {
      int8_t* dst = q.peers[p] + q.n_off + n_tile0 + col0 + piece * 16;
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + (lane >> 3);
        if ((rows_ok >> r) & 1u) {
          const int4 value =
              *reinterpret_cast<const int4*>(gather_stage + r * 128 + ((piece ^ (r & 7)) << 4));
          *reinterpret_cast<int4*>(dst + size_t(m_base + r) * q.ldc) = value;
        }
      }
    }
    __syncwarp();  // the tile is rewritten by the next call
  }
}

}  // namespace i8
}  // namespace texo
