// RMSNorm with residual add, and the same fused with INT8 activation quantisation, for B200.
//
//   z[n,j]   = x[n,j] + residual[n,j]                                   (FP32 add)
//   out[n,j] = z[n,j] * rsqrt(mean_j(z[n,j]^2) + eps) * weight[j]       (FP32)
//
// `solve` is a drop-in for frezcirno/Texo src/rms_norm_w_residual.cu:40-75 (same symbol,
// argument order, device pointers, legacy default stream, output fully overwritten).  The
// reference reads x and residual twice (once for the sum of squares, once for the output);
// here a row lives in registers between the two steps, so each input byte crosses HBM once.
//
// `texo_rms_norm_quant_solve` is the producer in front of the INT8 matmul (no counterpart in
// the reference): the normalised row is not written as FP32 but quantised on the spot,
//   q[n,j] = clamp(rint(out[n,j] / scale) + zero_point, -128, 127),
// to the int8 activations A the matmul consumes (scale_A / zero_point_A of mm_int8), and
// the updated residual stream z can be written alongside.  13 bytes per element become 9
// (or 13 with z), against 8 + 4 + 4 + 1 = 17 for the unfused sequence norm -> quantise.
//
// Both are bound by HBM bandwidth.  One CTA per row; float4 streaming loads, all issued
// before the first use; one block-wide reduction; streaming stores.
#include <algorithm>
#include <cstdint>
#include <cuda_runtime.h>

#include "host_common.h"
#include "ptx.cuh"
#include "requant.cuh"

namespace texo {
namespace rn {

constexpr int THREADS = 256;
constexpr int MAX_VEC = 16;  // float4 per thread kept in registers: rows up to 16384 floats

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];  // same order in every thread
  return total;
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (threadIdx.x % 32 == 0) scratch[threadIdx.x / 32] = v;
  __syncthreads();
  int total = 0;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
  return total;
}

struct QuantOut {
  float scale, rscale;
  int zero_point;
  int fast_div;  // scale inside the range of the branch-free exact division
};

__device__ __forceinline__ int quantize_one(float y, const QuantOut& qo) {
  // y / scale, correctly rounded either way (see requant.cuh); |y| is bounded by the caller's
  // data, and values outside the safe range take the IEEE division.
  const float a = fabsf(y);
  const bool in_range = qo.fast_div && ((a >= 0x1p-60f && a <= 0x1p60f) || a == 0.f);
  const float t = in_range ? i8::div_rn_inrange(y, qo.scale, qo.rscale) : __fdiv_rn(y, qo.scale);
  float r = __fadd_rn(rintf(t), float(qo.zero_point));
  r = fminf(fmaxf(r, -128.f), 127.f);
  return __float2int_rn(r);
}

// One row per CTA, the row held in registers.  VEC = float4 per thread (C <= THREADS*4*VEC).
// QUANT: write int8 q (and optionally z) instead of FP32 out.
template <int VEC, bool QUANT>
__global__ void __launch_bounds__(THREADS)
    row_kernel(const float* __restrict__ x, const float* __restrict__ residual,
               const float* __restrict__ weight, float* __restrict__ out, int8_t* __restrict__ q,
               float* __restrict__ z_out, int* __restrict__ q_row_sum, int C, float eps, QuantOut qo) {
  __shared__ float scratch[THREADS / 32];
  __shared__ int iscratch[THREADS / 32];
  const size_t row = size_t(blockIdx.x) * C;
  const int c4 = C / 4;
  int qsum = 0;
  const float4* x4 = reinterpret_cast<const float4*>(x + row);
  const float4* r4 = reinterpret_cast<const float4*>(residual + row);
  float4 z[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * THREADS;
    z[i] = c < c4 ? __ldcs(x4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < c4) {
      const float4 r = __ldcs(r4 + c);
      z[i].x = __fadd_rn(z[i].x, r.x);
      z[i].y = __fadd_rn(z[i].y, r.y);
      z[i].z = __fadd_rn(z[i].z, r.z);
      z[i].w = __fadd_rn(z[i].w, r.w);
      sum += z[i].x * z[i].x + z[i].y * z[i].y + z[i].z * z[i].z + z[i].w * z[i].w;
    }
  }
  const float inv_rms = rsqrtf(block_sum(sum, scratch) / float(C) + eps);
  const float4* w4 = reinterpret_cast<const float4*>(weight);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    const int c = threadIdx.x + i * THREADS;
    if (c < c4) {
      const float4 w = __ldg(w4 + c);
      float4 y;
      y.x = z[i].x * inv_rms * w.x;
      y.y = z[i].y * inv_rms * w.y;
      y.z = z[i].z * inv_rms * w.z;
      y.w = z[i].w * inv_rms * w.w;
      if (QUANT) {
        const uint32_t packed = i8::pack_sat_s8(quantize_one(y.x, qo), quantize_one(y.y, qo),
                                                quantize_one(y.z, qo), quantize_one(y.w, qo));
        qsum = __dp4a(int(packed), 0x01010101, qsum);
        __stcs(reinterpret_cast<unsigned int*>(q + row) + c, packed);
        if (z_out) __stcs(reinterpret_cast<float4*>(z_out + row) + c, z[i]);
      } else {
        __stcs(reinterpret_cast<float4*>(out + row) + c, y);
      }
    }
  }
  if (QUANT && q_row_sum) {
    const int total = block_sum_int(qsum, iscratch);
    if (threadIdx.x == 0) q_row_sum[blockIdx.x] = total;
  }
}

// Any C, any alignment: two passes over the row (the second mostly from L2).
template <bool QUANT>
__global__ void __launch_bounds__(THREADS)
    generic_kernel(const float* __restrict__ x, const float* __restrict__ residual,
                   const float* __restrict__ weight, float* __restrict__ out,
                   int8_t* __restrict__ q, float* __restrict__ z_out, int* __restrict__ q_row_sum,
                   int C, float eps, QuantOut qo) {
  __shared__ float scratch[THREADS / 32];
  __shared__ int iscratch[THREADS / 32];
  const size_t row = size_t(blockIdx.x) * C;
  int qsum = 0;
  float sum = 0.f;
  for (int j = threadIdx.x; j < C; j += THREADS) {
    const float z = __fadd_rn(x[row + j], residual[row + j]);
    sum += z * z;
  }
  const float inv_rms = rsqrtf(block_sum(sum, scratch) / float(C) + eps);
  for (int j = threadIdx.x; j < C; j += THREADS) {
    const float z = __fadd_rn(x[row + j], residual[row + j]);
    const float y = z * inv_rms * weight[j];
    if (QUANT) {
      const int v = quantize_one(y, qo);
      qsum += v;
      q[row + j] = int8_t(v);
      if (z_out) z_out[row + j] = z;
    } else {
      out[row + j] = y;
    }
  }
  if (QUANT && q_row_sum) {
    const int total = block_sum_int(qsum, iscratch);
    if (threadIdx.x == 0) q_row_sum[blockIdx.x] = total;
  }
}

inline int& last_path() {
  static int path = 0;
  return path;
}

template <bool QUANT>
static void launch(const float* x, const float* residual, const float* weight, float* out, int8_t* q,
                   float* z_out, int* q_row_sum, int N, int C, float eps, const QuantOut& qo) {
  if (N <= 0 || C <= 0) return;
  auto aligned = [](const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
  const bool vec = C % 4 == 0 && C <= THREADS * 4 * MAX_VEC && aligned(x, 16) && aligned(residual, 16) &&
                   aligned(weight, 16) && (QUANT ? aligned(q, 4) && (!z_out || aligned(z_out, 16))
                                                 : aligned(out, 16));
  if (vec) {
    const int need = (C / 4 + THREADS - 1) / THREADS;
    if (need <= 2)
      row_kernel<2, QUANT><<<N, THREADS>>>(x, residual, weight, out, q, z_out, q_row_sum, C, eps, qo);
    else if (need <= 4)
      row_kernel<4, QUANT><<<N, THREADS>>>(x, residual, weight, out, q, z_out, q_row_sum, C, eps, qo);
    else if (need <= 8)
      row_kernel<8, QUANT><<<N, THREADS>>>(x, residual, weight, out, q, z_out, q_row_sum, C, eps, qo);
    else
      row_kernel<MAX_VEC, QUANT><<<N, THREADS>>>(x, residual, weight, out, q, z_out, q_row_sum, C, eps, qo);
    last_path() = 2;
  } else {
    generic_kernel<QUANT><<<N, THREADS>>>(x, residual, weight, out, q, z_out, q_row_sum, C, eps, qo);
    last_path() = 1;
  }
  ++launch_counter();
}

}  // namespace rn
}  // namespace texo

// x, residual [N,C], weight [C], out [N,C]: FP32 device pointers.
extern "C" void solve(const float* x, const float* residual, const float* weight, float* out, int N,
                      int C, float eps) {
  using namespace texo;
  if (N <= 0 || C <= 0) return;
  if (!x || !residual || !weight || !out) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  const int slot = profile_start();
  rn::launch<false>(x, residual, weight, out, nullptr, nullptr, nullptr, N, C, eps,
                    rn::QuantOut{1.f, 1.f, 0, 0});
  profile_stop(slot);
}

// q [N,C] int8 = quantised RMSNorm(x + residual) * weight; z_out [N,C] FP32 (may be null)
// receives x + residual; q_row_sum [N] int32 (may be null) receives sum_j q[n,j], which the
// INT8 matmul needs for its zero-point correction (texo_mm_int8_solve_presummed) and would
// otherwise recompute by reading q again.  scale must be finite and non-zero.
extern "C" void texo_rms_norm_quant_solve(const float* x, const float* residual, const float* weight,
                                          int8_t* q, float* z_out, int* q_row_sum, int N, int C,
                                          float eps, float scale, int zero_point) {
  using namespace texo;
  if (N <= 0 || C <= 0) return;
  if (!x || !residual || !weight || !q || !(scale == scale) || scale == 0.f) {
    note_host_error(STATUS_BAD_ARGUMENT);
    return;
  }
  rn::QuantOut qo{scale, 0.f, zero_point, 0};
  const float a = scale < 0 ? -scale : scale;
  if (a >= 0x1p-60f && a <= 0x1p60f) {
    qo.rscale = 1.0f / scale;
    qo.fast_div = 1;
  }
  const int slot = profile_start();
  rn::launch<true>(x, residual, weight, nullptr, q, z_out, q_row_sum, N, C, eps, qo);
  profile_stop(slot);
}

extern "C" int texo_rms_norm_last_path() { return texo::rn::last_path(); }
