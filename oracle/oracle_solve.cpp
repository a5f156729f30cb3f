// `solve` of each hot-path operator bound to the CPU oracle (qmm_oracle.c), with the exact
// prototypes the reference harnesses declare (tests/mm_int8.cpp:5-6, tests/mm_int4.cpp:7-8,
// tests/dequantization.cpp:4 of frezcirno/Texo).  Compiled three times, once per operator
// (-DORACLE_SOLVE_MM_INT8 / _MM_INT4 / _DEQUANTIZATION), and linked with the unchanged
// harness source and host_cudart.cpp.  TEST INFRASTRUCTURE, never part of the product.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {
int oracle_mm_int8_rows(const int8_t* A, const int8_t* B, int8_t* C_rows, int M, int N, int K,
                        float sa, float sb, float sc, int za, int zb, int zc, int row0, int row1,
                        int mode);
int oracle_mm_int4_rows(const uint16_t* x, const uint8_t* w_q, const uint16_t* scales,
                        double* Y_rows, int M, int N, int K, int G, int row0, int row1);
int oracle_dequantization(const float* X, const float* S, double* Y, int M, int N, int T);
}

#if defined(ORACLE_SOLVE_MM_INT8)
// mode 0: the normative form (exact integer dot + the FP32 epilogue of src/mm_int8.cu:12-25)
extern "C" void solve(const int8_t* A, const int8_t* B, int8_t* C, int M, int N, int K,
                      float scale_A, float scale_B, float scale_C, int zero_point_A,
                      int zero_point_B, int zero_point_C) {
  oracle_mm_int8_rows(A, B, C, M, N, K, scale_A, scale_B, scale_C, zero_point_A, zero_point_B,
                      zero_point_C, 0, M, 0);
}
#elif defined(ORACLE_SOLVE_MM_INT4)
// double -> FP16 bits, round to nearest even (the harness reads y as FP16)
static uint16_t to_half_bits(double v) {
  const float f = float(v);
  uint32_t u;
  std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const int32_t exp = int32_t((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffffu;
  if (((u >> 23) & 0xff) == 0xff) return uint16_t(sign | 0x7c00u | (man ? 0x200u : 0u));
  if (exp >= 31) return uint16_t(sign | 0x7c00u);
  if (exp <= 0) {
    if (exp < -10) return uint16_t(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t half = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return uint16_t(sign | half);
  }
  uint32_t half = (uint32_t(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return uint16_t(sign | half);
}
extern "C" void solve(const uint16_t* x, const uint8_t* w_q, const uint16_t* scales, uint16_t* y,
                      int M, int N, int K, int group_size) {
  if (M <= 0 || N <= 0) return;
  std::vector<double> out(size_t(M) * N);
  oracle_mm_int4_rows(x, w_q, scales, out.data(), M, N, K, group_size, 0, M);
  for (size_t i = 0; i < out.size(); ++i) y[i] = to_half_bits(out[i]);
}
#elif defined(ORACLE_SOLVE_DEQUANTIZATION)
extern "C" void solve(const float* X, const float* S, float* Y, int M, int N, int T) {
  std::vector<double> out(size_t(M) * N);
  oracle_dequantization(X, S, out.data(), M, N, T);
  for (size_t i = 0; i < out.size(); ++i) Y[i] = float(out[i]);
}
#else
#error "define ORACLE_SOLVE_MM_INT8, ORACLE_SOLVE_MM_INT4 or ORACLE_SOLVE_DEQUANTIZATION"
#endif
