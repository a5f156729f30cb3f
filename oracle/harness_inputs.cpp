// Input generators of the reference harnesses, restated (TEST INFRASTRUCTURE).
//
// The reference tests draw their inputs from std::mt19937 through libstdc++'s
// distributions; reproducing the same byte streams needs the same library algorithms,
// hence this small C++ file next to the C oracle.
//   int8 : tests/mm_int8.cpp:20-27   (one uniform_int_distribution<int>(lo,hi) draw per byte)
//   int4 : tests/mm_int4.cpp:19-33   (one engine: all x ~ N(0,1), then all bytes, then scales)
//   fp32 : tests/test_utils.h:51-57  (uniform_real_distribution<float>(-8,8))
#include <cmath>
#include <cstdint>
#include <cstring>
#include <random>

namespace {
// float -> IEEE binary16 bits, round to nearest even (what __float2half_rn does).
uint16_t float_to_half_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return uint16_t(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return uint16_t(sign | 0x7c00u);  // rounds to infinity
  if (x < 0x33000001u) return uint16_t(sign);              // rounds to zero
  int exp = int(x >> 23) - 127;
  uint32_t man = (x & 0x7fffffu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) {  // subnormal half
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = uint32_t(exp + 15) << 10;
    man &= 0x7fffffu;
  }
  uint32_t q = man >> shift, rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) ++q;
  return uint16_t(sign | (base + q));  // a mantissa carry correctly bumps the exponent
}
}  // namespace

extern "C" {

void harness_random_int8(int8_t* out, size_t size, unsigned seed, int lo, int hi) {
  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> dist(lo, hi);
  for (size_t i = 0; i < size; ++i) out[i] = int8_t(dist(rng));
}

void harness_int4_inputs(int m, int n, int k, int g, unsigned seed, int zero_x,
                         uint16_t* x, uint8_t* w, uint16_t* scales) {
  std::mt19937 rng(seed);
  std::normal_distribution<float> normal(0.f, 1.f);
  std::uniform_int_distribution<int> byte(0, 255);
  std::uniform_real_distribution<float> unit(0.f, 1.f);
  for (size_t i = 0; i < size_t(m) * k; ++i)
    x[i] = float_to_half_bits(zero_x ? 0.f : normal(rng));
  for (size_t i = 0; i < size_t(n) * (k / 2); ++i) w[i] = uint8_t(byte(rng));
  for (size_t i = 0; i < size_t(n) * (k / g); ++i)
    scales[i] = float_to_half_bits(unit(rng) * 0.1f + 0.01f);
}

void harness_random_values(float* out, size_t n, unsigned seed) {
  std::mt19937 rng(seed);
  std::uniform_real_distribution<float> dist(-8.0f, 8.0f);
  for (size_t i = 0; i < n; ++i) out[i] = dist(rng);
}

uint16_t harness_float_to_half(float f) { return float_to_half_bits(f); }

}  // extern "C"
