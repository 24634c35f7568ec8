// inferop (B200 build): software E4M3 codec, usable on host and device.
//
// Drop-in for the reference's include/inferop/fp8.h (decode :40-59, encode
// :62-96): OCP FP8 E4M3 with finite saturation.  S.EEEE.MMM, bias 7, largest
// finite value 448 (0x7E), NaN = S.1111.111, denormals m * 2^-9.  The encoder
// rounds to nearest with ties to even and saturates to +-448; NaN keeps its
// sign.  The CUDA kernels use the hardware converter (cvt.rn.satfinite.e4m3x2)
// on the hot path; this integer version defines the bytes it must reproduce.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define INFEROP_HD __host__ __device__
#else
#define INFEROP_HD
#endif

namespace inferop {
namespace fp8 {

constexpr float kE4M3Max = 448.0f;

namespace detail {
INFEROP_HD inline uint32_t f32_to_u32(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
INFEROP_HD inline float u32_to_f32(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
}  // namespace detail

INFEROP_HD inline float e4m3_to_float(uint8_t b) {
  const uint32_t sign = static_cast<uint32_t>(b & 0x80u) << 24;
  const uint32_t exp = (b >> 3) & 0xFu, man = b & 7u;
  if (exp == 15u && man == 7u) return detail::u32_to_f32(sign | 0x7FC00000u);
  if (exp != 0u) return detail::u32_to_f32(sign | ((exp + 120u) << 23) | (man << 20));
  // denormal row: man * 2^-9, the product is exact in fp32
  const float mag = static_cast<float>(man) * 0.001953125f;
  return detail::u32_to_f32(sign | detail::f32_to_u32(mag));
}

INFEROP_HD inline uint8_t float_to_e4m3_rn_sat(float f) {
  const uint32_t u = detail::f32_to_u32(f);
  const uint32_t sign = (u >> 24) & 0x80u;
  const uint32_t mag = u & 0x7FFFFFFFu;
  if (mag > 0x7F800000u) return static_cast<uint8_t>(sign | 0x7Fu);
  const int e = static_cast<int>(mag >> 23) - 127;
  if (e >= 9) return static_cast<uint8_t>(sign | 0x7Eu);
  if (e < -10) return static_cast<uint8_t>(sign);
  // Grid spacing is 2^(e-3), with e clamped at -6 for the denormal row; count
  // grid steps with one RNE rounding and offset by the binade's first code.
  const uint32_t sig = (mag & 0x7FFFFFu) | 0x800000u;
  const uint32_t shift = (e >= -6) ? 20u : static_cast<uint32_t>(14 - e);
  uint32_t steps = sig >> shift;
  const uint32_t rest = sig & ((1u << shift) - 1u), half = 1u << (shift - 1u);
  if (rest > half || (rest == half && (steps & 1u))) ++steps;
  uint32_t code = (e >= -6) ? ((static_cast<uint32_t>(e + 7) << 3) + steps - 8u) : steps;
  if (code > 0x7Eu) code = 0x7Eu;
  return static_cast<uint8_t>(sign | code);
}

}  // namespace fp8
}  // namespace inferop
