// inferop (B200 build): element types and host-side number-format helpers.
//
// Drop-in for the reference's include/inferop/common.h: the same names in the
// same namespaces with the same meaning (reference: common.h:13 for the dtype
// enum, :25-33 dtype_bytes, :55-61 bf16, :63-101 fp16), written independently.
// Stays free of CUDA so CPU-only translation units can include it.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>

namespace inferop {

// Values are part of the ABI: the C entry points take them as int32_t.
enum class dtype : int32_t { fp32 = 0, fp16 = 1, bf16 = 2, fp8_e4m3 = 3 };

inline int dtype_bytes(dtype d) {
  return d == dtype::fp32 ? 4 : (d == dtype::fp16 || d == dtype::bf16) ? 2 : d == dtype::fp8_e4m3 ? 1 : 0;
}

inline const char* dtype_name(dtype d) {
  static const char* const names[] = {"fp32", "fp16", "bf16", "fp8_e4m3"};
  int i = static_cast<int>(d);
  return (i >= 0 && i < 4) ? names[i] : "unknown";
}

namespace bitcast {
inline uint32_t f32_to_u32(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float u32_to_f32(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
}  // namespace bitcast

namespace host_convert {

// bf16 is the upper half of an fp32 word.
inline float bf16_to_float(uint16_t h) { return bitcast::u32_to_f32(static_cast<uint32_t>(h) << 16); }

// Round to nearest, ties to even: bias by 0x7FFF plus the parity of the kept part.
inline uint16_t float_to_bf16_rn(float f) {
  uint32_t u = bitcast::f32_to_u32(f);
  return static_cast<uint16_t>((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// IEEE binary16 -> fp32, exact.
inline float half_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const int exp = (h >> 10) & 0x1F;
  const uint32_t frac = h & 0x3FFu;
  if (exp == 31) return bitcast::u32_to_f32(sign | 0x7F800000u | (frac ? 0x400000u | (frac << 13) : 0u));
  if (exp == 0) {
    const float mag = std::ldexp(static_cast<float>(frac), -24);
    return sign ? -mag : mag;
  }
  return bitcast::u32_to_f32(sign | (static_cast<uint32_t>(exp + 112) << 23) | (frac << 13));
}

// fp32 -> IEEE binary16, round to nearest even, overflow to infinity.
inline uint16_t float_to_half_rn(float f) {
  const uint32_t u = bitcast::f32_to_u32(f);
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  const uint32_t mag = u & 0x7FFFFFFFu;
  if (mag > 0x7F800000u) return 0x7E00;                       // NaN
  if (mag >= 0x477FF000u) return sign | 0x7C00;               // rounds to >= 2^16 -> inf
  if (mag < 0x33000001u) return sign;                         // <= 2^-25 -> zero
  const int e = static_cast<int>(mag >> 23) - 127;
  const uint32_t sig = (mag & 0x7FFFFFu) | 0x800000u;
  const int shift = (e >= -14) ? 13 : (-1 - e);               // denormal row keeps fewer bits
  uint32_t kept = sig >> shift;
  const uint32_t rest = sig & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rest > half || (rest == half && (kept & 1u))) ++kept;
  const uint32_t code = (e >= -14) ? ((static_cast<uint32_t>(e + 15) << 10) + kept - 1024u) : kept;
  return static_cast<uint16_t>(sign | code);
}

}  // namespace host_convert
}  // namespace inferop
