// Arithmetic of the per-token-group quantiser shared by the stand-alone kernel (quant.cu) and
// the GEMM prologue that quantises activations on the fly (gemm_decode_sm100.cu).  Both must
// produce the bytes and scales of reference/reference.cpp:65-80 bit for bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace ib200 {

// Two floats -> two E4M3 bytes (low byte = a) with the hardware converter:
// round to nearest even, saturate to +-448.
__device__ __forceinline__ uint32_t cvt2(float a, float b) {
  return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3));
}

// Rare path: a quotient was NaN.  The hardware converter writes 0x7F for any
// NaN; the reference keeps the sign of a NaN input and, for the invalid
// operation Inf/Inf (an infinite group maximum), produces the x86 default NaN,
// whose sign bit is set.
__device__ __forceinline__ uint32_t nan_byte(float x) {
  return (x != x) ? (0x7Fu | ((__float_as_uint(x) >> 24) & 0x80u)) : 0xFFu;
}

// x / scale, correctly rounded, from a correctly rounded reciprocal rcp = RN(1/scale):
// q0 = RN(x * rcp) is within an ulp or so of the quotient, the residual x - q0 * scale is
// exact in one FMA, and adding residual * rcp back lands on RN(x / scale).  Used only where
// kFastDivOk says the operands are far from overflow and underflow, and only for 16-bit
// inputs, for which the whole domain (every group maximum x every element value) is checked
// against __fdiv_rn by inferop_selftest_quant_div.
__device__ __forceinline__ float div_by_rcp(float x, float scale, float rcp) {
  const float q0 = __fmul_rn(x, rcp);
  // the residual is kept negated (q0 * scale - x) so that a zero x keeps its sign:
  // (-0) - (-0) * ... ends in -0 + -0 = -0, where x - q0 * scale would give +0
  const float neg_r = __fmaf_rn(q0, scale, -x);
  return __fmaf_rn(-neg_r, rcp, q0);
}
// amax in [2^-100, 2^127): scale, its reciprocal, every quotient and every residual are
// normal numbers.  amax == 0 (scale 1, every element +-0) is exact as well and keeps the
// signs of the zeros.
__device__ __forceinline__ bool fast_div_ok(float amax) {
  return (amax >= 7.888609052e-31f && amax < 1.701411835e38f) || amax == 0.0f;
}

template <bool kFast>
__device__ __forceinline__ uint2 quantise8(const float (&f)[8], float scale, float rcp) {
  float q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = kFast ? div_by_rcp(f[i], scale, rcp) : __fdiv_rn(f[i], scale);
  uint32_t w0 = cvt2(q[0], q[1]) | (cvt2(q[2], q[3]) << 16);
  uint32_t w1 = cvt2(q[4], q[5]) | (cvt2(q[6], q[7]) << 16);
  // any byte equal to 0x7F / 0xFF marks a NaN quotient
  if (__vcmpeq4(w0 & 0x7F7F7F7Fu, 0x7F7F7F7Fu) | __vcmpeq4(w1 & 0x7F7F7F7Fu, 0x7F7F7F7Fu)) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (q[i] != q[i]) {
        uint32_t& w = (i < 4) ? w0 : w1;
        const int sh = (i & 3) * 8;
        w = (w & ~(0xFFu << sh)) | (nan_byte(f[i]) << sh);
      }
    }
  }
  return make_uint2(w0, w1);
}

// Fast path for eight 16-bit inputs (raw = the four bf16x2 / f16x2 words, f = the same values
// widened): the division through the reciprocal, two elements per instruction
// (mul.f32x2 / fma.f32x2), the hardware converter, and the sign of every byte taken from its
// input.  The quotient of x by a positive scale has the sign of x, so overriding the sign bit
// is exact; it also restores what the arithmetic and the converter lose: the sign of a -0
// input (x - q0 * scale gives +0) and the sign of a NaN input.  Valid under fast_div_ok only.
__device__ __forceinline__ uint2 quantise8_fast16(const uint4& raw, const float (&f)[8], float scale,
                                                 float rcp) {
  const float2 rcp2 = make_float2(rcp, rcp);
  const float2 nscale2 = make_float2(-scale, -scale);
  uint32_t c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = make_float2(f[2 * i], f[2 * i + 1]);
    const float2 q0 = __fmul2_rn(x, rcp2);
    const float2 r = __ffma2_rn(q0, nscale2, x);   // x - q0 * scale, exact
    const float2 q1 = __ffma2_rn(r, rcp2, q0);
    c[i] = cvt2(q1.x, q1.y);
  }
  // the high byte of every 16-bit input carries its sign in bit 7
  const uint32_t s0 = __byte_perm(raw.x, raw.y, 0x7531) & 0x80808080u;
  const uint32_t s1 = __byte_perm(raw.z, raw.w, 0x7531) & 0x80808080u;
  return make_uint2(((c[0] | (c[1] << 16)) & 0x7F7F7F7Fu) | s0, ((c[2] | (c[3] << 16)) & 0x7F7F7F7Fu) | s1);
}

// max |x| over the eight 16-bit inputs of a lane, on the packed words (a NaN never wins:
// __hmax2 returns the other operand)
template <typename T2>
__device__ __forceinline__ float absmax8_packed(const uint4& raw) {
  const T2 a = __habs2(*reinterpret_cast<const T2*>(&raw.x));
  const T2 b = __habs2(*reinterpret_cast<const T2*>(&raw.y));
  const T2 c = __habs2(*reinterpret_cast<const T2*>(&raw.z));
  const T2 d = __habs2(*reinterpret_cast<const T2*>(&raw.w));
  const T2 m = __hmax2(__hmax2(a, b), __hmax2(c, d));
  const float2 mf = (sizeof(T2) == sizeof(__half2) && std::is_same<T2, __half2>::value)
                        ? __half22float2(*reinterpret_cast<const __half2*>(&m))
                        : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&m));
  return fmaxf(0.0f, fmaxf(mf.x, mf.y));   // fmaxf drops a NaN that survived (all eight NaN)
}

// scale of a group from its maximum magnitude (reference/reference.cpp:73)
__device__ __forceinline__ float group_scale(float amax) {
  return (amax == 0.0f) ? 1.0f : __fmul_rn(amax, 1.0f / 448.0f);
}

}  // namespace ib200
