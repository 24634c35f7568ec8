// SwiGLU arithmetic shared by the stand-alone kernels (moe.cu) and the gate_up GEMM epilogue
// that applies it in place (gemm_sm100.cu).  Both must produce the same bits:
//   out[i] = silu(gate[i]) * up[i],  silu(g) = g / (1 + exp(-g)),
// computed in fp32 from inputs already rounded to the 16-bit type T and rounded once to T
// (reference kernels/silu_mul.cu:16-28, reference/reference.cpp:55-63).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ib200 {
namespace swiglu {

// For 16-bit outputs: exponential and division from the special-function unit (about 2 units in
// the last place of fp32 each, a thousandth of the 16-bit rounding step), a third of the
// instructions.  Below g = -87 the quotient underflows to zero (exact value: under 1e-36 times
// the up-projection).
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}

// eight 16-bit values of one 16-byte word <-> floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&f)[8]);
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2_rn(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2_rn<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// eight SwiGLU outputs from eight gates and eight ups, rounded to T and packed
template <typename T>
__device__ __forceinline__ uint4 silu_mul8(const uint4& g_raw, const uint4& u_raw) {
  float g[8], u[8];
  unpack8<T>(g_raw, g);
  unpack8<T>(u_raw, u);
  uint4 o;
  o.x = pack2_rn<T>(silu_mul_fast(g[0], u[0]), silu_mul_fast(g[1], u[1]));
  o.y = pack2_rn<T>(silu_mul_fast(g[2], u[2]), silu_mul_fast(g[3], u[3]));
  o.z = pack2_rn<T>(silu_mul_fast(g[4], u[4]), silu_mul_fast(g[5], u[5]));
  o.w = pack2_rn<T>(silu_mul_fast(g[6], u[6]), silu_mul_fast(g[7], u[7]));
  return o;
}

}  // namespace swiglu
}  // namespace ib200
