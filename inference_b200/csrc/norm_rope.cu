// RMSNorm, residual add + RMSNorm, and the NeoX rotary embedding for sm_100: the operators that sit
// in front of the quantise + GEMM path in a transformer block (reference kernels/rmsnorm.cu:21-59,
// kernels/rope.cu:19-41; CPU golden reference/reference.cpp:11-53).  All three are HBM-bound:
// every element is read once and written once.
//
//   * rmsnorm_vec_kernel: a row lives in registers between the two passes the reference makes over
//     it (16-byte loads, up to eight vectors per thread), so it is read from memory once; 32 to 256
//     threads per row depending on its length, several rows per CTA when rows are short.
//   * rope_kernel: the angle of (position, i) does not depend on the head, so a CTA computes the
//     cos / sin table of its token once and applies it to a block of heads with 16-byte accesses.
//     The frequencies come from the host (the C library's powf, as in the CPU golden: at position
//     100 000 two units in the last place of a device powf would be 0.02 rad).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "internal.h"
#include "quant_math.cuh"

namespace ib200 {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 8;   // 16-byte vectors of a row that one thread keeps in registers

template <typename T>
struct VecOf {
  static constexpr int N = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__device__ __forceinline__ void unpack(const uint4& raw, float (&f)[VecOf<T>::N]) {
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < VecOf<T>::N; ++i) f[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack(const float (&f)[VecOf<T>::N]) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < VecOf<T>::N; ++i) e[i] = from_f32<T>(f[i]);
  return raw;
}

// kAdd: residual[r, :] += x[r, :] first (stored in T), then the norm of the sum.  As in the
// reference's kernel the sum of squares uses the unrounded sums and the output the stored ones.
// tpr = threads per row (a power of two, 32 .. 256); rows per CTA = 256 / tpr; NV = 16-byte
// vectors of the row per thread, kept packed in registers between the two passes.
template <typename T, bool kAdd, int NV>
__global__ void __launch_bounds__(kThreads)
rmsnorm_vec_kernel(T* __restrict__ out, T* __restrict__ residual, const T* __restrict__ in,
                   const T* __restrict__ weight, float eps, int64_t rows, int cols, int tpr) {
  constexpr int V = VecOf<T>::N;
  __shared__ float red[kThreads / 32];
  const int lane_in_row = threadIdx.x & (tpr - 1);
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / tpr) + (threadIdx.x / tpr);
  const bool live = row < rows;
  const int nvec = cols / V;
  const uint4* src = reinterpret_cast<const uint4*>(in + (live ? row : 0) * cols);
  uint4* res = kAdd ? reinterpret_cast<uint4*>(residual + (live ? row : 0) * cols) : nullptr;

  uint4 raw[NV], rraw[kAdd ? NV : 1];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int j = lane_in_row + k * tpr;
    const bool have = live && j < nvec;
    raw[k] = have ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
    if constexpr (kAdd) rraw[k] = have ? res[j] : make_uint4(0u, 0u, 0u, 0u);
  }
  float partial = 0.0f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float v[V];
    unpack<T>(raw[k], v);
    if constexpr (kAdd) {
      float r[V];
      unpack<T>(rraw[k], r);
#pragma unroll
      for (int i = 0; i < V; ++i) r[i] = __fadd_rn(r[i], v[i]);
#pragma unroll
      for (int i = 0; i < V; ++i) partial = fmaf(r[i], r[i], partial);
      raw[k] = pack<T>(r);   // what is stored; the output is computed from it
      const int j = lane_in_row + k * tpr;
      if (live && j < nvec) res[j] = raw[k];
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) partial = fmaf(v[i], v[i], partial);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) partial += __shfl_xor_sync(0xFFFFFFFFu, partial, o);
  if (tpr > 32) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = partial;
    __syncthreads();
    const int w0 = (threadIdx.x / tpr) * (tpr >> 5);
    partial = 0.0f;
    for (int w = 0; w < (tpr >> 5); ++w) partial += red[w0 + w];
  }
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial, static_cast<float>(cols)), eps)));
  uint4* dst = reinterpret_cast<uint4*>(out + (live ? row : 0) * cols);
  const uint4* wv = reinterpret_cast<const uint4*>(weight);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int j = lane_in_row + k * tpr;
    if (live && j < nvec) {
      float v[V], w[V], y[V];
      unpack<T>(raw[k], v);
      unpack<T>(__ldg(wv + j), w);
#pragma unroll
      for (int i = 0; i < V; ++i) y[i] = __fmul_rn(__fmul_rn(v[i], inv), w[i]);
      dst[j] = pack<T>(y);
    }
  }
}

// RMSNorm (or residual add + RMSNorm) with the 1 x 128 FP8 quantisation of the result in the same
// pass: q / scales are what quant_fp8_per_token_group gives on the 16-bit output of the norm, bit
// for bit (the normalised value is rounded to T first, then quantised by the quantiser's own
// functions), and the 16-bit matrix between the two never exists.  A group of 128 elements is 16
// consecutive vectors, i.e. the 16 lanes of a half warp.  16-bit T, cols % 128 == 0.
template <typename T, bool kAdd, int NV>
__global__ void __launch_bounds__(kThreads)
rmsnorm_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, T* __restrict__ residual,
                     const T* __restrict__ in, const T* __restrict__ weight, float eps, int64_t rows, int cols,
                     int tpr) {
  constexpr int V = 8;
  using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
  __shared__ float red[kThreads / 32];
  const int lane_in_row = threadIdx.x & (tpr - 1);
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / tpr) + (threadIdx.x / tpr);
  const bool live = row < rows;
  const int nvec = cols / V;
  const uint4* src = reinterpret_cast<const uint4*>(in + (live ? row : 0) * cols);
  uint4* res = kAdd ? reinterpret_cast<uint4*>(residual + (live ? row : 0) * cols) : nullptr;

  uint4 raw[NV], rraw[kAdd ? NV : 1];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int j = lane_in_row + k * tpr;
    const bool have = live && j < nvec;
    raw[k] = have ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
    if constexpr (kAdd) rraw[k] = have ? res[j] : make_uint4(0u, 0u, 0u, 0u);
  }
  float partial = 0.0f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float v[V];
    unpack<T>(raw[k], v);
    if constexpr (kAdd) {
      float r[V];
      unpack<T>(rraw[k], r);
#pragma unroll
      for (int i = 0; i < V; ++i) r[i] = __fadd_rn(r[i], v[i]);
#pragma unroll
      for (int i = 0; i < V; ++i) partial = fmaf(r[i], r[i], partial);
      raw[k] = pack<T>(r);
      const int j = lane_in_row + k * tpr;
      if (live && j < nvec) res[j] = raw[k];
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) partial = fmaf(v[i], v[i], partial);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) partial += __shfl_xor_sync(0xFFFFFFFFu, partial, o);
  if (tpr > 32) {
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = partial;
    __syncthreads();
    const int w0 = (threadIdx.x / tpr) * (tpr >> 5);
    partial = 0.0f;
    for (int w = 0; w < (tpr >> 5); ++w) partial += red[w0 + w];
  }
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial, static_cast<float>(cols)), eps)));
  const uint4* wv = reinterpret_cast<const uint4*>(weight);
  uint8_t* qrow = q + (live ? row : 0) * cols;
  float* srow = scales + (live ? row : 0) * (cols >> 7);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int j = lane_in_row + k * tpr;
    const bool have = live && j < nvec;   // the same for the 16 lanes of a group (nvec % 16 == 0)
    float v[V], w[V], y[V];
    unpack<T>(raw[k], v);
    unpack<T>(have ? __ldg(wv + j) : make_uint4(0u, 0u, 0u, 0u), w);
#pragma unroll
    for (int i = 0; i < V; ++i) y[i] = __fmul_rn(__fmul_rn(v[i], inv), w[i]);
    const uint4 yraw = pack<T>(y);        // the norm's output as it would have been stored
    float f[V];
    unpack<T>(yraw, f);
    float amax = absmax8_packed<T2>(yraw);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float scale = group_scale(amax);
    if (have) {
      const uint2 bytes = fast_div_ok(amax) ? quantise8_fast16(yraw, f, scale, __frcp_rn(scale))
                                            : quantise8<false>(f, scale, 0.0f);
      *reinterpret_cast<uint2*>(qrow + j * V) = bytes;
      if ((lane_in_row & 15) == 0) srow[j >> 4] = scale;
    }
  }
}

// Any shape and alignment: one CTA per row, two strided passes (the reference's own scheme).
template <typename T, bool kAdd>
__global__ void __launch_bounds__(kThreads)
rmsnorm_any_kernel(T* __restrict__ out, T* __restrict__ residual, const T* __restrict__ in,
                   const T* __restrict__ weight, float eps, int cols) {
  __shared__ float red[kThreads / 32];
  const int64_t row = blockIdx.x;
  const T* x = in + row * cols;
  T* res = kAdd ? residual + row * cols : nullptr;
  float partial = 0.0f;
  for (int i = threadIdx.x; i < cols; i += kThreads) {
    float v = to_f32<T>(x[i]);
    if constexpr (kAdd) {
      v = __fadd_rn(to_f32<T>(res[i]), v);
      res[i] = from_f32<T>(v);   // the same thread reads it back below
    }
    partial = fmaf(v, v, partial);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) partial += __shfl_xor_sync(0xFFFFFFFFu, partial, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = partial;
  __syncthreads();
  partial = 0.0f;
  for (int w = 0; w < kThreads / 32; ++w) partial += red[w];
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial, static_cast<float>(cols)), eps)));
  T* y = out + row * cols;
  for (int i = threadIdx.x; i < cols; i += kThreads) {
    const float v = to_f32<T>(kAdd ? res[i] : x[i]);
    y[i] = from_f32<T>(__fmul_rn(__fmul_rn(v, inv), to_f32<T>(weight[i])));
  }
}

template <typename T, bool kAdd>
int launch_rmsnorm_t(void* out, void* residual, const void* in, const void* weight, int64_t rows, int64_t cols,
                     float eps, cudaStream_t stream) {
  constexpr int V = VecOf<T>::N;
  const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(in) |
                         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(residual)) & 15u) == 0;
  const int64_t nvec = cols / V;
  if (aligned && cols % V == 0 && nvec <= static_cast<int64_t>(kThreads) * kMaxVec) {
    int tpr = 32;
    while (tpr < kThreads && static_cast<int64_t>(tpr) * 4 < nvec) tpr <<= 1;   // about four vectors per thread
    const int per_thread = static_cast<int>((nvec + tpr - 1) / tpr);
    const int rows_per_cta = kThreads / tpr;
    const int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
    if (grid > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
    T* o = static_cast<T*>(out);
    T* r = static_cast<T*>(residual);
    const T* i = static_cast<const T*>(in);
    const T* w = static_cast<const T*>(weight);
    const unsigned g = static_cast<unsigned>(grid);
    const int c = static_cast<int>(cols);
    if (per_thread <= 1) rmsnorm_vec_kernel<T, kAdd, 1><<<g, kThreads, 0, stream>>>(o, r, i, w, eps, rows, c, tpr);
    else if (per_thread <= 2) rmsnorm_vec_kernel<T, kAdd, 2><<<g, kThreads, 0, stream>>>(o, r, i, w, eps, rows, c, tpr);
    else if (per_thread <= 4) rmsnorm_vec_kernel<T, kAdd, 4><<<g, kThreads, 0, stream>>>(o, r, i, w, eps, rows, c, tpr);
    else rmsnorm_vec_kernel<T, kAdd, kMaxVec><<<g, kThreads, 0, stream>>>(o, r, i, w, eps, rows, c, tpr);
  } else {
    if (rows > 0x7FFFFFFFLL || cols > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
    rmsnorm_any_kernel<T, kAdd><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(
        static_cast<T*>(out), static_cast<T*>(residual), static_cast<const T*>(in), static_cast<const T*>(weight),
        eps, static_cast<int>(cols));
  }
  return check_launch();
}

template <typename T, bool kAdd>
int launch_rmsnorm_quant_t(void* q, void* scales, void* residual, const void* in, const void* weight, int64_t rows,
                           int64_t cols, float eps, cudaStream_t stream) {
  const int64_t nvec = cols / 8;
  int tpr = 32;
  while (tpr < kThreads && static_cast<int64_t>(tpr) * 4 < nvec) tpr <<= 1;
  const int per_thread = static_cast<int>((nvec + tpr - 1) / tpr);
  const int rows_per_cta = kThreads / tpr;
  const int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
  if (grid > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  uint8_t* qp = static_cast<uint8_t*>(q);
  float* sp = static_cast<float*>(scales);
  T* r = static_cast<T*>(residual);
  const T* i = static_cast<const T*>(in);
  const T* w = static_cast<const T*>(weight);
  const unsigned g = static_cast<unsigned>(grid);
  const int c = static_cast<int>(cols);
  if (per_thread <= 1) rmsnorm_quant_kernel<T, kAdd, 1><<<g, kThreads, 0, stream>>>(qp, sp, r, i, w, eps, rows, c, tpr);
  else if (per_thread <= 2) rmsnorm_quant_kernel<T, kAdd, 2><<<g, kThreads, 0, stream>>>(qp, sp, r, i, w, eps, rows, c, tpr);
  else if (per_thread <= 4) rmsnorm_quant_kernel<T, kAdd, 4><<<g, kThreads, 0, stream>>>(qp, sp, r, i, w, eps, rows, c, tpr);
  else rmsnorm_quant_kernel<T, kAdd, kMaxVec><<<g, kThreads, 0, stream>>>(qp, sp, r, i, w, eps, rows, c, tpr);
  return check_launch();
}

// ------------------------------------------------------------------------------------- rotary embedding
constexpr int kRopeThreads = 128;
constexpr int kRopeMaxHalf = 512;   // rotary_dim up to 1024

// The frequencies base^(-2 i / rotary_dim) * yarn depend on i only: the launcher computes them on the
// host with the C library's powf, the very function the CPU golden calls, and passes them in the
// kernel's parameter block.
struct RopeFreq {
  float f[kRopeMaxHalf];
};

// grid (tokens, ceil(heads / heads_per_cta)).  kVec: 16-byte accesses (rotary_dim / 2 a multiple of the
// vector length, rows 16-byte aligned); otherwise element by element.
template <typename T, bool kVec>
__global__ void __launch_bounds__(kRopeThreads)
rope_kernel(T* __restrict__ qkv, const int64_t* __restrict__ positions, int heads, int head_dim, int rotary_dim,
            int heads_per_cta, const __grid_constant__ RopeFreq freq) {
  constexpr int V = VecOf<T>::N;
  constexpr int kItems = 4;             // vector pairs a thread handles per CTA (the launcher sizes the head block so)
  __shared__ float2 cs[kRopeMaxHalf];   // (cos, sin) of this token's angles
  const int half = rotary_dim >> 1;
  const int64_t t = blockIdx.x;
  const int h0 = blockIdx.y * heads_per_cta;
  const int h1 = min(heads, h0 + heads_per_cta);
  T* tok = qkv + t * heads * head_dim;
  // the operands are requested before the table is computed, so that the two latencies overlap
  uint4 r0[kVec ? kItems : 1], r1[kVec ? kItems : 1];
  if constexpr (kVec) {
    const int vec_per_head = half / V;
    const int work = (h1 - h0) * vec_per_head;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const int wi = threadIdx.x + k * kRopeThreads;
      if (wi < work) {
        const int h = h0 + wi / vec_per_head, j = wi % vec_per_head;
        r0[k] = *(reinterpret_cast<const uint4*>(tok + h * head_dim) + j);
        r1[k] = *(reinterpret_cast<const uint4*>(tok + h * head_dim + half) + j);
      }
    }
  }
  const float pos = static_cast<float>(__ldg(positions + t));
  for (int i = threadIdx.x; i < half; i += kRopeThreads) {
    float sn, c;
    sincosf(__fmul_rn(pos, freq.f[i]), &sn, &c);   // the accurate version: angles reach 1e5 rad
    cs[i] = make_float2(c, sn);
  }
  __syncthreads();
  if constexpr (kVec) {
    const int vec_per_head = half / V;
    const int work = (h1 - h0) * vec_per_head;
#pragma unroll
    for (int k = 0; k < kItems; ++k) {
      const int wi = threadIdx.x + k * kRopeThreads;
      if (wi < work) {
        const int h = h0 + wi / vec_per_head, j = wi % vec_per_head;
        float x0[V], x1[V], y0[V], y1[V];
        unpack<T>(r0[k], x0);
        unpack<T>(r1[k], x1);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float2 a = cs[j * V + i];
          y0[i] = __fsub_rn(__fmul_rn(x0[i], a.x), __fmul_rn(x1[i], a.y));
          y1[i] = __fadd_rn(__fmul_rn(x1[i], a.x), __fmul_rn(x0[i], a.y));
        }
        *(reinterpret_cast<uint4*>(tok + h * head_dim) + j) = pack<T>(y0);
        *(reinterpret_cast<uint4*>(tok + h * head_dim + half) + j) = pack<T>(y1);
      }
    }
  } else {
    const int work = (h1 - h0) * half;
    for (int wi = threadIdx.x; wi < work; wi += kRopeThreads) {
      const int h = h0 + wi / half, i = wi % half;
      T* p = tok + h * head_dim;
      const float x0 = to_f32<T>(p[i]), x1 = to_f32<T>(p[i + half]);
      const float2 a = cs[i];
      p[i] = from_f32<T>(__fsub_rn(__fmul_rn(x0, a.x), __fmul_rn(x1, a.y)));
      p[i + half] = from_f32<T>(__fadd_rn(__fmul_rn(x1, a.x), __fmul_rn(x0, a.y)));
    }
  }
}

template <typename T>
int launch_rope_t(void* qkv, const int64_t* positions, int64_t tokens, int heads, int head_dim, int rotary_dim,
                  float base, float yarn, cudaStream_t stream) {
  constexpr int V = VecOf<T>::N;
  const int half = rotary_dim / 2;
  RopeFreq freq;
  for (int i = 0; i < half; ++i) {
    // reference/reference.cpp:44: std::pow(base, -2.0f * float(i) / float(rotary_dim)) * yarn_factor
    volatile float e = -2.0f * static_cast<float>(i) / static_cast<float>(rotary_dim);
    volatile float pw = powf(base, e);
    freq.f[i] = pw * yarn;
  }
  for (int i = half; i < kRopeMaxHalf; ++i) freq.f[i] = 0.0f;
  const bool vec = (reinterpret_cast<uintptr_t>(qkv) & 15u) == 0 && half % V == 0 &&
                   (static_cast<int64_t>(head_dim) * sizeof(T)) % 16 == 0;
  // at most four work items per thread and CTA (the vector kernel holds that many in registers);
  // a token's table is computed once per CTA
  const int items_per_head = vec ? half / V : half;
  int hpc = 4 * kRopeThreads / items_per_head;
  if (hpc > heads) hpc = heads;
  if (hpc < 1) hpc = 1;
  const int chunks = (heads + hpc - 1) / hpc;
  if (chunks > 65535) return INFEROP_ERR_LIMIT;
  const dim3 grid(static_cast<unsigned>(tokens), static_cast<unsigned>(chunks));
  if (vec) {
    rope_kernel<T, true><<<grid, kRopeThreads, 0, stream>>>(static_cast<T*>(qkv), positions, heads, head_dim,
                                                            rotary_dim, hpc, freq);
  } else {
    rope_kernel<T, false><<<grid, kRopeThreads, 0, stream>>>(static_cast<T*>(qkv), positions, heads, head_dim,
                                                             rotary_dim, hpc, freq);
  }
  return check_launch();
}

}  // namespace

int launch_rmsnorm(void* out, void* residual, const void* in, const void* weight, int32_t dt, int64_t rows,
                   int64_t cols, float eps, cudaStream_t stream) {
  const bool add = residual != nullptr;
  switch (dt) {
    case 0: return add ? launch_rmsnorm_t<float, true>(out, residual, in, weight, rows, cols, eps, stream)
                       : launch_rmsnorm_t<float, false>(out, nullptr, in, weight, rows, cols, eps, stream);
    case 1: return add ? launch_rmsnorm_t<__half, true>(out, residual, in, weight, rows, cols, eps, stream)
                       : launch_rmsnorm_t<__half, false>(out, nullptr, in, weight, rows, cols, eps, stream);
    case 2: return add ? launch_rmsnorm_t<__nv_bfloat16, true>(out, residual, in, weight, rows, cols, eps, stream)
                       : launch_rmsnorm_t<__nv_bfloat16, false>(out, nullptr, in, weight, rows, cols, eps, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

int launch_rmsnorm_quant(void* q, void* scales, void* residual, const void* in, const void* weight, int32_t dt,
                         int64_t rows, int64_t cols, float eps, cudaStream_t stream) {
  if (cols % 128 != 0 || cols / 8 > static_cast<int64_t>(kThreads) * kMaxVec) return INFEROP_ERR_SHAPE;
  const bool add = residual != nullptr;
  switch (dt) {
    case 1: return add ? launch_rmsnorm_quant_t<__half, true>(q, scales, residual, in, weight, rows, cols, eps, stream)
                       : launch_rmsnorm_quant_t<__half, false>(q, scales, nullptr, in, weight, rows, cols, eps, stream);
    case 2: return add ? launch_rmsnorm_quant_t<__nv_bfloat16, true>(q, scales, residual, in, weight, rows, cols, eps, stream)
                       : launch_rmsnorm_quant_t<__nv_bfloat16, false>(q, scales, nullptr, in, weight, rows, cols, eps, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

int launch_rope_neox(void* qkv, const int64_t* positions, int32_t dt, int64_t tokens, int heads, int head_dim,
                     int rotary_dim, float base, float yarn, cudaStream_t stream) {
  if (rotary_dim / 2 > kRopeMaxHalf) return INFEROP_ERR_LIMIT;
  if (tokens > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  switch (dt) {
    case 0: return launch_rope_t<float>(qkv, positions, tokens, heads, head_dim, rotary_dim, base, yarn, stream);
    case 1: return launch_rope_t<__half>(qkv, positions, tokens, heads, head_dim, rotary_dim, base, yarn, stream);
    case 2: return launch_rope_t<__nv_bfloat16>(qkv, positions, tokens, heads, head_dim, rotary_dim, base, yarn, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

}  // namespace ib200
