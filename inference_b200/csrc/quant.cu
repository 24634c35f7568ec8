// Per-token-group FP8 (E4M3) quantisation and its inverse for sm_100a.
//
// Replaces the reference's kernels/quant.cu (quant_fp8_kernel :16-35,
// dequant_fp8_kernel :37-46) and must reproduce reference/reference.cpp:65-80
// bit for bit:
//     amax  = max |x| over the group (NaN never wins)
//     scale = amax * fl(1/448), exactly 1 for an all-zero group
//     q     = e4m3_rn_sat(x / scale)       <- IEEE fp32 division
//
// Layout.  With cols % 128 == 0 and row-major storage, group g of the
// flattened [rows * cols/128] group index space starts at element g*128 of x
// and q and at scales[g]; the kernel therefore treats the tensor as a flat
// array of 128-element groups.  Sixteen lanes own one group: each lane loads
// 8 consecutive elements with one 16-byte load (two for fp32), the absmax is
// reduced with four xor-shuffles inside the half warp, each lane converts its
// 8 values with cvt.rn.satfinite.e4m3x2.f32 and writes them with one 8-byte
// store, so a warp reads 512 contiguous bytes and writes 256.  Every thread
// keeps kUnroll independent groups in flight.
//
// HBM traffic per element: 2 B read + 1 B written + 4/128 B of scale = 3.03 B.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "inferop/fp8.h"
#include "internal.h"
#include "quant_math.cuh"

namespace ib200 {
namespace {

constexpr int kThreads = 256;
#ifndef IB200_QUANT_UNROLL
#define IB200_QUANT_UNROLL 4
#endif
#ifndef IB200_QUANT_MIN_CTAS
#define IB200_QUANT_MIN_CTAS 4
#endif
constexpr int kUnroll = IB200_QUANT_UNROLL;        // groups in flight per half warp
constexpr int kMinCtas = IB200_QUANT_MIN_CTAS;     // resident CTAs per SM the register budget allows

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  uint4 raw;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    raw = __ldg(reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
  }
};
template <>
struct Vec8<__half> {
  uint4 raw;
  __device__ __forceinline__ void load(const __half* p) {
    raw = __ldg(reinterpret_cast<const uint4*>(p));
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
};
template <>
struct Vec8<float> {
  float4 lo, hi;
  __device__ __forceinline__ void load(const float* p) {
    lo = __ldg(reinterpret_cast<const float4*>(p));
    hi = __ldg(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    f[0] = lo.x; f[1] = lo.y; f[2] = lo.z; f[3] = lo.w;
    f[4] = hi.x; f[5] = hi.y; f[6] = hi.z; f[7] = hi.w;
  }
};

template <typename T>
__global__ void __launch_bounds__(kThreads, kMinCtas)
quant128_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const T* __restrict__ x,
                int64_t groups) {
  // a GEMM queued behind this kernel may begin its preamble (barriers, tensor memory, weight
  // prefetch); it waits for this kernel's completion before it reads q or scales
  pdl_launch_dependents();
  // launched with programmatic stream serialisation this kernel may itself have started under the
  // tail of the kernel before it (a GEMM that still reads q and scales, or the producer of x):
  // nothing is read or written before that kernel has completed (a no-op after an ordinary launch)
  pdl_wait();
  const int sub = threadIdx.x & 15;
  const int64_t hw = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 4;
  const int64_t hw_total = (static_cast<int64_t>(gridDim.x) * kThreads) >> 4;
  // the two half warps of a warp own neighbouring groups; loop on the warp's
  // first group so that the shuffles below always run with all 32 lanes
  const int64_t warp_first = hw & ~int64_t(1);
  for (int64_t base = 0; warp_first + base < groups; base += hw_total * kUnroll) {
    Vec8<T> v[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      live[u] = g < groups;
      if (live[u]) v[u].load(x + g * 128 + sub * 8);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      float f[8];
      if (live[u]) {
        v[u].unpack(f);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = 0.0f;
      }
      float amax;
      if constexpr (sizeof(T) == 2) {
        using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
        amax = live[u] ? absmax8_packed<T2>(v[u].raw) : 0.0f;
      } else {
        amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float scale = group_scale(amax);
      if (live[u]) {
        uint2 bytes;
        // 16-bit inputs whose group maximum is far from the ends of the fp32 range divide
        // through the reciprocal, two elements per instruction; everything else uses IEEE division
        if constexpr (sizeof(T) == 2) {
          bytes = fast_div_ok(amax) ? quantise8_fast16(v[u].raw, f, scale, __frcp_rn(scale))
                                    : quantise8<false>(f, scale, 0.0f);
        } else {
          bytes = quantise8<false>(f, scale, 0.0f);
        }
        *reinterpret_cast<uint2*>(q + g * 128 + sub * 8) = bytes;
        if (sub == 0) scales[g] = scale;
      }
    }
  }
}

// Any other group size: one warp per group, strided lanes.  Correctness path
// only; the library's hot path always uses 128.
template <typename T>
__device__ __forceinline__ float widen(T v);
template <>
__device__ __forceinline__ float widen(float v) { return v; }
template <>
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
quant_any_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const T* __restrict__ x,
                 int64_t groups, int gs) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
  for (int64_t g = warp; g < groups; g += warps) {
    const T* gx = x + g * gs;
    float amax = 0.0f;
    for (int i = lane; i < gs; i += 32) amax = fmaxf(amax, fabsf(widen(gx[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float scale = group_scale(amax);
    if (lane == 0) scales[g] = scale;
    for (int i = lane; i < gs; i += 32) {
      const float xv = widen(gx[i]);
      const float r = __fdiv_rn(xv, scale);
      uint32_t b = cvt2(r, 0.0f) & 0xFFu;
      if (r != r) b = nan_byte(xv);
      q[g * gs + i] = static_cast<uint8_t>(b);
    }
  }
}

// E4M3 byte -> fp32, exact (hardware e4m3x2 -> f16x2 conversion, then widen).
__device__ __forceinline__ float decode_e4m3(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
template <typename T>
__device__ __forceinline__ T narrow(float v);
template <>
__device__ __forceinline__ float narrow(float v) { return v; }
template <>
__device__ __forceinline__ __half narrow(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 narrow(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
dequant_kernel(T* __restrict__ x, const uint8_t* __restrict__ q, const float* __restrict__ scales,
               int64_t total, int gs) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += stride) {
    x[i] = narrow<T>(__fmul_rn(decode_e4m3(q[i]), __ldg(scales + i / gs)));
  }
}

// Self-test: hardware converter against the software encoder of
// include/inferop/fp8.h on every fp32 bit pattern in [lo, hi).  NaN inputs are
// counted separately (the hardware drops their sign; quantise8 restores it).
__global__ void __launch_bounds__(kThreads)
cvt_selftest_kernel(uint64_t lo, uint64_t hi, unsigned long long* counts) {
  unsigned long long bad = 0, bad_nan = 0;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads;
  for (uint64_t u = lo + static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x; u < hi;
       u += stride) {
    const float f = __uint_as_float(static_cast<uint32_t>(u));
    const uint32_t hw = cvt2(f, 0.0f) & 0xFFu;
    const uint32_t sw = inferop::fp8::float_to_e4m3_rn_sat(f);
    if (hw != sw) {
      if (f != f) ++bad_nan; else ++bad;
    }
  }
  if (bad) atomicAdd(&counts[0], bad);
  if (bad_nan) atomicAdd(&counts[1], bad_nan);
}

// Self-test of div_by_rcp: for every finite positive 16-bit group maximum (bf16 when
// is_bf16, else fp16) that takes the fast path, and every 16-bit element value no larger in
// magnitude, the E4M3 byte from the reciprocal path must equal the byte from __fdiv_rn.
__global__ void __launch_bounds__(kThreads)
div_selftest_kernel(int is_bf16, unsigned long long* counts) {
  unsigned long long bad = 0, pairs = 0;
  for (uint32_t a = blockIdx.x; a < 0x8000u; a += gridDim.x) {   // a == 0: the all-zero group
    const float amax = is_bf16 ? __uint_as_float(a << 16)
                               : __half2float(__ushort_as_half(static_cast<unsigned short>(a)));
    if (!(amax == amax) || !fast_div_ok(amax)) continue;  // NaN / Inf / out of the fast range
    const float scale = group_scale(amax);
    const float rcp = __frcp_rn(scale);
    for (uint32_t xb = threadIdx.x; xb < 0x10000u; xb += kThreads) {
      const float x = is_bf16 ? __uint_as_float(xb << 16)
                              : __half2float(__ushort_as_half(static_cast<unsigned short>(xb)));
      if (!(fabsf(x) <= amax)) continue;
      ++pairs;
      // the kernels' fast path, element 0 of the eight (the other seven are zeros)
      const uint4 raw = make_uint4(xb, 0u, 0u, 0u);
      const float f8[8] = {x, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
      const uint32_t fast = quantise8_fast16(raw, f8, scale, rcp).x & 0xFFu;
      const uint32_t slow = cvt2(__fdiv_rn(x, scale), 0.0f) & 0xFFu;
      if (fast != slow) {
        ++bad;
        counts[2] = (static_cast<unsigned long long>(a) << 32) | xb;  // one example: group maximum, element
      }
    }
  }
  if (bad) atomicAdd(&counts[0], bad);
  atomicAdd(&counts[1], pairs);
}

int grid_for(int64_t work_items_per_thread_block, int sms) {
  int64_t want = work_items_per_thread_block;
  int64_t cap = static_cast<int64_t>(sms) * 8;  // 8 resident 256-thread CTAs per SM
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  return static_cast<int>(want);
}

}  // namespace

int launch_quant(void* q, void* scales, const void* x, int32_t dt, int64_t rows, int64_t cols,
                 int32_t gs, cudaStream_t stream, int sms) {
  const int64_t groups = rows * (cols / gs);
  uint8_t* qp = static_cast<uint8_t*>(q);
  float* sp = static_cast<float*>(scales);
  const bool vec_ok = gs == 128 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                      (reinterpret_cast<uintptr_t>(q) % 8 == 0);
  if (vec_ok) {
    const int64_t groups_per_block = (kThreads / 16) * kUnroll;
    const int grid = grid_for((groups + groups_per_block - 1) / groups_per_block, sms);
    // programmatic stream serialisation: the launch itself may overlap the tail of the kernel
    // queued before it when that kernel lets its dependents start early (the small-M GEMM does)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = options().quant_pdl ? 1 : 0;
    cudaError_t e;
    switch (dt) {
      case 0: e = cudaLaunchKernelEx(&cfg, quant128_kernel<float>, qp, sp, static_cast<const float*>(x), groups); break;
      case 1: e = cudaLaunchKernelEx(&cfg, quant128_kernel<__half>, qp, sp, static_cast<const __half*>(x), groups); break;
      case 2: e = cudaLaunchKernelEx(&cfg, quant128_kernel<__nv_bfloat16>, qp, sp, static_cast<const __nv_bfloat16*>(x), groups); break;
      default: return INFEROP_ERR_DTYPE;
    }
    if (e != cudaSuccess) return note_cuda_error(e);
  } else {
    const int64_t groups_per_block = kThreads / 32;
    const int grid = grid_for((groups + groups_per_block - 1) / groups_per_block, sms);
    switch (dt) {
      case 0: quant_any_kernel<float><<<grid, kThreads, 0, stream>>>(qp, sp, static_cast<const float*>(x), groups, gs); break;
      case 1: quant_any_kernel<__half><<<grid, kThreads, 0, stream>>>(qp, sp, static_cast<const __half*>(x), groups, gs); break;
      case 2: quant_any_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(qp, sp, static_cast<const __nv_bfloat16*>(x), groups, gs); break;
      default: return INFEROP_ERR_DTYPE;
    }
  }
  return check_launch();
}

int run_cvt_selftest(uint64_t lo, uint64_t hi, uint64_t* out2, int sms) {
  unsigned long long* d = nullptr;
  cudaError_t e = cudaMalloc(&d, 16);
  if (e != cudaSuccess) return note_cuda_error(e);
  cudaMemset(d, 0, 16);
  cvt_selftest_kernel<<<sms * 8, kThreads>>>(lo, hi, d);
  e = cudaMemcpy(out2, d, 16, cudaMemcpyDeviceToHost);
  cudaFree(d);
  return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
}

int run_div_selftest(int is_bf16, uint64_t* out3, int sms) {
  unsigned long long* d = nullptr;
  cudaError_t e = cudaMalloc(&d, 24);
  if (e != cudaSuccess) return note_cuda_error(e);
  cudaMemset(d, 0, 24);
  div_selftest_kernel<<<sms * 8, kThreads>>>(is_bf16, d);
  e = cudaMemcpy(out3, d, 24, cudaMemcpyDeviceToHost);
  cudaFree(d);
  return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
}

int launch_dequant(void* x, int32_t dt, const void* q, const void* scales, int64_t rows,
                   int64_t cols, int32_t gs, cudaStream_t stream, int sms) {
  const int64_t total = rows * cols;
  const int grid = grid_for((total + kThreads - 1) / kThreads, sms);
  const uint8_t* qp = static_cast<const uint8_t*>(q);
  const float* sp = static_cast<const float*>(scales);
  switch (dt) {
    case 0: dequant_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<float*>(x), qp, sp, total, gs); break;
    case 1: dequant_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(x), qp, sp, total, gs); break;
    case 2: dequant_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(x), qp, sp, total, gs); break;
    default: return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

}  // namespace ib200
