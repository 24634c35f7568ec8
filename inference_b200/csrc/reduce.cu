// Second half of the reduce-scatter of the row-parallel (K-sharded) GEMM: the owner of a block
// of output rows adds the fp32 partial results that every rank's GEMM epilogue stored into its
// slots, in rank order (so the sum never depends on arrival order), and rounds once to the
// output type.  HBM-bound: ranks * 4 bytes read + sizeof(out) written per element.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "internal.h"

namespace ib200 {
namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ void store4(T* out, int64_t i4, const float4& v);
template <>
__device__ __forceinline__ void store4(float* out, int64_t i4, const float4& v) {
  reinterpret_cast<float4*>(out)[i4] = v;
}
template <>
__device__ __forceinline__ void store4(__half* out, int64_t i4, const float4& v) {
  const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  reinterpret_cast<uint2*>(out)[i4] =
      make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}
template <>
__device__ __forceinline__ void store4(__nv_bfloat16* out, int64_t i4, const float4& v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  reinterpret_cast<uint2*>(out)[i4] =
      make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
}

// slots [ranks][elems] fp32, elems % 4 == 0
template <typename T>
__global__ void __launch_bounds__(kThreads)
reduce_slots_kernel(T* __restrict__ out, const float* __restrict__ slots, int ranks, int64_t elems4) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < elems4;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    float4 acc = __ldcs(reinterpret_cast<const float4*>(slots) + i);
    for (int r = 1; r < ranks; ++r) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(slots) + r * elems4 + i);
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    store4<T>(out, i, acc);
  }
}

}  // namespace

int launch_reduce_slots(void* out, int32_t out_dt, const void* slots, int32_t ranks, int64_t elems,
                        cudaStream_t stream, int sms) {
  const int64_t e4 = elems / 4;
  int64_t blocks = (e4 + kThreads - 1) / kThreads;
  const int64_t cap = static_cast<int64_t>(sms) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const int grid = static_cast<int>(blocks);
  const float* s = static_cast<const float*>(slots);
  switch (out_dt) {
    case 0: reduce_slots_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<float*>(out), s, ranks, e4); break;
    case 1: reduce_slots_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(out), s, ranks, e4); break;
    case 2: reduce_slots_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(out), s, ranks, e4); break;
    default: return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

}  // namespace ib200
