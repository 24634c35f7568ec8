// Mixture-of-experts kernels around the grouped blockwise-FP8 GEMM, for sm_100a:
//
//   topk_softmax           routing: softmax over the expert logits + top-k
//                          (reference kernels/moe/topk_softmax.cu:18-97, CPU reference/reference.cpp:152-181)
//   moe_align              expert histogram, row offsets, M-tile table and the stable
//                          expert-sorted position of every (token, k) pair, all on the device
//   moe_scatter_quant      quantise each token row once (1x128 groups, bit-identical to
//                          quant_fp8_per_token_group) and write it to its top-k sorted positions
//   silu_and_mul           SwiGLU between the two expert GEMMs
//                          (reference kernels/silu_mul.cu:16-28, CPU reference/reference.cpp:55-63)
//   silu_and_mul_quant     the same followed by the per-token-group quantisation, in one pass
//   moe_combine            out[t] = sum_k w[t,k] * y[position(t,k)]
//
// All of them are HBM-bound (or latency-bound at these sizes); none touches the tensor cores.
// Nothing here synchronises with the host: the row counts of the experts never leave the
// device, the grouped GEMM reads the tile table that moe_align wrote.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <algorithm>

#include "internal.h"
#include "ptx.cuh"
#include "quant_math.cuh"
#include "swiglu_math.cuh"

namespace ib200 {
namespace {

constexpr int kThreads = 256;

// ---------------------------------------------------------------------------------------------
// Routing.  One warp per token; lane l holds experts l, l + 32, ... in registers, so the row is
// read once with coalesced loads and nothing goes through shared memory.  Ordering rule of the
// reference (reference.cpp:166-170): higher probability first, lower expert index on equal
// probabilities; the comparison is made on the fp32 probabilities exp(logit - max), as there.
// weight = p / sum(p), divided again by the sum of the k weights when `renorm`.
template <int kPerLane>
__global__ void __launch_bounds__(kThreads)
topk_softmax_kernel(int32_t* __restrict__ ids, float* __restrict__ weights,
                    const float* __restrict__ logits, int tokens, int experts, int topk, int renorm) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (t >= tokens) return;
  const float* row = logits + static_cast<int64_t>(t) * experts;
  float p[kPerLane];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    p[j] = e < experts ? __ldg(row + e) : -CUDART_INF_F;
    mx = fmaxf(mx, p[j]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  float l = 0.0f;
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = j * 32 + lane;
    if (e < experts) {
      p[j] = expf(p[j] - mx);
      l += p[j];
    } else {
      p[j] = -1.0f;  // below every probability: never selected
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xFFFFFFFFu, l, o);

  float wsum = 0.0f;
  int32_t* my_ids = ids + static_cast<int64_t>(t) * topk;
  float* my_w = weights + static_cast<int64_t>(t) * topk;
  for (int k = 0; k < topk; ++k) {
    float bv = -1.0f;
    int bi = 0x7FFFFFFF;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      if (p[j] > bv) {  // ascending index inside the lane: the lower index keeps a tie
        bv = p[j];
        bi = j * 32 + lane;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, o);
      const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    // every lane now holds the winner; its owner retires it
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      if (j * 32 + lane == bi) p[j] = -1.0f;
    }
    const float w = bv / l;
    wsum += w;
    if (lane == 0) {
      my_ids[k] = bi;
      my_w[k] = w;
    }
  }
  if (renorm && wsum > 0.0f) {
    __syncwarp();
    for (int k = lane; k < topk; k += 32) my_w[k] = my_w[k] / wsum;
  }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU.  gate_up [rows, 2d]: out[r, i] = silu(gate_up[r, i]) * gate_up[r, d + i], computed in
// fp32 (silu(g) = g / (1 + exp(-g))) and rounded once to the output type.
__device__ __forceinline__ float silu_mul(float g, float u) {
  return (g / (1.0f + expf(-g))) * u;
}
using swiglu::silu_mul_fast;
template <typename T>
__device__ __forceinline__ float silu_mul_as(float g, float u) {
  return sizeof(T) == 2 ? silu_mul_fast(g, u) : silu_mul(g, u);
}

template <typename T>
__device__ __forceinline__ float ld_f32(const T* p);
template <>
__device__ __forceinline__ float ld_f32(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f32(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float ld_f32(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ T st_from_f32(float v);
template <>
__device__ __forceinline__ float st_from_f32(float v) { return v; }
template <>
__device__ __forceinline__ __half st_from_f32(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 st_from_f32(float v) { return __float2bfloat16_rn(v); }

using swiglu::unpack8;
using swiglu::pack2_rn;
using swiglu::silu_mul8;

// 16-bit types, d % 8 == 0, 16-byte aligned: one thread per 8 outputs
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int64_t rows, int64_t d8) {
  const int64_t total = rows * d8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / d8, c = i - r * d8;
    const uint4* row = reinterpret_cast<const uint4*>(gate_up) + r * 2 * d8;
    const uint4 g = __ldg(row + c);
    const uint4 u = __ldg(row + d8 + c);
    reinterpret_cast<uint4*>(out)[i] = silu_mul8<T>(g, u);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_mul_any_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int64_t rows, int64_t d) {
  const int64_t total = rows * d;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / d, c = i - r * d;
    const T* row = gate_up + r * 2 * d;
    out[i] = st_from_f32<T>(silu_mul_as<T>(ld_f32(row + c), ld_f32(row + d + c)));
  }
}

// SwiGLU + per-token-group quantisation (groups of 128 outputs): sixteen lanes own one group,
// each lane 8 outputs.  The SwiGLU result is rounded to T first, exactly as the two separate
// kernels would store and reload it, so bytes and scales equal theirs bit for bit.
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_mul_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales,
                      const T* __restrict__ gate_up, int64_t rows, int64_t d) {
  using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
  const int sub = threadIdx.x & 15;
  const int64_t gpr = d / 128;  // groups per row
  const int64_t groups = rows * gpr;
  const int64_t hw = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 4;
  const int64_t hw_total = (static_cast<int64_t>(gridDim.x) * kThreads) >> 4;
  const int64_t warp_first = hw & ~int64_t(1);
  constexpr int kUnroll = 2;
  for (int64_t base = 0; warp_first + base < groups; base += hw_total * kUnroll) {
    uint4 graw[kUnroll], uraw[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      live[u] = g < groups;
      graw[u] = uraw[u] = make_uint4(0u, 0u, 0u, 0u);
      if (live[u]) {
        const int64_t r = g / gpr, c = g - r * gpr;
        const T* row = gate_up + r * 2 * d + c * 128 + sub * 8;
        graw[u] = __ldg(reinterpret_cast<const uint4*>(row));
        uraw[u] = __ldg(reinterpret_cast<const uint4*>(row + d));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      const uint4 h = silu_mul8<T>(graw[u], uraw[u]);   // zeros for a lane without a group
      float f[8];
      unpack8<T>(h, f);
      float amax = absmax8_packed<T2>(h);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float scale = group_scale(amax);
      if (live[u]) {
        const uint2 bytes = fast_div_ok(amax) ? quantise8_fast16(h, f, scale, __frcp_rn(scale))
                                              : quantise8<false>(f, scale, 0.0f);
        *reinterpret_cast<uint2*>(q + g * 128 + sub * 8) = bytes;
        if (sub == 0) scales[g] = scale;
      }
    }
  }
}

int grid_for(int64_t blocks, int sms, int per_sm) {
  const int64_t cap = static_cast<int64_t>(sms) * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

int launch_topk_softmax(int32_t* ids, float* weights, const float* logits, int32_t tokens,
                        int32_t experts, int32_t topk, int32_t renorm, cudaStream_t stream) {
  const int grid = (tokens + kThreads / 32 - 1) / (kThreads / 32);
#define IB200_TOPK(N)                                                                            \
  topk_softmax_kernel<N><<<grid, kThreads, 0, stream>>>(ids, weights, logits, tokens, experts, \
                                                        topk, renorm)
  if (experts <= 32) IB200_TOPK(1);
  else if (experts <= 64) IB200_TOPK(2);
  else if (experts <= 128) IB200_TOPK(4);
  else if (experts <= 256) IB200_TOPK(8);
  else if (experts <= 512) IB200_TOPK(16);
  else IB200_TOPK(32);
#undef IB200_TOPK
  return check_launch();
}

int launch_silu_and_mul(void* out, const void* gate_up, int32_t dt, int64_t rows, int64_t d,
                        cudaStream_t stream, int sms) {
  const bool vec = dt != 0 && d % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(gate_up) % 16 == 0;
  if (vec) {
    const int64_t d8 = d / 8;
    const int grid = grid_for((rows * d8 + kThreads - 1) / kThreads, sms, 8);
    if (dt == 1) {
      silu_mul_vec_kernel<__half><<<grid, kThreads, 0, stream>>>(
          static_cast<__half*>(out), static_cast<const __half*>(gate_up), rows, d8);
    } else {
      silu_mul_vec_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
          static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), rows, d8);
    }
    return check_launch();
  }
  const int grid = grid_for((rows * d + kThreads - 1) / kThreads, sms, 8);
  switch (dt) {
    case 0: silu_mul_any_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<float*>(out), static_cast<const float*>(gate_up), rows, d); break;
    case 1: silu_mul_any_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(out), static_cast<const __half*>(gate_up), rows, d); break;
    case 2: silu_mul_any_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), rows, d); break;
    default: return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

int launch_silu_and_mul_quant(void* q, void* scales, const void* gate_up, int32_t dt, int64_t rows,
                              int64_t d, cudaStream_t stream, int sms) {
  const int64_t groups = rows * (d / 128);
  const int grid = grid_for((groups + (kThreads / 16) * 2 - 1) / ((kThreads / 16) * 2), sms, 8);
  if (dt == 1) {
    silu_mul_quant_kernel<__half><<<grid, kThreads, 0, stream>>>(
        static_cast<uint8_t*>(q), static_cast<float*>(scales), static_cast<const __half*>(gate_up), rows, d);
  } else if (dt == 2) {
    silu_mul_quant_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        static_cast<uint8_t*>(q), static_cast<float*>(scales), static_cast<const __nv_bfloat16*>(gate_up), rows, d);
  } else {
    return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

namespace {

// ---------------------------------------------------------------------------------------------
// moe_align: everything the grouped GEMM and the scatter / combine kernels need to know about a
// routing, computed without leaving the device by one thread-block cluster of up to 8 CTAs of
// 1024 threads (one CTA for small routings).
//   counts[e]        rows routed to expert e
//   offsets[e]       first row of expert e in the expert-sorted order (offsets[experts] = pairs)
//   pos[i]           sorted row of pair i = token * topk + k; inside an expert the pairs keep
//                    their order of i (a stable counting sort), so the layout is deterministic
//   src_token[r]     token whose copy sits in sorted row r
//   tile_row0/meta   the experts' rows cut into M-tiles of up to 128 rows (first row, and
//                    (expert << 8) | (rows - 1)); num_mtiles[0] = how many
// The warps of the cluster, numbered CTA by CTA, take contiguous chunks of the pairs.  Every warp
// counts its chunk into its own histogram; a CTA's per-expert totals are read by the other CTAs
// through distributed shared memory, so every CTA knows how many rows of an expert lie in the
// CTAs before it and in all of them.  An exclusive scan over the experts (repeated by each CTA,
// it is 1024 values) and the scan over the warps give every (warp, expert) its first row; each
// warp then walks its chunk in order, 32 pairs at a time, ranking equal experts by lane.
constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;
constexpr int kAlignMaxCtas = 8;          // the portable cluster size

__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ int32_t ld_cluster_s32(uint32_t cluster_addr) {
  int32_t v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}

__global__ void __launch_bounds__(kAlignThreads, 1)
moe_align_kernel(const int32_t* __restrict__ ids, int pairs, int topk, int experts,
                 int32_t* __restrict__ counts, int32_t* __restrict__ offsets, int32_t* __restrict__ pos,
                 int32_t* __restrict__ src_token, int32_t* __restrict__ tile_row0,
                 int32_t* __restrict__ tile_meta, int32_t* __restrict__ num_mtiles) {
  extern __shared__ int32_t align_smem[];
  int32_t* hist = align_smem;                                   // [kAlignWarps][experts]
  int32_t* cta_total = hist + kAlignWarps * experts;            // [1024], read by the other CTAs
  unsigned long long* scan = reinterpret_cast<unsigned long long*>(cta_total + kAlignThreads);  // [1024]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = static_cast<int>(cluster_ctarank()), nranks = static_cast<int>(cluster_nctarank());
  for (int i = tid; i < kAlignWarps * experts; i += kAlignThreads) hist[i] = 0;
  __syncthreads();

  const int all_warps = nranks * kAlignWarps;
  const int chunk = ((pairs + all_warps - 1) / all_warps + 31) & ~31;
  const long long first = static_cast<long long>(rank * kAlignWarps + warp) * chunk;
  const int begin = static_cast<int>(min(static_cast<long long>(pairs), first));
  const int end = static_cast<int>(min(static_cast<long long>(pairs), first + chunk));
  int32_t* my_hist = hist + warp * experts;
  for (int i0 = begin; i0 < end; i0 += 256) {   // eight loads in flight per lane
    int ev[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * 32 + lane;
      ev[u] = i < end ? __ldg(ids + i) : -1;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (ev[u] >= 0 && ev[u] < experts) atomicAdd(&my_hist[ev[u]], 1);
    }
  }
  __syncthreads();

  // per expert: rows of this CTA's warps before each warp, and the CTA's total
  int mine = 0;
  if (tid < experts) {
    for (int w = 0; w < kAlignWarps; ++w) {
      const int c = hist[w * experts + tid];
      hist[w * experts + tid] = mine;
      mine += c;
    }
  }
  cta_total[tid] = mine;
  cluster_sync_all();
  // rows of the expert in the CTAs before this one, and in the whole cluster
  int count = 0, before = 0;
  if (tid < experts) {
    const uint32_t local = smem_u32(cta_total + tid);
    for (int r = 0; r < nranks; ++r) {
      const int c = r == rank ? mine : ld_cluster_s32(mapa_shared(local, static_cast<uint32_t>(r)));
      before += r < rank ? c : 0;
      count += c;
    }
  }
  // nobody reads another CTA's shared memory after this point; the matching wait stands at the
  // end of the kernel, so that no CTA leaves while a neighbour may still read its totals
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  const int tiles = (count + 127) >> 7;
  // inclusive scan over the experts of (tiles, rows) packed into one 64-bit word: by shuffles
  // inside a warp, then over the 32 warp sums
  unsigned long long v = (static_cast<unsigned long long>(tiles) << 32) | static_cast<unsigned>(count);
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, v, o);
    if (lane >= o) v += up;
  }
  if (lane == 31) scan[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long s = scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long up = __shfl_up_sync(0xFFFFFFFFu, s, o);
      if (lane >= o) s += up;
    }
    scan[lane] = s;
  }
  __syncthreads();
  if (warp > 0) v += scan[warp - 1];
  const int row_first = static_cast<int>(v & 0xFFFFFFFFull) - count;   // exclusive
  const int tile_first = static_cast<int>(v >> 32) - tiles;
  if (tid < experts) {
    for (int w = 0; w < kAlignWarps; ++w) hist[w * experts + tid] += row_first + before;
    if (rank == 0) {
      counts[tid] = count;
      offsets[tid] = row_first;
      for (int j = 0; j < tiles; ++j) {
        tile_row0[tile_first + j] = row_first + j * 128;
        tile_meta[tile_first + j] = (tid << 8) | (min(128, count - j * 128) - 1);
      }
    }
  }
  if (rank == 0 && tid == kAlignThreads - 1) {
    offsets[experts] = static_cast<int>(v & 0xFFFFFFFFull);
    num_mtiles[0] = static_cast<int>(v >> 32);
  }
  __syncthreads();

  const int id_bits = 32 - __clz(max(experts - 1, 1));
  // the ids of four steps are requested together, so their latency is paid once per four steps
  for (int i0 = begin; i0 < end; i0 += 128) {
    int ev[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * 32 + lane;
      ev[u] = i < end ? __ldg(ids + i) : -1;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = i0 + u * 32 + lane;
      if (i0 + u * 32 >= end) break;                      // warp-uniform
      int e = ev[u];
      if (e >= experts) e = -1;
      // lanes of this step that hold the same expert: one ballot per bit of the expert index
      // (far cheaper than match.any when most of the 32 values differ)
      unsigned peers = __ballot_sync(0xFFFFFFFFu, e >= 0);
      for (int b = 0; b < id_bits; ++b) {
        const unsigned bal = __ballot_sync(0xFFFFFFFFu, (e >> b) & 1);
        peers &= ((e >> b) & 1) ? bal : ~bal;
      }
      int row = -1;
      if (e >= 0) row = my_hist[e] + __popc(peers & ((1u << lane) - 1u));
      __syncwarp();
      if (e >= 0 && lane == 31 - __clz(peers)) my_hist[e] = row + 1;   // the last of the equals
      __syncwarp();
      if (i < end) {
        pos[i] = row;
        if (row >= 0) src_token[row] = i / topk;
      }
    }
  }
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// moe_scatter_quant: x [tokens, cols] (bf16 / fp16) -> q [pairs, cols], scales [pairs, cols/128]
// in expert-sorted row order.  A token row is quantised once (the arithmetic of quant128_kernel)
// and its bytes and scales are written to the sorted rows of its top-k copies.
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_scatter_quant_kernel(uint8_t* __restrict__ q, float* __restrict__ scales, const T* __restrict__ x,
                         const int32_t* __restrict__ pos, int64_t tokens, int64_t cols, int topk) {
  using T2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
  constexpr int kUnroll = 2;
  const int sub = threadIdx.x & 15;
  const int64_t gpr = cols / 128;
  const int64_t groups = tokens * gpr;
  const int64_t hw = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 4;
  const int64_t hw_total = (static_cast<int64_t>(gridDim.x) * kThreads) >> 4;
  const int64_t warp_first = hw & ~int64_t(1);
  for (int64_t base = 0; warp_first + base < groups; base += hw_total * kUnroll) {
    uint4 raw[kUnroll];
    bool live[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      live[u] = g < groups;
      raw[u] = live[u] ? __ldg(reinterpret_cast<const uint4*>(x + g * 128 + sub * 8)) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t g = hw + base + u * hw_total;
      float f[8];
      unpack8<T>(raw[u], f);
      float amax = absmax8_packed<T2>(raw[u]);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
      const float scale = group_scale(amax);
      if (live[u]) {
        const uint2 bytes = fast_div_ok(amax) ? quantise8_fast16(raw[u], f, scale, __frcp_rn(scale))
                                              : quantise8<false>(f, scale, 0.0f);
        const int64_t t = g / gpr, c = g - t * gpr;
        for (int k = 0; k < topk; ++k) {
          const int64_t r = __ldg(pos + t * topk + k);
          if (r < 0) continue;
          *reinterpret_cast<uint2*>(q + r * cols + c * 128 + sub * 8) = bytes;
          if (sub == 0) scales[r * gpr + c] = scale;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// moe_combine: out[t, :] = sum over k (in order) of w[t, k] * y[pos[t, k], :], every product and
// every sum rounded to fp32, the result rounded once to the output type.  One thread per 8 columns.
template <typename T>
__global__ void __launch_bounds__(kThreads)
moe_combine_kernel(T* __restrict__ out, const T* __restrict__ y, const float* __restrict__ w,
                   const int32_t* __restrict__ pos, int64_t tokens, int64_t h8, int topk) {
  const int64_t total = tokens * h8;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t t = i / h8, c = i - t * h8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
    for (int k = 0; k < topk; ++k) {
      const int64_t r = __ldg(pos + t * topk + k);
      if (r < 0) continue;
      const float wk = __ldg(w + t * topk + k);
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(y) + r * h8 + c);
      float f[8];
      unpack8<T>(raw, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(wk, f[j]));
    }
    uint4 o;
    o.x = pack2_rn<T>(acc[0], acc[1]);
    o.y = pack2_rn<T>(acc[2], acc[3]);
    o.z = pack2_rn<T>(acc[4], acc[5]);
    o.w = pack2_rn<T>(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace

int64_t moe_max_mtiles(int64_t pairs, int64_t experts) {
  // every expert adds at most one partly filled tile to the full ones
  return pairs / 128 + experts;
}

int launch_moe_align(const int32_t* ids, int64_t tokens, int32_t topk, int32_t experts, int32_t* counts,
                     int32_t* offsets, int32_t* pos, int32_t* src_token, int32_t* tile_row0,
                     int32_t* tile_meta, int32_t* num_mtiles, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(kAlignWarps) * experts * 4 + kAlignThreads * 4 + kAlignThreads * 8;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(moe_align_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kAlignWarps * 1024 * 4 + kAlignThreads * 12);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  // one CTA per 4096 pairs (four steps of 32 per warp), up to the portable cluster size
  const int64_t pairs = tokens * topk;
  int ctas = static_cast<int>(std::min<int64_t>(kAlignMaxCtas, (pairs + 4095) / 4096));
  if (options().align_ctas > 0) ctas = std::min(options().align_ctas, kAlignMaxCtas);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kAlignThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, moe_align_kernel, ids, static_cast<int>(pairs), static_cast<int>(topk),
                                     static_cast<int>(experts), counts, offsets, pos, src_token, tile_row0,
                                     tile_meta, num_mtiles);
  if (e != cudaSuccess) return note_cuda_error(e);
  return check_launch();
}

int launch_moe_scatter_quant(void* q, void* scales, const void* x, int32_t dt, const int32_t* pos,
                             int64_t tokens, int64_t cols, int32_t topk, cudaStream_t stream, int sms) {
  const int64_t groups = tokens * (cols / 128);
  const int grid = grid_for((groups + (kThreads / 16) * 2 - 1) / ((kThreads / 16) * 2), sms, 8);
  if (dt == 1) {
    moe_scatter_quant_kernel<__half><<<grid, kThreads, 0, stream>>>(
        static_cast<uint8_t*>(q), static_cast<float*>(scales), static_cast<const __half*>(x), pos, tokens, cols, topk);
  } else if (dt == 2) {
    moe_scatter_quant_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        static_cast<uint8_t*>(q), static_cast<float*>(scales), static_cast<const __nv_bfloat16*>(x), pos, tokens, cols, topk);
  } else {
    return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

namespace {
// Rows of row_bytes bytes moved by a permutation: scatter (dst[perm[i]] = src[i]) or gather
// (dst[i] = src[perm[i]]); rows with perm < 0 are skipped.  16 bytes per thread and step.
// Expert-parallel layers use it to bring rows received from other ranks into expert-sorted
// order and the experts' outputs back into the order they arrived in.
template <bool kGather>
__global__ void __launch_bounds__(kThreads)
permute_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, const int32_t* __restrict__ perm,
                    int64_t rows, int64_t vec_per_row) {
  const int64_t total = rows * vec_per_row;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t r = i / vec_per_row, c = i - r * vec_per_row;
    const int64_t pr = __ldg(perm + r);
    if (pr < 0) continue;
    if (kGather) dst[i] = __ldg(src + pr * vec_per_row + c);
    else dst[pr * vec_per_row + c] = __ldg(src + i);
  }
}
}  // namespace

int launch_permute_rows(void* dst, const void* src, const int32_t* perm, int64_t rows, int64_t row_bytes,
                        int32_t gather, cudaStream_t stream, int sms) {
  const int64_t vec = row_bytes / 16;
  const int grid = grid_for((rows * vec + kThreads - 1) / kThreads, sms, 8);
  if (gather) {
    permute_rows_kernel<true><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src),
                                                             perm, rows, vec);
  } else {
    permute_rows_kernel<false><<<grid, kThreads, 0, stream>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src),
                                                              perm, rows, vec);
  }
  return check_launch();
}

int launch_moe_combine(void* out, const void* y, const float* w, const int32_t* pos, int32_t dt,
                       int64_t tokens, int64_t hidden, int32_t topk, cudaStream_t stream, int sms) {
  const int64_t h8 = hidden / 8;
  const int grid = grid_for((tokens * h8 + kThreads - 1) / kThreads, sms, 8);
  if (dt == 1) {
    moe_combine_kernel<__half><<<grid, kThreads, 0, stream>>>(static_cast<__half*>(out), static_cast<const __half*>(y), w, pos, tokens, h8, topk);
  } else if (dt == 2) {
    moe_combine_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(y), w, pos, tokens, h8, topk);
  } else {
    return INFEROP_ERR_DTYPE;
  }
  return check_launch();
}

}  // namespace ib200

