// Paged attention, single-token decode with grouped-query heads, for sm_100 (reference
// kernels/attention/paged_attn_decode.cu:26-118; CPU golden reference/reference.cpp:112-150).
//
//   q / out  [batch, heads, head_dim]
//   k / v    [blocks, block_size, kv_heads, head_dim]   (paged; block_tables int32 [batch, max_blocks])
//
// The step is a stream of the sequence's K and V rows from HBM, so the mapping follows the bytes:
//   * the query heads that share a KV head are processed together (up to four per CTA), so a K / V
//     row is fetched once for the group; the reference launches one block per query head and reads
//     the cache once per head.
//   * a K or V row is one coalesced access of a group of lanes, 16 bytes each (8 / 16 / 32 lanes
//     for 64 / 128 / 256 16-bit elements); such a lane group is an independent token stream with
//     its own running maximum, denominator and accumulator (online softmax), four tokens in
//     flight per step.  No block-wide synchronisation inside the token loop.
//   * long sequences are cut into `splits` token ranges, one CTA each, so that a small batch
//     still fills the GPU; the CTA's streams are merged through shared memory, the splits by a
//     second small kernel (log-sum-exp merge, fixed order: reproducible).
// Scores are kept in the base-2 domain (q is pre-multiplied by scale * log2 e), probabilities by
// exp2f: softmax is unchanged.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "internal.h"

namespace ib200 {
namespace {

constexpr int kThreads = 128;
constexpr int kBatch = 4;   // tokens of a stream per step
constexpr int kDepth = 3;   // steps in flight (shared-memory ring)

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

// 2^x for x <= 0 by the special-function unit alone (results below the normal range flush to 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// the elements of one 16-byte vector as floats (16-bit types: pure bit operations / packed converts)
template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4& raw, float* f);
template <>
__device__ __forceinline__ void unpack_vec<float>(const uint4& raw, float* f) {
  f[0] = __uint_as_float(raw.x);
  f[1] = __uint_as_float(raw.y);
  f[2] = __uint_as_float(raw.z);
  f[3] = __uint_as_float(raw.w);
}
template <>
__device__ __forceinline__ void unpack_vec<__nv_bfloat16>(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void unpack_vec<__half>(const uint4& raw, float* f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

template <typename T, int D>
struct ACfg {
  static constexpr int EV = 16 / sizeof(T);                                  // elements per 16-byte vector
  static constexpr int kVecPerRow = D / EV;
  static constexpr int LPT = kVecPerRow > 32 ? 32 : kVecPerRow;              // lanes per token
  static constexpr int VPL = kVecPerRow / LPT;                               // vectors per lane and row
  static constexpr int EPL = VPL * EV;                                       // elements per lane and row
  static constexpr int TPW = 32 / LPT;                                       // token streams per warp
  static constexpr int NS = (kThreads / 32) * TPW;                           // token streams per CTA
};

struct AttnParams {
  void* out;
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* block_tables;
  const int32_t* seq_lens;
  float* partial;   // [batch][heads][splits][D + 2]: accumulator, running maximum (base 2), denominator
  int num_heads, num_kv_heads, block_size, block_shift, max_blocks_per_seq, splits;   // block_shift: log2(block_size) or -1
  float scale_log2e;
};

// element e (0 .. EPL) of a lane's share of a row -> index inside the row
template <typename C>
__device__ __forceinline__ int elem_index(int sub, int e) {
  return ((e / C::EV) * C::LPT + sub) * C::EV + (e % C::EV);
}

template <typename T, int D, int GT>
__global__ void __launch_bounds__(kThreads, 4)
paged_attn_kernel(const AttnParams p) {
  using C = ACfg<T, D>;
  extern __shared__ float sm[];   // [NS][GT][D + 2] at the end: the streams' states
  const int split = blockIdx.x;
  const int groups_per_kvh = (p.num_heads / p.num_kv_heads) / GT;
  const int kvh = blockIdx.y / groups_per_kvh;
  const int hg = blockIdx.y % groups_per_kvh;
  const int b = blockIdx.z;
  const int head0 = kvh * (p.num_heads / p.num_kv_heads) + hg * GT;   // first query head of this CTA

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % C::LPT;                    // position inside the lane group of a token
  const int stream = warp * C::TPW + lane / C::LPT;  // token stream of this lane group

  int len = __ldg(p.seq_lens + b);
  const int cap = p.max_blocks_per_seq * p.block_size;
  len = len < 0 ? 0 : (len > cap ? cap : len);
  const int per_split = (len + p.splits - 1) / p.splits;
  const int t0 = split * per_split;
  const int t1 = min(len, t0 + per_split);
  const int32_t* bt = p.block_tables + static_cast<int64_t>(b) * p.max_blocks_per_seq;

  // this lane's share of the group's query rows, pre-multiplied so that scores come out in base 2
  float qf[GT][C::EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    const T* qrow = static_cast<const T*>(p.q) + (static_cast<int64_t>(b) * p.num_heads + head0 + g) * D;
#pragma unroll
    for (int e = 0; e < C::EPL; ++e) qf[g][e] = to_f32<T>(qrow[elem_index<C>(sub, e)]) * p.scale_log2e;
  }
  float m[GT], l[GT], acc[GT][C::EPL];
#pragma unroll
  for (int g = 0; g < GT; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.0f;
#pragma unroll
    for (int e = 0; e < C::EPL; ++e) acc[g][e] = 0.0f;
  }

  const T* kc = static_cast<const T*>(p.k_cache);
  const T* vc = static_cast<const T*>(p.v_cache);
  // K and V rows travel through a ring in shared memory by cp.async, kDepth steps ahead of the
  // arithmetic: every lane copies the 16-byte pieces it will itself consume, so the only
  // synchronisation is the lane's own wait for its copy groups, and the bytes in flight are not
  // limited by registers.  Layout: [step % kDepth][token of the step][K, V][vector][thread].
  constexpr int kSlotVecs = kBatch * 2 * C::VPL;           // 16-byte pieces per thread and step
  uint4* ring = reinterpret_cast<uint4*>(sm);              // the streams' final states reuse this memory
  auto issue = [&](int step_tb0, int slot) {
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      const int t = step_tb0 + stream + c * C::NS;
      if (t < t1) {
        // (a power-of-two block size, the usual case, needs no division)
        const int bi = p.block_shift >= 0 ? t >> p.block_shift : t / p.block_size;
        const int off = p.block_shift >= 0 ? t & (p.block_size - 1) : t - bi * p.block_size;
        const int blk = __ldg(bt + bi);
        const int64_t row = ((static_cast<int64_t>(blk) * p.block_size + off) * p.num_kv_heads + kvh) * D;
#pragma unroll
        for (int v = 0; v < C::VPL; ++v) {
          uint4* dk = ring + (static_cast<size_t>(slot) * kSlotVecs + (c * 2 + 0) * C::VPL + v) * kThreads + threadIdx.x;
          uint4* dv = ring + (static_cast<size_t>(slot) * kSlotVecs + (c * 2 + 1) * C::VPL + v) * kThreads + threadIdx.x;
          const uint4* sk = reinterpret_cast<const uint4*>(kc + row) + v * C::LPT + sub;
          const uint4* sv = reinterpret_cast<const uint4*>(vc + row) + v * C::LPT + sub;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dk)), "l"(sk) : "memory");
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dv)), "l"(sv) : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per step, empty or not
  };
  constexpr int kStep = C::NS * kBatch;                    // tokens of the CTA per step
#pragma unroll
  for (int j = 0; j < kDepth - 1; ++j) issue(t0 + j * kStep, j);

  // the trip count is the same for every lane of the CTA (the shuffles below need whole warps);
  // a stream whose tokens of a step all lie beyond the range skips the update
  int slot = 0;
  for (int tb0 = t0; tb0 < t1; tb0 += kStep) {
    const int tb = tb0 + stream;
    {
      int ahead = slot + kDepth - 1;
      if (ahead >= kDepth) ahead -= kDepth;
      issue(tb0 + (kDepth - 1) * kStep, ahead);
    }
    asm volatile("cp.async.wait_group %0;" ::"n"(kDepth - 1) : "memory");
    uint4 kr[kBatch][C::VPL], vr[kBatch][C::VPL];
    bool valid[kBatch];
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      valid[c] = tb + c * C::NS < t1;
#pragma unroll
      for (int v = 0; v < C::VPL; ++v) {
        kr[c][v] = ring[(static_cast<size_t>(slot) * kSlotVecs + (c * 2 + 0) * C::VPL + v) * kThreads + threadIdx.x];
        vr[c][v] = ring[(static_cast<size_t>(slot) * kSlotVecs + (c * 2 + 1) * C::VPL + v) * kThreads + threadIdx.x];
      }
    }
    if (++slot == kDepth) slot = 0;
    // ---- scores of the batch for every head of the group: this lane's partial dot products ...
    constexpr int NV = GT * kBatch;   // values to be summed over the LPT lanes of the token group
    float val[NV];
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      // (the slot of a token beyond the range holds stale bytes: its scores are masked below)
      float kf[C::EPL];
#pragma unroll
      for (int v = 0; v < C::VPL; ++v) unpack_vec<T>(kr[c][v], kf + v * C::EV);
#pragma unroll
      for (int g = 0; g < GT; ++g) {
        float part = 0.0f;
#pragma unroll
        for (int e = 0; e < C::EPL; ++e) part = fmaf(qf[g][e], kf[e], part);
        val[g * kBatch + c] = part;
      }
    }
    // ... summed by a reduce-scatter butterfly (every step halves the values a lane carries:
    // NV - 1 shuffles instead of NV log2(LPT); the warp shuffle unit is the scarce resource here)
    // and handed back to all lanes of the group from their owners
    {
      int cnt = NV;
#pragma unroll
      for (int o = C::LPT / 2; o > 0; o >>= 1) {
        if (cnt > 1) {
          const bool upper = (sub & o) != 0;
          cnt >>= 1;
#pragma unroll
          for (int i = 0; i < NV / 2; ++i) {
            if (i < cnt) {
              const float keep = upper ? val[i + cnt] : val[i];
              const float send = upper ? val[i] : val[i + cnt];
              val[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
            }
          }
        } else {
          val[0] += __shfl_xor_sync(0xFFFFFFFFu, val[0], o);
        }
      }
    }
    float s2[GT][kBatch];
    {
      constexpr int CF = NV >= C::LPT ? NV / C::LPT : 1;      // totals a lane owns after the butterfly
      constexpr int LF = NV >= C::LPT ? 1 : C::LPT / NV;      // lanes that hold the same total
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        const float tot = __shfl_sync(0xFFFFFFFFu, val[v % CF], (v / CF) * LF, C::LPT);
        s2[v / kBatch][v % kBatch] = valid[v % kBatch] ? tot : -INFINITY;
      }
    }
    // ---- online softmax update (with valid[0] the maxima are finite)
    if (!valid[0]) continue;
    float pr[GT][kBatch];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
      float m_new = m[g];
#pragma unroll
      for (int c = 0; c < kBatch; ++c) m_new = fmaxf(m_new, s2[g][c]);
      if (m_new > m[g]) {
        // a new maximum (always so in a stream's first step, where m = -inf and alpha = 0; rare
        // later in a long sequence): the state is rescaled
        const float alpha = ex2(m[g] - m_new);
        l[g] *= alpha;
#pragma unroll
        for (int e = 0; e < C::EPL; ++e) acc[g][e] *= alpha;
        m[g] = m_new;
      }
      float ps = 0.0f;
#pragma unroll
      for (int c = 0; c < kBatch; ++c) {
        pr[g][c] = ex2(s2[g][c] - m_new);        // 0 for a missing token
        ps += pr[g][c];
      }
      l[g] += ps;
    }
#pragma unroll
    for (int c = 0; c < kBatch; ++c) {
      if (valid[c]) {
        float vf[C::EPL];
#pragma unroll
        for (int v = 0; v < C::VPL; ++v) unpack_vec<T>(vr[c][v], vf + v * C::EV);
#pragma unroll
        for (int g = 0; g < GT; ++g) {
#pragma unroll
          for (int e = 0; e < C::EPL; ++e) acc[g][e] = fmaf(pr[g][c], vf[e], acc[g][e]);
        }
      }
    }
  }

  // ---- merge the CTA's streams: every stream leaves its state in shared memory (the ring's)
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  constexpr int kRec = D + 2;
  float* mine = sm + (static_cast<size_t>(stream) * GT) * kRec;
#pragma unroll
  for (int g = 0; g < GT; ++g) {
#pragma unroll
    for (int e = 0; e < C::EPL; ++e) mine[g * kRec + elem_index<C>(sub, e)] = acc[g][e];
    if (sub == 0) {
      mine[g * kRec + D] = m[g];
      mine[g * kRec + D + 1] = l[g];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < GT * D; idx += kThreads) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
    for (int s = 0; s < C::NS; ++s) mm = fmaxf(mm, sm[(s * GT + g) * kRec + D]);
    float a = 0.0f, ll = 0.0f;
    for (int s = 0; s < C::NS; ++s) {
      const float* rec = sm + (s * GT + g) * kRec;
      const float w = rec[D] == -INFINITY ? 0.0f : exp2f(rec[D] - mm);
      a = fmaf(rec[d], w, a);
      ll = fmaf(rec[D + 1], w, ll);
    }
    const int64_t head = static_cast<int64_t>(b) * p.num_heads + head0 + g;
    if (p.splits == 1) {
      static_cast<T*>(p.out)[head * D + d] = from_f32<T>(ll == 0.0f ? 0.0f : a / ll);
    } else {
      float* dst = p.partial + (head * p.splits + split) * kRec;
      dst[d] = a;
      if (d == 0) {
        dst[D] = mm;
        dst[D + 1] = ll;
      }
    }
  }
}

// out[b, h, :] from the `splits` partial states of the head; grid (heads, batch), D threads.
template <typename T, int D>
__global__ void __launch_bounds__(D)
paged_attn_merge_kernel(const AttnParams p) {
  constexpr int kRec = D + 2;
  const int64_t head = static_cast<int64_t>(blockIdx.y) * p.num_heads + blockIdx.x;
  const float* base = p.partial + head * p.splits * kRec;
  const int d = threadIdx.x;
  float mm = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, base[s * kRec + D]);
  float a = 0.0f, ll = 0.0f;
  for (int s = 0; s < p.splits; ++s) {
    const float* rec = base + s * kRec;
    const float w = rec[D] == -INFINITY ? 0.0f : exp2f(rec[D] - mm);
    a = fmaf(rec[d], w, a);
    ll = fmaf(rec[D + 1], w, ll);
  }
  static_cast<T*>(p.out)[head * D + d] = from_f32<T>(ll == 0.0f ? 0.0f : a / ll);
}

template <typename T, int D, int GT>
int launch_attn_gt(const AttnParams& p, int batch, cudaStream_t stream) {
  using C = ACfg<T, D>;
  const size_t states = static_cast<size_t>(C::NS) * GT * (D + 2) * sizeof(float);
  const size_t ring = static_cast<size_t>(kDepth) * kBatch * 2 * C::VPL * kThreads * 16;
  const size_t smem = states > ring ? states : ring;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(paged_attn_kernel<T, D, GT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(smem));
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  const int groups = p.num_kv_heads * ((p.num_heads / p.num_kv_heads) / GT);
  const dim3 grid(static_cast<unsigned>(p.splits), static_cast<unsigned>(groups), static_cast<unsigned>(batch));
  paged_attn_kernel<T, D, GT><<<grid, kThreads, smem, stream>>>(p);
  int rc = check_launch();
  if (rc != INFEROP_OK || p.splits == 1) return rc;
  paged_attn_merge_kernel<T, D><<<dim3(static_cast<unsigned>(p.num_heads), static_cast<unsigned>(batch)), D, 0, stream>>>(p);
  return check_launch();
}

int heads_per_cta(int group) {
  const int forced = options().attn_heads_per_cta;
  if ((forced == 1 || forced == 2 || forced == 4) && group % forced == 0) return forced;
  return group % 4 == 0 ? 4 : (group % 2 == 0 ? 2 : 1);
}

template <typename T, int D>
int launch_attn_d(const AttnParams& p, int batch, cudaStream_t stream) {
  switch (heads_per_cta(p.num_heads / p.num_kv_heads)) {
    case 4: return launch_attn_gt<T, D, 4>(p, batch, stream);
    case 2: return launch_attn_gt<T, D, 2>(p, batch, stream);
    default: return launch_attn_gt<T, D, 1>(p, batch, stream);
  }
}

template <typename T>
int launch_attn_t(const AttnParams& p, int batch, int head_dim, cudaStream_t stream) {
  switch (head_dim) {
    case 64: return launch_attn_d<T, 64>(p, batch, stream);
    case 128: return launch_attn_d<T, 128>(p, batch, stream);
    case 256: return launch_attn_d<T, 256>(p, batch, stream);
    default: return INFEROP_ERR_SHAPE;
  }
}

}  // namespace

int paged_attn_splits(int sm_count, int batch, int num_heads, int num_kv_heads, int block_size, int max_blocks_per_seq) {
  const int g = num_heads / num_kv_heads;
  const int gt = heads_per_cta(g);
  const int64_t base = static_cast<int64_t>(batch) * num_kv_heads * (g / gt);
  if (options().attn_splits > 0) return options().attn_splits > 128 ? 128 : options().attn_splits;
  int64_t splits = (4LL * sm_count + base - 1) / base;                       // about four CTAs per SM, as many as are resident
  const int64_t by_len = (static_cast<int64_t>(max_blocks_per_seq) * block_size + 255) / 256;   // 256 tokens per CTA at least
  if (splits > by_len) splits = by_len;
  if (splits > 64) splits = 64;   // (128 ranges of one 65536-token sequence measured 25 % slower than 64)
  if (splits < 1) splits = 1;
  return static_cast<int>(splits);
}

size_t paged_attn_workspace_bytes(int splits, int batch, int num_heads, int head_dim) {
  return splits <= 1 ? 0 : static_cast<size_t>(batch) * num_heads * splits * (head_dim + 2) * sizeof(float);
}

int launch_paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                             const int32_t* block_tables, const int32_t* seq_lens, int32_t dt, int batch,
                             int num_heads, int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                             float scale, int splits, float* workspace, cudaStream_t stream) {
  AttnParams p;
  p.out = out;
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.block_tables = block_tables;
  p.seq_lens = seq_lens;
  p.partial = workspace;
  p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads;
  p.block_size = block_size;
  p.block_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == block_size) p.block_shift = sh;
  p.max_blocks_per_seq = max_blocks_per_seq;
  p.splits = splits;
  p.scale_log2e = scale * 1.4426950408889634f;
  switch (dt) {
    case 0: return launch_attn_t<float>(p, batch, head_dim, stream);
    case 1: return launch_attn_t<__half>(p, batch, head_dim, stream);
    case 2: return launch_attn_t<__nv_bfloat16>(p, batch, head_dim, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

}  // namespace ib200
