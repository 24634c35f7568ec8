// Small-M ("decode") variant of the blockwise-FP8 W8A8 GEMM for sm_100a.
//
// Same arithmetic contract as gemm_sm100.cu (reference kernels/gemm/w8a8_block_fp8.cu:100-114,
// reference/reference.cpp:93-110), different mapping.  With a handful of tokens the work is a
// pure stream of the weight matrix from HBM, so:
//   * operands are swapped: a 128-row weight tile is the M side of tcgen05.mma (UMMA M=128)
//     and the tokens, padded to MP in {16, 32, 64, 128}, are its N side.  The accumulator of one
//     K block is a [128 weight rows] x [MP tokens] slice of tensor memory; 512 / MP (at most 8)
//     slices are in flight, so the MMA -> promotion -> MMA round trip never limits the stream.
//   * work is dealt in whole pieces: with at least as many weight tiles as CTAs every CTA takes
//     a contiguous run of whole tiles; with fewer, every tile's K range is cut into `splits`
//     equal parts, one CTA each (split-K).  A CTA of a split tile writes an fp32 partial to a
//     workspace; the last CTA to finish the tile adds the parts in a fixed order
//     (deterministic) and writes the output.  HBM, not the SM count, bounds this kernel, so
//     leaving a few SMs idle costs nothing, while ragged pieces would cost a second partial
//     flush per CTA.
//
// CTA layout (256 threads, one CTA per SM):
//   warp 0  allocates / frees tensor memory; one thread is the TMA producer: weight tile
//           [128 x 128 B] + token tile [MP x 128 B] per K block into a deep ring
//   warps 1, 3  MMA issuers (warp-uniform loops, one elected lane each, alternating units):
//           4 x tcgen05.mma (M=128, N=MP, K=32) per unit
//   warp 2  scale warp: writes sa[m, kb] * sb[tile, kb] for the MP tokens of each unit to a
//           small shared ring, one vector per TMEM slice
//   warps 4-7  promotion + epilogue: thread = one weight row (= output column), MP accumulators
//
// HBM traffic (algorithmic): N*K weight bytes + M*K token bytes + scales + 2*M*N output bytes;
// split tiles add 2 x 4*128*MP bytes of workspace traffic per extra segment.
//
// Every wait is bounded (ptx.cuh: mbar_wait); see gemm_sm100.cu for the wind-down rules.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <type_traits>

#include "internal.h"
#include "quant_math.cuh"

namespace ib200 {
namespace {

constexpr int TN = 128;   // weight rows per tile (UMMA M)
constexpr int BK = 128;
constexpr int kThreads = 256;
constexpr int kFusedThreads = 384;   // fused prologue: four more warps that quantise the token tile
constexpr int kBytesW = TN * BK;
constexpr int kMaxStages = 12;       // barrier slots of the ring
constexpr int kFusedMaxSmem = 227 * 1024;   // fused prologue: dynamic shared memory the launcher may ask for
constexpr int kMaxSlots = 16;        // fused prologue: barrier slots of the token-tile ring

template <int MP>
struct DCfg {
  static constexpr int kBytesA = MP * BK;
  static constexpr int kStageBytes = kBytesW + kBytesA;
  // (twelve stages of 18 KiB fit too and measured 3 % slower than ten)
  static constexpr int kStages = (200 * 1024 / kStageBytes) < 10 ? (200 * 1024 / kStageBytes) : 10;
  static_assert(kStages % 2 == 0, "the two MMA issuer warps alternate units: a stage must always belong to the same warp");
  static_assert(kStages % 2 == 0, "the two MMA issuer warps alternate units: a stage must always belong to the same warp");
  static constexpr int kBufs = (512 / MP) < 8 ? (512 / MP) : 8;
  static constexpr int kTmemCols = (kBufs * MP) < 32 ? 32 : (kBufs * MP);
  static constexpr int kScaleBytes = kBufs * MP * 4;
  static constexpr int kBarrierBytes = 512;
  static constexpr int kSmemBytes = kStages * kStageBytes + kScaleBytes + kBarrierBytes + 1024;
};

struct DecodeParams {
  const float* a_scales;   // [M, KB]
  const void* a_src;       // fused prologue only: unquantised activations [M, K] (bf16 / fp16)
  const float* b_scales;   // [ceil(N/128), KB]
  // Output: the [M, N] result goes to columns [col0, col0 + N) of n_dst row-major buffers with
  // row pitch ldc elements.  A plain call has one destination (c, ldc = N, col0 = 0); the
  // all-gather form lists every rank's buffer (peer-mapped addresses, plain stores).
  void* dst[8];
  int n_dst, ldc, col0;
  float* workspace;        // [gridDim.x][2][MP][128] fp32 partials (slot 0: the CTA's first tile, slot 1: its last)
  int splits;              // 0: units dealt evenly (below); else K parts per tile (1 = runs of whole tiles)
  int stages, a_slots;     // fused prologue: depth of the weight ring and of the token-tile ring
  int* counters;           // [n_tiles], zero between launches
  int m, n, kb, n_tiles;
  long long units;         // n_tiles * kb
  int no_loads;            // test hook: the producer issues no load
  int trigger;    // let kernels queued behind this one with programmatic stream serialisation start early
  DeviceStatus* status;
};

enum : uint32_t {
  kSiteDProducerEmpty = 0x111,
  kSiteDMmaFull = 0x211,
  kSiteDMmaTmemEmpty = 0x212,
  kSiteDScaleEmpty = 0x411,
  kSiteDPromoFull = 0x311,
  kSiteDPromoScale = 0x312,
  kSiteDQuantEmpty = 0x511,
  kSiteDQuantTmem = 0x512,
};

template <typename OutT>
__device__ __forceinline__ OutT cvt_out(float v);

template <>
__device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Column gn of the result (MP values, one per token, in registers) to every destination.  The
// destination loop is the outer one so that the token loop stays fully unrolled over registers;
// with the usual single destination it runs once.
template <int MP, typename OutT>
__device__ __forceinline__ void store_column(const DecodeParams& p, int gn, const float (&v)[MP]) {
  for (int d = 0; d < p.n_dst; ++d) {
    OutT* col = static_cast<OutT*>(p.dst[d]) + p.col0 + gn;
#pragma unroll
    for (int m = 0; m < MP; ++m)
      if (m < p.m) col[static_cast<int64_t>(m) * p.ldc] = cvt_out<OutT>(v[m]);
  }
}

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]);
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_32x16(taddr, r); }
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_32x32(taddr, r); }

template <int N>
__device__ __forceinline__ void tmem_wait_pin(uint32_t (&r)[N]) {
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+r"(r[i])::"memory");
}

// 8 consecutive 16-bit activations -> 8 floats
template <typename AT>
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
template <>
__device__ __forceinline__ void unpack8<void>(const uint4&, float (&)[8]) {}

// AT = void: the token tile arrives quantised through TMA and a scale warp prepares the scale
// vectors.  AT = bf16 / fp16 (the fused prologue): warps 8-11 quantise the token tile of every
// unit themselves, straight from the unquantised activations, into a ring of their own in
// shared memory (swizzled [MP x 128 B] tiles, the layout a TMA load would have produced, plus
// the group scales), running ahead of the weight stream by up to the ring's depth; the producer
// streams weights only.  The stand-alone quantisation kernel, its launch and its q / scales
// round trip through HBM disappear.
template <int MP, typename OutT, typename AT>
__global__ void __launch_bounds__(std::is_same<AT, void>::value ? kThreads : kFusedThreads, 1)
w8a8_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   const DecodeParams p) {
  using C = DCfg<MP>;
  constexpr bool kFused = !std::is_same<AT, void>::value;
  constexpr int kQuantWarps = 4;
  constexpr int CH = (MP < 32) ? MP : 32;   // columns per tensor-memory load
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  // ring stages: weight tile + token tile; fused: weight tile only, depth chosen by the launcher
  const uint32_t nst = kFused ? static_cast<uint32_t>(p.stages) : static_cast<uint32_t>(C::kStages);
  constexpr uint32_t kStride = kFused ? kBytesW : C::kStageBytes;
  const uint32_t a_slots = kFused ? static_cast<uint32_t>(p.a_slots) : 0u;  // fused: ring of quantised token tiles (a power of two)
  const uint32_t a_mask = a_slots - 1u, a_shift = 31u - static_cast<uint32_t>(__clz(static_cast<int>(a_slots | 1u)));
  uint8_t* a_res = smem + nst * kStride;                                    // [a_slots][MP x 128 B], swizzled
  float* sa_res = reinterpret_cast<float*>(a_res + a_slots * (MP * BK));     // [a_slots][MP] group scales
  float* sv = sa_res + a_slots * MP;                                         // [kBufs][MP]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sv) + C::kScaleBytes);
  uint64_t* full = bars;                         // [kMaxStages] TMA -> MMA
  uint64_t* empty = full + kMaxStages;           // [kMaxStages] MMA -> TMA
  uint64_t* tmem_full = empty + kMaxStages;      // [kBufs]   MMA -> promotion
  uint64_t* tmem_empty = tmem_full + C::kBufs;   // [kBufs]   promotion -> MMA, scale warp
  uint64_t* sv_full = tmem_empty + C::kBufs;     // [kBufs]   scale warp -> promotion
  uint64_t* a_full = sv_full + C::kBufs;         // [a_slots] fused: quantising warps -> MMA, scale warp
  uint64_t* a_empty = a_full + (kFused ? kMaxSlots : 0);   // [a_slots] fused: MMA + scale warp -> quantising warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(a_empty + (kFused ? kMaxSlots : 0));
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* last_flag = tmem_slot + 2;

  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (uint32_t s = 0; s < nst; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (uint32_t j = 0; j < a_slots; ++j) {
      mbar_init(&a_full[j], 1);
      mbar_init(&a_empty[j], 2);   // the unit's MMAs have read the tile, the scale warp its scales
    }
    for (int b = 0; b < C::kBufs; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);
      mbar_init(&sv_full[b], 1);
    }
    *abort_flag = 0u;
    mbar_init_fence();
    tma_prefetch_desc(&map_w);
    if (!kFused) tma_prefetch_desc(&map_a);
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_slot, 0);
  // A kernel queued behind this one with programmatic stream serialisation (the quantiser of the
  // next step, and behind it the next GEMM) may be launched from now on: it takes SMs as this
  // grid's CTAs leave them and waits for this grid's completion before it touches memory.
  if (p.trigger) pdl_launch_dependents();

  // This CTA's piece: tiles [t_first, ...) from K block kb_first, `count` units in all.  A unit
  // is one (weight tile, K block) pair = 16 KiB of weights.  Default: the n_tiles * kb units are
  // dealt evenly, CTA c takes units [c U / G, (c + 1) U / G), so every SM streams the same number
  // of bytes whatever the tile count; a piece may start and end inside a tile, and the K parts of
  // a tile are then added in CTA order by the last CTA to finish (deterministic).
  int t_first, kb_first;
  uint32_t count;
  if (p.splits == 0) {
    const long long g = gridDim.x, c = blockIdx.x;
    const long long u0 = c * p.units / g, u1 = (c + 1) * p.units / g;
    t_first = static_cast<int>(u0 / p.kb);
    kb_first = static_cast<int>(u0 - static_cast<long long>(t_first) * p.kb);
    count = static_cast<uint32_t>(u1 - u0);
  } else if (p.splits == 1) {
    const long long g = gridDim.x, c = blockIdx.x;
    t_first = static_cast<int>(c * p.n_tiles / g);
    kb_first = 0;
    count = static_cast<uint32_t>(((c + 1) * p.n_tiles / g - t_first) * p.kb);
  } else {
    const int part = blockIdx.x % p.splits;
    t_first = blockIdx.x / p.splits;
    kb_first = part * p.kb / p.splits;
    count = static_cast<uint32_t>((part + 1) * p.kb / p.splits - kb_first);
  }

  if (warp == 0) {
    // ------------------------------ TMA producer (warp-uniform loop) ------
    // The weights never depend on the kernel queued before this one, the token tile may (it
    // is usually the output of the quantisation kernel).  So the first ring-full of weight
    // tiles is requested at once, then the producer waits for the preceding kernel
    // (programmatic dependent launch; a no-op otherwise) and only then asks for token tiles.
    int t = t_first, kb = kb_first;
    uint32_t armed = 0;
    bool ok = true;
    const uint32_t head = count < nst ? count : nst;
    if (p.no_loads) {
      // test hook: nothing is ever loaded, so every other role's wait runs out
    } else if (!kFused) {
      int th = t, kh = kb;
      for (uint32_t i = 0; i < head; ++i) {
        uint8_t* dst = smem + i * C::kStageBytes;
        if (elect_one()) {
          mbar_arrive_expect_tx(&full[i], C::kStageBytes);
          tma_load_2d(dst, &map_w, &full[i], kh * BK, th * TN);
        }
        __syncwarp();
        if (++kh == p.kb) {
          kh = 0;
          ++th;
        }
      }
      armed = head;
      pdl_wait();
      for (uint32_t i = 0; i < head; ++i) {
        uint8_t* dst = smem + i * C::kStageBytes;
        if (elect_one()) tma_load_2d(dst + kBytesW, &map_a, &full[i], kb * BK, 0);
        __syncwarp();
        if (++kb == p.kb) {
          kb = 0;
          ++t;
        }
      }
    }
    // (fused: this warp touches weights only, which never depend on the kernel queued before)
    for (uint32_t i = (kFused ? 0u : head); i < count && !p.no_loads; ++i) {
      const uint32_t stage = i % nst;
      const uint32_t phase = (i / nst) & 1u;
      if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, kSiteDProducerEmpty)) {
        ok = false;
        break;
      }
      __syncwarp();
      uint8_t* dst = smem + stage * kStride;
      if (elect_one()) {
        mbar_arrive_expect_tx(&full[stage], kStride);
        tma_load_2d(dst, &map_w, &full[stage], kb * BK, t * TN);
        if (!kFused) tma_load_2d(dst + kBytesW, &map_a, &full[stage], kb * BK, 0);
      }
      __syncwarp();
      armed = i + 1;
      if (++kb == p.kb) {
        kb = 0;
        ++t;
      }
    }
    if (!ok && lane == 0) {
      // wind-down: let the copies this warp started land before the CTA exits
      const uint32_t lo = armed > nst ? armed - nst : 0u;
      for (uint32_t i = lo; i < armed; ++i) {
        const long long t0 = clock64();
        while (!mbar_test_wait(&full[i % nst], (i / nst) & 1u)) {
          if (clock64() - t0 > kWaitBudgetCycles) break;
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------ MMA issuers (warp-uniform) ------------
    // warp 1 issues the even units of the range, warp 3 the odd ones: waiting, building
    // descriptors, 4 MMAs and 2 commits cost one thread about 650 cycles per unit, more than
    // the time the unit's 18 KiB take to arrive from HBM
    constexpr uint32_t idesc = umma_idesc_e4m3_f32(TN, MP);
    const uint32_t smem_base = smem_u32(smem);
    for (uint32_t i = (warp == 3) ? 1u : 0u; i < count; i += 2) {
      const uint32_t stage = i % nst;
      const uint32_t phase = (i / nst) & 1u;
      const uint32_t buf = i % C::kBufs;
      const uint32_t use = i / C::kBufs;
      const uint32_t slot = kFused ? (i & a_mask) : 0u;   // fused: the unit's slot in the token-tile ring
      if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kSiteDMmaFull)) break;
      if (kFused && !mbar_wait(&a_full[slot], (i >> a_shift) & 1u, abort_flag, p.status, kSiteDQuantEmpty)) break;
      if (!mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, p.status, kSiteDMmaTmemEmpty)) break;
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t w_addr = smem_base + stage * kStride;
      const uint64_t dw = umma_desc_k_sw128(w_addr);
      const uint64_t da = umma_desc_k_sw128(kFused ? smem_u32(a_res) + slot * (MP * BK) : w_addr + kBytesW);
      const uint32_t d_tmem = tmem_base + buf * MP;
      if (elect_one()) {
#pragma unroll
        for (int k4 = 0; k4 < BK / 32; ++k4) {
          umma_f8_ss(d_tmem, dw + 2u * k4, da + 2u * k4, idesc, k4 > 0 ? 1u : 0u);
        }
        umma_commit(&tmem_full[buf]);
        umma_commit(&empty[stage]);
        if (kFused) umma_commit(&a_empty[slot]);
      }
      __syncwarp();
    }
  } else if (kFused && warp >= 8) {
    // ------------------------------ quantising prologue (fused) -----------
    // Warp w takes the units w, w + 4, ...: all token rows of the unit's K block, two per step (a
    // half warp owns one row's 128-wide group: 16 lanes x 8 elements), the next unit's
    // activations in flight while the current one is quantised.  Rows beyond M are zero: they are
    // written once, before the loop, and never touched again.
    if constexpr (kFused) {
      constexpr int STEPS = MP / 2;
      const int qw = warp - 8, hw = lane >> 4, sub = lane & 15;
      const AT* src = static_cast<const AT*>(p.a_src);
      const int64_t ld = static_cast<int64_t>(p.kb) * BK;
      const int live_steps = (p.m + 1) >> 1;   // steps that hold at least one real row
      for (uint32_t j = qw; j < a_slots; j += kQuantWarps) {
#pragma unroll
        for (int s2 = 0; s2 < STEPS; ++s2) {
          const int r = 2 * s2 + hw;
          if (r >= p.m) {
            *reinterpret_cast<uint2*>(a_res + j * (MP * BK) + r * 128 + (((sub >> 1) ^ (r & 7)) << 4) + ((sub & 1) << 3)) =
                make_uint2(0u, 0u);
            if (sub == 0) sa_res[j * MP + r] = 0.0f;
          }
        }
      }
      uint4 cur[STEPS], nxt[STEPS];
      pdl_wait();   // the activations may come from the kernel queued before this one
      auto fetch = [&](uint4 (&dst)[STEPS], uint32_t unit) {
        const int kbx = static_cast<int>((static_cast<uint32_t>(kb_first) + unit) % static_cast<uint32_t>(p.kb));
#pragma unroll
        for (int s2 = 0; s2 < STEPS; ++s2) {
          const int r = 2 * s2 + hw;
          if (s2 < live_steps) {
            dst[s2] = (r < p.m && unit < count)
                          ? __ldg(reinterpret_cast<const uint4*>(src + r * ld + kbx * BK + sub * 8))
                          : make_uint4(0u, 0u, 0u, 0u);
          }
        }
      };
      fetch(cur, qw);
      for (uint32_t i = qw; i < count; i += kQuantWarps) {
        fetch(nxt, i + kQuantWarps);
        const uint32_t slot = (i & a_mask);
        if (!mbar_wait(&a_empty[slot], ((i >> a_shift) & 1u) ^ 1u, abort_flag, p.status, kSiteDQuantEmpty)) break;
        __syncwarp();
        uint8_t* tile = a_res + slot * (MP * BK);
#pragma unroll
        for (int s2 = 0; s2 < STEPS; ++s2) {
          if (s2 < live_steps) {
            const int r = 2 * s2 + hw;
            float f[8];
            unpack8<AT>(cur[s2], f);
            float amax = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
            const float scale = group_scale(amax);
            const uint2 bytes = fast_div_ok(amax) ? quantise8_fast16(cur[s2], f, scale, __frcp_rn(scale))
                                                  : quantise8<false>(f, scale, 0.0f);
            if (r < p.m) {
              // swizzled K-major layout of a TMA SWIZZLE_128B load: 16-byte chunk c of row r sits at
              // chunk c ^ (r & 7); this lane's 8 bytes are half of chunk sub / 2
              *reinterpret_cast<uint2*>(tile + r * 128 + (((sub >> 1) ^ (r & 7)) << 4) + ((sub & 1) << 3)) = bytes;
              if (sub == 0) sa_res[slot * MP + r] = scale;
            }
          }
        }
        fence_proxy_async_smem();   // the tensor core reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[slot]);
#pragma unroll
        for (int s2 = 0; s2 < STEPS; ++s2) cur[s2] = nxt[s2];
      }
    }
  } else if (warp == 2) {
    // ------------------------------ scale warp ----------------------------
    if (!kFused) pdl_wait();   // a_scales may come from the kernel queued before this one
    int t = t_first, kb = kb_first;
    for (uint32_t i = 0; i < count; ++i) {
      const uint32_t buf = i % C::kBufs;
      const uint32_t use = i / C::kBufs;
      if (!mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, p.status, kSiteDScaleEmpty)) break;
      const float sb = __ldg(p.b_scales + static_cast<int64_t>(t) * p.kb + kb);
      // fused: the group scales of this unit are in shared memory once its tile is published
      const uint32_t slot = kFused ? (i & a_mask) : 0u;
      if (kFused && !mbar_wait(&a_full[slot], (i >> a_shift) & 1u, abort_flag, p.status, kSiteDQuantTmem)) break;
#pragma unroll
      for (int m0 = 0; m0 < MP; m0 += 32) {
        const int m = m0 + lane;
        if (m < MP) {
          float sa;
          if (kFused) sa = sa_res[slot * MP + m];
          else sa = (m < p.m) ? __ldg(p.a_scales + static_cast<int64_t>(m) * p.kb + kb) : 0.0f;
          sv[buf * MP + m] = sa * sb;
        }
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&sv_full[buf]);
        if (kFused) mbar_arrive(&a_empty[slot]);
      }
      if (++kb == p.kb) {
        kb = 0;
        ++t;
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------ promotion + epilogue ------------------
    const int quarter = warp - 4;            // == warp % 4: TMEM lane quarter
    const int row = quarter * 32 + lane;     // weight row inside the tile
    const int ct = threadIdx.x - 128;        // 0..127 among the promotion threads
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    float acc[MP];
#pragma unroll
    for (int j = 0; j < MP; ++j) acc[j] = 0.0f;
    pdl_wait();   // the output, workspace and counters may still be in use by the preceding kernel
    int t = t_first, kb = kb_first, seg_kb0 = kb_first;
    bool ok = true;
    for (uint32_t i = 0; i < count; ++i) {
      const uint32_t buf = i % C::kBufs;
      const uint32_t par = (i / C::kBufs) & 1u;
      // a warp whose wait ran out skips the work of the remaining units of its segment (without
      // waiting) and meets its siblings at the segment's end, where the four warps agree to leave
      if (ok && (!mbar_wait(&tmem_full[buf], par, abort_flag, p.status, kSiteDPromoFull) ||
                 !mbar_wait(&sv_full[buf], par, abort_flag, p.status, kSiteDPromoScale))) {
        ok = false;
      }
      if (ok) {
        __syncwarp();
        tc_fence_after_sync();
        const float4* svb = reinterpret_cast<const float4*>(sv + buf * MP);
        // all loads of up to 64 columns are issued before the single wait, so that their
        // latencies overlap; 128 columns go in two such halves (register budget)
        constexpr int HALF = (MP < 64) ? MP : 64;
#pragma unroll
        for (int h0 = 0; h0 < MP; h0 += HALF) {
          uint32_t v[HALF / CH][CH];
#pragma unroll
          for (int q = 0; q < HALF / CH; ++q) tmem_ld_cols<CH>(lane_base + buf * MP + h0 + q * CH, v[q]);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < HALF / CH; ++q) {
#pragma unroll
            for (int j = 0; j < CH; ++j) asm volatile("" : "+r"(v[q][j])::"memory");
          }
#pragma unroll
          for (int q = 0; q < HALF / CH; ++q) {
#pragma unroll
            for (int j = 0; j < CH; j += 4) {
              const int c = h0 + q * CH + j;
              const float4 s4 = svb[c >> 2];
              acc[c + 0] = fmaf(__uint_as_float(v[q][j + 0]), s4.x, acc[c + 0]);
              acc[c + 1] = fmaf(__uint_as_float(v[q][j + 1]), s4.y, acc[c + 1]);
              acc[c + 2] = fmaf(__uint_as_float(v[q][j + 2]), s4.z, acc[c + 2]);
              acc[c + 3] = fmaf(__uint_as_float(v[q][j + 3]), s4.w, acc[c + 3]);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);
      }

      const bool seg_end = (kb == p.kb - 1) || (i + 1 == count);
      if (seg_end) {
        if (named_bar_or(2, 128, !ok)) break;   // agreed: the piece is abandoned, nobody waits at the barriers below
        const int gn = t * TN + row;
        const bool whole = (seg_kb0 == 0 && kb == p.kb - 1);
        if (whole) {
          if (gn < p.n) store_column<MP, OutT>(p, gn, acc);
        } else {
          // one K part of a split tile: a slot of this CTA in the workspace (slot 0 for the tile
          // the piece starts in, slot 1 for the tile it ends in)
          const int64_t my_slot = p.splits == 0 ? static_cast<int64_t>(blockIdx.x) * 2 + (t == t_first ? 0 : 1)
                                                : static_cast<int64_t>(blockIdx.x);
          float* wp = p.workspace + my_slot * (MP * TN);
#pragma unroll
          for (int m = 0; m < MP; ++m) __stcg(wp + m * TN + row, acc[m]);
          __threadfence();
          // which CTAs hold parts of tile t: with even dealing, the CTA that owns unit u is
          // ceil((u + 1) G / U) - 1
          int c_lo = 0, c_hi = 0;
          if (p.splits == 0) {
            const long long g = gridDim.x;
            c_lo = static_cast<int>(((static_cast<long long>(t) * p.kb + 1) * g + p.units - 1) / p.units) - 1;
            c_hi = static_cast<int>(((static_cast<long long>(t + 1) * p.kb) * g + p.units - 1) / p.units) - 1;
          }
          const int parts = p.splits == 0 ? c_hi - c_lo + 1 : p.splits;
          named_bar_sync(1, 128);
          if (ct == 0) {
            const int prev = atomicAdd(p.counters + t, 1);
            *last_flag = (prev == parts - 1) ? 1u : 0u;
          }
          named_bar_sync(1, 128);
          if (*last_flag != 0u) {
            __threadfence();
            float sum[MP];
#pragma unroll
            for (int m = 0; m < MP; ++m) sum[m] = 0.0f;
            for (int part = 0; part < parts; ++part) {   // fixed order: the result does not depend on arrival order
              int64_t slot;
              if (p.splits == 0) {
                const long long c2 = c_lo + part;
                const int tf = static_cast<int>((c2 * p.units / gridDim.x) / p.kb);   // the tile CTA c2 starts in
                slot = c2 * 2 + (tf == t ? 0 : 1);
              } else {
                slot = static_cast<int64_t>(t) * p.splits + part;
              }
              const float* rp = p.workspace + slot * (MP * TN);
#pragma unroll
              for (int m = 0; m < MP; ++m) sum[m] += __ldcg(rp + m * TN + row);
            }
            if (gn < p.n) store_column<MP, OutT>(p, gn, sum);
            if (ct == 0) p.counters[t] = 0;   // ready for the next launch
          }
          named_bar_sync(1, 128);   // last_flag may be rewritten only after everyone has read it
        }
#pragma unroll
        for (int j = 0; j < MP; ++j) acc[j] = 0.0f;
        seg_kb0 = 0;
      }
      if (++kb == p.kb) {
        kb = 0;
        ++t;
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

template <int MP, typename OutT, typename AT = void>
int launch_decode_t(const CUtensorMap& mw, const CUtensorMap& ma, const DecodeParams& p, int ctas,
                    cudaStream_t stream, int smem_bytes = 0) {
  using C = DCfg<MP>;
  constexpr bool kFused = !std::is_same<AT, void>::value;
  if (!kFused) smem_bytes = C::kSmemBytes;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_decode_kernel<MP, OutT, AT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kFused ? kFusedMaxSmem : C::kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  // programmatic dependent launch: the preamble and the weight prefetch of this kernel may
  // overlap the tail of the kernel queued before it (in practice the quantisation kernel)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(std::is_same<AT, void>::value ? kThreads : kFusedThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().decode_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, w8a8_decode_kernel<MP, OutT, AT>, mw, ma, p);
  if (e != cudaSuccess) return note_cuda_error(e);
  return check_launch();
}

template <typename OutT, typename AT>
int launch_decode_fused_mp(int mp, const CUtensorMap& mw, const DecodeParams& p, int ctas,
                           cudaStream_t stream, int smem_bytes) {
  return mp == 16 ? launch_decode_t<16, OutT, AT>(mw, mw, p, ctas, stream, smem_bytes)
                  : launch_decode_t<32, OutT, AT>(mw, mw, p, ctas, stream, smem_bytes);
}
template <typename AT>
int launch_decode_fused_out(int out_dt, int mp, const CUtensorMap& mw, const DecodeParams& p, int ctas,
                            cudaStream_t stream, int smem_bytes) {
  switch (out_dt) {
    case 0: return launch_decode_fused_mp<float, AT>(mp, mw, p, ctas, stream, smem_bytes);
    case 1: return launch_decode_fused_mp<__half, AT>(mp, mw, p, ctas, stream, smem_bytes);
    case 2: return launch_decode_fused_mp<__nv_bfloat16, AT>(mp, mw, p, ctas, stream, smem_bytes);
    default: return INFEROP_ERR_DTYPE;
  }
}

template <typename OutT>
int launch_decode_mp(int mp, const CUtensorMap& mw, const CUtensorMap& ma, const DecodeParams& p,
                     int ctas, cudaStream_t stream) {
  switch (mp) {
    case 16: return launch_decode_t<16, OutT>(mw, ma, p, ctas, stream);
    case 32: return launch_decode_t<32, OutT>(mw, ma, p, ctas, stream);
    case 64: return launch_decode_t<64, OutT>(mw, ma, p, ctas, stream);
    default: return launch_decode_t<128, OutT>(mw, ma, p, ctas, stream);
  }
}

}  // namespace

size_t decode_workspace_bytes(int ctas) { return static_cast<size_t>(ctas) * 2 * kDecodeMaxM * TN * 4; }

int launch_gemm_decode_fused(DeviceCtx* ctx, float* workspace, int* counters, void* c, const void* a,
                             int32_t a_dt, const void* b_q, const void* b_scales, int64_t m, int64_t n,
                             int64_t k, int32_t out_dt, cudaStream_t stream) {
  const int mp = m <= 16 ? 16 : 32;
  DecodeParams p;
  p.a_scales = nullptr;
  p.a_src = a;
  p.b_scales = static_cast<const float*>(b_scales);
  p.dst[0] = c;
  p.n_dst = 1;
  p.ldc = static_cast<int>(n);
  p.col0 = 0;
  p.workspace = workspace;
  p.counters = counters;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.kb = static_cast<int>(k / 128);
  p.n_tiles = static_cast<int>((n + TN - 1) / TN);
  p.units = static_cast<long long>(p.n_tiles) * p.kb;
  p.no_loads = options().debug_no_loads;
  p.trigger = options().pdl_trigger;
  p.status = ctx->status;
  CUtensorMap mw;
  const int rc = make_tensor_map_2d(&mw, b_q, 1, n, k, k, TN, BK, true);
  if (rc != INFEROP_OK) return rc;
  const Options& opt = options();
  int max_ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (max_ctas > ctx->sm_count) max_ctas = ctx->sm_count;
  int ctas;
  if (p.n_tiles >= max_ctas) {
    p.splits = 1;
    ctas = max_ctas;
  } else {
    p.splits = max_ctas / p.n_tiles;
    if (p.splits > p.kb) p.splits = p.kb;
    if (opt.decode_splits > 0 && opt.decode_splits <= p.splits) p.splits = opt.decode_splits;
    ctas = p.n_tiles * p.splits;
  }
  // token-tile ring of 32 KiB beside a full-depth weight ring
  p.a_slots = 32 * 1024 / (mp * BK);
  if (p.a_slots > kMaxSlots) p.a_slots = kMaxSlots;
  const int bufs = (512 / mp) < 8 ? (512 / mp) : 8;
  const int fixed = p.a_slots * mp * (BK + 4) + bufs * mp * 4 + 1024 /* barriers */ + 1024 /* alignment slack */;
  p.stages = 10;
  const int smem_bytes = p.stages * kBytesW + fixed;
  if (a_dt == 2) return launch_decode_fused_out<__nv_bfloat16>(out_dt, mp, mw, p, ctas, stream, smem_bytes);
  if (a_dt == 1) return launch_decode_fused_out<__half>(out_dt, mp, mw, p, ctas, stream, smem_bytes);
  return INFEROP_ERR_DTYPE;
}

int launch_gemm_decode(DeviceCtx* ctx, float* workspace, int* counters, void* c, const void* a_q,
                       const void* a_scales, const void* b_q, const void* b_scales, int64_t m,
                       int64_t n, int64_t k, int32_t out_dt, cudaStream_t stream, int clear_counters) {
  void* const dst[1] = {c};
  return launch_gemm_decode_to(ctx, workspace, counters, dst, 1, n, 0, a_q, a_scales, b_q, b_scales, m, n,
                               k, out_dt, stream, clear_counters);
}

int launch_gemm_decode_to(DeviceCtx* ctx, float* workspace, int* counters, void* const* dst, int n_dst,
                          int64_t ldc, int64_t col0, const void* a_q, const void* a_scales,
                          const void* b_q, const void* b_scales, int64_t m, int64_t n, int64_t k,
                          int32_t out_dt, cudaStream_t stream, int clear_counters) {
  const int mp = m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128;
  DecodeParams p;
  p.a_src = nullptr;
  p.stages = 0;
  p.a_slots = 0;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  if (n_dst < 1 || n_dst > 8) return INFEROP_ERR_SHAPE;
  for (int d = 0; d < 8; ++d) p.dst[d] = dst[d < n_dst ? d : 0];
  p.n_dst = n_dst;
  p.ldc = static_cast<int>(ldc);
  p.col0 = static_cast<int>(col0);
  p.workspace = workspace;
  p.counters = counters;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.kb = static_cast<int>(k / 128);
  p.n_tiles = static_cast<int>((n + TN - 1) / TN);
  p.units = static_cast<long long>(p.n_tiles) * p.kb;
  p.no_loads = options().debug_no_loads;
  p.trigger = options().pdl_trigger;
  p.status = ctx->status;

  CUtensorMap mw, ma;
  int rc = make_tensor_map_2d(&mw, b_q, 1, n, k, k, TN, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&ma, a_q, 1, m, k, k, mp, BK, true);
  if (rc != INFEROP_OK) return rc;
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  if (clear_counters > 0) {
    // everything that can reject the call has been checked: nothing is left on the stream by a rejected call
    const cudaError_t e = cudaMemsetAsync(counters, 0, static_cast<size_t>(clear_counters) * sizeof(int), stream);
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  const Options& opt = options();
  int max_ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (max_ctas > ctx->sm_count) max_ctas = ctx->sm_count;   // the workspace is sized for one CTA per SM
  int ctas;
  if (opt.decode_deal == 0) {
    // every (tile, K block) unit dealt evenly over one CTA per SM
    p.splits = 0;
    ctas = p.units < max_ctas ? static_cast<int>(p.units) : max_ctas;
  } else if (p.n_tiles >= max_ctas) {
    p.splits = 1;
    ctas = max_ctas;
  } else {
    p.splits = max_ctas / p.n_tiles;
    if (p.splits > p.kb) p.splits = p.kb;
    if (opt.decode_splits > 0 && opt.decode_splits <= p.splits) p.splits = opt.decode_splits;
    ctas = p.n_tiles * p.splits;
  }
  switch (out_dt) {
    case 0: return launch_decode_mp<float>(mp, mw, ma, p, ctas, stream);
    case 1: return launch_decode_mp<__half>(mp, mw, ma, p, ctas, stream);
    case 2: return launch_decode_mp<__nv_bfloat16>(mp, mw, ma, p, ctas, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

}  // namespace ib200

// ---------------------------------------------------------------------------
// Entry point that allocates nothing.
//
// Some callers cannot let a library call cudaMalloc on their behalf: a serving process that
// handed all of the device's memory to its own pool at start-up (weights, KV cache) has none
// left for the driver to give out, and a latency-critical loop cannot afford an allocation
// call that may take driver locks or synchronise the device.  For them the split-tile scratch
// of the small-M kernel lives in a fixed array inside the library image instead of in memory
// obtained at run time.  Every GPU that loads the library carries the array (about 5.3 MB)
// until the process exits, which is why it is kept small: M <= 32 tokens, at most 4096 weight
// tiles (N <= 524288) and at most 160 SMs.
// ---------------------------------------------------------------------------
namespace ib200 {
namespace {

constexpr int kFixedMaxM = 32;
constexpr int kFixedMaxCtas = 160;
constexpr int kFixedMaxTiles = 4096;

struct FixedScratch {
  float partials[kFixedMaxCtas * 2 * kFixedMaxM * TN];  // two K parts of split tiles per CTA
  int counters[kFixedMaxTiles];                     // arrivals per tile; zero between launches
  DeviceStatus status;                              // bounded-wait record of this entry point
};

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress; the
// device address obtained from it is what the kernel receives.
static __device__ __align__(256) unsigned char g_fixed_scratch[sizeof(FixedScratch)];

struct FixedScratchPtr {
  FixedScratch* ptr = nullptr;
  int sm_count = 0;
  int sm_version = 0;
};

FixedScratchPtr g_fixed_cache[64];
std::mutex g_fixed_mutex;

FixedScratch* fixed_scratch_cached(int dev) {
  std::lock_guard<std::mutex> lock(g_fixed_mutex);
  return g_fixed_cache[dev].ptr;
}

// Device address of the scratch on the current device, resolved once per device.
int fixed_scratch_for_current_device(FixedScratchPtr* out) {
  FixedScratchPtr* cache = g_fixed_cache;
  std::mutex& m = g_fixed_mutex;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return note_cuda_error(e);
  if (dev < 0 || dev >= 64) return INFEROP_ERR_LIMIT;
  std::lock_guard<std::mutex> lock(m);
  if (!cache[dev].ptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_fixed_scratch);
    if (e != cudaSuccess || !p) return note_cuda_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e);
    int major = 0, minor = 0, sms = 0;
    if ((e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) {
      return note_cuda_error(e);
    }
    cache[dev].sm_version = major * 10 + minor;
    cache[dev].sm_count = sms;
    cache[dev].ptr = static_cast<FixedScratch*>(p);
  }
  *out = cache[dev];
  return INFEROP_OK;
}

}  // namespace
}  // namespace ib200

extern "C" int inferop_w8a8_block_fp8_gemm_fixed_scratch(void* c, const void* a_q, const void* a_scales,
                                                         const void* b_q, const void* b_scales, int64_t m,
                                                         int64_t n, int64_t k, int32_t group_size,
                                                         int32_t block_n, int32_t out_dt, void* stream) {
  using namespace ib200;
  if (group_size != 128 || block_n != 128 || k < 0 || k % 128 != 0 || m <= 0 || n <= 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  if (m > kFixedMaxM || (n + TN - 1) / TN > kFixedMaxTiles || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!c) return INFEROP_ERR_POINTER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (k == 0) {  // empty sum: zeros, as the regular entry point (and the reference's kernel) stores
    const cudaError_t e = cudaMemsetAsync(c, 0, static_cast<size_t>(m) * n * (out_dt == 0 ? 4 : 2), s);
    return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
  }
  if (!a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  FixedScratchPtr fs;
  const int rc = fixed_scratch_for_current_device(&fs);
  if (rc != INFEROP_OK) return rc;
  if (fs.sm_version != 100) return INFEROP_ERR_ARCH;
  if (fs.sm_count > kFixedMaxCtas) return INFEROP_ERR_LIMIT;
  DeviceCtx local;  // carries the SM count and the status slot to the launcher; owns nothing
  local.ordinal = 0;
  local.sm_version = fs.sm_version;
  local.sm_count = fs.sm_count;
  local.status = &fs.ptr->status;
  // the array keeps whatever the last call left: the launcher zeroes the arrival counters of this
  // call's tiles on the stream, after its last check and before the kernel
  const int tiles = static_cast<int>((n + TN - 1) / TN);
  return launch_gemm_decode(&local, fs.ptr->partials, fs.ptr->counters, c, a_q, a_scales, b_q, b_scales,
                            m, n, k, out_dt, s, tiles);
}

// The bounded-wait record of the fixed-scratch entry point on the current device, for
// inferop_device_status: nothing is read (and *used = false) when that entry point has not
// run on this device yet.  Allocates nothing.
int ib200::fixed_scratch_status(DeviceStatus* out, bool reset, bool* used) {
  *used = false;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return note_cuda_error(e);
  if (dev < 0 || dev >= 64) return INFEROP_OK;
  FixedScratch* ptr = fixed_scratch_cached(dev);
  if (!ptr) return INFEROP_OK;
  e = cudaMemcpy(out, &ptr->status, kStatusRecordBytes, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return note_cuda_error(e);
  if (reset) {
    e = cudaMemset(&ptr->status, 0, kStatusRecordBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
  }
  *used = true;
  return INFEROP_OK;
}
