// Blockwise-FP8 W8A8 GEMM for sm_100a on CTA pairs: two CTAs of one cluster compute one
// 256 x 256 tile of C with tcgen05.mma.cta_group::2.
//
// Same arithmetic contract, data layout and role split as gemm_sm100.cu (reference
// kernels/gemm/w8a8_block_fp8.cu:100-114, reference/reference.cpp:93-110); what changes is who
// loads what.  With one CTA per 128 x 256 tile every SM pulls 16 KiB of A and 32 KiB of B per K
// block through L2.  Here CTA r of a pair loads rows [128 r, 128 r + 128) of the tile's A panel
// and rows [128 r, 128 r + 128) of its B panel (16 + 16 KiB); the tensor cores of both SMs read
// both B halves (the peer's through distributed shared memory), and each SM keeps the
// accumulator of its own 128 rows x 256 columns in its own tensor memory.  Two thirds of the
// operand bytes per flop, the same promotion work per SM.  Every CTA issues plain TMA loads
// of its own boxes: nothing is multicast and nothing is loaded from another GPU.
//
// Per CTA (384 threads):
//   warp 0      tensor-memory allocation for the pair; one thread is the TMA producer of this
//               CTA's halves.  The byte counts of both CTAs are credited to the LEADER's
//               (rank 0) `full` barrier of the stage.
//   warps 1, 2  leader only: MMA issuers (even / odd K blocks), 4 x (M256 N256 K32) per K block
//               into accumulator buffer kb & 1 of both CTAs; commits arrive on `tmem_full` and
//               `empty` of BOTH CTAs.
//   warps 4-11  promotion + epilogue of this CTA's 128 rows, exactly as in gemm_sm100.cu; the
//               `tmem_empty` arrivals of both CTAs go to the leader's barrier.
//
// Every wait is bounded (ptx.cuh: mbar_wait).  A role that gives up sets its CTA's abort flag;
// the promotion warps of a column half agree on abandoning a tile through a reducing barrier,
// so no warp is left alone at a named barrier.  Both CTAs meet at a cluster barrier before the
// tensor memory is freed.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "internal.h"

#define IB200_TRACE_TAG pair
#include "trace.cuh"

namespace ib200 {
namespace {

constexpr int PM = 128;                 // rows of C per CTA; the pair's tile has 2 * PM rows
constexpr int PN = 256;                 // columns of C per tile
constexpr int BK = 128;
constexpr int kPromoWarps = 8;
constexpr int kThreads = 128 + 32 * kPromoWarps;
constexpr int kBytesA = PM * BK;        // this CTA's rows of the A panel
constexpr int kBytesB = (PN / 2) * BK;  // this CTA's half of the weight rows
constexpr int kStageBytes = kBytesA + kBytesB;
constexpr int kStages = 6;
constexpr int kSlices = 2;              // accumulator buffers of PN columns in tensor memory
constexpr int kTmemCols = 512;
constexpr int CT = PN / 2;              // columns per promotion thread
constexpr int kStoreBufBytes = 128 * 128;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStoreBufBytes + kBarrierBytes + 1024;
static_assert(kSmemBytes <= 232448, "shared memory of one CTA");

struct PairParams {
  const float* a_scales;
  const float* b_scales;
  void* c;
  int m, n, kb, nb;
  int tiles_m, tiles_n, num_tiles;   // tiles of 256 x 256
  int group_m;                       // M-tiles per rasterisation band
  int tma_store;
  int no_loads;   // test hook: the producers issue no load
  DeviceStatus* status;
};

enum : uint32_t {
  kSitePProducerEmpty = 0x121,
  kSitePMmaFull = 0x221,
  kSitePMmaTmemEmpty = 0x222,
  kSitePPromoTmemFull = 0x321,
};

template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<float>(float, float) { return 0u; }

template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ void tmem_ld_wait_pin(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                 "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                 "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]),
                 "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

__device__ __forceinline__ void promote32(float2* acc, const uint32_t (&v)[32], float s) {
  const float2 s2 = make_float2(s, s);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), s2,
                        acc[j]);
  }
}

// tile t of the launch -> first row and first column (bands of group_m M-tiles, N-tiles
// outermost inside a band, so a band's A panel stays in L2 while the weights stream past once)
__device__ __forceinline__ void tile_origin(int t, const PairParams& p, int& row0, int& col0) {
  const int per_band = p.group_m * p.tiles_n;
  const int band = t / per_band;
  const int first_m = band * p.group_m;
  const int band_m = min(p.group_m, p.tiles_m - first_m);
  const int r = t - band * per_band;
  row0 = (first_m + r % band_m) * (2 * PM);
  col0 = (r / band_m) * PN;
}

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
w8a8_pair_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_c, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* store_buf = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_buf + 2 * kStoreBufBytes);
  uint64_t* full = bars;                        // [kStages]  leader's: both CTAs' TMA bytes -> MMA
  uint64_t* empty = bars + kStages;             // [kStages]  MMA -> this CTA's producer
  uint64_t* tmem_full = bars + 2 * kStages;     // [kSlices]  MMA -> this CTA's promotion warps
  uint64_t* tmem_empty = tmem_full + kSlices;   // [kSlices]  leader's: promotion warps of both CTAs -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + kSlices);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kSlices; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * kPromoWarps);
    }
    *abort_flag = 0u;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.tma_store) tma_prefetch_desc(&map_c);
  }
  if (warp == 0) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  // the peer's barriers must exist before anything of this CTA signals them
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_slot, 0);
  const uint32_t my_tiles = pair < p.num_tiles ? (p.num_tiles - pair + num_pairs - 1) / num_pairs : 0u;

  if (warp < 4) {
    reg_dealloc<56>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------
      pdl_wait();   // the A panel is usually the output of the kernel queued before this one
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; ok && !p.no_loads && t < p.num_tiles; t += num_pairs) {
        int row0, col0;
        tile_origin(t, p, row0, col0);
        const int a_row = row0 + static_cast<int>(rank) * PM;
        const int b_row = col0 + static_cast<int>(rank) * (PN / 2);
        for (int kb = 0; kb < p.kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, kSitePProducerEmpty)) {
            ok = false;
            break;
          }
          TRACE(rank, pair == 0, 0, static_cast<uint32_t>((t - pair) / num_pairs * p.kb + kb), 0);
          uint8_t* sa = smem + stage * kStageBytes;
          const uint32_t leader_full = mapa_shared(smem_u32(&full[stage]), 0u);
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2 * kStageBytes);
          tma_load_2d_pair(sa, &map_a, leader_full, kb * BK, a_row);
          tma_load_2d_pair(sa + kBytesA, &map_b, leader_full, kb * BK, b_row);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // wind-down: copies this thread started credit the leader's barriers; give them time to
        // land before this CTA's shared memory goes away (the cluster barrier below also keeps
        // the leader alive until then)
        const long long t0 = clock64();
        while (clock64() - t0 < (1LL << 22)) {
        }
      }
    } else if (rank == 0 && (warp == 1 || warp == 2)) {
      // ------------------------------ MMA issuers (leader CTA) ------------
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(2 * PM, PN);
      const uint32_t total = my_tiles * static_cast<uint32_t>(p.kb);
      const uint32_t smem_base = smem_u32(smem);
      uint32_t stage = warp - 1, phase = 0, buf = warp - 1, use = 0;
      for (uint32_t it = warp - 1; it < total; it += 2, stage += 2, buf += 2) {
        if (stage >= static_cast<uint32_t>(kStages)) {
          stage -= kStages;
          phase ^= 1u;
        }
        if (buf >= static_cast<uint32_t>(kSlices)) {
          buf -= kSlices;
          ++use;
        }
        const uint32_t d_tmem = tmem_base + buf * PN;
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kSitePMmaFull)) break;
        TRACE(rank, pair == 0 && lane == 0, 1, it, 0);
        if (!mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, p.status, kSitePMmaTmemEmpty)) break;
        TRACE(rank, pair == 0 && lane == 0, 1, it, 1);
        __syncwarp();
        tc_fence_after_sync();
        const uint32_t a_addr = smem_base + stage * kStageBytes;
        const uint64_t da = umma_desc_k_sw128(a_addr);
        const uint64_t db = umma_desc_k_sw128(a_addr + kBytesA);
        if (elect_one()) {
#pragma unroll
          for (int k4 = 0; k4 < BK / 32; ++k4) {
            umma_f8_ss_pair(d_tmem, da + 2u * k4, db + 2u * k4, idesc, k4 > 0 ? 1u : 0u);
          }
          umma_commit_pair(&tmem_full[buf], 3);
          umma_commit_pair(&empty[stage], 3);
        }
        __syncwarp();
        TRACE(rank, pair == 0 && lane == 0, 1, it, 2);
      }
    }
  } else {
    reg_alloc<224>();
    // ------------------------------ promotion + epilogue ------------------
    const int pw = warp - 4;
    const int quarter = pw & 3;  // == warp % 4: the TMEM lane quarter this warp may read
    const int half = pw >> 2;    // column half of the tile (inside one weight-scale block)
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * CT;
    uint8_t* my_buf = store_buf + half * kStoreBufBytes;
    const bool issuer = (quarter == 0 && lane == 0);
    const uint32_t leader_tmem_empty = mapa_shared(smem_u32(&tmem_empty[0]), 0u);
    uint32_t kiter = 0;
    pdl_wait();   // a_scales come from the kernel queued before this one, which may also still read C
    for (int t = pair; t < p.num_tiles; t += num_pairs) {
      int row0, col0;
      tile_origin(t, p, row0, col0);
      const int a_row = row0 + static_cast<int>(rank) * PM;
      const int gm = a_row + row;
      const int nbi = (col0 + half * CT) / 128;
      const bool have = gm < p.m && nbi < p.nb;
      const float* sa_ptr = p.a_scales + static_cast<int64_t>(have ? gm : 0) * p.kb;
      const float* sb_ptr = p.b_scales + static_cast<int64_t>(have ? nbi : 0) * p.kb;

      float2 acc[CT / 2];
#pragma unroll
      for (int j = 0; j < CT / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);

      // the scales of a K block are requested three blocks before the product that uses them, by
      // loads the compiler cannot move next to their use (see gemm_sm100.cu): a warp that waits
      // for its scale holds up the accumulator buffer for all sixteen of the pair
      float sa_q0 = 0.0f, sa_q1 = 0.0f, sa_q2 = 0.0f, sb_q0 = 0.0f, sb_q1 = 0.0f, sb_q2 = 0.0f;
      if (have) {
        sa_q0 = ld_nc_f32_pinned(sa_ptr);
        sb_q0 = ld_nc_f32_pinned(sb_ptr);
        if (p.kb > 1) {
          sa_q1 = ld_nc_f32_pinned(sa_ptr + 1);
          sb_q1 = ld_nc_f32_pinned(sb_ptr + 1);
        }
        if (p.kb > 2) {
          sa_q2 = ld_nc_f32_pinned(sa_ptr + 2);
          sb_q2 = ld_nc_f32_pinned(sb_ptr + 2);
        }
      }
      bool ok = true;
      for (int kb = 0; kb < p.kb; ++kb, ++kiter) {
        const float s = sa_q0 * sb_q0;
        sa_q0 = sa_q1;
        sb_q0 = sb_q1;
        sa_q1 = sa_q2;
        sb_q1 = sb_q2;
        if (kb + 3 < p.kb && have) {
          sa_q2 = ld_nc_f32_pinned(sa_ptr + kb + 3);
          sb_q2 = ld_nc_f32_pinned(sb_ptr + kb + 3);
        }
        const uint32_t buf = kiter % kSlices;
        if (!mbar_wait(&tmem_full[buf], (kiter / kSlices) & 1u, abort_flag, p.status, kSitePPromoTmemFull)) {
          ok = false;
          break;
        }
        TRACE(rank, pair == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 0);
        __syncwarp();
        tc_fence_after_sync();
        const uint32_t taddr = lane_base + buf * PN;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait_pin(v0);
        tmem_ld_wait_pin(v1);
        TRACE(rank, pair == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 1);
        promote32(acc, v0, s);
        tmem_ld_32x32(taddr + 64, v0);
        promote32(acc + 16, v1, s);
        tmem_ld_32x32(taddr + 96, v1);
        tmem_ld_wait_pin(v0);
        tmem_ld_wait_pin(v1);
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_tmem_empty + buf * 8u);
        TRACE(rank, pair == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 2);
        promote32(acc + 32, v0, s);
        promote32(acc + 48, v1, s);
        TRACE(rank, pair == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 3);
      }
      // the four warps of a column half leave together or not at all
      if (named_bar_or(1 + half, 128, !ok)) break;

      // ---- epilogue: this thread holds C[gm, col .. col + 128) in fp32
#pragma unroll
      for (int ch = 0; ch < CT / 64; ++ch) {
        const float* accf = reinterpret_cast<const float*>(acc) + ch * 64;
        const int c0 = col0 + half * CT + ch * 64;
        if (sizeof(OutT) == 2 && p.tma_store) {
          if (issuer) tma_store_wait_read0();   // the staging buffer may still be read by the previous store
          named_bar_sync(1 + half, 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 w;
            const float* a8 = accf + j * 8;
            w.x = pack2<OutT>(a8[0], a8[1]);
            w.y = pack2<OutT>(a8[2], a8[3]);
            w.z = pack2<OutT>(a8[4], a8[5]);
            w.w = pack2<OutT>(a8[6], a8[7]);
            // 128-byte swizzle: 16-byte chunk j of row r lives at chunk j ^ (r & 7)
            *reinterpret_cast<uint4*>(my_buf + row * 128 + ((j ^ (row & 7)) << 4)) = w;
          }
          fence_proxy_async_smem();
          named_bar_sync(1 + half, 128);
          if (issuer && c0 < p.n && a_row < p.m) {
            tma_store_2d(&map_c, my_buf, c0, a_row);
            tma_store_commit();
          }
        } else if (gm < p.m) {
          OutT* crow = static_cast<OutT*>(p.c) + static_cast<int64_t>(gm) * p.n;
          constexpr int kVec = 16 / sizeof(OutT);
#pragma unroll
          for (int j = 0; j < 64; j += kVec) {
            const int col = c0 + j;
            alignas(16) OutT tmp[kVec];
#pragma unroll
            for (int e = 0; e < kVec; ++e) tmp[e] = to_out<OutT>(accf[j + e]);
            if (col + kVec <= p.n && (reinterpret_cast<uintptr_t>(crow + col) & 15u) == 0) {
              *reinterpret_cast<uint4*>(crow + col) = *reinterpret_cast<const uint4*>(tmp);
            } else {
#pragma unroll
              for (int e = 0; e < kVec; ++e)
                if (col + e < p.n) crow[col + e] = tmp[e];
            }
          }
        }
      }
    }
    if (issuer) tma_store_wait_all();
  }

  // nobody frees tensor memory or leaves while the peer may still use this CTA's shared memory,
  // barriers or accumulators
  __syncwarp();
  tc_fence_before_sync();
  cluster_sync_all();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc_pair(tmem_base, kTmemCols);
}

template <typename OutT>
int launch_pair_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const PairParams& p,
                  int pairs, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_pair_gemm_kernel<OutT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = options().gemm_pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, w8a8_pair_gemm_kernel<OutT>, ma, mb, mc, p);
  if (e != cudaSuccess) return note_cuda_error(e);
  return check_launch();
}

}  // namespace

// Whether a plain GEMM call goes to the pair kernel: from two 128-row M-tiles on.
bool use_pair_kernel(int64_t m) {
  const int forced = options().gemm_pair;
  if (forced == 0) return false;
  if (forced == 1) return true;
  return m > 128;
}

int launch_gemm_pair(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales, const void* b_q,
                     const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                     cudaStream_t stream) {
  const Options& opt = options();
  const int out_bytes = (out_dt == 0) ? 4 : 2;
  bool tma_store = out_bytes == 2 && (n * out_bytes) % 16 == 0 && (reinterpret_cast<uintptr_t>(c) % 16 == 0);
  if (opt.gemm_tma_store == 0) tma_store = false;

  PairParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = c;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>((n + 127) / 128);
  p.tiles_m = static_cast<int>((m + 2 * PM - 1) / (2 * PM));
  p.tiles_n = static_cast<int>((n + PN - 1) / PN);
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = tma_store ? 1 : 0;
  // bands of 4096 rows like the single-CTA kernel (option gemm_group_m counts 128-row tiles)
  p.group_m = opt.gemm_group_m > 0 ? (opt.gemm_group_m + 1) / 2 : 16;
  p.no_loads = opt.debug_no_loads;
  p.status = ctx->status;

  CUtensorMap ma, mb, mc;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m, k, k, PM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, n, k, k, PN / 2, BK, true);
  if (rc != INFEROP_OK) return rc;
  if (tma_store) {
    rc = make_tensor_map_2d(&mc, c, 2, m, n, n * 2, 128, 64, true);
    if (rc != INFEROP_OK) return rc;
  } else {
    mc = ma;  // unused by the kernel
  }
  int pairs = (opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count) / 2;
  if (pairs < 1) pairs = 1;
  if (pairs > p.num_tiles) pairs = p.num_tiles;
  switch (out_dt) {
    case 0: return launch_pair_t<float>(ma, mb, mc, p, pairs, stream);
    case 1: return launch_pair_t<__half>(ma, mb, mc, p, pairs, stream);
    case 2: return launch_pair_t<__nv_bfloat16>(ma, mb, mc, p, pairs, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

}  // namespace ib200
