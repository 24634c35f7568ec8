// Blockwise-FP8 W8A8 GEMM for sm_100a: TMA -> swizzled shared memory ->
// tcgen05.mma (E4M3 x E4M3 -> fp32 in tensor memory) -> per-K-block scale
// promotion into fp32 registers -> bf16/fp16/fp32 output.
//
// Replaces the reference's kernels/gemm/w8a8_block_fp8.cu (CUDA-core kernel
// :27-126, run-time tile dispatch :128-159) with one persistent, warp-
// specialised kernel.  The arithmetic contract is the reference's
// (w8a8_block_fp8.cu:100-114, reference/reference.cpp:93-110):
//     C[m,n] = sum_kb ( sa[m,kb] * sb[n/128,kb] ) * sum_{k in kb} A_q[m,k] * B_q[n,k]
// The inner sum over one 128-wide K block is exact-product fp32 accumulation
// on the tensor core; the outer sum is an fp32 FMA per output element per K
// block on the CUDA cores ("promotion"), so no scale is ever folded into a
// reduced-precision accumulator.  Output is rounded once (RNE).
//
// Tile: 128 rows x 256 columns of C per CTA, K in blocks of 128.  One K block is
// 4 MMAs (M=128, N=256, K=32) into one of two 256-column accumulator buffers in
// tensor memory (buffer = K block parity), so the tensor core works on block
// kb+1 while block kb is being promoted.
//
// CTA layout (384 threads, one CTA per SM, persistent over output tiles):
//   warp 0      allocates / frees tensor memory; one thread is the TMA producer:
//               A tile [128 x 128 B] and B tile [256 x 128 B] per K block into a
//               4-deep ring (128-byte swizzle, K-major)
//   warps 1, 2  MMA issuers: warp 1 the even K blocks of the CTA's work list,
//               warp 2 the odd ones.  Their instruction streams write different
//               TMEM buffers and need no ordering between them.
//   warps 4-11  promotion + epilogue.  Warp w reads TMEM lane quarter w % 4
//               (its 32 rows); warps 4-7 take columns 0-127 (the left
//               weight-scale block), warps 8-11 columns 128-255.  A thread owns
//               one output row segment of 128 columns in registers.
//
// Shared memory (dynamic, 1024-byte aligned):
//   [4 x (A 16 KiB | B 32 KiB)] [2 x 16 KiB output staging] [barriers]
//
// HBM traffic per call (algorithmic): M*K + N*K operand bytes, 4*M*K/128 +
// 4*ceil(N/128)*K/128 scale bytes, M*N*sizeof(out) output bytes; operand
// re-reads by other tiles are served by L2 (tiles are rasterised in bands of
// 32 M-tiles: a band's A panel stays in L2 while the weights stream past it once).
//
// Every wait is bounded (ptx.cuh: mbar_wait).  A wait that runs out sets the
// CTA's abort flag and the device status record; all roles then fall through
// to the common exit, tensor memory is freed, and the kernel returns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include <atomic>

#include "internal.h"
#include "quant_math.cuh"
#include "swiglu_math.cuh"

#define IB200_TRACE_TAG single
#include "trace.cuh"

namespace ib200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 128;
constexpr int kPromoWarps = 8;
constexpr int kThreads = 128 + 32 * kPromoWarps;
constexpr int kBytesA = BM * BK;
constexpr int kTmemCols = 512;             // all of tensor memory: 512 / BN accumulator buffers
constexpr int kStoreBufBytes = 128 * 128;  // 128 rows x 64 two-byte columns
constexpr int kBarrierBytes = 256;

// Two tile widths.  256 columns: the fewest operand bytes per flop; the default.  128 columns:
// half the promotion work and half the weight bytes per K block, six ring stages instead of four
// and four accumulator buffers instead of two; it pays only when M fits one M-tile (see
// pick_block_n), where it doubles the number of tiles that share the SMs.
template <int TBN>
struct Tile {
  static constexpr int BN = TBN;
  static constexpr int CT = TBN / 2;            // columns per promotion thread (two column halves)
  static constexpr int kStages = TBN == 256 ? 4 : 6;
  static constexpr int kBytesB = TBN * BK;
  static constexpr int kStageBytes = kBytesA + kBytesB;
  static constexpr int kSlices = kTmemCols / TBN;   // TMEM accumulator buffers, one K block each
  static constexpr int kSmemBytes =
      kStages * kStageBytes + 2 * kStoreBufBytes + kBarrierBytes + 1024 /* alignment slack */;
};
static_assert(Tile<256>::kSmemBytes == Tile<128>::kSmemBytes, "both variants fill shared memory");
constexpr int kSmemBytes = Tile<256>::kSmemBytes;

struct GemmParams {
  const float* a_scales;
  const float* b_scales;
  void* c;
  int m, n, k;
  int kb;        // K / 128
  int nb;        // ceil(N / 128): rows of b_scales
  int tiles_m, tiles_n, num_tiles;
  int group_m;   // M-tiles per rasterisation band: a band's A panel stays in L2 while W streams past once
  int tma_store; // 1: epilogue goes through shared memory + TMA store
  int no_loads;  // test hook: the producer issues no load
  // Grouped launches with a device tile list: tiles are claimed from this counter (zeroed before the
  // launch) instead of being dealt round-robin, nullptr = static dealing.  See gemm_body.
  int* sched = nullptr;
  int rep = 0;   // grouped launches: M-tiles of at most 32 rows run in the replicated form (gemm_body)
  // SwiGLU launches only: c receives E4M3 bytes [rows, n / 2], c_scales one fp32 per 128 of them
  float* c_scales;
  DeviceStatus* status;
};

// wait sites reported in DeviceStatus::code
enum : uint32_t {
  kSiteProducerEmpty = 0x101,
  kSiteProducerDrain = 0x102,
  kSiteMmaTmemEmpty = 0x201,
  kSiteMmaFull = 0x202,
  kSitePromoTmemFull = 0x301,
  kSiteSchedEmpty = 0x401,
  kSiteSchedFull = 0x402,
};
constexpr int kSchedSlots = 4;   // claimed tiles the producer may be ahead of the slowest consumer warp

// Grouped (MoE) launches: the rows of A and C are the concatenation of the groups' rows, the
// weights are [groups][N][K].  The host cuts every group into 128-row M-tiles and passes the
// list by value; tile t of the launch is M-tile t / tiles_n, N-tile t % tiles_n.
constexpr int kMaxGroupTiles = 2040;
struct GroupTable {
  int row0[kMaxGroupTiles];   // first row (in A and C) of the M-tile
  int meta[kMaxGroupTiles];   // (group << 8) | (rows - 1): which group, how many valid rows
};

// All-gather launches (column-parallel sharding): this rank's [M, n] result is written into the
// full [M, n * ranks] row-major result of EVERY rank, at column offset rank * n, by one TMA store
// per destination from the same staging buffer.  The destinations are peer-mapped device
// addresses; the list is rotated on the host (first destination = rank + 1, own buffer last) so
// that the ranks do not all write to the same GPU at the same moment.
constexpr int kMaxPeers = 8;
struct PeerMaps {
  CUtensorMap map[kMaxPeers];  // [M, n * ranks] two-byte row-major, box 128 rows x 64 columns
  int count;
  int col_offset;              // rank * n
  // scatter launches only (below)
  int rows_per_owner;
  int rank;
};

// Scatter launches (row-parallel sharding, the first half of a reduce-scatter): this rank holds a
// K shard of both operands, so its result is a PARTIAL sum over K of the whole [M, N] output.  It
// stays in fp32 and goes, tile by tile, to the rank that owns those rows of the final result:
// rows [d * M/G, (d + 1) * M/G) belong to rank d, which keeps one [M/G, N] fp32 slot per source
// rank; map[d] describes rank d's slots as one [G * M/G, N] fp32 tensor (box 128 rows x 32
// columns) and this rank writes slot `rank` of it.  The owner adds its slots in rank order
// afterwards (reduce_slots), so the sum does not depend on arrival order.
// SwiGLU launches (the gate_up projection of an expert layer): a grouped launch whose weights are
// [groups][2 I][K] with the gate rows first and the up rows second (the reference's layout,
// kernels/silu_mul.cu:16-28).  Tile tn takes gate rows [128 tn, 128 tn + 128) as its left 128
// columns and up rows [I + 128 tn, ...) as its right 128, so one tile holds everything one
// 128-wide output group needs: the epilogue rounds both halves to the 16-bit type, applies
// silu(gate) * up, quantises the 128 results of each row (one scale per row and tile) and writes
// E4M3 bytes + scales, bit for bit what silu_and_mul_quant makes of the GEMM's 16-bit output.
enum : int { kModePlain = 0, kModeGrouped = 1, kModeGather = 2, kModeScatter = 3, kModeSwiglu = 4 };

struct TileInfo {
  int a_row;     // first row of the tile in A / a_scales / C
  int row_end;   // rows at and beyond this index are not this tile's
  int b_row;     // first row of the tile in the (stacked) weight matrix
  int b_row_hi;  // SwiGLU launches: first weight row of the right column half (the up rows)
  int sb_row;    // row of b_scales for the tile's left half
  int sb_step;   // rows of b_scales between the left and the right column half
  int sb_rows;   // one past the last valid b_scales row for this tile's group
  int col;       // first output column
  int rep;       // 1: the tile has at most 32 rows and runs in the replicated form
};

// The tile list of a grouped launch as the kernel sees it: either the by-value GroupTable or
// arrays that a kernel wrote to device memory (no host round trip for the experts' row counts).
struct TileList {
  const int* row0;
  const int* meta;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int per_band = group_m * tiles_n;
  const int band = t / per_band;
  const int first_m = band * group_m;
  const int band_m = min(group_m, tiles_m - first_m);
  const int r = t - band * per_band;
  tm = first_m + r % band_m;
  tn = r / band_m;
}

template <bool kGrouped, int BN, bool kSwiglu = false>
__device__ __forceinline__ TileInfo tile_info(int t, const GemmParams& p, const TileList& tab) {
  TileInfo ti;
  ti.sb_step = (BN / 2) / 128;
  ti.b_row_hi = 0;
  ti.rep = 0;
  if (kSwiglu) {
    // p.n = 2 I weight rows per group, p.tiles_n = I / 128 tiles, 128 output columns per tile
    const int mt = t / p.tiles_n, tn = t - mt * p.tiles_n;
    const int meta = tab.meta[mt];
    const int group = meta >> 8;
    const int inter = p.n >> 1;
    ti.a_row = tab.row0[mt];
    ti.row_end = ti.a_row + (meta & 0xFF) + 1;
    ti.b_row = group * p.n + tn * 128;
    ti.b_row_hi = ti.b_row + inter;
    ti.sb_row = group * p.nb + tn;
    ti.sb_step = inter >> 7;
    ti.sb_rows = (group + 1) * p.nb;
    ti.col = tn * 128;
    ti.rep = (p.rep && (meta & 0xFF) < 32) ? 1 : 0;
  } else if (kGrouped) {
    const int mt = t / p.tiles_n, tn = t - mt * p.tiles_n;
    const int meta = tab.meta[mt];
    const int group = meta >> 8;
    ti.a_row = tab.row0[mt];
    ti.row_end = ti.a_row + (meta & 0xFF) + 1;
    ti.b_row = group * p.n + tn * BN;
    ti.sb_row = group * p.nb + tn * (BN / 128);
    ti.sb_rows = (group + 1) * p.nb;
    ti.col = tn * BN;
    ti.rep = (BN == 256 && p.rep && (meta & 0xFF) < 32) ? 1 : 0;
  } else {
    int tm, tn;
    tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
    ti.a_row = tm * BM;
    ti.row_end = p.m;
    ti.b_row = tn * BN;
    ti.sb_row = tn * (BN / 128);
    ti.sb_rows = p.nb;
    ti.col = tn * BN;
  }
  return ti;
}

template <typename OutT>
__device__ __forceinline__ OutT to_out(float v);
template <>
__device__ __forceinline__ float to_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// two floats -> one 32-bit word of two 16-bit outputs (low half = a)
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

// Pin the 32 registers of a tensor-memory load behind the wait: nothing that
// reads them may be scheduled before tcgen05.wait::ld.
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

// acc[0..31] += v[0..31] * s, two lanes per instruction (fma.rn.f32x2)
__device__ __forceinline__ void promote32(float2* acc, const uint32_t (&v)[32], float s) {
  const float2 s2 = make_float2(s, s);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    acc[j] = __ffma2_rn(make_float2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), s2,
                        acc[j]);
  }
}

template <typename OutT, int kMode, int TBN>
__device__ __forceinline__ void gemm_body(const CUtensorMap* map_a, const CUtensorMap* map_b,
                                          const CUtensorMap* map_c, const GemmParams& p,
                                          const TileList tab, const PeerMaps* peers,
                                          const int* num_mtiles_dev, const CUtensorMap* map_a32 = nullptr) {
  constexpr bool kSwiglu = kMode == kModeSwiglu;
  constexpr bool kGrouped = kMode == kModeGrouped || kSwiglu;
  constexpr bool kGather = kMode == kModeGather;
  constexpr bool kScatter = kMode == kModeScatter;
  using TL = Tile<TBN>;
  constexpr int BN = TL::BN, CT = TL::CT, kStages = TL::kStages, kStageBytes = TL::kStageBytes,
                kSlices = TL::kSlices;
  // The two MMA issuer warps alternate K blocks.  With an even number of stages (and of
  // accumulator buffers) a stage always belongs to the same warp, whose parity waits on its
  // barrier follow one another in program order.  With an odd number a stage would alternate
  // between the warps, and one warp's wait could be answered by the phase the other warp is still
  // waiting for whenever two TMA loads complete out of order (seen as a launch failure at full
  // size on 4 GPUs in a three-stage experiment); such a variant needs one barrier per stage AND warp.
  static_assert(kStages % 2 == 0 && kSlices % 2 == 0, "a ring stage must always belong to the same issuer warp");
  // Registers per thread after the role split (setmaxnreg; ptxas allocates each branch against its
  // own figure).  The CTA owns what it was launched with, 384 threads x 168 registers, and
  // setmaxnreg.inc waits until that pool can serve it: the 128 threads of warps 0-3 must give back
  // at least what the 256 promotion threads take, or the kernel never gets past the role split.
  // The 256-column tile needs every register it can get for its 128 accumulators and two
  // 32-column loads in flight; with the 128-column tile the producer and MMA warps keep 80, which
  // is what their branch needs to stay free of spills.
  constexpr int kLaunchRegs = 168;
  constexpr int kLowRegs = TBN == 256 ? 56 : 80;
  constexpr int kHighRegs = TBN == 256 ? 224 : 208;
  static_assert(128 * (kLaunchRegs - kLowRegs) >= 256 * (kHighRegs - kLaunchRegs),
                "warps 0-3 must release at least the registers the promotion warps request");
  // a device-built tile list comes with its length in device memory (at most p.tiles_m entries)
  const int num_tiles =
      (kGrouped && num_mtiles_dev != nullptr) ? min(__ldg(num_mtiles_dev), p.tiles_m) * p.tiles_n
                                              : p.num_tiles;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  uint8_t* store_buf = smem + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(store_buf + 2 * kStoreBufBytes);
  uint64_t* full = bars;                            // [kStages]  TMA -> MMA
  uint64_t* empty = bars + kStages;                 // [kStages]  MMA (both issuers) -> TMA
  uint64_t* tmem_full = bars + 2 * kStages;         // [kSlices]  MMA -> promotion
  uint64_t* tmem_empty = tmem_full + kSlices;       // [kSlices]  promotion -> MMA
  uint64_t* sched_full = tmem_empty + kSlices;      // [kSchedSlots]  producer -> MMA and promotion warps
  uint64_t* sched_empty = sched_full + kSchedSlots; // [kSchedSlots]  the ten consumer warps -> producer
  volatile int* sched_tile = reinterpret_cast<volatile int*>(sched_empty + kSchedSlots);   // [kSchedSlots]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(const_cast<int*>(sched_tile) + kSchedSlots);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  static_assert((2 * kStages + 2 * kSlices + 2 * kSchedSlots) * 8 + kSchedSlots * 4 + 8 <= kBarrierBytes,
                "barriers, tile slots and flags must fit their corner of shared memory");
  // Tiles claimed from a device counter.  Dealt round-robin, the CTAs drift apart by tens of
  // microseconds over a launch, and the two M-tiles of one expert, which stream the same weights,
  // end up so far apart that the second reader misses L2 (1.45 times the weight bytes came from
  // HBM on a 256-expert layer).  With a counter, tiles next to each other in the list start within
  // microseconds of each other whatever happened before.  The producer claims a tile when it has
  // issued the last load of the previous one and publishes it to the other warps through a small
  // ring of slots; -1 ends the list.  The results do not depend on who computes which tile.
  const bool dyn = kGrouped && p.sched != nullptr;

  // the shuffle tells the compiler that the warp index is uniform across the warp
  const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < kSlices; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], kPromoWarps);
    }
    for (int q = 0; q < kSchedSlots; ++q) {
      mbar_init(&sched_full[q], 1);
      mbar_init(&sched_empty[q], 2 + kPromoWarps);
    }
    *abort_flag = 0u;
    mbar_init_fence();
    tma_prefetch_desc(map_a);
    tma_prefetch_desc(map_b);
    if constexpr (kGather || kScatter) {
      for (int d = 0; d < peers->count; ++d) tma_prefetch_desc(&peers->map[d]);
    } else {
      if (p.tma_store) tma_prefetch_desc(map_c);
    }
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_slot, 0);

  // the next tile of this CTA as an MMA or promotion warp sees it: -1 at the end of the list, -2
  // when the wait for the producer's slot ran out
  uint32_t sched_i = 0;
  auto next_tile = [&](int prev) -> int {
    if (!dyn) {
      const int t = prev < 0 ? static_cast<int>(blockIdx.x) : prev + static_cast<int>(gridDim.x);
      return t < num_tiles ? t : -1;
    }
    const uint32_t q = sched_i % kSchedSlots;
    if (!mbar_wait(&sched_full[q], (sched_i / kSchedSlots) & 1u, abort_flag, p.status, kSiteSchedFull)) return -2;
    const int t = sched_tile[q];
    __syncwarp();
    if (lane == 0) mbar_arrive(&sched_empty[q]);
    ++sched_i;
    return t;
  };

  if (warp < 4) {
    reg_dealloc<kLowRegs>();
    if (warp == 0 && lane == 0) {
      // ------------------------------ TMA producer ------------------------
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0, armed_phase = 0;
      bool ok = true;
      uint32_t claim_i = 0;
      for (int t = blockIdx.x; ok && !p.no_loads; t += gridDim.x) {
        if (dyn) {
          const uint32_t q = claim_i % kSchedSlots;
          if (!mbar_wait(&sched_empty[q], ((claim_i / kSchedSlots) & 1u) ^ 1u, abort_flag, p.status,
                         kSiteSchedEmpty)) {
            ok = false;
            break;
          }
          t = atomicAdd(p.sched, 1);
          if (t >= num_tiles) t = -1;
          sched_tile[q] = t;
          mbar_arrive(&sched_full[q]);
          ++claim_i;
          if (t < 0) break;
        } else if (t >= num_tiles) {
          break;
        }
        const TileInfo ti = tile_info<kGrouped, BN, kSwiglu>(t, p, tab);
        for (int kb = 0; kb < p.kb; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, p.status, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          mbar_arrive_expect_tx(&full[stage], kStageBytes);
          if (kGrouped && ti.rep) {
            // the tile's (at most) 32 rows four times over: every quarter of the 128 accumulator
            // lanes then holds the same rows, and each quarter's warps promote other columns
#pragma unroll
            for (int q = 0; q < 4; ++q) tma_load_2d(sa + q * 32 * BK, map_a32, &full[stage], kb * BK, ti.a_row);
          } else {
            tma_load_2d(sa, map_a, &full[stage], kb * BK, ti.a_row);
          }
          if constexpr (kSwiglu) {
            // two 128-row boxes of the weights: the gate rows, then the up rows of the same block
            tma_load_2d(sa + kBytesA, map_b, &full[stage], kb * BK, ti.b_row);
            tma_load_2d(sa + kBytesA + 128 * BK, map_b, &full[stage], kb * BK, ti.b_row_hi);
          } else {
            tma_load_2d(sa + kBytesA, map_b, &full[stage], kb * BK, ti.b_row);
          }
          armed |= 1u << stage;
          armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // wind-down: let the copies this thread started land before the CTA exits
        for (int s = 0; s < kStages; ++s) {
          if (!(armed & (1u << s))) continue;
          const uint32_t par = (armed_phase >> s) & 1u;
          const long long t0 = clock64();
          while (!mbar_test_wait(&full[s], par)) {
            if (clock64() - t0 > wait_budget(p.status)) {
              atomicCAS(&p.status->code, 0u, kSiteProducerDrain);
              break;
            }
          }
        }
      }
    } else if (warp == 1 || warp == 2) {
      // ------------------------------ MMA issuers -------------------------
      // Warp 1 issues the even K blocks of this CTA's work list (TMEM buffer 0), warp 2 the
      // odd ones (buffer 1); the two streams write different buffers and need no ordering.
      // Each warp runs its loop with all 32 lanes: warp-uniform control flow keeps the
      // descriptors in uniform registers, which makes issuing cheap (about 76 cycles per MMA
      // and 92 per commit, against more than 120 per MMA from divergent single-lane code);
      // one elected lane issues the tcgen05 instructions.
      constexpr uint32_t idesc = umma_idesc_e4m3_f32(BM, BN);
      const uint32_t smem_base = smem_u32(smem);
      // K blocks of the tiles seen so far (the warps learn of a tile from next_tile)
      uint32_t total = 0;
      int mma_t = -1;
      // K block `it` uses ring stage it % kStages and accumulator buffer it % kSlices; this warp
      // steps by two, so it keeps running counters instead of dividing (kStages and kSlices are even)
      uint32_t stage = warp - 1, phase = 0, buf = warp - 1, use = 0;
      for (uint32_t it = warp - 1;; it += 2, stage += 2, buf += 2) {
        while (it >= total && mma_t != -2) {
          mma_t = next_tile(mma_t);
          if (mma_t < 0) {
            mma_t = -2;
            break;
          }
          total += static_cast<uint32_t>(p.kb);
        }
        if (it >= total) break;
        if (stage >= static_cast<uint32_t>(kStages)) {
          stage -= kStages;
          phase ^= 1u;
        }
        if (buf >= static_cast<uint32_t>(kSlices)) {
          buf -= kSlices;
          ++use;
        }
        const uint32_t d_tmem = tmem_base + buf * BN;
        // operands first (normally long there), then the accumulator buffer (the late one)
        if (!mbar_wait(&full[stage], phase, abort_flag, p.status, kSiteMmaFull)) break;
        TRACE(0, blockIdx.x == 0 && lane == 0, 1, it, 0);
        if (!mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag, p.status, kSiteMmaTmemEmpty)) break;
        TRACE(0, blockIdx.x == 0 && lane == 0, 1, it, 1);
        __syncwarp();
        tc_fence_after_sync();
        const uint32_t a_addr = smem_base + stage * kStageBytes;
        const uint64_t da = umma_desc_k_sw128(a_addr);
        const uint64_t db = umma_desc_k_sw128(a_addr + kBytesA);
        if (elect_one()) {
#pragma unroll
          for (int k4 = 0; k4 < BK / 32; ++k4) {
            // 32 E4M3 elements = 32 bytes along K inside the swizzle atom: +2 in 16-byte units
            umma_f8_ss(d_tmem, da + 2u * k4, db + 2u * k4, idesc, k4 > 0 ? 1u : 0u);
          }
          umma_commit(&tmem_full[buf]);
          umma_commit(&empty[stage]);
        }
        __syncwarp();
        TRACE(0, blockIdx.x == 0 && lane == 0, 1, it, 2);
      }
    }
  } else {
    reg_alloc<kHighRegs>();
    // ------------------------------ promotion + epilogue ------------------
    const int pw = warp - 4;
    const int quarter = pw & 3;  // == warp % 4: the TMEM lane quarter this warp may read
    const int half = pw >> 2;    // which column half of the tile (CT columns, inside one weight-scale block)
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + half * CT;
    uint8_t* my_buf = store_buf + half * kStoreBufBytes;
    const bool issuer = (quarter == 0 && lane == 0);
    uint32_t kiter = 0;
    bool gave_up = false;
    for (int t = next_tile(-1);; t = next_tile(t)) {
      if (t < 0) {
        gave_up = t == -2;
        break;
      }
      bool ok = true;
      const TileInfo ti = tile_info<kGrouped, BN, kSwiglu>(t, p, tab);
      // Replicated form of a tile with at most 32 rows (grouped launches, 256-column tiles): the
      // producer loaded the same 32 rows into all four row quarters of the A tile, so the four
      // lane quarters of the accumulator hold the same 32 x 256 block.  Lane l of every warp owns
      // tile row l, and the warp of quarter q promotes columns [32 q, 32 q + 32) of its column
      // half: a quarter of the work per warp, with the same arithmetic per element.  Without it a
      // small tile costs the promotion warps as much as a full one (two of the eight do it all).
      const bool rep = kGrouped && CT == 128 && ti.rep;
      if constexpr (kGrouped && CT == 128) {
        if (rep) {
          // the whole replicated path is kept apart from the full one: 32 accumulators instead of
          // 128, and nothing of it inside the full path's loop
          const int gm = ti.a_row + lane;
          const int nbi = ti.sb_row + half * ti.sb_step;
          const bool have = gm < ti.row_end && nbi < ti.sb_rows;
          const float* sa_ptr = p.a_scales + static_cast<int64_t>(have ? gm : 0) * p.kb;
          const float* sb_ptr = p.b_scales + static_cast<int64_t>(have ? nbi : 0) * p.kb;
          float2 acc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = make_float2(0.0f, 0.0f);
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
            if (!mbar_wait(&tmem_full[buf], (kiter / kSlices) & 1u, abort_flag, p.status,
                           kSitePromoTmemFull)) {
              ok = false;
              break;
            }
            __syncwarp();
            tc_fence_after_sync();
            uint32_t v0[32];
            tmem_ld_32x32(lane_base + buf * BN + quarter * 32, v0);
            tmem_ld_wait_pin(v0);
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[buf]);
            promote32(acc, v0, s);
          }
          if (!ok) {
            gave_up = true;
            break;
          }
          const float* accf = reinterpret_cast<const float*>(acc);
          if constexpr (kSwiglu) {
            named_bar_sync(3, 256);   // the previous tile's readers are done with the staging memory
            // replicated form: this thread holds 32 columns (four 16-byte chunks) of tile row `lane`;
            // the 128-wide output group of a row is spread over the four quarters' warps, which
            // exchange their partial maxima through shared memory
            using T2 = typename std::conditional<std::is_same<OutT, __half>::value, __half2, __nv_bfloat162>::type;
            uint8_t* exr = store_buf + lane * 256;
            float* amax_sh = reinterpret_cast<float*>(store_buf + 32 * 256);   // [4][32]
            if (half == 1) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 w;
                const float* a8 = accf + j * 8;
                w.x = pack2<OutT>(a8[0], a8[1]);
                w.y = pack2<OutT>(a8[2], a8[3]);
                w.z = pack2<OutT>(a8[4], a8[5]);
                w.w = pack2<OutT>(a8[6], a8[7]);
                *reinterpret_cast<uint4*>(exr + (((quarter * 4 + j) ^ (lane & 15)) << 4)) = w;
              }
            }
            named_bar_sync(3, 256);
            uint4 h[4];
            float amax = 0.0f;
            if (half == 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint4 g;
                const float* a8 = accf + j * 8;
                g.x = pack2<OutT>(a8[0], a8[1]);
                g.y = pack2<OutT>(a8[2], a8[3]);
                g.z = pack2<OutT>(a8[4], a8[5]);
                g.w = pack2<OutT>(a8[6], a8[7]);
                const uint4 u = *reinterpret_cast<const uint4*>(exr + (((quarter * 4 + j) ^ (lane & 15)) << 4));
                h[j] = swiglu::silu_mul8<OutT>(g, u);
                amax = fmaxf(amax, absmax8_packed<T2>(h[j]));
              }
              amax_sh[quarter * 32 + lane] = amax;
            }
            named_bar_sync(3, 256);
            if (half == 0 && gm < ti.row_end) {
              amax = fmaxf(fmaxf(amax_sh[lane], amax_sh[32 + lane]), fmaxf(amax_sh[64 + lane], amax_sh[96 + lane]));
              const float scale = group_scale(amax);
              const bool fast = fast_div_ok(amax);
              const float rcp = __frcp_rn(scale);
              uint8_t* qrow = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(gm) * (p.n >> 1) + ti.col + quarter * 32;
#pragma unroll
              for (int j = 0; j < 4; j += 2) {
                float f0[8], f1[8];
                swiglu::unpack8<OutT>(h[j], f0);
                swiglu::unpack8<OutT>(h[j + 1], f1);
                const uint2 b0 = fast ? quantise8_fast16(h[j], f0, scale, rcp) : quantise8<false>(f0, scale, 0.0f);
                const uint2 b1 = fast ? quantise8_fast16(h[j + 1], f1, scale, rcp) : quantise8<false>(f1, scale, 0.0f);
                *reinterpret_cast<uint4*>(qrow + j * 8) = make_uint4(b0.x, b0.y, b1.x, b1.y);
              }
              if (quarter == 0) p.c_scales[static_cast<int64_t>(gm) * (p.n >> 8) + (ti.col >> 7)] = scale;
            }
          } else {
            // replicated form: 32 columns of tile row `lane`, stored straight from the registers
            if (gm < ti.row_end) {
              const int col0 = ti.col + half * CT + quarter * 32;
              OutT* crow = static_cast<OutT*>(p.c) + static_cast<int64_t>(gm) * p.n;
              constexpr int kVec = 16 / sizeof(OutT);
#pragma unroll
              for (int j = 0; j < 32; j += kVec) {
                const int col = col0 + j;
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
          continue;
        }
      }
      const int gm = ti.a_row + row;
      const int nbi = ti.sb_row + half * ti.sb_step;
      const bool have = gm < ti.row_end && nbi < ti.sb_rows;
      // a TMA store writes whole 128-row boxes (clipped only at the end of C): a grouped tile
      // with fewer rows must not spill into the next group's rows
      const bool tma_store = p.tma_store && (!kGrouped || ti.row_end - ti.a_row == BM);
      const float* sa_ptr = p.a_scales + static_cast<int64_t>(have ? gm : 0) * p.kb;
      const float* sb_ptr = p.b_scales + static_cast<int64_t>(have ? nbi : 0) * p.kb;

      float2 acc[CT / 2];
#pragma unroll
      for (int j = 0; j < CT / 2; ++j) acc[j] = make_float2(0.0f, 0.0f);

      // The scales of a K block are requested three blocks before the product that uses them, so
      // an L2 round trip (and most of an HBM one: expert rows' scales are used by one wave of
      // N-tiles only) never stalls this warp; a warp that waits holds up the accumulator buffer
      // for all eight.  The loads are pinned where they are written.  Measured on expert tiles of
      // 128 rows, consecutive builds: 2.09 ms with pinned loads one block ahead, 1.35 ms with this
      // queue; several builds with plain loads one block ahead also ran at 1.7-2.3 ms.
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
        if (!mbar_wait(&tmem_full[buf], (kiter / kSlices) & 1u, abort_flag, p.status,
                       kSitePromoTmemFull)) {
          ok = false;
          break;
        }
        TRACE(0, blockIdx.x == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 0);
        __syncwarp();
        tc_fence_after_sync();
        const uint32_t taddr = lane_base + buf * BN;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait_pin(v0);
        tmem_ld_wait_pin(v1);
        if constexpr (CT == 128) {
          TRACE(0, blockIdx.x == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 1);
          promote32(acc, v0, s);
          tmem_ld_32x32(taddr + 64, v0);
          promote32(acc + 16, v1, s);
          tmem_ld_32x32(taddr + 96, v1);
          tmem_ld_wait_pin(v0);
          tmem_ld_wait_pin(v1);
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
          TRACE(0, blockIdx.x == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 2);
          promote32(acc + 32, v0, s);
          promote32(acc + 48, v1, s);
          TRACE(0, blockIdx.x == 0 && lane == 0 && quarter == 0, 2 + half, kiter, 3);
        } else {
          // 64 columns per thread: one round of loads, the buffer is free before the FMAs
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[buf]);
          promote32(acc, v0, s);
          promote32(acc + 16, v1, s);
        }
      }
      if (!ok) {
        gave_up = true;
        break;
      }

      // ---- epilogue: this thread holds C[gm, col .. col + 128) in fp32
      if constexpr (kSwiglu) {
        // The right column half (up) parks its 128 values per row, rounded to the 16-bit type, in
        // the staging memory: row r = 256 bytes, 16-byte chunk j at position j ^ (r & 15), which
        // keeps both the row-per-thread writes and reads free of bank conflicts.  The left half
        // (gate) then owns one whole 128-wide output group per thread.
        named_bar_sync(3, 256);   // the previous tile's readers are done with the staging memory
        const float* accf = reinterpret_cast<const float*>(acc);
        uint8_t* ex = store_buf + row * 256;
        if (half == 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            uint4 w;
            const float* a8 = accf + j * 8;
            w.x = pack2<OutT>(a8[0], a8[1]);
            w.y = pack2<OutT>(a8[2], a8[3]);
            w.z = pack2<OutT>(a8[4], a8[5]);
            w.w = pack2<OutT>(a8[6], a8[7]);
            *reinterpret_cast<uint4*>(ex + ((j ^ (row & 15)) << 4)) = w;
          }
        }
        named_bar_sync(3, 256);
        if (half == 0) {
          using T2 = typename std::conditional<std::is_same<OutT, __half>::value, __half2, __nv_bfloat162>::type;
          uint4 h[16];
          float amax = 0.0f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            uint4 g;
            const float* a8 = accf + j * 8;
            g.x = pack2<OutT>(a8[0], a8[1]);
            g.y = pack2<OutT>(a8[2], a8[3]);
            g.z = pack2<OutT>(a8[4], a8[5]);
            g.w = pack2<OutT>(a8[6], a8[7]);
            const uint4 u = *reinterpret_cast<const uint4*>(ex + ((j ^ (row & 15)) << 4));
            h[j] = swiglu::silu_mul8<OutT>(g, u);
            amax = fmaxf(amax, absmax8_packed<T2>(h[j]));
          }
          const float scale = group_scale(amax);
          if (gm < ti.row_end) {
            const bool fast = fast_div_ok(amax);
            const float rcp = __frcp_rn(scale);
            uint8_t* qrow = static_cast<uint8_t*>(p.c) + static_cast<int64_t>(gm) * (p.n >> 1) + ti.col;
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              float f0[8], f1[8];
              swiglu::unpack8<OutT>(h[j], f0);
              swiglu::unpack8<OutT>(h[j + 1], f1);
              const uint2 b0 = fast ? quantise8_fast16(h[j], f0, scale, rcp) : quantise8<false>(f0, scale, 0.0f);
              const uint2 b1 = fast ? quantise8_fast16(h[j + 1], f1, scale, rcp) : quantise8<false>(f1, scale, 0.0f);
              *reinterpret_cast<uint4*>(qrow + j * 8) = make_uint4(b0.x, b0.y, b1.x, b1.y);
            }
            p.c_scales[static_cast<int64_t>(gm) * (p.n >> 8) + (ti.col >> 7)] = scale;
          }
        }
        continue;
      }
      if constexpr (kScatter) {
        // fp32 partial sums to slot `rank` of the rows' owner, 32 columns (128 bytes) per store
        const int owner = ti.a_row / peers->rows_per_owner;
        const int slot_row = peers->rank * peers->rows_per_owner + (ti.a_row - owner * peers->rows_per_owner);
#pragma unroll
        for (int ch = 0; ch < CT / 32; ++ch) {
          const float* accf = reinterpret_cast<const float*>(acc) + ch * 32;
          const int col0 = ti.col + half * CT + ch * 32;
          if (issuer) tma_store_wait_read0();
          named_bar_sync(1 + half, 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 w = make_uint4(__float_as_uint(accf[j * 4]), __float_as_uint(accf[j * 4 + 1]),
                                       __float_as_uint(accf[j * 4 + 2]), __float_as_uint(accf[j * 4 + 3]));
            *reinterpret_cast<uint4*>(my_buf + row * 128 + ((j ^ (row & 7)) << 4)) = w;
          }
          fence_proxy_async_smem();
          named_bar_sync(1 + half, 128);
          if (issuer && col0 < p.n) {
            tma_store_2d(&peers->map[owner], my_buf, col0, slot_row);
            tma_store_commit();
          }
        }
        continue;
      }
#pragma unroll
      for (int ch = 0; ch < CT / 64; ++ch) {
        const float* accf = reinterpret_cast<const float*>(acc) + ch * 64;
        const int col0 = ti.col + half * CT + ch * 64;
        if (sizeof(OutT) == 2 && tma_store) {
          // the staging buffer may still be read by the previous TMA store
          if (issuer) tma_store_wait_read0();
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
          if (issuer && col0 < p.n) {
            if constexpr (kGather) {
              for (int d = 0; d < peers->count; ++d)
                tma_store_2d(&peers->map[d], my_buf, peers->col_offset + col0, ti.a_row);
            } else {
              tma_store_2d(map_c, my_buf, col0, ti.a_row);
            }
            tma_store_commit();
          }
        } else if (kGrouped && sizeof(OutT) == 2 && p.tma_store) {
          // A group's ragged tile: a TMA store would write all 128 rows and run into the next
          // group, so the block is staged the same way and copied out by the 128 threads of this
          // column half with row-guarded 16-byte stores, 8 lanes per 128-byte row segment
          // (coalesced; the per-thread-row stores below touch 32 rows per instruction).
          if (issuer) tma_store_wait_read0();
          named_bar_sync(1 + half, 128);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 w;
            const float* a8 = accf + j * 8;
            w.x = pack2<OutT>(a8[0], a8[1]);
            w.y = pack2<OutT>(a8[2], a8[3]);
            w.z = pack2<OutT>(a8[4], a8[5]);
            w.w = pack2<OutT>(a8[6], a8[7]);
            *reinterpret_cast<uint4*>(my_buf + row * 128 + ((j ^ (row & 7)) << 4)) = w;
          }
          named_bar_sync(1 + half, 128);
          if (col0 < p.n) {
            const int chunk = row & 7;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = (row >> 3) + 16 * i;
              if (ti.a_row + r < ti.row_end) {
                const uint4 w = *reinterpret_cast<const uint4*>(my_buf + r * 128 + ((chunk ^ (r & 7)) << 4));
                OutT* dst = static_cast<OutT*>(p.c) + static_cast<int64_t>(ti.a_row + r) * p.n + col0 + chunk * 8;
                *reinterpret_cast<uint4*>(dst) = w;
              }
            }
          }
        } else if (gm < ti.row_end) {
          OutT* crow = static_cast<OutT*>(p.c) + static_cast<int64_t>(gm) * p.n;
          constexpr int kVec = 16 / sizeof(OutT);
          // fully unrolled: the accumulators must stay in registers
#pragma unroll
          for (int j = 0; j < 64; j += kVec) {
            const int col = col0 + j;
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
    if (gave_up) {
      // This warp's wait ran out (the CTA's abort flag is set, the call will report
      // INFEROP_ERR_DEVICE_WAIT).  A sibling whose own wait on the same barrier succeeded a moment
      // later may already stand at one of the named barriers of the tile's epilogue, waiting for
      // this warp.  It must not wait for ever: arrive at those barriers, without blocking, as
      // often as an epilogue has barriers, with pauses in which the siblings move on.  They then
      // fail their next wait (the MMA warps stop without this warp's releases) and come here too.
      for (int i = 0; i < 8; ++i) {
        named_bar_arrive(kSwiglu ? 3 : 1 + half, kSwiglu ? 256 : 128);
        const long long t0 = clock64();
        while (clock64() - t0 < 4096) {
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

template <typename OutT, int TBN>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  gemm_body<OutT, kModePlain, TBN>(&map_a, &map_b, &map_c, p, TileList{nullptr, nullptr}, nullptr, nullptr);
}

template <typename OutT, int TBN>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const GemmParams p,
                         const __grid_constant__ GroupTable tab) {
  gemm_body<OutT, kModeGrouped, TBN>(&map_a, &map_b, &map_c, p, TileList{tab.row0, tab.meta}, nullptr, nullptr);
}

// grouped launch whose tile list (and its length) was written to device memory by moe_align
template <typename OutT, int TBN>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_grouped_dev_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                             const __grid_constant__ CUtensorMap map_c, const GemmParams p,
                             const int* __restrict__ row0, const int* __restrict__ meta,
                             const int* __restrict__ num_mtiles, const __grid_constant__ CUtensorMap map_a32) {
  gemm_body<OutT, kModeGrouped, TBN>(&map_a, &map_b, &map_c, p, TileList{row0, meta}, nullptr, num_mtiles,
                                     &map_a32);
}

// SwiGLU launch: grouped tile list from device memory, output = E4M3 bytes + scales
template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_swiglu_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const GemmParams p, const int* __restrict__ row0, const int* __restrict__ meta,
                        const int* __restrict__ num_mtiles, const __grid_constant__ CUtensorMap map_a32) {
  gemm_body<T, kModeSwiglu, 256>(&map_a, &map_b, nullptr, p, TileList{row0, meta}, nullptr, num_mtiles, &map_a32);
}

template <typename T>
int launch_swiglu_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& ma32, const GemmParams& p,
                    const int* row0, const int* meta, const int* num_mtiles, int ctas, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_swiglu_gemm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_swiglu_gemm_kernel<T><<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, p, row0, meta, num_mtiles, ma32);
  return check_launch();
}

template <typename OutT, int TBN>
int launch_grouped_dev_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                         const CUtensorMap& ma32, const GemmParams& p, const int* row0, const int* meta, const int* num_mtiles,
                         int ctas, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_grouped_dev_gemm_kernel<OutT, TBN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_grouped_dev_gemm_kernel<OutT, TBN><<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, mc, p, row0, meta,
                                                                             num_mtiles, ma32);
  return check_launch();
}

template <typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
w8a8_gather_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const GemmParams p, const __grid_constant__ PeerMaps peers) {
  gemm_body<OutT, kModeGather, 256>(&map_a, &map_b, nullptr, p, TileList{nullptr, nullptr}, &peers, nullptr);
}

__global__ void __launch_bounds__(kThreads, 1)
w8a8_scatter_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         const GemmParams p, const __grid_constant__ PeerMaps peers) {
  gemm_body<float, kModeScatter, 256>(&map_a, &map_b, nullptr, p, TileList{nullptr, nullptr}, &peers, nullptr);
}

template <typename OutT>
int launch_gather_t(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p,
                    const PeerMaps& peers, int ctas, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gather_gemm_kernel<OutT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_gather_gemm_kernel<OutT><<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, p, peers);
  return check_launch();
}

template <typename OutT, int TBN>
int launch_grouped_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                     const GemmParams& p, const GroupTable& tab, int ctas, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_grouped_gemm_kernel<OutT, TBN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_grouped_gemm_kernel<OutT, TBN><<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, mc, p, tab);
  return check_launch();
}

template <typename OutT, int TBN>
int launch_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
             const GemmParams& p, int ctas, cudaStream_t stream) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_gemm_kernel<OutT, TBN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_gemm_kernel<OutT, TBN><<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, mc, p);
  return check_launch();
}

}  // namespace

namespace {
// Tile width of a launch: option gemm_block_n forces 128 or 256.  Measured on M x 18432 x 7168:
// with a single M-tile (M <= 128) the 128-column tile is 14 % faster (30.4 against 35.4 us: twice
// as many tiles to spread over the SMs, deeper ring); from two M-tiles on, and for expert groups
// (1.82 against 2.07 ms on 256 experts x 4096 x 7168), the 256-column tile wins by 15-40 %.
int pick_block_n(bool grouped, int64_t m) {
  const int forced = options().gemm_block_n;
  if (forced == 128 || forced == 256) return forced;
  return (!grouped && m <= BM) ? 128 : 256;
}
}  // namespace

int launch_gemm(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales, const void* b_q,
                const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                cudaStream_t stream) {
  const Options& opt = options();
  const int out_bytes = (out_dt == 0) ? 4 : 2;
  bool tma_store = out_bytes == 2 && (n * out_bytes) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(c) % 16 == 0);
  if (opt.gemm_tma_store == 0) tma_store = false;

  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = c;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>((n + 127) / 128);
  const int BN = pick_block_n(false, m);
  p.tiles_m = static_cast<int>((m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = tma_store ? 1 : 0;
  p.group_m = opt.gemm_group_m > 0 ? opt.gemm_group_m : 32;
  p.no_loads = opt.debug_no_loads;
  p.c_scales = nullptr;
  p.status = ctx->status;

  CUtensorMap ma, mb, mc;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, n, k, k, BN, BK, true);
  if (rc != INFEROP_OK) return rc;
  if (tma_store) {
    rc = make_tensor_map_2d(&mc, c, 2, m, n, n * 2, 128, 64, true);
    if (rc != INFEROP_OK) return rc;
  } else {
    mc = ma;  // unused by the kernel
  }
  int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (ctas > p.num_tiles) ctas = p.num_tiles;

  switch (out_dt) {
    case 0: return BN == 128 ? launch_t<float, 128>(ma, mb, mc, p, ctas, stream)
                             : launch_t<float, 256>(ma, mb, mc, p, ctas, stream);
    case 1: return BN == 128 ? launch_t<__half, 128>(ma, mb, mc, p, ctas, stream)
                             : launch_t<__half, 256>(ma, mb, mc, p, ctas, stream);
    case 2: return BN == 128 ? launch_t<__nv_bfloat16, 128>(ma, mb, mc, p, ctas, stream)
                             : launch_t<__nv_bfloat16, 256>(ma, mb, mc, p, ctas, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

namespace {
// A zeroed tile counter for one launch (see gemm_body): the context's counters in rotation, so
// that launches in flight on different streams do not share one.  A launch captured in a graph
// keeps its counter: such a graph must not run concurrently with itself.
int claim_tile_counter(DeviceCtx* ctx, cudaStream_t stream, int** out) {
  static std::atomic<unsigned> next{0};
  int* c = ctx->tile_counters + (next.fetch_add(1) % DeviceCtx::kTileCounters);
  cudaError_t e = cudaMemsetAsync(c, 0, sizeof(int), stream);
  if (e != cudaSuccess) return note_cuda_error(e);
  *out = c;
  return INFEROP_OK;
}
}  // namespace

int launch_gemm_grouped(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales,
                        const void* b_q, const void* b_scales, const int64_t* m_per_group,
                        int64_t groups, int64_t n, int64_t k, int32_t out_dt, cudaStream_t stream) {
  const Options& opt = options();
  const int out_bytes = (out_dt == 0) ? 4 : 2;
  int64_t m_total = 0;
  for (int64_t g = 0; g < groups; ++g) m_total += m_per_group[g];
  if (m_total == 0) return INFEROP_OK;
  bool tma_store = out_bytes == 2 && (n * out_bytes) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(c) % 16 == 0);
  if (opt.gemm_tma_store == 0) tma_store = false;

  // cut the groups into M-tiles; launch in chunks when the list outgrows one parameter block
  static thread_local GroupTable tab;
  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = c;
  p.m = static_cast<int>(m_total);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(n / 128);
  const int BN = pick_block_n(true, m_total);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  p.tma_store = tma_store ? 1 : 0;
  p.group_m = 32;
  p.no_loads = opt.debug_no_loads;
  p.c_scales = nullptr;
  p.status = ctx->status;

  CUtensorMap ma, mb, mc;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m_total, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, groups * n, k, k, BN, BK, true);
  if (rc != INFEROP_OK) return rc;
  if (tma_store) {
    rc = make_tensor_map_2d(&mc, c, 2, m_total, n, n * 2, 128, 64, true);
    if (rc != INFEROP_OK) return rc;
  } else {
    mc = ma;
  }
  auto flush = [&](int n_mtiles) -> int {
    if (n_mtiles == 0) return INFEROP_OK;
    p.tiles_m = n_mtiles;
    p.num_tiles = n_mtiles * p.tiles_n;
    int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
    if (ctas > p.num_tiles) ctas = p.num_tiles;
    p.sched = nullptr;
    if (opt.grouped_dynamic) {
      const int crc = claim_tile_counter(ctx, stream, &p.sched);
      if (crc != INFEROP_OK) return crc;
    }
    switch (out_dt) {
      case 0: return BN == 128 ? launch_grouped_t<float, 128>(ma, mb, mc, p, tab, ctas, stream)
                               : launch_grouped_t<float, 256>(ma, mb, mc, p, tab, ctas, stream);
      case 1: return BN == 128 ? launch_grouped_t<__half, 128>(ma, mb, mc, p, tab, ctas, stream)
                               : launch_grouped_t<__half, 256>(ma, mb, mc, p, tab, ctas, stream);
      case 2: return BN == 128 ? launch_grouped_t<__nv_bfloat16, 128>(ma, mb, mc, p, tab, ctas, stream)
                               : launch_grouped_t<__nv_bfloat16, 256>(ma, mb, mc, p, tab, ctas, stream);
      default: return INFEROP_ERR_DTYPE;
    }
  };
  int count = 0;
  int64_t row = 0;
  for (int64_t g = 0; g < groups; ++g) {
    for (int64_t r = 0; r < m_per_group[g]; r += BM) {
      if (count == kMaxGroupTiles) {
        rc = flush(count);
        if (rc != INFEROP_OK) return rc;
        count = 0;
      }
      const int64_t rows = (m_per_group[g] - r) < BM ? (m_per_group[g] - r) : BM;
      tab.row0[count] = static_cast<int>(row + r);
      tab.meta[count] = static_cast<int>((g << 8) | (rows - 1));
      ++count;
    }
    row += m_per_group[g];
  }
  return flush(count);
}

// Shared by the all-gather launch and the strided-output launch: this call's [m, n] result goes
// to columns [col_offset, col_offset + n) of `count` row-major two-byte buffers of n_total
// columns each (dsts in the order the stores are issued).
static int launch_gemm_to_wide(DeviceCtx* ctx, void* const* dsts, int count, int64_t n_total, int64_t col_offset,
                               const void* a_q, const void* a_scales, const void* b_q, const void* b_scales,
                               int64_t m, int64_t n, int64_t k, int32_t out_dt, cudaStream_t stream) {
  const Options& opt = options();
  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = nullptr;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(n / 128);
  constexpr int BN = 256;
  p.tiles_m = static_cast<int>((m + BM - 1) / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = 1;
  p.group_m = opt.gemm_group_m > 0 ? opt.gemm_group_m : 32;
  p.no_loads = opt.debug_no_loads;
  p.c_scales = nullptr;
  p.status = ctx->status;

  CUtensorMap ma, mb;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, n, k, k, BN, BK, true);
  if (rc != INFEROP_OK) return rc;
  static thread_local PeerMaps peers;
  peers.count = count;
  peers.col_offset = static_cast<int>(col_offset);
  for (int i = 0; i < count; ++i) {
    rc = make_tensor_map_2d(&peers.map[i], dsts[i], 2, m, n_total, n_total * 2, 128, 64, true);
    if (rc != INFEROP_OK) return rc;
  }
  for (int i = count; i < kMaxPeers; ++i) peers.map[i] = peers.map[0];
  int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (ctas > p.num_tiles) ctas = p.num_tiles;
  return out_dt == 1 ? launch_gather_t<__half>(ma, mb, p, peers, ctas, stream)
                     : launch_gather_t<__nv_bfloat16>(ma, mb, p, peers, ctas, stream);
}

int launch_gemm_allgather(DeviceCtx* ctx, void* const* c_peers, int32_t n_peers, int32_t rank,
                          const void* a_q, const void* a_scales, const void* b_q,
                          const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                          cudaStream_t stream) {
  if (out_dt != 1 && out_dt != 2) return INFEROP_ERR_DTYPE;
  if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return INFEROP_ERR_SHAPE;
  // a store box is 64 columns wide and must not reach into the next rank's columns; the weight
  // scales of a shard are whole 128-row blocks
  if (n % 128 != 0) return INFEROP_ERR_SHAPE;
  const int64_t n_total = n * n_peers;
  if (n_total > 0x7FFFFFFF) return INFEROP_ERR_LIMIT;
  void* dsts[kMaxPeers];
  for (int i = 0; i < n_peers; ++i) {
    dsts[i] = c_peers[(rank + 1 + i) % n_peers];   // own buffer last
    if (dsts[i] == nullptr || reinterpret_cast<uintptr_t>(dsts[i]) % 16 != 0) return INFEROP_ERR_POINTER;
  }
  return launch_gemm_to_wide(ctx, dsts, n_peers, n_total, static_cast<int64_t>(rank) * n, a_q, a_scales, b_q,
                             b_scales, m, n, k, out_dt, stream);
}

int launch_gemm_into(DeviceCtx* ctx, void* c_base, int64_t ldc, int64_t col0, const void* a_q,
                     const void* a_scales, const void* b_q, const void* b_scales, int64_t m, int64_t n, int64_t k,
                     int32_t out_dt, cudaStream_t stream) {
  if (out_dt != 1 && out_dt != 2) return INFEROP_ERR_DTYPE;
  if (n % 128 != 0 || col0 % 8 != 0 || ldc % 8 != 0 || col0 < 0 || col0 + n > ldc) return INFEROP_ERR_SHAPE;
  if (ldc > 0x7FFFFFFF) return INFEROP_ERR_LIMIT;
  if (c_base == nullptr || reinterpret_cast<uintptr_t>(c_base) % 16 != 0) return INFEROP_ERR_POINTER;
  void* dsts[1] = {c_base};
  return launch_gemm_to_wide(ctx, dsts, 1, ldc, col0, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, stream);
}

int launch_gemm_grouped_dev(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales,
                            const void* b_q, const void* b_scales, const int32_t* tile_row0,
                            const int32_t* tile_meta, const int32_t* num_mtiles, int64_t max_mtiles,
                            int64_t m_total, int64_t groups, int64_t n, int64_t k, int32_t out_dt,
                            cudaStream_t stream) {
  const Options& opt = options();
  const int out_bytes = (out_dt == 0) ? 4 : 2;
  bool tma_store = out_bytes == 2 && (n * out_bytes) % 16 == 0 &&
                   (reinterpret_cast<uintptr_t>(c) % 16 == 0);
  if (opt.gemm_tma_store == 0) tma_store = false;
  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = c;
  p.m = static_cast<int>(m_total);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(n / 128);
  const int BN = pick_block_n(true, m_total);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  p.tiles_m = static_cast<int>(max_mtiles);   // upper bound; the real count is read on the device
  const int64_t tiles = max_mtiles * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = tma_store ? 1 : 0;
  p.group_m = 32;
  p.no_loads = opt.debug_no_loads;
  p.c_scales = nullptr;
  p.status = ctx->status;

  p.rep = (opt.grouped_rep && BN == 256) ? 1 : 0;
  CUtensorMap ma, mb, mc, ma32;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m_total, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&ma32, a_q, 1, m_total, k, k, 32, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, groups * n, k, k, BN, BK, true);
  if (rc != INFEROP_OK) return rc;
  if (tma_store) {
    rc = make_tensor_map_2d(&mc, c, 2, m_total, n, n * 2, 128, 64, true);
    if (rc != INFEROP_OK) return rc;
  } else {
    mc = ma;
  }
  int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (ctas > p.num_tiles) ctas = p.num_tiles;
  if (opt.grouped_dynamic) {
    rc = claim_tile_counter(ctx, stream, &p.sched);
    if (rc != INFEROP_OK) return rc;
  }
  switch (out_dt) {
    case 0: return BN == 128 ? launch_grouped_dev_t<float, 128>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream)
                             : launch_grouped_dev_t<float, 256>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream);
    case 1: return BN == 128 ? launch_grouped_dev_t<__half, 128>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream)
                             : launch_grouped_dev_t<__half, 256>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream);
    case 2: return BN == 128 ? launch_grouped_dev_t<__nv_bfloat16, 128>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream)
                             : launch_grouped_dev_t<__nv_bfloat16, 256>(ma, mb, mc, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream);
    default: return INFEROP_ERR_DTYPE;
  }
}

int launch_gemm_swiglu(DeviceCtx* ctx, void* q, float* q_scales, const void* a_q, const void* a_scales,
                       const void* b_q, const void* b_scales, const int32_t* tile_row0,
                       const int32_t* tile_meta, const int32_t* num_mtiles, int64_t max_mtiles,
                       int64_t m_total, int64_t groups, int64_t inter, int64_t k, int32_t mid_dt,
                       cudaStream_t stream) {
  const Options& opt = options();
  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = q;
  p.c_scales = q_scales;
  p.m = static_cast<int>(m_total);
  p.n = static_cast<int>(2 * inter);          // weight rows per group: gate rows, then up rows
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>(2 * inter / 128);
  p.tiles_n = static_cast<int>(inter / 128);
  p.tiles_m = static_cast<int>(max_mtiles);
  const int64_t tiles = max_mtiles * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = 0;
  p.group_m = 32;
  p.no_loads = opt.debug_no_loads;
  p.status = ctx->status;
  p.rep = opt.grouped_rep ? 1 : 0;
  CUtensorMap ma, mb, ma32;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m_total, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&ma32, a_q, 1, m_total, k, k, 32, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, groups * 2 * inter, k, k, 128, BK, true);
  if (rc != INFEROP_OK) return rc;
  int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (ctas > p.num_tiles) ctas = p.num_tiles;
  if (opt.grouped_dynamic) {
    rc = claim_tile_counter(ctx, stream, &p.sched);
    if (rc != INFEROP_OK) return rc;
  }
  return mid_dt == 1 ? launch_swiglu_t<__half>(ma, mb, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream)
                     : launch_swiglu_t<__nv_bfloat16>(ma, mb, ma32, p, tile_row0, tile_meta, num_mtiles, ctas, stream);
}

int launch_gemm_scatter(DeviceCtx* ctx, void* const* slot_peers, int32_t n_peers, int32_t rank,
                        const void* a_q, const void* a_scales, const void* b_q, const void* b_scales,
                        int64_t m, int64_t n, int64_t k, cudaStream_t stream) {
  const Options& opt = options();
  if (n_peers < 1 || n_peers > kMaxPeers || rank < 0 || rank >= n_peers) return INFEROP_ERR_SHAPE;
  // a tile's 128 rows must belong to one owner; a row of fp32 must be a whole number of 16 bytes
  if (m % (static_cast<int64_t>(BM) * n_peers) != 0 || n % 4 != 0) return INFEROP_ERR_SHAPE;
  for (int d = 0; d < n_peers; ++d) {
    if (slot_peers[d] == nullptr || reinterpret_cast<uintptr_t>(slot_peers[d]) % 16 != 0) return INFEROP_ERR_POINTER;
  }
  GemmParams p;
  p.a_scales = static_cast<const float*>(a_scales);
  p.b_scales = static_cast<const float*>(b_scales);
  p.c = nullptr;
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.kb = static_cast<int>(k / 128);
  p.nb = static_cast<int>((n + 127) / 128);
  constexpr int BN = 256;
  p.tiles_m = static_cast<int>(m / BM);
  p.tiles_n = static_cast<int>((n + BN - 1) / BN);
  const int64_t tiles = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (tiles > 0x7FFFFFFF || tiles * p.kb > 0x7FFFFFFFLL) return INFEROP_ERR_LIMIT;
  p.num_tiles = static_cast<int>(tiles);
  p.tma_store = 1;
  p.group_m = opt.gemm_group_m > 0 ? opt.gemm_group_m : 32;
  p.no_loads = opt.debug_no_loads;
  p.c_scales = nullptr;
  p.status = ctx->status;

  CUtensorMap ma, mb;
  int rc = make_tensor_map_2d(&ma, a_q, 1, m, k, k, BM, BK, true);
  if (rc != INFEROP_OK) return rc;
  rc = make_tensor_map_2d(&mb, b_q, 1, n, k, k, BN, BK, true);
  if (rc != INFEROP_OK) return rc;
  static thread_local PeerMaps peers;
  peers.count = n_peers;
  peers.col_offset = 0;
  peers.rows_per_owner = static_cast<int>(m / n_peers);
  peers.rank = rank;
  for (int d = 0; d < n_peers; ++d) {
    rc = make_tensor_map_2d(&peers.map[d], slot_peers[d], 4, m, n, n * 4, 128, 32, true);
    if (rc != INFEROP_OK) return rc;
  }
  for (int i = n_peers; i < kMaxPeers; ++i) peers.map[i] = peers.map[0];
  int ctas = opt.gemm_ctas > 0 ? opt.gemm_ctas : ctx->sm_count;
  if (ctas > p.num_tiles) ctas = p.num_tiles;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w8a8_scatter_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return note_cuda_error(e);
    attr_done[dev] = true;
  }
  w8a8_scatter_gemm_kernel<<<ctas, kThreads, kSmemBytes, stream>>>(ma, mb, p, peers);
  return check_launch();
}

}  // namespace ib200
