// Declarations shared by the translation units of libinferop_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "inferop_b200.h"
#include "ptx.cuh"

namespace ib200 {

// Records a failed CUDA call for inferop_last_cuda_error() and maps it to a status.
int note_cuda_error(cudaError_t e);
// cudaGetLastError() after a launch -> INFEROP_OK / INFEROP_ERR_CUDA.
int check_launch();

// Per-device facts and library-owned device objects, created on first use.
struct DeviceCtx {
  int ordinal = -1;
  int sm_version = 0;
  int sm_count = 0;
  DeviceStatus* status = nullptr;  // device memory, zero-initialised
  // Tile counters of the grouped GEMM launches that claim their tiles on the device: kTileCounters
  // ints behind the status record, one per launch in rotation (zeroed on the stream before the launch).
  static constexpr int kTileCounters = 64;
  int* tile_counters = nullptr;
  // Scratch of the small-M GEMM path, one set per stream that has used it (launches on one
  // stream run in order and may share a set; launches on different streams may overlap).
  static constexpr int kMaxStreams = 64;
  int n_scratch = 0;
  cudaStream_t scratch_stream[kMaxStreams] = {};
  float* scratch_ws[kMaxStreams] = {};
  int* scratch_counters[kMaxStreams] = {};
  // Quantised activations of the one-call quantise + GEMM entry point for large M, one pair of
  // buffers per stream, grown on demand (never shrunk).
  int n_qscratch = 0;
  cudaStream_t qscratch_stream[kMaxStreams] = {};
  void* qscratch_q[kMaxStreams] = {};
  void* qscratch_s[kMaxStreams] = {};
  size_t qscratch_q_bytes[kMaxStreams] = {};
  size_t qscratch_s_bytes[kMaxStreams] = {};
};
// Context of the current device (nullptr + *err set when there is none / wrong arch).
DeviceCtx* current_ctx(int* err);

struct Options {
  int gemm_block_n = 0;    // 0 auto, 128, 256
  int gemm_tma_store = -1; // -1 auto, 0 off, 1 on
  int gemm_ctas = 0;       // 0 = one per SM
  int gemm_group_m = 0;    // M-tiles per rasterisation band of the large-tile kernel (0 = default 32)
  int decode_pdl = 1;      // small-M kernel: launch with programmatic stream serialisation
  int decode_deal = 1;     // small-M kernel: 1 whole tiles / equal K parts per CTA (default); 0 (tile, K block) units dealt evenly
  int decode_splits = 0;   // with decode_deal 1: 0 auto, else K parts per tile (capped by SMs / tiles)
  int gemm_path = 0;       // 0 auto, 1 always the large-tile kernel, 2 small-M kernel whenever M <= 128
  int gemm_pair = -1;      // large-tile GEMM on CTA pairs (256 x 256 tiles): -1 auto, 0 never, 1 always
  int pdl_trigger = 1;     // small-M GEMM: a dependent launch (the next step's quantiser) may start under its tail
  int fused_prologue = 0;  // one-call quantise + GEMM, M <= 32: 1 = quantise inside the small-M kernel (one launch; slower than the chained pair except at M = 1)
  int attn_heads_per_cta = 0;  // paged attention: query heads of a KV head per CTA (0 = auto: 4, 2 or 1)
  int attn_splits = 0;     // paged attention: token ranges per sequence (0 = auto)
  int grouped_rep = 1;     // grouped GEMMs with a device tile list: M-tiles of at most 32 rows in the replicated form
  int grouped_dynamic = 1; // grouped GEMMs with a device tile list: tiles claimed from a device counter (0: dealt round-robin)
  int align_ctas = 0;      // moe_align: CTAs of its cluster (0 = auto: one per 4096 pairs, at most 8)
  int quant_pdl = 1;       // quantiser: launch with programmatic stream serialisation
  int gemm_pdl = 1;        // pair kernel: launch with programmatic stream serialisation
  int debug_no_loads = 0;  // test hook: the TMA producers of the GEMM kernels issue no load (every wait runs out)
};
Options& options();
bool decode_scratch(DeviceCtx* ctx, cudaStream_t stream, float** ws, int** counters);
// Buffers of at least q_bytes / s_bytes for `stream` (INFEROP_OK, or ERR_LIMIT / ERR_CUDA).
int quant_scratch(DeviceCtx* ctx, cudaStream_t stream, size_t q_bytes, size_t s_bytes, void** q, void** s);

// quant.cu
int launch_quant(void* q, void* scales, const void* x, int32_t dt, int64_t rows, int64_t cols,
                 int32_t gs, cudaStream_t stream, int sms);
int launch_dequant(void* x, int32_t dt, const void* q, const void* scales, int64_t rows,
                   int64_t cols, int32_t gs, cudaStream_t stream, int sms);

int run_cvt_selftest(uint64_t lo, uint64_t hi, uint64_t* out2, int sms);
int run_div_selftest(int is_bf16, uint64_t* out3, int sms);

// gemm_sm100.cu
int launch_gemm(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales, const void* b_q,
                const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                cudaStream_t stream);

// gemm_pair_sm100.cu : the same GEMM on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles)
bool use_pair_kernel(int64_t m);
int launch_gemm_pair(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales, const void* b_q,
                     const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                     cudaStream_t stream);

// Grouped launch: group g has m_per_group[g] (host array) rows of A / C, stacked in group
// order; b_q is [groups][n][k], b_scales [groups][n/128][k/128].
int launch_gemm_grouped(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales,
                        const void* b_q, const void* b_scales, const int64_t* m_per_group,
                        int64_t groups, int64_t n, int64_t k, int32_t out_dt, cudaStream_t stream);

// All-gather launch (column-parallel sharding): this rank's [m, n] result goes to columns
// [rank * n, (rank + 1) * n) of the [m, n * n_peers] two-byte row-major buffer of every peer;
// c_peers (host array) holds the n_peers base addresses as mapped in this process.
int launch_gemm_allgather(DeviceCtx* ctx, void* const* c_peers, int32_t n_peers, int32_t rank,
                          const void* a_q, const void* a_scales, const void* b_q,
                          const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt,
                          cudaStream_t stream);

// Strided-output launch: the [m, n] result goes to columns [col0, col0 + n) of a row-major
// two-byte buffer with ldc columns (n % 128 == 0, col0 and ldc multiples of 8).
int launch_gemm_into(DeviceCtx* ctx, void* c_base, int64_t ldc, int64_t col0, const void* a_q,
                     const void* a_scales, const void* b_q, const void* b_scales, int64_t m, int64_t n, int64_t k,
                     int32_t out_dt, cudaStream_t stream);

// Grouped launch whose M-tile list and its length live in device memory (written by moe_align);
// max_mtiles bounds the list, m_total is the number of rows of a_q / c.
int launch_gemm_grouped_dev(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales,
                            const void* b_q, const void* b_scales, const int32_t* tile_row0,
                            const int32_t* tile_meta, const int32_t* num_mtiles, int64_t max_mtiles,
                            int64_t m_total, int64_t groups, int64_t n, int64_t k, int32_t out_dt,
                            cudaStream_t stream);

// Grouped launch of a gate_up projection whose epilogue applies SwiGLU and quantises the result
// per 1 x 128 group: q [m_total, inter] E4M3 + q_scales [m_total, inter / 128]; b_q is
// [groups][2 * inter][k], gate rows first.
int launch_gemm_swiglu(DeviceCtx* ctx, void* q, float* q_scales, const void* a_q, const void* a_scales,
                       const void* b_q, const void* b_scales, const int32_t* tile_row0,
                       const int32_t* tile_meta, const int32_t* num_mtiles, int64_t max_mtiles,
                       int64_t m_total, int64_t groups, int64_t inter, int64_t k, int32_t mid_dt,
                       cudaStream_t stream);

// Scatter launch (row-parallel sharding): fp32 partial results of this rank's K shard, stored
// tile by tile into slot `rank` of the rank that owns the rows; slot_peers[d] (host array) is the
// base of rank d's [n_peers][m / n_peers][n] fp32 slots as mapped in this process.
int launch_gemm_scatter(DeviceCtx* ctx, void* const* slot_peers, int32_t n_peers, int32_t rank,
                        const void* a_q, const void* a_scales, const void* b_q, const void* b_scales,
                        int64_t m, int64_t n, int64_t k, cudaStream_t stream);
// reduce.cu : out[i] = sum over ranks (in order) of slots[r][i], rounded once
int launch_reduce_slots(void* out, int32_t out_dt, const void* slots, int32_t ranks, int64_t elems,
                        cudaStream_t stream, int sms);

// moe.cu
int launch_topk_softmax(int32_t* ids, float* weights, const float* logits, int32_t tokens,
                        int32_t experts, int32_t topk, int32_t renorm, cudaStream_t stream);
// norm_rope.cu : RMSNorm (residual == nullptr) or residual += in followed by RMSNorm of the sum,
// and the NeoX rotary embedding in place.
int launch_rmsnorm(void* out, void* residual, const void* in, const void* weight, int32_t dt, int64_t rows,
                   int64_t cols, float eps, cudaStream_t stream);
// the same followed by the 1 x 128 FP8 quantisation of the (16-bit) result, in one pass
int launch_rmsnorm_quant(void* q, void* scales, void* residual, const void* in, const void* weight, int32_t dt,
                         int64_t rows, int64_t cols, float eps, cudaStream_t stream);
int launch_rope_neox(void* qkv, const int64_t* positions, int32_t dt, int64_t tokens, int heads, int head_dim,
                     int rotary_dim, float base, float yarn, cudaStream_t stream);
// attention.cu : paged attention decode.  `splits` token ranges per sequence (paged_attn_splits),
// `workspace` of paged_attn_workspace_bytes for the partial states when splits > 1.
int paged_attn_splits(int sm_count, int batch, int num_heads, int num_kv_heads, int block_size, int max_blocks_per_seq);
size_t paged_attn_workspace_bytes(int splits, int batch, int num_heads, int head_dim);
int launch_paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                             const int32_t* block_tables, const int32_t* seq_lens, int32_t dt, int batch,
                             int num_heads, int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq,
                             float scale, int splits, float* workspace, cudaStream_t stream);
int launch_silu_and_mul(void* out, const void* gate_up, int32_t dt, int64_t rows, int64_t d,
                        cudaStream_t stream, int sms);
int launch_silu_and_mul_quant(void* q, void* scales, const void* gate_up, int32_t dt, int64_t rows,
                              int64_t d, cudaStream_t stream, int sms);
int64_t moe_max_mtiles(int64_t pairs, int64_t experts);
int launch_moe_align(const int32_t* ids, int64_t tokens, int32_t topk, int32_t experts, int32_t* counts,
                     int32_t* offsets, int32_t* pos, int32_t* src_token, int32_t* tile_row0,
                     int32_t* tile_meta, int32_t* num_mtiles, cudaStream_t stream);
int launch_moe_scatter_quant(void* q, void* scales, const void* x, int32_t dt, const int32_t* pos,
                             int64_t tokens, int64_t cols, int32_t topk, cudaStream_t stream, int sms);
int launch_permute_rows(void* dst, const void* src, const int32_t* perm, int64_t rows, int64_t row_bytes,
                        int32_t gather, cudaStream_t stream, int sms);
int launch_moe_combine(void* out, const void* y, const float* w, const int32_t* pos, int32_t dt,
                       int64_t tokens, int64_t hidden, int32_t topk, cudaStream_t stream, int sms);

// gemm_decode_sm100.cu : small-M path (M <= kDecodeMaxM).  workspace holds
// decode_workspace_bytes(sm_count) bytes, counters kDecodeMaxTiles zeroed ints; both are
// owned by the caller of launch_gemm_decode and must not be shared by launches that can
// overlap on the device.
constexpr int kDecodeMaxM = 128;
constexpr int kDecodeMaxTiles = 1 << 16;
size_t decode_workspace_bytes(int ctas);
// clear_counters > 0: that many counters are zeroed on the stream after the call's last check.
int launch_gemm_decode(DeviceCtx* ctx, float* workspace, int* counters, void* c, const void* a_q,
                       const void* a_scales, const void* b_q, const void* b_scales, int64_t m,
                       int64_t n, int64_t k, int32_t out_dt, cudaStream_t stream, int clear_counters = 0);
// Bounded-wait record of the allocation-free entry point on the current device (if it has run).
int fixed_scratch_status(DeviceStatus* out, bool reset, bool* used);
// Context of the current device if one has been created already; never allocates.
DeviceCtx* peek_ctx();

// The same with the [m, n] result written to columns [col0, col0 + n) of n_dst (<= 8) row-major
// buffers of row pitch ldc elements (host array `dst`; peer-mapped addresses allowed).
int launch_gemm_decode_to(DeviceCtx* ctx, float* workspace, int* counters, void* const* dst, int n_dst,
                          int64_t ldc, int64_t col0, const void* a_q, const void* a_scales,
                          const void* b_q, const void* b_scales, int64_t m, int64_t n, int64_t k,
                          int32_t out_dt, cudaStream_t stream, int clear_counters = 0);

// Fused prologue: `a` holds unquantised activations (a_dt 1 = fp16, 2 = bf16), M <= kFusedMaxM.
constexpr int kFusedMaxM = 32;
int launch_gemm_decode_fused(DeviceCtx* ctx, float* workspace, int* counters, void* c, const void* a,
                             int32_t a_dt, const void* b_q, const void* b_scales, int64_t m, int64_t n,
                             int64_t k, int32_t out_dt, cudaStream_t stream);

// tensormap.cu : cuTensorMapEncodeTiled through the runtime's driver entry point.
// 2-D row-major tensor [rows, cols] of elem_bytes-wide elements with row pitch
// pitch_bytes; box = [box_rows, box_cols]; 128-byte swizzle when swizzle128.
int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows,
                       uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                       bool swizzle128);

}  // namespace ib200
