// inferop (B200 build): C++ host API for the blockwise-FP8 W8A8 path.
//
// Drop-in for the part of the reference's include/inferop/ops.h that this
// library implements: identical names, namespaces, argument order, defaults
// and error behaviour (reference: ops.h:19-25 device queries, :54-55 SwiGLU,
// :64-70 quant / dequant, :81-84 GEMM, :108-110 MoE routing).  Tensor arguments are caller-owned device pointers on
// the current device; `stream` is a cudaStream_t passed as void* (nullptr = the
// default stream); calls enqueue work and return without synchronising.
//
// This build targets NVIDIA B200 (sm_100a) only.  There is no fallback: on any
// other device, or without a device, the operators print one line to stderr
// and do nothing, and has_cuda() tells the caller beforehand.
//
// The functions are thin wrappers over the C entry points in inferop_b200.h,
// which return status codes instead of failing silently.
#pragma once

#include "inferop/common.h"

#if defined(__GNUC__)
#define INFEROP_EXPORT __attribute__((visibility("default")))
#else
#define INFEROP_EXPORT
#endif

namespace inferop {

INFEROP_EXPORT bool has_cuda();                          // a usable device is visible
INFEROP_EXPORT int device_count();                       // number of visible CUDA devices
INFEROP_EXPORT const char* device_name(int ordinal = 0); // "-" when out of range
INFEROP_EXPORT int device_sm_version(int ordinal = 0);   // major*10+minor, -1 when out of range

// x [rows, cols] (fp32 / fp16 / bf16)  ->  q [rows, cols] E4M3 bytes and
// scales [rows, cols/group_size] fp32, one scale per run of group_size
// elements of a row:  scale = absmax * fl(1/448) (1 for an all-zero group),
// q = e4m3_rn_sat(x / scale).  Bytes and scales are bit-identical to the
// reference's CPU implementation.  Invalid shapes (non-positive sizes,
// cols % group_size != 0) and other dtypes are a silent no-op.
INFEROP_EXPORT void quant_fp8_per_token_group(void* q, void* scales, const void* x, dtype dt, int64_t rows,
                               int64_t cols, int group_size = 128, void* stream = nullptr);

// x = decode(q) * scale, written as dt.
INFEROP_EXPORT void dequant_fp8_per_token_group(void* x, dtype dt, const void* q, const void* scales,
                                 int64_t rows, int64_t cols, int group_size = 128,
                                 void* stream = nullptr);

// C[m, n] = sum_k  A_q[m,k] * sa[m, k/128]  *  B_q[n,k] * sb[n/128, k/128]
//   a_q [M, K] E4M3, a_scales [M, K/128] fp32
//   b_q [N, K] E4M3, b_scales [ceil(N/128), K/128] fp32
//   c   [M, N] in out_dt (fp32 / fp16 / bf16), fp32 accumulation
// Requires group_size == 128, block_n == 128, K % 128 == 0, M > 0, N > 0;
// anything else prints one "[inferop]" line to stderr and does nothing.
// M and N may be ragged.
INFEROP_EXPORT void w8a8_block_fp8_gemm(void* c, const void* a_q, const void* a_scales, const void* b_q,
                         const void* b_scales, int64_t m, int64_t n, int64_t k,
                         int group_size = 128, int block_n = 128, dtype out_dt = dtype::bf16,
                         void* stream = nullptr);

// out[r, c] = weight[c] * in[r, c] / sqrt(mean(in[r, :]^2) + eps); in / out [rows, cols], weight [cols] in dt.
INFEROP_EXPORT void rmsnorm(void* out, const void* in, const void* weight, dtype dt, int64_t rows,
             int64_t cols, float eps = 1e-6f, void* stream = nullptr);

// residual[r, c] += x[r, c] (in place);  out = rmsnorm(residual).
INFEROP_EXPORT void fused_add_rmsnorm(void* residual, void* out, const void* x, const void* weight,
                       dtype dt, int64_t rows, int64_t cols, float eps = 1e-6f,
                       void* stream = nullptr);

// Rotary position embedding (GPT-NeoX style, half-dim rotation, in place) on qkv
// [tokens, heads, head_dim]; positions int64 [tokens]; rotary_dim <= head_dim, even;
// theta = position * base^(-2 i / rotary_dim) * yarn_factor.  A bad rotary_dim is a silent no-op.
INFEROP_EXPORT void rope_neox(void* qkv, const int64_t* positions, dtype dt, int64_t tokens, int heads,
               int head_dim, int rotary_dim, float base = 10000.0f, float yarn_factor = 1.0f,
               void* stream = nullptr);

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, d + i];  gate_up [tokens, 2d], out [tokens, d] in dt.
INFEROP_EXPORT void silu_and_mul(void* out, const void* gate_up, dtype dt, int64_t tokens, int64_t d,
                  void* stream = nullptr);

// Paged attention (single-token decode, GQA):
//   q / out [batch, num_heads, head_dim], k_cache / v_cache [num_blocks, block_size, num_kv_heads, head_dim] (dt),
//   block_tables int32 [batch, max_blocks_per_seq], seq_lens int32 [batch].
// head_dim in {64, 128, 256}; num_heads % num_kv_heads == 0; anything else is a silent no-op.
INFEROP_EXPORT void paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                       const int32_t* block_tables, const int32_t* seq_lens, dtype dt,
                       int batch, int num_heads, int num_kv_heads, int head_dim,
                       int block_size, int max_blocks_per_seq, float scale,
                       void* stream = nullptr);

// MoE routing: softmax over logits [tokens, num_experts] (fp32) + top-k.
//   topk_weights fp32 [tokens, topk] (softmax probability, renormalised over the k when asked)
//   topk_ids     int32 [tokens, topk]; equal probabilities: the lower expert index first
// num_experts <= 1024, topk <= num_experts; anything else is a silent no-op.
INFEROP_EXPORT void topk_softmax(int32_t* topk_ids, void* topk_weights, const void* logits, int tokens,
                  int num_experts, int topk, bool renormalize = true, void* stream = nullptr);

}  // namespace inferop
