// C entry points over the reference's own CUDA kernels (kernels/quant.cu, kernels/gemm/w8a8_block_fp8.cu,
// kernels/rmsnorm.cu, kernels/rope.cu, kernels/attention/paged_attn_decode.cu), compiled unmodified from
// the reference tree for sm_100.
// TEST / BENCHMARK INFRASTRUCTURE ONLY: the secondary GPU baseline of bench.py (the reference's
// CUDA-core kernels timed on the same B200) and a cross-check of results.  Nothing in the
// shipped package links or loads this.
#include <stdint.h>

#include "internal.h"   // the reference's kernels/internal.h (dispatch entries per translation unit)

extern "C" {

__attribute__((visibility("default"))) void refcuda_quant_fp8_per_token_group(
    void* q, void* scales, const void* x, int32_t dt, int64_t rows, int64_t cols, int32_t group_size, void* stream) {
  inferop::kernels::quant_fp8_per_token_group_impl(q, scales, x, static_cast<inferop::dtype>(dt), rows, cols,
                                                   group_size, stream);
}

__attribute__((visibility("default"))) void refcuda_w8a8_block_fp8_gemm(
    void* c, const void* a_q, const void* a_scales, const void* b_q, const void* b_scales, int64_t m, int64_t n,
    int64_t k, int32_t group_size, int32_t block_n, int32_t out_dt, void* stream) {
  inferop::kernels::w8a8_block_fp8_gemm_impl(c, a_q, a_scales, b_q, b_scales, m, n, k, group_size, block_n,
                                             static_cast<inferop::dtype>(out_dt), stream);
}

__attribute__((visibility("default"))) void refcuda_rmsnorm(void* out, const void* in, const void* weight, int32_t dt,
                                                            int64_t rows, int64_t cols, float eps, void* stream) {
  inferop::kernels::rmsnorm_impl(out, in, weight, static_cast<inferop::dtype>(dt), rows, cols, eps, stream);
}

__attribute__((visibility("default"))) void refcuda_rope_neox(void* qkv, const int64_t* positions, int32_t dt,
                                                              int64_t tokens, int32_t heads, int32_t head_dim,
                                                              int32_t rotary_dim, float base, float yarn, void* stream) {
  inferop::kernels::rope_neox_impl(qkv, positions, static_cast<inferop::dtype>(dt), tokens, heads, head_dim, rotary_dim,
                                   base, yarn, stream);
}

__attribute__((visibility("default"))) void refcuda_paged_attn_decode(
    void* out, const void* q, const void* k_cache, const void* v_cache, const int32_t* block_tables,
    const int32_t* seq_lens, int32_t dt, int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
    int32_t block_size, int32_t max_blocks_per_seq, float scale, void* stream) {
  inferop::kernels::paged_attn_decode_impl(out, q, k_cache, v_cache, block_tables, seq_lens,
                                           static_cast<inferop::dtype>(dt), batch, num_heads, num_kv_heads, head_dim,
                                           block_size, max_blocks_per_seq, scale, stream);
}

}  // extern "C"
