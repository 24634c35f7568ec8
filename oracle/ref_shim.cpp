// C entry points over the reference's own CPU golden code.  TEST INFRASTRUCTURE ONLY.
//
// This translation unit is compiled together with the reference project's
// reference/reference.cpp (taken from the reference tree where it lies, never
// copied into this repository) into oracle/_ref/libinferop_ref.so.  It adds
// nothing numerical: each function forwards to inferop::ref / inferop::fp8 /
// inferop::host_convert so that Python can call the unmodified reference and
// compare the in-tree oracle with it.  The *_mt variants run the same
// reference function on disjoint row slices from several host threads; that is
// the "all host cores" CPU baseline the benchmark reports.
#include <cstdint>
#include <thread>
#include <vector>

#include "reference/reference.h"

namespace r = inferop::ref;

extern "C" {

uint8_t ref_f32_to_e4m3(float f) { return inferop::fp8::float_to_e4m3_rn_sat(f); }
float ref_e4m3_to_f32(uint8_t b) { return inferop::fp8::e4m3_to_float(b); }
uint16_t ref_f32_to_bf16(float f) { return inferop::host_convert::float_to_bf16_rn(f); }
float ref_bf16_to_f32(uint16_t h) { return inferop::host_convert::bf16_to_float(h); }

void ref_e4m3_encode_array(uint8_t* out, const float* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = inferop::fp8::float_to_e4m3_rn_sat(in[i]);
}

void ref_quant_fp8_per_token_group(uint8_t* q, float* scales, const float* x, int64_t rows,
                                   int64_t cols, int gs) {
  r::quant_fp8_per_token_group(q, scales, x, rows, cols, gs);
}

void ref_dequant_fp8_per_token_group(float* x, const uint8_t* q, const float* scales, int64_t rows,
                                     int64_t cols, int gs) {
  r::dequant_fp8_per_token_group(x, q, scales, rows, cols, gs);
}

void ref_w8a8_block_fp8_gemm(float* c, const uint8_t* aq, const float* as, const uint8_t* bq,
                             const float* bs, int64_t m, int64_t n, int64_t k, int gs, int bn) {
  r::w8a8_block_fp8_gemm(c, aq, as, bq, bs, m, n, k, gs, bn);
}

void ref_topk_softmax(int32_t* ids, float* w, const float* logits, int64_t tokens, int experts,
                      int topk, int renorm) {
  r::topk_softmax(ids, w, logits, tokens, experts, topk, renorm != 0);
}

void ref_rmsnorm(float* out, const float* in, const float* weight, int64_t rows, int64_t cols, float eps) {
  r::rmsnorm(out, in, weight, rows, cols, eps);
}
void ref_fused_add_rmsnorm(float* residual, float* out, const float* x, const float* weight, int64_t rows,
                           int64_t cols, float eps) {
  r::fused_add_rmsnorm(residual, out, x, weight, rows, cols, eps);
}
void ref_rope_neox(float* qkv, const int64_t* positions, int64_t tokens, int heads, int head_dim, int rotary_dim,
                   float base, float yarn_factor) {
  r::rope_neox(qkv, positions, tokens, heads, head_dim, rotary_dim, base, yarn_factor);
}
void ref_paged_attn_decode(float* out, const float* q, const float* k_cache, const float* v_cache,
                           const int32_t* block_tables, const int32_t* seq_lens, int batch, int num_heads,
                           int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq, float scale) {
  r::paged_attn_decode(out, q, k_cache, v_cache, block_tables, seq_lens, batch, num_heads, num_kv_heads, head_dim,
                       block_size, max_blocks_per_seq, scale);
}
void ref_silu_and_mul(float* out, const float* gate_up, int64_t tokens, int64_t d) {
  r::silu_and_mul(out, gate_up, tokens, d);
}

// Row-sliced multi-thread drivers.  Rows of A (and of x for quant) are
// independent in both operators, so slice t handles rows [t*m/T, (t+1)*m/T).
int ref_w8a8_block_fp8_gemm_mt(float* c, const uint8_t* aq, const float* as, const uint8_t* bq,
                               const float* bs, int64_t m, int64_t n, int64_t k, int gs, int bn,
                               int threads) {
  if (threads <= 0) threads = int(std::thread::hardware_concurrency());
  if (threads <= 0) threads = 1;
  if (threads > m) threads = int(m);
  std::vector<std::thread> pool;
  int64_t kb = k / gs;
  for (int t = 0; t < threads; ++t) {
    int64_t r0 = m * t / threads, r1 = m * (t + 1) / threads;
    pool.emplace_back([=] {
      r::w8a8_block_fp8_gemm(c + r0 * n, aq + r0 * k, as + r0 * kb, bq, bs, r1 - r0, n, k, gs, bn);
    });
  }
  for (auto& th : pool) th.join();
  return threads;
}

int ref_quant_fp8_per_token_group_mt(uint8_t* q, float* scales, const float* x, int64_t rows,
                                     int64_t cols, int gs, int threads) {
  if (threads <= 0) threads = int(std::thread::hardware_concurrency());
  if (threads <= 0) threads = 1;
  if (threads > rows) threads = int(rows);
  std::vector<std::thread> pool;
  int64_t g = cols / gs;
  for (int t = 0; t < threads; ++t) {
    int64_t r0 = rows * t / threads, r1 = rows * (t + 1) / threads;
    pool.emplace_back([=] {
      r::quant_fp8_per_token_group(q + r0 * cols, scales + r0 * g, x + r0 * cols, r1 - r0, cols, gs);
    });
  }
  for (auto& th : pool) th.join();
  return threads;
}

// Exhaustive codec comparison: counts the fp32 bit patterns in [lo, hi) on which
// `other` (any encoder with this signature, e.g. the in-tree oracle's) disagrees
// with the reference encoder.  The whole 2^32 range takes a few seconds on 8 cores.
uint64_t ref_encode_mismatches(uint8_t (*other)(float), uint64_t lo, uint64_t hi, int threads) {
  if (threads <= 0) threads = int(std::thread::hardware_concurrency());
  if (threads <= 0) threads = 1;
  std::vector<uint64_t> bad(size_t(threads), 0);
  std::vector<std::thread> pool;
  for (int t = 0; t < threads; ++t) {
    uint64_t a = lo + (hi - lo) * uint64_t(t) / uint64_t(threads);
    uint64_t b = lo + (hi - lo) * uint64_t(t + 1) / uint64_t(threads);
    pool.emplace_back([=, &bad] {
      uint64_t n = 0;
      for (uint64_t u = a; u < b; ++u) {
        float f = inferop::bitcast::u32_to_f32(uint32_t(u));
        n += other(f) != inferop::fp8::float_to_e4m3_rn_sat(f);
      }
      bad[size_t(t)] = n;
    });
  }
  for (auto& th : pool) th.join();
  uint64_t total = 0;
  for (auto v : bad) total += v;
  return total;
}

int ref_hardware_threads() { return int(std::thread::hardware_concurrency()); }

}  // extern "C"
