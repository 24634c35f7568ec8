/*
 * CPU oracle for the blockwise-FP8 path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a from-scratch C restatement of the reference's CPU golden
 * code for the two operators on the path plus the number formats they use.
 * It is the checker the CUDA kernels are compared with; nothing in the
 * shipped library links, loads or calls it.  Only the test-suite, the smoke
 * check and the benchmark's cpu_baseline leg may use it.
 *
 * Parity is pinned: the test-suite compares this file bit-for-bit with the
 * reference's own reference/reference.cpp (compiled into oracle/_ref/ where
 * the reference tree is present), with the reference's E4M3 known-answer
 * grid (tests/test_fp8.cpp, scripts/check_fp8.py) and with vectors generated
 * from the reference and committed under tests/golden/.
 *
 * Each function names the reference lines it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- bf16 <-> fp32 (include/inferop/common.h:55-61) ------------------- */
/* widen: the 16 stored bits are the top half of the fp32 word */
float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* narrow: round to nearest, ties to even, by adding 0x7FFF plus the lowest
 * kept bit and truncating (no special-casing of NaN, like the reference) */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u = f2u(f);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* ---- E4M3 (OCP FP8, finite-saturating) -------------------------------- */
/* decode: include/inferop/fp8.h:40-59.  S.EEEE.MMM, bias 7; E=0 is the
 * denormal row m*2^-9; E=15,m=7 is NaN; everything else (8+m)*2^(E-10). */
float orc_e4m3_to_f32(uint8_t b) {
  int e = (b >> 3) & 15, m = b & 7;
  float v;
  if (e == 15 && m == 7) return u2f(0x7FC00000u | ((uint32_t)(b >> 7) << 31));
  v = (e == 0) ? ldexpf((float)m, -9) : ldexpf((float)(8 + m), e - 10);
  return (b & 0x80) ? -v : v;
}

/* encode: include/inferop/fp8.h:62-96.  Round-to-nearest-even onto the
 * E4M3 grid, saturating to +-448 (0x7E), NaN -> sign|0x7F.
 *
 * Restated as one rounding step: the grid spacing around |f| is 2^(e-3)
 * with e clamped below at -6 (the denormal row shares the spacing of the
 * first normal binade), so n = RNE(|f| / 2^(e-3)) counts grid steps and the
 * code is the step count offset by the binade's first code.  A carry out of
 * the mantissa (n == 16, or n == 8 in the denormal row) lands on the next
 * binade's first code by plain addition. */
uint8_t orc_f32_to_e4m3(float f) {
  uint32_t u = f2u(f);
  uint32_t sign = (u >> 24) & 0x80u;
  uint32_t mag = u & 0x7FFFFFFFu;
  int e;
  uint32_t sig, shift, n, rest, half, code;
  if (mag > 0x7F800000u) return (uint8_t)(sign | 0x7Fu);
  e = (int)(mag >> 23) - 127;
  if (e >= 9) return (uint8_t)(sign | 0x7Eu);  /* includes +-Inf */
  if (e < -10) return (uint8_t)sign;           /* below half the smallest step */
  sig = (mag & 0x7FFFFFu) | 0x800000u;
  shift = (e >= -6) ? 20u : (uint32_t)(14 - e);
  n = sig >> shift;
  rest = sig & ((1u << shift) - 1u);
  half = 1u << (shift - 1u);
  if (rest > half || (rest == half && (n & 1u))) n += 1u;
  code = (e >= -6) ? (((uint32_t)(e + 7) << 3) + n - 8u) : n;
  if (code > 0x7Eu) code = 0x7Eu;
  return (uint8_t)(sign | code);
}

void orc_e4m3_decode_array(float* out, const uint8_t* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_e4m3_to_f32(in[i]);
}
void orc_e4m3_encode_array(uint8_t* out, const float* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_e4m3(in[i]);
}
void orc_bf16_widen_array(float* out, const uint16_t* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_bf16_to_f32(in[i]);
}
void orc_bf16_narrow_array(uint16_t* out, const float* in, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_bf16(in[i]);
}

/* ---- per-token-group quantisation (reference/reference.cpp:65-80) ------
 * For every run of `gs` consecutive elements of a row:
 *   amax  = max |x|   (a NaN never replaces the running maximum)
 *   scale = amax * fl(1/448), or exactly 1 when the group is all zero
 *   q     = e4m3(x / scale)  -- a true fp32 division, not a reciprocal
 * Returns 0, or -1 for a shape the reference treats as a no-op
 * (kernels/quant.cu:52). */
int orc_quant_fp8_per_token_group(uint8_t* q, float* scales, const float* x, int64_t rows,
                                  int64_t cols, int gs) {
  if (rows <= 0 || cols <= 0 || gs <= 0 || cols % gs != 0) return -1;
  const float inv448 = 1.0f / 448.0f;
  int64_t groups = rows * (cols / gs);
  for (int64_t g = 0; g < groups; ++g) {
    const float* gx = x + g * gs;
    uint8_t* gq = q + g * gs;
    float amax = 0.0f;
    for (int i = 0; i < gs; ++i) {
      float a = fabsf(gx[i]);
      if (amax < a) amax = a;
    }
    volatile float scale = (amax == 0.0f) ? 1.0f : amax * inv448;
    scales[g] = scale;
    for (int i = 0; i < gs; ++i) {
      volatile float r = gx[i] / scale;
      gq[i] = orc_f32_to_e4m3(r);
    }
  }
  return 0;
}

/* inverse (reference/reference.cpp:82-91): x = decode(q) * scale, in fp32 */
int orc_dequant_fp8_per_token_group(float* x, const uint8_t* q, const float* scales, int64_t rows,
                                    int64_t cols, int gs) {
  if (rows <= 0 || cols <= 0 || gs <= 0 || cols % gs != 0) return -1;
  int64_t n = rows * cols;
  for (int64_t i = 0; i < n; ++i) x[i] = orc_e4m3_to_f32(q[i]) * scales[i / gs];
  return 0;
}

/* ---- weight block quantiser (tests/test_gemm.cpp:28-45) ----------------
 * One scale per (bn x gs) block of W[N,K]; N may be ragged (the last block
 * row is short).  Unlike the activation path this one multiplies by the
 * rounded reciprocal of the scale. */
int orc_block_quant_weights(uint8_t* bq, float* bs, const float* w, int64_t n, int64_t k, int gs,
                            int bn) {
  if (n <= 0 || k <= 0 || gs <= 0 || bn <= 0 || k % gs != 0) return -1;
  const float inv448 = 1.0f / 448.0f;
  int64_t kb = k / gs, nb = (n + bn - 1) / bn;
  for (int64_t b = 0; b < nb; ++b) {
    int64_t r0 = b * bn, r1 = (r0 + bn < n) ? r0 + bn : n;
    for (int64_t g = 0; g < kb; ++g) {
      float amax = 0.0f;
      for (int64_t r = r0; r < r1; ++r)
        for (int i = 0; i < gs; ++i) {
          float a = fabsf(w[r * k + g * gs + i]);
          if (amax < a) amax = a;
        }
      volatile float scale = (amax == 0.0f) ? 1.0f : amax * inv448;
      volatile float inv = 1.0f / scale;
      bs[b * kb + g] = scale;
      for (int64_t r = r0; r < r1; ++r)
        for (int i = 0; i < gs; ++i) {
          volatile float p = w[r * k + g * gs + i] * inv;
          bq[r * k + g * gs + i] = orc_f32_to_e4m3(p);
        }
    }
  }
  return 0;
}

/* ---- fp64 golden GEMM (reference/reference.cpp:93-110) -----------------
 *   C[m,n] = sum over k, in index order, of
 *            double( fl32(dec(A[m,k]) * sa[m,k/gs]) ) * double( fl32(dec(B[n,k]) * sb[n/bn,k/gs]) )
 * accumulated in double and narrowed to float once at the end.  The order
 * of the k loop is kept so the sum is bit-identical to the reference; speed
 * comes from dequantising each operand row once and from running eight
 * independent column sums side by side.
 *
 * rows/cols select a sub-matrix (NULL = all): out is [n_rows, n_cols]
 * row-major.  That is how the big shapes are spot-checked. */
int orc_w8a8_block_fp8_gemm(float* out, const uint8_t* aq, const float* as, const uint8_t* bq,
                            const float* bs, int64_t m, int64_t n, int64_t k, int gs, int bn,
                            const int64_t* rows, int64_t n_rows, const int64_t* cols,
                            int64_t n_cols) {
  if (m <= 0 || n <= 0 || k <= 0 || gs <= 0 || bn <= 0 || k % gs != 0) return -1;
  if (!rows) n_rows = m;
  if (!cols) n_cols = n;
  int64_t kb = k / gs;
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_to_f32((uint8_t)i);
  /* dequantised copy of the selected weight rows, [n_cols, k] */
  float* bv = (float*)malloc((size_t)n_cols * (size_t)k * sizeof(float));
  float* av = (float*)malloc((size_t)k * sizeof(float));
  if (!bv || !av) { free(bv); free(av); return -2; }
  for (int64_t j = 0; j < n_cols; ++j) {
    int64_t c = cols ? cols[j] : j;
    const uint8_t* src = bq + c * k;
    const float* s = bs + (c / bn) * kb;
    for (int64_t i = 0; i < k; ++i) bv[j * k + i] = lut[src[i]] * s[i / gs];
  }
  for (int64_t r = 0; r < n_rows; ++r) {
    int64_t row = rows ? rows[r] : r;
    const uint8_t* src = aq + row * k;
    const float* s = as + row * kb;
    for (int64_t i = 0; i < k; ++i) av[i] = lut[src[i]] * s[i / gs];
    int64_t j = 0;
    for (; j + 8 <= n_cols; j += 8) {
      double acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      const float* b0 = bv + j * k;
      for (int64_t i = 0; i < k; ++i) {
        double a = (double)av[i];
        for (int t = 0; t < 8; ++t) acc[t] += a * (double)b0[t * k + i];
      }
      for (int t = 0; t < 8; ++t) out[r * n_cols + j + t] = (float)acc[t];
    }
    for (; j < n_cols; ++j) {
      double acc = 0.0;
      const float* b0 = bv + j * k;
      for (int64_t i = 0; i < k; ++i) acc += (double)av[i] * (double)b0[i];
      out[r * n_cols + j] = (float)acc;
    }
  }
  free(bv);
  free(av);
  return 0;
}

/* ---- MoE routing (reference/reference.cpp:152-181) ---------------------
 * softmax over the expert logits in fp32 (subtract the row maximum, expf,
 * sum in index order), then the top-k experts by probability with the lower
 * index winning ties, weights p/l, optionally renormalised by their sum. */
int orc_topk_softmax(int32_t* ids, float* weights, const float* logits, int64_t tokens,
                     int experts, int topk, int renorm) {
  if (tokens < 0 || experts <= 0 || topk <= 0 || topk > experts) return -1;
  float* p = (float*)malloc((size_t)experts * sizeof(float));
  char* used = (char*)malloc((size_t)experts);
  if (!p || !used) { free(p); free(used); return -2; }
  for (int64_t t = 0; t < tokens; ++t) {
    const float* row = logits + t * experts;
    float mx = -INFINITY;
    for (int e = 0; e < experts; ++e) if (mx < row[e]) mx = row[e];
    volatile float l = 0.0f;
    for (int e = 0; e < experts; ++e) { p[e] = expf(row[e] - mx); l += p[e]; }
    memset(used, 0, (size_t)experts);
    volatile float wsum = 0.0f;
    for (int j = 0; j < topk; ++j) {
      int best = -1;
      for (int e = 0; e < experts; ++e)
        if (!used[e] && (best < 0 || p[e] > p[best])) best = e;
      used[best] = 1;
      ids[t * topk + j] = best;
      volatile float w = p[best] / l;
      weights[t * topk + j] = w;
      wsum += w;
    }
    if (renorm && wsum > 0.0f)
      for (int j = 0; j < topk; ++j) weights[t * topk + j] /= wsum;
  }
  free(p);
  free(used);
  return 0;
}

/* ---- SwiGLU (reference/reference.cpp:55-63) -----------------------------
 * out[t, i] = (g / (1 + expf(-g))) * u with g = gate_up[t, i], u = gate_up[t, d + i], every
 * operation in fp32. */
int orc_silu_and_mul(float* out, const float* gate_up, int64_t tokens, int64_t d) {
  if (tokens < 0 || d <= 0) return -1;
  for (int64_t t = 0; t < tokens; ++t) {
    const float* row = gate_up + t * 2 * d;
    for (int64_t i = 0; i < d; ++i) {
      volatile float den = 1.0f + expf(-row[i]);
      volatile float s = row[i] / den;
      out[t * d + i] = s * row[d + i];
    }
  }
  return 0;
}

/* ---- RMSNorm (reference/reference.cpp:11-21) -----------------------------
 * Per row: ss = sum of x^2 accumulated left to right in fp32, inv = 1 / sqrtf(ss / cols + eps),
 * y = (x * inv) * w, every operation rounded to fp32. */
int orc_rmsnorm(float* out, const float* in, const float* weight, int64_t rows, int64_t cols, float eps) {
  if (rows < 0 || cols <= 0) return -1;
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * cols;
    float* y = out + r * cols;
    volatile float ss = 0.0f;
    for (int64_t c = 0; c < cols; ++c) {
      volatile float sq = x[c] * x[c];
      ss = ss + sq;
    }
    volatile float mean = ss / (float)cols;
    volatile float den = sqrtf(mean + eps);
    const float inv = 1.0f / den;
    for (int64_t c = 0; c < cols; ++c) {
      volatile float t = x[c] * inv;
      y[c] = t * weight[c];
    }
  }
  return 0;
}

/* ---- residual add + RMSNorm (reference/reference.cpp:23-35) ---------------
 * residual += x (in place), then RMSNorm of the updated residual. */
int orc_fused_add_rmsnorm(float* residual, float* out, const float* x, const float* weight, int64_t rows,
                          int64_t cols, float eps) {
  if (rows < 0 || cols <= 0) return -1;
  for (int64_t r = 0; r < rows; ++r) {
    float* res = residual + r * cols;
    const float* xr = x + r * cols;
    for (int64_t c = 0; c < cols; ++c) res[c] = res[c] + xr[c];
  }
  return orc_rmsnorm(out, residual, weight, rows, cols, eps);
}

/* ---- rotary embedding, GPT-NeoX layout (reference/reference.cpp:37-53) ------
 * In place on qkv [tokens, heads, head_dim]: for i < rotary_dim / 2,
 * freq = powf(base, -2 i / rotary_dim) * yarn_factor, theta = (float)position * freq,
 * (x_i, x_{i+half}) rotated by theta; elements from rotary_dim on are left alone. */
int orc_rope_neox(float* qkv, const int64_t* positions, int64_t tokens, int heads, int head_dim, int rotary_dim,
                  float base, float yarn_factor) {
  if (tokens < 0 || heads <= 0 || head_dim <= 0 || rotary_dim <= 0 || rotary_dim > head_dim || (rotary_dim & 1))
    return -1;
  const int half = rotary_dim / 2;
  for (int64_t t = 0; t < tokens; ++t) {
    for (int h = 0; h < heads; ++h) {
      float* p = qkv + (t * heads + h) * head_dim;
      for (int i = 0; i < half; ++i) {
        volatile float e = -2.0f * (float)i / (float)rotary_dim;
        volatile float pw = powf(base, e);
        volatile float freq = pw * yarn_factor;
        volatile float theta = (float)positions[t] * freq;
        const float c = cosf(theta), s = sinf(theta);
        const float x0 = p[i], x1 = p[i + half];
        volatile float a = x0 * c, b = x1 * s, d = x1 * c, g = x0 * s;
        p[i] = a - b;
        p[i + half] = d + g;
      }
    }
  }
  return 0;
}

/* ---- paged attention, single-token decode, GQA (reference/reference.cpp:112-150) --------------
 * q / out [batch, heads, head_dim]; k_cache / v_cache [blocks, block_size, kv_heads, head_dim];
 * block_tables int32 [batch, max_blocks_per_seq]; seq_lens int32 [batch].  Per (sequence, head):
 * scores = (q . k) * scale with the dot product accumulated left to right in fp32, m = max score,
 * p = expf(score - m), l = sum p, out = (sum p * v) / l (0 for an empty sequence). */
int orc_paged_attn_decode(float* out, const float* q, const float* k_cache, const float* v_cache,
                          const int32_t* block_tables, const int32_t* seq_lens, int batch, int num_heads,
                          int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq, float scale) {
  if (batch < 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || head_dim <= 0 ||
      block_size <= 0)
    return -1;
  for (int b = 0; b < batch; ++b) {
    const int len = seq_lens[b];
    const int32_t* bt = block_tables + (int64_t)b * max_blocks_per_seq;
    float* scores = (float*)malloc(sizeof(float) * (size_t)(len > 0 ? len : 1));
    float* acc = (float*)malloc(sizeof(float) * (size_t)head_dim);
    if (!scores || !acc) {
      free(scores);
      free(acc);
      return -2;
    }
    for (int h = 0; h < num_heads; ++h) {
      const int kvh = h / (num_heads / num_kv_heads);
      const float* qv = q + ((int64_t)b * num_heads + h) * head_dim;
      float m = -INFINITY;
      for (int key = 0; key < len; ++key) {
        const int blk = bt[key / block_size], off = key % block_size;
        const float* krow = k_cache + (((int64_t)blk * block_size + off) * num_kv_heads + kvh) * head_dim;
        volatile float dot = 0.0f;
        for (int d = 0; d < head_dim; ++d) {
          volatile float pr = qv[d] * krow[d];
          dot = dot + pr;
        }
        scores[key] = dot * scale;
        if (scores[key] > m) m = scores[key];
      }
      for (int d = 0; d < head_dim; ++d) acc[d] = 0.0f;
      volatile float l = 0.0f;
      for (int key = 0; key < len; ++key) {
        const float p = expf(scores[key] - m);
        l = l + p;
        const int blk = bt[key / block_size], off = key % block_size;
        const float* vrow = v_cache + (((int64_t)blk * block_size + off) * num_kv_heads + kvh) * head_dim;
        for (int d = 0; d < head_dim; ++d) {
          volatile float pr = p * vrow[d];
          acc[d] = acc[d] + pr;
        }
      }
      float* o = out + ((int64_t)b * num_heads + h) * head_dim;
      const float inv = (l == 0.0f) ? 0.0f : 1.0f / l;
      for (int d = 0; d < head_dim; ++d) o[d] = acc[d] * inv;
    }
    free(scores);
    free(acc);
  }
  return 0;
}
