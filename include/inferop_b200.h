/*
 * inferop_b200: C ABI of the B200 (sm_100a) blockwise-FP8 W8A8 path.
 *
 * This is the boundary a foreign-function binding attaches to: plain C,
 * pointers and sizes only.  Every tensor pointer is caller-owned device memory
 * on the current CUDA device unless a comment says "host".  `stream` is a
 * cudaStream_t passed as void* (NULL = the default stream).  Calls enqueue
 * work and return; they never synchronise unless stated.
 *
 * Return value: INFEROP_OK (0) when the work was enqueued, otherwise one of
 * the INFEROP_ERR_* codes and nothing was launched.  There is no CPU or
 * generic-GPU fallback: without an sm_100 device every operator returns
 * INFEROP_ERR_NO_DEVICE / INFEROP_ERR_ARCH.
 *
 * dtype codes (reference include/inferop/common.h:13):
 *   0 = fp32, 1 = fp16, 2 = bf16, 3 = fp8_e4m3.
 */
#ifndef INFEROP_B200_H_
#define INFEROP_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define INFEROP_API __attribute__((visibility("default")))
#else
#define INFEROP_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
  INFEROP_OK = 0,
  INFEROP_ERR_SHAPE = 1,      /* sizes the reference treats as a no-op / contract violation */
  INFEROP_ERR_DTYPE = 2,      /* dtype code not supported by this operator */
  INFEROP_ERR_POINTER = 3,    /* NULL tensor pointer */
  INFEROP_ERR_NO_DEVICE = 4,  /* no CUDA device visible */
  INFEROP_ERR_ARCH = 5,       /* current device is not sm_100 */
  INFEROP_ERR_CUDA = 6,       /* a CUDA runtime/driver call failed; see inferop_last_cuda_error */
  INFEROP_ERR_LIMIT = 7,      /* size beyond a documented limit of the entry point */
  INFEROP_ERR_DEVICE_WAIT = 8 /* a bounded wait inside a kernel ran out (inferop_device_status) */
};

/* Human-readable name of a status code. */
INFEROP_API const char* inferop_status_string(int status);
/* cudaError_t of the most recent failed CUDA call on this thread (0 if none). */
INFEROP_API int inferop_last_cuda_error(void);

/* ---- device queries (reference include/inferop/ops.h:19-25, kernels/api.cu:12-50) ---- */
INFEROP_API int inferop_has_cuda(void);                 /* 1 when at least one device is visible */
INFEROP_API int inferop_device_count(void);
INFEROP_API const char* inferop_device_name(int ordinal);   /* "-" when out of range */
INFEROP_API int inferop_device_sm_version(int ordinal);     /* major*10+minor, -1 when out of range */

/* ---- per-token-group quantisation
 * Replaces inferop::quant_fp8_per_token_group (reference include/inferop/ops.h:64-65,
 * kernels/api.cu:73-76, kernels/quant.cu:50-75).
 *   x [rows, cols] in dt (0/1/2) -> q [rows, cols] uint8, scales [rows, cols/group_size] fp32.
 * Bit-exact against reference/reference.cpp:65-80.  Any group_size dividing cols is
 * accepted; 128 takes the vectorised kernel. */
INFEROP_API int inferop_quant_fp8_per_token_group(void* q, void* scales, const void* x, int32_t dt,
                                      int64_t rows, int64_t cols, int32_t group_size,
                                      void* stream);

/* Replaces inferop::dequant_fp8_per_token_group (reference include/inferop/ops.h:68-70,
 * kernels/quant.cu:77-103):  x = decode(q) * scale, stored as dt. */
INFEROP_API int inferop_dequant_fp8_per_token_group(void* x, int32_t dt, const void* q, const void* scales,
                                        int64_t rows, int64_t cols, int32_t group_size,
                                        void* stream);

/* ---- blockwise-FP8 GEMM
 * Replaces inferop::w8a8_block_fp8_gemm (reference include/inferop/ops.h:81-84,
 * kernels/api.cu:83-88, kernels/gemm/w8a8_block_fp8.cu:163-188).
 *   a_q [M,K] E4M3, a_scales [M,K/128] fp32, b_q [N,K] E4M3,
 *   b_scales [ceil(N/128), K/128] fp32, c [M,N] in out_dt (0/1/2).
 * Contract as in the reference: group_size == 128, block_n == 128, K % 128 == 0,
 * M > 0, N > 0 (else INFEROP_ERR_SHAPE).  a_q and b_q must be 16-byte aligned
 * (INFEROP_ERR_POINTER otherwise); c may have any alignment and N any value.
 * Calls with few tokens (M <= 32, and M <= 64 when ceil(N/128) is below 3/4 of the SM count)
 * take a weight-streaming kernel that keeps a library-owned scratch
 * buffer (about 19 MB) per stream; it is allocated by the first such call on a stream, so
 * make that call before capturing the stream into a CUDA graph (up to 64 streams per device
 * get scratch; calls on further streams are served by the large-tile kernel).  Calls with
 * M > 128 take the CTA-pair kernel (clusters of two CTAs, tcgen05.mma.cta_group::2).
 *
 * Programmatic dependent launch: the weight-streaming and the CTA-pair kernels are launched
 * with programmatic stream serialisation and may start their set-up while the kernel queued
 * before them on the stream is still running; the weight-streaming kernel also requests its
 * first weight tiles (b_q) before it waits for that kernel.  a_q, a_scales and c are touched
 * only after the wait.  So b_q and b_scales must not be PRODUCED by the kernel queued
 * immediately before the call if that kernel triggers its dependents early
 * (griddepcontrol.launch_dependents), as this library's quantiser does; weights written by an
 * ordinary kernel, a copy, or anything earlier on the stream are fine.  A caller that rewrites
 * weights with such a kernel right before the GEMM sets the options "decode_pdl" and
 * "gemm_pdl" to 0 (inferop_set_option).  The same holds for the fused-quant, all-gather,
 * strided-output and fixed-scratch entry points. */
INFEROP_API int inferop_w8a8_block_fp8_gemm(void* c, const void* a_q, const void* a_scales, const void* b_q,
                                const void* b_scales, int64_t m, int64_t n, int64_t k,
                                int32_t group_size, int32_t block_n, int32_t out_dt,
                                void* stream);

/* ---- quantisation as the GEMM's A-operand prologue: one call for quantise + GEMM
 * Same result, bit for bit, as inferop_quant_fp8_per_token_group (group 128) followed by
 * inferop_w8a8_block_fp8_gemm (reference include/inferop/ops.h:64-65 then :81-84).
 * a [M, K] in a_dt (1 = fp16, 2 = bf16), 16-byte aligned.
 *   M <= 32: one launch, without the q / scales round trip: the small-M kernel's prologue warps
 *     quantise each K block of the activations on the fly (scratch as for the small-M GEMM path).
 *   M > 32: quantising inside the GEMM would repeat the work once per column tile (N / 256
 *     times), so the call is two launches chained by programmatic dependent launch: the
 *     quantiser writes into library-owned scratch of this stream (M * K + 4 * M * K / 128 bytes,
 *     grown by a cudaMalloc whenever a call is larger than any before it on the stream: make the
 *     largest call before a stream capture) and the GEMM sets itself up underneath it. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_fused_quant(void* c, const void* a, int32_t a_dt, const void* b_q,
                                            const void* b_scales, int64_t m, int64_t n, int64_t k,
                                            int32_t group_size, int32_t block_n, int32_t out_dt,
                                            void* stream);

/* ---- grouped blockwise-FP8 GEMM (MoE expert GEMMs in one launch)
 * Equivalent to one inferop_w8a8_block_fp8_gemm call per group (which is how the reference runs
 * expert GEMMs: include/inferop/ops.h:81-84 once per expert; a grouped GEMM is only on its
 * roadmap, docs/ROADMAP.md:39):
 *   for g in 0..groups-1:  C[r_g : r_g + m_g, :] = gemm(A_q[r_g : r_g + m_g], B_q[g], ...)
 * with r_g the running sum of m_per_group.  a_q [sum m_g, K], a_scales [sum m_g, K/128] and
 * c [sum m_g, N] hold the groups' rows one after the other; b_q is [groups, N, K] and b_scales
 * [groups, N/128, K/128].  m_per_group is a HOST array of `groups` entries (zeros allowed) and
 * is read before the call returns.  N % 128 == 0 is required in addition to the GEMM contract. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_grouped(void* c, const void* a_q, const void* a_scales, const void* b_q,
                                        const void* b_scales, const int64_t* m_per_group,
                                        int64_t groups, int64_t n, int64_t k, int32_t group_size,
                                        int32_t block_n, int32_t out_dt, void* stream);

/* ---- blockwise-FP8 GEMM of one column shard, all-gathered by its own epilogue
 * Column-parallel use of inferop_w8a8_block_fp8_gemm (reference include/inferop/ops.h:81-84; the
 * reference is single-GPU and has no collective): rank `rank` of `n_peers` holds the weight rows
 * b_q [n, K] / b_scales [n/128, K/128] of its shard and the full activations, and the result
 * [M, n] is written to columns [rank * n, (rank + 1) * n) of the row-major [M, n * n_peers]
 * buffer of EVERY rank, straight from the kernel's epilogue (one TMA store per destination over
 * NVLink), instead of a local store followed by an all-gather.
 * c_peers is a HOST array of n_peers device addresses, entry d = the base of rank d's buffer as
 * mapped into this process (CUDA IPC, virtual-memory export or symmetric memory; entry `rank` is
 * the local buffer), each 16-byte aligned; it is read before the call returns.  n % 128 == 0,
 * n_peers <= 8, out_dt 1 (fp16) or 2 (bf16).  Few tokens (the rule of the plain GEMM) run the weight-streaming kernel of the
 * plain GEMM (plain stores to the peers, same per-stream scratch), larger M the large-tile kernel
 * (one TMA store per destination).  The call does not synchronise the ranks: a rank's
 * buffer is complete when every rank's call has finished, so the ranks must meet (a barrier, a
 * collective, or stream-ordered signals) after the call before any of them reads its buffer, and
 * before the call overwrites a buffer that a peer may still be reading. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_allgather(void* const* c_peers, int32_t n_peers, int32_t rank,
                                          const void* a_q, const void* a_scales, const void* b_q,
                                          const void* b_scales, int64_t m, int64_t n, int64_t k,
                                          int32_t group_size, int32_t block_n, int32_t out_dt,
                                          void* stream);

/* ---- blockwise-FP8 GEMM of one K shard, reduce-scattered (row-parallel sharding)
 * The partner of the column-parallel form (reference include/inferop/ops.h:81-84 on a K shard of
 * both operands; the reference is single-GPU and has no collective): rank `rank` of `n_peers`
 * holds columns of the activations a_q [M, k] / a_scales [M, k/128] and of the weights
 * b_q [N, k] / b_scales [ceil(N/128), k/128] for its K range, so its product is a partial sum of
 * the whole [M, N] result.  Rank d owns rows [d * M/n_peers, (d + 1) * M/n_peers) of the final
 * result and keeps, for them, one fp32 slot per source rank: slots [n_peers][M/n_peers][N].
 * inferop_w8a8_block_fp8_gemm_scatter stores this rank's partial tiles straight from the GEMM's
 * epilogue into slot `rank` of each owner (TMA stores over NVLink; slot_peers is a HOST array,
 * entry d = base of rank d's slots as mapped in this process, 16-byte aligned).  After the ranks
 * have met, each owner calls inferop_reduce_slots, which adds its slots in rank order and rounds
 * once to out_dt: out [M/n_peers, N].  The sum is fp32 over K blocks within a rank (as in the plain
 * GEMM) and fp32 over the ranks, so it equals the unsharded GEMM up to fp32 reassociation, and it
 * is reproducible.  M % (128 * n_peers) == 0, N % 4 == 0, n_peers <= 8. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_scatter(void* const* slot_peers, int32_t n_peers, int32_t rank,
                                        const void* a_q, const void* a_scales, const void* b_q,
                                        const void* b_scales, int64_t m, int64_t n, int64_t k,
                                        int32_t group_size, int32_t block_n, void* stream);
INFEROP_API int inferop_reduce_slots(void* out, int32_t out_dt, const void* slots, int32_t n_peers, int64_t rows,
                         int64_t n, void* stream);

/* inferop_w8a8_block_fp8_gemm (reference include/inferop/ops.h:81-84) with a strided output: the
 * [M, N] result goes to columns [col0, col0 + N) of a row-major buffer c_base with ldc columns
 * (out_dt 1 fp16 / 2 bf16; N % 128 == 0; col0 and ldc multiples of 8; c_base 16-byte aligned).
 * A column shard's GEMM can so write straight into its place in the full [M, N_total] result. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_into(void* c_base, int64_t ldc, int64_t col0, const void* a_q,
                                     const void* a_scales, const void* b_q, const void* b_scales, int64_t m,
                                     int64_t n, int64_t k, int32_t group_size, int32_t block_n, int32_t out_dt,
                                     void* stream);

/* 2-D copy by the copy engines (cudaMemcpy2DAsync, device to device, peer-mapped addresses
 * allowed): `rows` rows of width_bytes from src (row pitch src_pitch_bytes) to dst (row pitch
 * dst_pitch_bytes), enqueued on `stream`.  No counterpart in the reference (it has no multi-GPU
 * code); used to push finished row panels of a column shard's result into every rank's [M, N]
 * buffer while the tensor cores work on the next panel, without taking SMs or epilogue time
 * from the GEMM. */
INFEROP_API int inferop_copy_2d_async(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                          int64_t width_bytes, int64_t rows, void* stream);

/* ---- mixture-of-experts layer around the grouped GEMM
 * Every step stays on the device: the experts' row counts are never copied to the host, the
 * grouped GEMM reads the M-tile list that inferop_moe_align wrote.  The steps of a layer:
 *   inferop_topk_softmax -> inferop_moe_align -> inferop_moe_scatter_quant ->
 *   inferop_w8a8_block_fp8_gemm_grouped_tiles (gate_up) -> inferop_silu_and_mul_quant ->
 *   inferop_w8a8_block_fp8_gemm_grouped_tiles (down) -> inferop_moe_combine
 */

/* Routing (reference include/inferop/ops.h:108-110, kernels/moe/topk_softmax.cu:18-97, CPU
 * reference/reference.cpp:152-181): softmax over logits [tokens, num_experts] (fp32), the topk
 * experts by probability (lower index first on equal probabilities) into topk_ids
 * [tokens, topk] (int32) and their probabilities into topk_weights [tokens, topk] (fp32),
 * divided by their sum when `renormalize`.  num_experts <= 1024, topk <= num_experts;
 * anything else is INFEROP_ERR_SHAPE (the reference: silent no-op).  Logits must be finite. */
INFEROP_API int inferop_topk_softmax(int32_t* topk_ids, void* topk_weights, const void* logits, int32_t tokens,
                         int32_t num_experts, int32_t topk, int32_t renormalize, void* stream);

/* RMSNorm (reference include/inferop/ops.h:30-31, kernels/rmsnorm.cu:21-36, CPU
 * reference/reference.cpp:11-21): out[r, c] = in[r, c] / sqrt(mean(in[r, :]^2) + eps) * weight[c]
 * for in / out [rows, cols] and weight [cols] in dt (0 fp32, 1 fp16, 2 bf16), computed in fp32. */
INFEROP_API int inferop_rmsnorm(void* out, const void* in, const void* weight, int32_t dt, int64_t rows,
                    int64_t cols, float eps, void* stream);

/* Residual add + RMSNorm (reference ops.h:35-37, kernels/rmsnorm.cu:38-59, CPU
 * reference.cpp:23-35): residual[r, :] += x[r, :] in place (stored in dt), out = RMSNorm of the
 * sum.  As in the reference's kernel the mean uses the unrounded sums and the output the stored ones. */
INFEROP_API int inferop_fused_add_rmsnorm(void* residual, void* out, const void* x, const void* weight, int32_t dt,
                              int64_t rows, int64_t cols, float eps, void* stream);

/* RMSNorm (residual == NULL) or residual add + RMSNorm (residual[r, :] += in[r, :] in place) with the
 * 1 x 128 FP8 quantisation of the result in the same pass: q [rows, cols] E4M3 and scales
 * [rows, cols / 128] are, bit for bit, what inferop_quant_fp8_per_token_group gives on the output of
 * inferop_rmsnorm / inferop_fused_add_rmsnorm (reference ops.h:30-37 then :64-65), and the 16-bit matrix
 * between the two never exists (3 bytes per element instead of 7).  dt 1 fp16 / 2 bf16 (the type of in,
 * weight, residual and of the intermediate rounding); group_size == 128; cols % 128 == 0, cols <= 16384;
 * in / weight / residual 16-byte aligned, q 8-byte aligned.  No counterpart in the reference. */
INFEROP_API int inferop_rmsnorm_quant(void* q, void* scales, void* residual, const void* in, const void* weight,
                          int32_t dt, int64_t rows, int64_t cols, int32_t group_size, float eps, void* stream);

/* Rotary position embedding, GPT-NeoX layout, in place (reference ops.h:46-48, kernels/rope.cu:19-41,
 * CPU reference.cpp:37-53): qkv [tokens, heads, head_dim] in dt, positions int64 [tokens] (device);
 * for i < rotary_dim / 2: theta = position * base^(-2 i / rotary_dim) * yarn_factor and
 * (x_i, x_{i + rotary_dim/2}) is rotated by theta; elements from rotary_dim on are untouched.
 * rotary_dim even, 2 <= rotary_dim <= head_dim, rotary_dim <= 1024 (INFEROP_ERR_LIMIT beyond);
 * the reference returns silently on a bad rotary_dim, this returns INFEROP_ERR_SHAPE. */
INFEROP_API int inferop_rope_neox(void* qkv, const int64_t* positions, int32_t dt, int64_t tokens, int32_t heads,
                      int32_t head_dim, int32_t rotary_dim, float base, float yarn_factor, void* stream);

/* Paged attention, single-token decode with grouped-query heads (reference ops.h:96-100,
 * kernels/attention/paged_attn_decode.cu:26-118, CPU reference.cpp:112-150):
 *   q / out [batch, num_heads, head_dim] in dt; k_cache / v_cache [blocks, block_size, num_kv_heads,
 *   head_dim] in dt (16-byte aligned); block_tables int32 [batch, max_blocks_per_seq]; seq_lens int32
 *   [batch] (clamped to max_blocks_per_seq * block_size); out = softmax(q k^T * scale) v per head, an
 *   empty sequence gives zeros.  head_dim in {64, 128, 256} (the reference's list; anything else is
 *   INFEROP_ERR_SHAPE where the reference does nothing), num_heads % num_kv_heads == 0, batch <= 65535.
 * Long sequences are processed as several token ranges whose partial results live in scratch of the
 * stream (allocated by the first call that needs it: make one call before capturing a CUDA graph). */
INFEROP_API int inferop_paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                              const int32_t* block_tables, const int32_t* seq_lens, int32_t dt, int32_t batch,
                              int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                              int32_t max_blocks_per_seq, float scale, void* stream);

/* SwiGLU (reference include/inferop/ops.h:54-55, kernels/silu_mul.cu:16-28, CPU
 * reference/reference.cpp:55-63): out[t, i] = silu(gate_up[t, i]) * gate_up[t, d + i] for
 * gate_up [tokens, 2d] and out [tokens, d] in dt (0 fp32, 1 fp16, 2 bf16), computed in fp32. */
INFEROP_API int inferop_silu_and_mul(void* out, const void* gate_up, int32_t dt, int64_t tokens, int64_t d,
                         void* stream);

/* inferop_silu_and_mul followed by inferop_quant_fp8_per_token_group in one pass, bit for bit
 * the result of the two calls (reference ops.h:54-55 then :64-65): q [tokens, d] E4M3 and scales
 * [tokens, d/128] from gate_up [tokens, 2d] in dt (1 fp16, 2 bf16; the SwiGLU value is rounded
 * to dt before it is quantised, as the separate kernels store it).  d % 128 == 0, group 128,
 * gate_up 16-byte and q 8-byte aligned. */
INFEROP_API int inferop_silu_and_mul_quant(void* q, void* scales, const void* gate_up, int32_t dt, int64_t tokens,
                               int64_t d, int32_t group_size, void* stream);

/* Upper bound on the M-tiles inferop_moe_align can produce: size of tile_row0 / tile_meta. */
INFEROP_API int64_t inferop_moe_max_mtiles(int64_t tokens, int32_t topk, int32_t num_experts);

/* Expert-sorted layout of a routing (no reference counterpart: the reference runs one GEMM per
 * expert from the host).  From topk_ids [tokens, topk] (device):
 *   counts [num_experts]       rows per expert
 *   offsets [num_experts + 1]  first sorted row of each expert, offsets[num_experts] = pairs
 *   pos [tokens * topk]        sorted row of pair (token, k); pairs of one expert keep their
 *                              (token, k) order; -1 for an id outside [0, num_experts)
 *   src_token [tokens * topk]  token of each sorted row
 *   tile_row0 / tile_meta [inferop_moe_max_mtiles]  M-tiles of up to 128 rows that never span
 *                              two experts: first row, and (expert << 8) | (rows - 1)
 *   num_mtiles [1]             how many tiles were written
 * all int32 device arrays.  One launch (a cluster of up to 8 CTAs); num_experts <= 1024. */
INFEROP_API int inferop_moe_align(const int32_t* topk_ids, int64_t tokens, int32_t topk, int32_t num_experts,
                      int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_token,
                      int32_t* tile_row0, int32_t* tile_meta, int32_t* num_mtiles, void* stream);

/* Quantise x [tokens, cols] (dt 1 fp16 / 2 bf16) per 1x128 group, exactly as
 * inferop_quant_fp8_per_token_group does, and write every token's bytes and scales to the
 * sorted rows pos[token * topk + k] of q [tokens * topk, cols] and scales
 * [tokens * topk, cols/128] (rows with pos < 0 are skipped). */
INFEROP_API int inferop_moe_scatter_quant(void* q, void* scales, const void* x, int32_t dt, const int32_t* pos,
                              int64_t tokens, int64_t cols, int32_t topk, int32_t group_size,
                              void* stream);

/* Rows of row_bytes bytes (a multiple of 16; dst and src 16-byte aligned) moved by a permutation
 * held in device memory: gather == 0: dst[perm[i]] = src[i]; gather != 0: dst[i] = src[perm[i]];
 * i in [0, rows), rows with perm[i] < 0 are skipped.  No counterpart in the reference; an
 * expert-parallel layer uses it to put the rows it received from the other ranks into
 * expert-sorted order (perm = the pos array of inferop_moe_align over the received expert ids)
 * and to put the experts' outputs back into arrival order for the way home. */
INFEROP_API int inferop_moe_permute_rows(void* dst, const void* src, const int32_t* perm, int64_t rows,
                             int64_t row_bytes, int32_t gather, void* stream);

/* out[t, :] = sum_k topk_weights[t, k] * y[pos[t * topk + k], :] for y [tokens * topk, hidden]
 * and out [tokens, hidden] in dt (1 fp16 / 2 bf16): products and sums in fp32, each rounded, in
 * the order of k, the result rounded once.  hidden % 8 == 0; out and y 16-byte aligned. */
INFEROP_API int inferop_moe_combine(void* out, const void* y, const void* topk_weights, const int32_t* pos, int32_t dt,
                        int64_t tokens, int64_t hidden, int32_t topk, void* stream);

/* inferop_w8a8_block_fp8_gemm_grouped with the tile list in device memory (as written by
 * inferop_moe_align) instead of host row counts: nothing is read on the host, so the call can
 * follow the routing kernels on the stream without a synchronisation.  a_q / c have m_total
 * rows; max_mtiles bounds the list (inferop_moe_max_mtiles), *num_mtiles is its length. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_grouped_tiles(void* c, const void* a_q, const void* a_scales,
                                              const void* b_q, const void* b_scales,
                                              const int32_t* tile_row0, const int32_t* tile_meta,
                                              const int32_t* num_mtiles, int64_t max_mtiles,
                                              int64_t m_total, int64_t groups, int64_t n, int64_t k,
                                              int32_t group_size, int32_t block_n, int32_t out_dt,
                                              void* stream);

/* The gate_up projection of an expert layer with SwiGLU and the 1x128 re-quantisation done in the
 * GEMM's epilogue: replaces inferop_w8a8_block_fp8_gemm_grouped_tiles (gate_up) followed by
 * inferop_silu_and_mul_quant, i.e. the reference's w8a8_block_fp8_gemm + silu_and_mul +
 * quant_fp8_per_token_group chain (include/inferop/ops.h:81-84, :54-55, :64-65;
 * kernels/silu_mul.cu:16-28), and produces the same bytes and scales bit for bit.
 *   b_q [groups][2 * inter][k] with the gate rows first and the up rows second (the layout
 *   silu_and_mul expects of the GEMM's output columns), b_scales [groups][2 * inter / 128][k / 128];
 *   q [m_total, inter] E4M3, q_scales [m_total, inter / 128] fp32;
 *   mid_dt (1 fp16 / 2 bf16): the 16-bit type the two-kernel chain would have stored gate_up in
 *   (both the GEMM result and the SwiGLU result are rounded to it before the quantisation).
 * inter % 128 == 0; q 16-byte aligned.  The 16-bit gate_up matrix is never written. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_grouped_tiles_swiglu(void* q, void* q_scales, const void* a_q,
                                                     const void* a_scales, const void* b_q,
                                                     const void* b_scales, const int32_t* tile_row0,
                                                     const int32_t* tile_meta, const int32_t* num_mtiles,
                                                     int64_t max_mtiles, int64_t m_total, int64_t groups,
                                                     int64_t inter, int64_t k, int32_t group_size,
                                                     int32_t block_n, int32_t mid_dt, void* stream);

/* ---- blockwise-FP8 GEMM for a few tokens, with no allocation
 * No counterpart in the reference: added for callers that must not trigger a device
 * allocation, such as a server that gave all device memory to its own pool at start-up, or a
 * latency-critical loop that cannot make an allocation call (driver locks, possible device
 * synchronisation).  Same arguments, contract and results as inferop_w8a8_block_fp8_gemm,
 * restricted to M <= 32, N <= 524288 and devices with at most 160 SMs (INFEROP_ERR_LIMIT
 * beyond).  The scratch the small-M kernel needs for split tiles is a fixed array of about
 * 5.3 MB inside the library image, resident on every GPU that loads the library until the
 * process exits; this call uses cudaMalloc, cudaFree and allocating library routines nowhere.
 * The first call on a device looks the array's device address up (once per device, with
 * that device current); make that first call before any stream capture.  All calls on a
 * device share the array: calls that can overlap on the GPU (different streams) race on it
 * and must be ordered by the caller.  If a wait inside the kernel ever runs out, the record is
 * kept inside the same array and inferop_device_status (which allocates nothing either)
 * reports and resets it. */
INFEROP_API int inferop_w8a8_block_fp8_gemm_fixed_scratch(void* c, const void* a_q, const void* a_scales,
                                              const void* b_q, const void* b_scales, int64_t m,
                                              int64_t n, int64_t k, int32_t group_size,
                                              int32_t block_n, int32_t out_dt, void* stream);

/* ---- diagnostics
 * Synchronises the current device and copies out the device-side status record
 * {code, block, aux0, aux1}.  code == 0 means no bounded wait has run out since
 * the last reset.  Two records exist per device: the one of the library-owned context (all
 * entry points but one) and the one inside the fixed scratch array of
 * inferop_w8a8_block_fp8_gemm_fixed_scratch; whichever is non-zero is reported (the context's
 * first), both are reset when `reset` is set.  The call itself allocates nothing.  Returns
 * INFEROP_OK, INFEROP_ERR_DEVICE_WAIT (record non-zero) or INFEROP_ERR_CUDA.  `out4` (host,
 * 4 x uint32) may be NULL.
 * Options that concern the waits (inferop_set_option): "wait_budget_us": how long a wait may
 * last before it gives up (0 = default, about a second), kept per device beside the record. */
INFEROP_API int inferop_device_status(uint32_t* out4, int reset);

/* Self-test of the hardware fp32 -> E4M3 converter used by the quantiser against the
 * software encoder of include/inferop/fp8.h (reference include/inferop/fp8.h:62-96) on every
 * fp32 bit pattern in [lo, hi), hi <= 2^32.  Synchronous.  out2 (host): [0] mismatches on
 * non-NaN inputs (must be 0), [1] mismatches on NaN inputs (sign handling, fixed up in the
 * quantiser). */
INFEROP_API int inferop_selftest_e4m3_cvt(uint64_t lo, uint64_t hi, uint64_t* out2);

/* Self-test of the quantiser's reciprocal-based division for 16-bit inputs (dt = 1 fp16,
 * 2 bf16): every finite group maximum on the fast path x every element value of that type
 * with |x| <= maximum, E4M3 byte through the reciprocal against the byte through IEEE
 * division (the oracle's x / scale, reference/reference.cpp:76).  Synchronous.
 * out3 (host, 3 x uint64): [0] mismatching pairs (must be 0), [1] pairs checked, [2] one
 * mismatching pair as (maximum bits << 32 | element bits). */
INFEROP_API int inferop_selftest_quant_div(int32_t dt, uint64_t* out3);

/* Tuning knobs for experiments and tests (process-wide, not thread-safe).
 * key: "gemm_tma_store" (-1 auto, 0, 1), "gemm_ctas" (0 = one per SM), "gemm_path" (0 auto,
 *      1 always the large-tile kernel, 2 the small-M kernel whenever M <= 128), "gemm_block_n"
 *      (0 auto, 128 or 256: tile width of the large-tile kernel; results do not depend on it),
 *      "gemm_group_m", "decode_splits", "decode_pdl", "align_ctas" (CTAs of the moe_align cluster:
 *      0 auto, 1..8; the layout does not depend on it), "grouped_rep" (1 or 0: M-tiles of at most
 *      32 rows in the replicated form) and "grouped_dynamic" (1 or 0: the grouped GEMMs with a
 *      device tile list claim their tiles from a device counter); results do not depend on them.  Returns INFEROP_ERR_SHAPE for an unknown
 *      key/value. */
INFEROP_API int inferop_set_option(const char* key, int64_t value);

#ifdef __cplusplus
}
#endif

#endif /* INFEROP_B200_H_ */
