// C ABI of libinferop_b200.so plus the C++ `namespace inferop` wrappers that
// make the library a drop-in for the reference's host API on this path
// (reference: kernels/api.cu:12-50 device info, :73-88 forwarding).
//
// The C entry points validate, return a status code and launch nothing on
// error.  The C++ wrappers reproduce the reference's observable behaviour:
// `void` return, silent no-op for an invalid quant shape or dtype
// (kernels/quant.cu:52,72), one "[inferop]" line on stderr for a GEMM contract
// violation (kernels/gemm/w8a8_block_fp8.cu:167-173).
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "inferop/ops.h"
#include "internal.h"

namespace ib200 {
namespace {

constexpr int kMaxDevices = 16;

struct DeviceTable {
  int count = 0;
  int sm[kMaxDevices] = {};
  int sms[kMaxDevices] = {};
  char name[kMaxDevices][128] = {};
  DeviceCtx ctx[kMaxDevices];
  std::mutex ctx_mutex;
};

DeviceTable& table() {
  static DeviceTable t;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n < 0) {
      cudaGetLastError();
      n = 0;
    }
    t.count = n;
    for (int i = 0; i < n && i < kMaxDevices; ++i) {
      cudaDeviceProp prop;
      if (cudaGetDeviceProperties(&prop, i) == cudaSuccess) {
        t.sm[i] = prop.major * 10 + prop.minor;
        t.sms[i] = prop.multiProcessorCount;
        snprintf(t.name[i], sizeof(t.name[i]), "%s", prop.name);
      }
    }
  });
  return t;
}

thread_local int g_last_cuda_error = 0;

}  // namespace

int note_cuda_error(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return INFEROP_ERR_CUDA;
}

int check_launch() {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
}

Options& options() {
  static Options o;
  return o;
}

DeviceCtx* current_ctx(int* err) {
  DeviceTable& t = table();
  if (t.count <= 0) {
    *err = INFEROP_ERR_NO_DEVICE;
    return nullptr;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *err = note_cuda_error(e);
    return nullptr;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    *err = INFEROP_ERR_LIMIT;
    return nullptr;
  }
  if (t.sm[dev] != 100) {
    *err = INFEROP_ERR_ARCH;
    return nullptr;
  }
  DeviceCtx* c = &t.ctx[dev];
  if (c->ordinal < 0) {
    std::lock_guard<std::mutex> lock(t.ctx_mutex);
    if (c->ordinal < 0) {
      DeviceStatus* st = nullptr;
      // the status record and, 256 bytes behind it, the tile counters
      constexpr size_t kCtxBytes = 256 + DeviceCtx::kTileCounters * sizeof(int);
      static_assert(sizeof(DeviceStatus) <= 256, "the tile counters start 256 bytes behind the status record");
      e = cudaMalloc(&st, kCtxBytes);
      if (e == cudaSuccess) e = cudaMemset(st, 0, kCtxBytes);
      if (e != cudaSuccess) {
        *err = note_cuda_error(e);
        return nullptr;
      }
      c->status = st;
      c->tile_counters = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(st) + 256);
      c->sm_version = t.sm[dev];
      c->sm_count = t.sms[dev];
      c->ordinal = dev;
    }
  }
  *err = INFEROP_OK;
  return c;
}

DeviceCtx* peek_ctx() {
  DeviceTable& t = table();
  int dev = -1;
  if (t.count <= 0 || cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  DeviceCtx* c = &t.ctx[dev];
  std::lock_guard<std::mutex> lock(t.ctx_mutex);
  return c->ordinal < 0 ? nullptr : c;
}

// Scratch set of `stream` on this device, created on first use.  False when none can be had.
bool decode_scratch(DeviceCtx* ctx, cudaStream_t stream, float** ws, int** counters) {
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  for (int i = 0; i < ctx->n_scratch; ++i) {
    if (ctx->scratch_stream[i] == stream) {
      *ws = ctx->scratch_ws[i];
      *counters = ctx->scratch_counters[i];
      return true;
    }
  }
  if (ctx->n_scratch >= DeviceCtx::kMaxStreams) return false;
  float* w = nullptr;
  int* c = nullptr;
  if (cudaMalloc(&w, decode_workspace_bytes(ctx->sm_count)) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  if (cudaMalloc(&c, kDecodeMaxTiles * sizeof(int)) != cudaSuccess ||
      cudaMemset(c, 0, kDecodeMaxTiles * sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(w);
    if (c) cudaFree(c);
    return false;
  }
  const int i = ctx->n_scratch++;
  ctx->scratch_stream[i] = stream;
  ctx->scratch_ws[i] = w;
  ctx->scratch_counters[i] = c;
  *ws = w;
  *counters = c;
  return true;
}

int quant_scratch(DeviceCtx* ctx, cudaStream_t stream, size_t q_bytes, size_t s_bytes, void** q, void** s) {
  static std::mutex m;
  std::lock_guard<std::mutex> lock(m);
  int i = 0;
  for (; i < ctx->n_qscratch; ++i)
    if (ctx->qscratch_stream[i] == stream) break;
  if (i == ctx->n_qscratch) {
    if (ctx->n_qscratch >= DeviceCtx::kMaxStreams) return INFEROP_ERR_LIMIT;
    ctx->qscratch_stream[i] = stream;
    ++ctx->n_qscratch;
  }
  if (ctx->qscratch_q_bytes[i] < q_bytes || ctx->qscratch_s_bytes[i] < s_bytes) {
    // growing: earlier calls on this stream may still read the old buffers
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (ctx->qscratch_q[i]) cudaFree(ctx->qscratch_q[i]);
    if (ctx->qscratch_s[i]) cudaFree(ctx->qscratch_s[i]);
    ctx->qscratch_q[i] = ctx->qscratch_s[i] = nullptr;
    ctx->qscratch_q_bytes[i] = ctx->qscratch_s_bytes[i] = 0;
    void *nq = nullptr, *ns = nullptr;
    e = cudaMalloc(&nq, q_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ns, s_bytes);
    if (e != cudaSuccess) {
      if (nq) cudaFree(nq);
      return note_cuda_error(e);
    }
    ctx->qscratch_q[i] = nq;
    ctx->qscratch_s[i] = ns;
    ctx->qscratch_q_bytes[i] = q_bytes;
    ctx->qscratch_s_bytes[i] = s_bytes;
  }
  *q = ctx->qscratch_q[i];
  *s = ctx->qscratch_s[i];
  return INFEROP_OK;
}

}  // namespace ib200

using namespace ib200;

extern "C" {

const char* inferop_status_string(int status) {
  switch (status) {
    case INFEROP_OK: return "ok";
    case INFEROP_ERR_SHAPE: return "invalid shape or contract violation";
    case INFEROP_ERR_DTYPE: return "unsupported dtype";
    case INFEROP_ERR_POINTER: return "null or misaligned pointer";
    case INFEROP_ERR_NO_DEVICE: return "no CUDA device";
    case INFEROP_ERR_ARCH: return "current device is not sm_100";
    case INFEROP_ERR_CUDA: return "CUDA call failed";
    case INFEROP_ERR_LIMIT: return "size beyond a documented limit";
    case INFEROP_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel ran out";
    default: return "unknown status";
  }
}

int inferop_last_cuda_error(void) { return g_last_cuda_error; }

int inferop_has_cuda(void) { return table().count > 0 ? 1 : 0; }
int inferop_device_count(void) { return table().count; }
const char* inferop_device_name(int ordinal) {
  DeviceTable& t = table();
  if (ordinal < 0 || ordinal >= t.count || ordinal >= kMaxDevices) return "-";
  return t.name[ordinal];
}
int inferop_device_sm_version(int ordinal) {
  DeviceTable& t = table();
  if (ordinal < 0 || ordinal >= t.count || ordinal >= kMaxDevices) return -1;
  return t.sm[ordinal];
}

int inferop_quant_fp8_per_token_group(void* q, void* scales, const void* x, int32_t dt,
                                      int64_t rows, int64_t cols, int32_t group_size,
                                      void* stream) {
  if (rows <= 0 || cols <= 0 || group_size <= 0 || cols % group_size != 0) return INFEROP_ERR_SHAPE;
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!q || !scales || !x) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_quant(q, scales, x, dt, rows, cols, group_size, static_cast<cudaStream_t>(stream),
                      ctx->sm_count);
}

int inferop_dequant_fp8_per_token_group(void* x, int32_t dt, const void* q, const void* scales,
                                        int64_t rows, int64_t cols, int32_t group_size,
                                        void* stream) {
  if (rows <= 0 || cols <= 0 || group_size <= 0 || cols % group_size != 0) return INFEROP_ERR_SHAPE;
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!q || !scales || !x) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_dequant(x, dt, q, scales, rows, cols, group_size,
                        static_cast<cudaStream_t>(stream), ctx->sm_count);
}

// Which kernel serves a plain GEMM call.  Measured on B200 (N x K = 18432 x 7168, 7168 x 18432,
// 24576 x 1536, 4096 x 7168, 36864 x 7168): up to 32 tokens the weight-streaming kernel is never
// slower; from 65 tokens on the large-tile kernel with 128-column tiles is 1.5-2.5 times faster;
// in between the large-tile kernel wins once there is about one 128-row weight tile per SM, and
// the weight-streaming kernel (which splits K over the idle SMs) wins below that.
static bool small_m_kernel(const DeviceCtx* ctx, int64_t m, int64_t n) {
  const int path = options().gemm_path;
  const int64_t tiles = (n + 127) / 128;
  if (path == 1 || m > kDecodeMaxM || tiles > kDecodeMaxTiles) return false;
  if (path == 2 || m <= 32) return true;
  if (m <= 64) return tiles * 4 < static_cast<int64_t>(ctx->sm_count) * 3;
  return false;
}

// Small M: the weight-streaming kernel, which needs scratch memory for split tiles.  The
// scratch is created on the first such call of each stream (a cudaMalloc: make that call
// before any stream capture); with more than DeviceCtx::kMaxStreams streams, or when the
// allocation fails, the large-tile kernel serves the call instead.  From two 128-row tiles on,
// the CTA-pair kernel.
static int gemm_dispatch(DeviceCtx* ctx, void* c, const void* a_q, const void* a_scales, const void* b_q,
                         const void* b_scales, int64_t m, int64_t n, int64_t k, int32_t out_dt, cudaStream_t s) {
  if (small_m_kernel(ctx, m, n)) {
    float* ws = nullptr;
    int* counters = nullptr;
    if (decode_scratch(ctx, s, &ws, &counters)) {
      return launch_gemm_decode(ctx, ws, counters, c, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
    }
  }
  if (use_pair_kernel(m)) return launch_gemm_pair(ctx, c, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
  return launch_gemm(ctx, c, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
}

int inferop_w8a8_block_fp8_gemm(void* c, const void* a_q, const void* a_scales, const void* b_q,
                                const void* b_scales, int64_t m, int64_t n, int64_t k,
                                int32_t group_size, int32_t block_n, int32_t out_dt,
                                void* stream) {
  if (group_size != 128 || block_n != 128 || k < 0 || k % 128 != 0 || m <= 0 || n <= 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  if (m > 0x7FFFFF00LL || n > 0x7FFFFF00LL || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!c) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (k == 0) {  // empty sum: the reference's kernel stores zeros
    const cudaError_t e = cudaMemsetAsync(c, 0, static_cast<size_t>(m) * n * (out_dt == 0 ? 4 : 2), s);
    return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
  }
  if (!a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  return gemm_dispatch(ctx, c, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
}

int inferop_w8a8_block_fp8_gemm_fused_quant(void* c, const void* a, int32_t a_dt, const void* b_q,
                                            const void* b_scales, int64_t m, int64_t n, int64_t k,
                                            int32_t group_size, int32_t block_n, int32_t out_dt,
                                            void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || m <= 0 || n <= 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt < 0 || out_dt > 2 || (a_dt != 1 && a_dt != 2)) return INFEROP_ERR_DTYPE;
  if (m > 0x7FFFFF00LL || n > 0x7FFFFF00LL || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (m <= kFusedMaxM && (n + 127) / 128 > kDecodeMaxTiles) return INFEROP_ERR_LIMIT;
  if (!c || !a || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (m <= kFusedMaxM && options().fused_prologue) {
    // A few tokens, on request (option fused_prologue): one launch.  Four warps of every CTA of the
    // small-M kernel quantise the token tiles of its units into a shared-memory ring, ahead of the
    // weight stream.  Level with the chained pair below at M = 1 and slower from M = 4 on (every CTA
    // repeats the quantisation and four warps do not keep up with the weight stream), so not the default.
    float* ws = nullptr;
    int* counters = nullptr;
    if (!decode_scratch(ctx, s, &ws, &counters)) return INFEROP_ERR_LIMIT;   // no scratch set left for this stream
    return launch_gemm_decode_fused(ctx, ws, counters, c, a, a_dt, b_q, b_scales, m, n, k, out_dt, s);
  }
  // More tokens (quantising inside the GEMM would repeat the work once per column tile): two launches.  The quantiser writes into scratch of this
  // stream (grown on demand: a cudaMalloc when a call is larger than any before it on the stream)
  // and signals its dependents at once; the GEMM, launched with programmatic stream
  // serialisation, sets itself up underneath it.  Same bits as the two separate calls.
  void *q = nullptr, *qs = nullptr;
  int rc = quant_scratch(ctx, s, static_cast<size_t>(m) * k, static_cast<size_t>(m) * (k / 128) * 4, &q, &qs);
  if (rc != INFEROP_OK) return rc;
  rc = launch_quant(q, qs, a, a_dt, m, k, 128, s, ctx->sm_count);
  if (rc != INFEROP_OK) return rc;
  return gemm_dispatch(ctx, c, q, qs, b_q, b_scales, m, n, k, out_dt, s);
}

int inferop_w8a8_block_fp8_gemm_grouped(void* c, const void* a_q, const void* a_scales, const void* b_q,
                                        const void* b_scales, const int64_t* m_per_group,
                                        int64_t groups, int64_t n, int64_t k, int32_t group_size,
                                        int32_t block_n, int32_t out_dt, void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 ||
      groups <= 0 || !m_per_group) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  int64_t m_total = 0;
  for (int64_t g = 0; g < groups; ++g) {
    if (m_per_group[g] < 0) return INFEROP_ERR_SHAPE;
    m_total += m_per_group[g];
  }
  if (m_total > 0x7FFFFF00LL || groups * n > 0x7FFFFF00LL || k > 0x7FFFFF00LL || groups >= (1 << 22)) {
    return INFEROP_ERR_LIMIT;
  }
  if (!c || !a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_gemm_grouped(ctx, c, a_q, a_scales, b_q, b_scales, m_per_group, groups, n, k, out_dt,
                             static_cast<cudaStream_t>(stream));
}

int inferop_w8a8_block_fp8_gemm_allgather(void* const* c_peers, int32_t n_peers, int32_t rank,
                                          const void* a_q, const void* a_scales, const void* b_q,
                                          const void* b_scales, int64_t m, int64_t n, int64_t k,
                                          int32_t group_size, int32_t block_n, int32_t out_dt,
                                          void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || m <= 0 || n <= 0 ||
      n % 128 != 0 || n_peers < 1 || n_peers > 8 || rank < 0 || rank >= n_peers) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt != 1 && out_dt != 2) return INFEROP_ERR_DTYPE;
  if (m > 0x7FFFFF00LL || n * n_peers > 0x7FFFFF00LL || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!c_peers || !a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // a few tokens: the weight-streaming kernel, storing straight into every rank's buffer
  if (small_m_kernel(ctx, m, n)) {
    float* ws;
    int* counters;
    if (decode_scratch(ctx, s, &ws, &counters)) {
      void* dst[8];
      for (int i = 0; i < n_peers; ++i) dst[i] = c_peers[(rank + 1 + i) % n_peers];   // own buffer last
      for (int i = 0; i < n_peers; ++i) {
        if (!dst[i] || (reinterpret_cast<uintptr_t>(dst[i]) & 15u)) return INFEROP_ERR_POINTER;
      }
      return launch_gemm_decode_to(ctx, ws, counters, dst, n_peers, n * n_peers, rank * n, a_q, a_scales,
                                   b_q, b_scales, m, n, k, out_dt, s);
    }
  }
  return launch_gemm_allgather(ctx, c_peers, n_peers, rank, a_q, a_scales, b_q, b_scales, m, n, k,
                               out_dt, s);
}

int inferop_w8a8_block_fp8_gemm_into(void* c_base, int64_t ldc, int64_t col0, const void* a_q, const void* a_scales,
                                     const void* b_q, const void* b_scales, int64_t m, int64_t n, int64_t k,
                                     int32_t group_size, int32_t block_n, int32_t out_dt, void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || m <= 0 || n <= 0 || n % 128 != 0 ||
      ldc <= 0 || col0 < 0 || col0 + n > ldc || col0 % 8 != 0 || ldc % 8 != 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt != 1 && out_dt != 2) return INFEROP_ERR_DTYPE;
  if (m > 0x7FFFFF00LL || ldc > 0x7FFFFF00LL || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!c_base || !a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u) ||
      (reinterpret_cast<uintptr_t>(c_base) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (small_m_kernel(ctx, m, n)) {
    float* ws;
    int* counters;
    if (decode_scratch(ctx, s, &ws, &counters)) {
      void* dst[1] = {c_base};
      return launch_gemm_decode_to(ctx, ws, counters, dst, 1, ldc, col0, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
    }
  }
  return launch_gemm_into(ctx, c_base, ldc, col0, a_q, a_scales, b_q, b_scales, m, n, k, out_dt, s);
}

int inferop_w8a8_block_fp8_gemm_scatter(void* const* slot_peers, int32_t n_peers, int32_t rank,
                                        const void* a_q, const void* a_scales, const void* b_q,
                                        const void* b_scales, int64_t m, int64_t n, int64_t k,
                                        int32_t group_size, int32_t block_n, void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || m <= 0 || n <= 0 || n % 4 != 0 ||
      n_peers < 1 || n_peers > 8 || rank < 0 || rank >= n_peers || m % (128 * n_peers) != 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (m > 0x7FFFFF00LL || n > 0x7FFFFF00LL || k > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!slot_peers || !a_q || !a_scales || !b_q || !b_scales) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_gemm_scatter(ctx, slot_peers, n_peers, rank, a_q, a_scales, b_q, b_scales, m, n, k,
                             static_cast<cudaStream_t>(stream));
}

int inferop_reduce_slots(void* out, int32_t out_dt, const void* slots, int32_t n_peers, int64_t rows,
                         int64_t n, void* stream) {
  if (n_peers < 1 || n_peers > 8 || rows <= 0 || n <= 0 || n % 4 != 0) return INFEROP_ERR_SHAPE;
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  if (!out || !slots) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(slots) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u)) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_reduce_slots(out, out_dt, slots, n_peers, rows * n, static_cast<cudaStream_t>(stream),
                             ctx->sm_count);
}

int inferop_copy_2d_async(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                          int64_t width_bytes, int64_t rows, void* stream) {
  if (width_bytes <= 0 || rows <= 0 || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes) {
    return INFEROP_ERR_SHAPE;
  }
  if (!dst || !src) return INFEROP_ERR_POINTER;
  const cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch_bytes), src,
                                          static_cast<size_t>(src_pitch_bytes), static_cast<size_t>(width_bytes),
                                          static_cast<size_t>(rows), cudaMemcpyDeviceToDevice,
                                          static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? INFEROP_OK : note_cuda_error(e);
}

int inferop_topk_softmax(int32_t* topk_ids, void* topk_weights, const void* logits, int32_t tokens,
                         int32_t num_experts, int32_t topk, int32_t renormalize, void* stream) {
  if (tokens <= 0 || num_experts <= 0 || num_experts > 1024 || topk <= 0 || topk > num_experts) {
    return INFEROP_ERR_SHAPE;
  }
  if (!topk_ids || !topk_weights || !logits) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_topk_softmax(topk_ids, static_cast<float*>(topk_weights), static_cast<const float*>(logits),
                             tokens, num_experts, topk, renormalize ? 1 : 0,
                             static_cast<cudaStream_t>(stream));
}

int inferop_rmsnorm(void* out, const void* in, const void* weight, int32_t dt, int64_t rows, int64_t cols,
                    float eps, void* stream) {
  if (rows <= 0 || cols <= 0) return INFEROP_ERR_SHAPE;
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!out || !in || !weight) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_rmsnorm(out, nullptr, in, weight, dt, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int inferop_fused_add_rmsnorm(void* residual, void* out, const void* x, const void* weight, int32_t dt,
                              int64_t rows, int64_t cols, float eps, void* stream) {
  if (rows <= 0 || cols <= 0) return INFEROP_ERR_SHAPE;
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!residual || !out || !x || !weight) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_rmsnorm(out, residual, x, weight, dt, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int inferop_rmsnorm_quant(void* q, void* scales, void* residual, const void* in, const void* weight, int32_t dt,
                          int64_t rows, int64_t cols, int32_t group_size, float eps, void* stream) {
  if (rows <= 0 || cols <= 0 || group_size != 128 || cols % 128 != 0 || cols > 16384) return INFEROP_ERR_SHAPE;
  if (dt != 1 && dt != 2) return INFEROP_ERR_DTYPE;
  if (!q || !scales || !in || !weight) return INFEROP_ERR_POINTER;
  if (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(residual)) & 15u) ||
      (reinterpret_cast<uintptr_t>(q) & 7u) || (reinterpret_cast<uintptr_t>(scales) & 3u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_rmsnorm_quant(q, scales, residual, in, weight, dt, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int inferop_rope_neox(void* qkv, const int64_t* positions, int32_t dt, int64_t tokens, int32_t heads,
                      int32_t head_dim, int32_t rotary_dim, float base, float yarn_factor, void* stream) {
  if (tokens <= 0 || heads <= 0 || head_dim <= 0 || rotary_dim <= 0 || rotary_dim > head_dim ||
      (rotary_dim & 1) != 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!qkv || !positions) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_rope_neox(qkv, positions, dt, tokens, heads, head_dim, rotary_dim, base, yarn_factor,
                          static_cast<cudaStream_t>(stream));
}

int inferop_paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                              const int32_t* block_tables, const int32_t* seq_lens, int32_t dt, int32_t batch,
                              int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                              int32_t max_blocks_per_seq, float scale, void* stream) {
  if (batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0 || block_size <= 0 ||
      max_blocks_per_seq <= 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256)) {
    return INFEROP_ERR_SHAPE;
  }
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (batch > 65535 || static_cast<int64_t>(max_blocks_per_seq) * block_size > 0x7FFFFF00LL) return INFEROP_ERR_LIMIT;
  if (!out || !q || !k_cache || !v_cache || !block_tables || !seq_lens) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(k_cache) & 15u) || (reinterpret_cast<uintptr_t>(v_cache) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int splits = paged_attn_splits(ctx->sm_count, batch, num_heads, num_kv_heads, block_size, max_blocks_per_seq);
  void *ws = nullptr, *unused = nullptr;
  if (splits > 1) {
    // partial states of the token ranges: scratch of this stream, grown on demand (a cudaMalloc when a
    // call needs more than any before it on the stream)
    const int rc = quant_scratch(ctx, s, paged_attn_workspace_bytes(splits, batch, num_heads, head_dim), 16, &ws, &unused);
    if (rc != INFEROP_OK) return rc;
  }
  return launch_paged_attn_decode(out, q, k_cache, v_cache, block_tables, seq_lens, dt, batch, num_heads, num_kv_heads,
                                  head_dim, block_size, max_blocks_per_seq, scale, splits, static_cast<float*>(ws), s);
}

int inferop_silu_and_mul(void* out, const void* gate_up, int32_t dt, int64_t tokens, int64_t d,
                         void* stream) {
  if (tokens <= 0 || d <= 0) return INFEROP_ERR_SHAPE;
  if (dt < 0 || dt > 2) return INFEROP_ERR_DTYPE;
  if (!out || !gate_up) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_silu_and_mul(out, gate_up, dt, tokens, d, static_cast<cudaStream_t>(stream), ctx->sm_count);
}

int inferop_silu_and_mul_quant(void* q, void* scales, const void* gate_up, int32_t dt, int64_t tokens,
                               int64_t d, int32_t group_size, void* stream) {
  if (tokens <= 0 || d <= 0 || group_size != 128 || d % 128 != 0) return INFEROP_ERR_SHAPE;
  if (dt != 1 && dt != 2) return INFEROP_ERR_DTYPE;
  if (!q || !scales || !gate_up) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(gate_up) & 15u) || (reinterpret_cast<uintptr_t>(q) & 7u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_silu_and_mul_quant(q, scales, gate_up, dt, tokens, d, static_cast<cudaStream_t>(stream),
                                   ctx->sm_count);
}

int64_t inferop_moe_max_mtiles(int64_t tokens, int32_t topk, int32_t num_experts) {
  if (tokens < 0 || topk <= 0 || num_experts <= 0) return 0;
  return moe_max_mtiles(tokens * topk, num_experts);
}

int inferop_moe_align(const int32_t* topk_ids, int64_t tokens, int32_t topk, int32_t num_experts,
                      int32_t* counts, int32_t* offsets, int32_t* pos, int32_t* src_token,
                      int32_t* tile_row0, int32_t* tile_meta, int32_t* num_mtiles, void* stream) {
  if (tokens <= 0 || topk <= 0 || num_experts <= 0 || num_experts > 1024) return INFEROP_ERR_SHAPE;
  if (tokens * topk > 0x7FFFFF00LL || num_experts >= (1 << 22)) return INFEROP_ERR_LIMIT;
  if (!topk_ids || !counts || !offsets || !pos || !src_token || !tile_row0 || !tile_meta || !num_mtiles) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_moe_align(topk_ids, tokens, topk, num_experts, counts, offsets, pos, src_token, tile_row0,
                          tile_meta, num_mtiles, static_cast<cudaStream_t>(stream));
}

int inferop_moe_scatter_quant(void* q, void* scales, const void* x, int32_t dt, const int32_t* pos,
                              int64_t tokens, int64_t cols, int32_t topk, int32_t group_size,
                              void* stream) {
  if (tokens <= 0 || cols <= 0 || topk <= 0 || group_size != 128 || cols % 128 != 0) return INFEROP_ERR_SHAPE;
  if (dt != 1 && dt != 2) return INFEROP_ERR_DTYPE;
  if (!q || !scales || !x || !pos) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 7u)) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_moe_scatter_quant(q, scales, x, dt, pos, tokens, cols, topk,
                                  static_cast<cudaStream_t>(stream), ctx->sm_count);
}

int inferop_moe_permute_rows(void* dst, const void* src, const int32_t* perm, int64_t rows, int64_t row_bytes,
                             int32_t gather, void* stream) {
  if (rows <= 0 || row_bytes <= 0 || row_bytes % 16 != 0) return INFEROP_ERR_SHAPE;
  if (!dst || !src || !perm) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(dst) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u)) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_permute_rows(dst, src, perm, rows, row_bytes, gather ? 1 : 0, static_cast<cudaStream_t>(stream),
                             ctx->sm_count);
}

int inferop_moe_combine(void* out, const void* y, const void* topk_weights, const int32_t* pos, int32_t dt,
                        int64_t tokens, int64_t hidden, int32_t topk, void* stream) {
  if (tokens <= 0 || hidden <= 0 || topk <= 0 || hidden % 8 != 0) return INFEROP_ERR_SHAPE;
  if (dt != 1 && dt != 2) return INFEROP_ERR_DTYPE;
  if (!out || !y || !topk_weights || !pos) return INFEROP_ERR_POINTER;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(y) & 15u)) return INFEROP_ERR_POINTER;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_moe_combine(out, y, static_cast<const float*>(topk_weights), pos, dt, tokens, hidden, topk,
                            static_cast<cudaStream_t>(stream), ctx->sm_count);
}

int inferop_w8a8_block_fp8_gemm_grouped_tiles(void* c, const void* a_q, const void* a_scales,
                                              const void* b_q, const void* b_scales,
                                              const int32_t* tile_row0, const int32_t* tile_meta,
                                              const int32_t* num_mtiles, int64_t max_mtiles,
                                              int64_t m_total, int64_t groups, int64_t n, int64_t k,
                                              int32_t group_size, int32_t block_n, int32_t out_dt,
                                              void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || n <= 0 || n % 128 != 0 ||
      groups <= 0 || m_total <= 0 || max_mtiles <= 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (out_dt < 0 || out_dt > 2) return INFEROP_ERR_DTYPE;
  if (m_total > 0x7FFFFF00LL || groups * n > 0x7FFFFF00LL || k > 0x7FFFFF00LL || groups >= (1 << 22)) {
    return INFEROP_ERR_LIMIT;
  }
  if (!c || !a_q || !a_scales || !b_q || !b_scales || !tile_row0 || !tile_meta || !num_mtiles) {
    return INFEROP_ERR_POINTER;
  }
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_gemm_grouped_dev(ctx, c, a_q, a_scales, b_q, b_scales, tile_row0, tile_meta, num_mtiles,
                                 max_mtiles, m_total, groups, n, k, out_dt, static_cast<cudaStream_t>(stream));
}

int inferop_w8a8_block_fp8_gemm_grouped_tiles_swiglu(void* q, void* q_scales, const void* a_q,
                                                     const void* a_scales, const void* b_q,
                                                     const void* b_scales, const int32_t* tile_row0,
                                                     const int32_t* tile_meta, const int32_t* num_mtiles,
                                                     int64_t max_mtiles, int64_t m_total, int64_t groups,
                                                     int64_t inter, int64_t k, int32_t group_size,
                                                     int32_t block_n, int32_t mid_dt, void* stream) {
  if (group_size != 128 || block_n != 128 || k <= 0 || k % 128 != 0 || inter <= 0 || inter % 128 != 0 ||
      groups <= 0 || m_total <= 0 || max_mtiles <= 0) {
    return INFEROP_ERR_SHAPE;
  }
  if (mid_dt != 1 && mid_dt != 2) return INFEROP_ERR_DTYPE;
  if (m_total > 0x7FFFFF00LL || groups * 2 * inter > 0x7FFFFF00LL || k > 0x7FFFFF00LL || groups >= (1 << 22)) {
    return INFEROP_ERR_LIMIT;
  }
  if (!q || !q_scales || !a_q || !a_scales || !b_q || !b_scales || !tile_row0 || !tile_meta || !num_mtiles) {
    return INFEROP_ERR_POINTER;
  }
  if ((reinterpret_cast<uintptr_t>(a_q) & 15u) || (reinterpret_cast<uintptr_t>(b_q) & 15u) ||
      (reinterpret_cast<uintptr_t>(q) & 15u)) {
    return INFEROP_ERR_POINTER;
  }
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return launch_gemm_swiglu(ctx, q, static_cast<float*>(q_scales), a_q, a_scales, b_q, b_scales, tile_row0,
                            tile_meta, num_mtiles, max_mtiles, m_total, groups, inter, k, mid_dt,
                            static_cast<cudaStream_t>(stream));
}

int inferop_device_status(uint32_t* out4, int reset) {
  // Allocates nothing: reads the record of the library-owned context if one exists on this
  // device, and the record inside the fixed scratch array if the allocation-free entry point
  // has run here.  The first non-zero record is reported.
  if (table().count <= 0) return INFEROP_ERR_NO_DEVICE;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return note_cuda_error(e);
  DeviceStatus host = {0, 0, 0, 0, 0};
  if (DeviceCtx* ctx = peek_ctx()) {
    e = cudaMemcpy(&host, ctx->status, kStatusRecordBytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return note_cuda_error(e);
    if (reset) {
      e = cudaMemset(ctx->status, 0, kStatusRecordBytes);   // the wait budget behind the record stays
      if (e != cudaSuccess) return note_cuda_error(e);
    }
  }
  DeviceStatus fixed = {0, 0, 0, 0, 0};
  bool used = false;
  const int rc = fixed_scratch_status(&fixed, reset != 0, &used);
  if (rc != INFEROP_OK) return rc;
  if (host.code == 0 && used && fixed.code != 0) host = fixed;
  if (out4) memcpy(out4, &host, kStatusRecordBytes);
  return host.code == 0 ? INFEROP_OK : INFEROP_ERR_DEVICE_WAIT;
}

int inferop_selftest_e4m3_cvt(uint64_t lo, uint64_t hi, uint64_t* out2) {
  if (!out2 || hi < lo || hi > (1ULL << 32)) return INFEROP_ERR_SHAPE;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return run_cvt_selftest(lo, hi, out2, ctx->sm_count);
}

int inferop_selftest_quant_div(int32_t dt, uint64_t* out3) {
  if (!out3 || (dt != 1 && dt != 2)) return INFEROP_ERR_SHAPE;
  int err;
  DeviceCtx* ctx = current_ctx(&err);
  if (!ctx) return err;
  return run_div_selftest(dt == 2 ? 1 : 0, out3, ctx->sm_count);
}

int inferop_set_option(const char* key, int64_t value) {
  if (!key) return INFEROP_ERR_SHAPE;
  Options& o = options();
  if (!strcmp(key, "gemm_block_n")) {
    if (value != 0 && value != 128 && value != 256) return INFEROP_ERR_SHAPE;
    o.gemm_block_n = static_cast<int>(value);
  } else if (!strcmp(key, "gemm_tma_store")) {
    if (value < -1 || value > 1) return INFEROP_ERR_SHAPE;
    o.gemm_tma_store = static_cast<int>(value);
  } else if (!strcmp(key, "gemm_group_m")) {
    if (value < 0 || value > 4096) return INFEROP_ERR_SHAPE;
    o.gemm_group_m = static_cast<int>(value);
  } else if (!strcmp(key, "decode_pdl")) {
    o.decode_pdl = value != 0;
  } else if (!strcmp(key, "decode_deal")) {
    if (value < 0 || value > 1) return INFEROP_ERR_SHAPE;
    o.decode_deal = static_cast<int>(value);
  } else if (!strcmp(key, "decode_splits")) {
    if (value < 0 || value > 1024) return INFEROP_ERR_SHAPE;
    o.decode_splits = static_cast<int>(value);
  } else if (!strcmp(key, "gemm_path")) {
    if (value < 0 || value > 2) return INFEROP_ERR_SHAPE;
    o.gemm_path = static_cast<int>(value);
  } else if (!strcmp(key, "debug_no_loads")) {
    o.debug_no_loads = value != 0;
  } else if (!strcmp(key, "wait_budget_us")) {
    // how long a wait inside a kernel may last before it gives up (0 = the default, about a second);
    // stored beside the status record of the current device
    if (value < 0 || value > 10000000) return INFEROP_ERR_SHAPE;
    int err;
    DeviceCtx* ctx = current_ctx(&err);
    if (!ctx) return err;
    const unsigned long long cycles = static_cast<unsigned long long>(value) * 2000ull;   // at about 2 GHz
    const cudaError_t e = cudaMemcpy(&ctx->status->budget_cycles, &cycles, sizeof(cycles), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return note_cuda_error(e);
  } else if (!strcmp(key, "gemm_pair")) {
    if (value < -1 || value > 1) return INFEROP_ERR_SHAPE;
    o.gemm_pair = static_cast<int>(value);
  } else if (!strcmp(key, "pdl_trigger")) {
    o.pdl_trigger = value != 0;
  } else if (!strcmp(key, "fused_prologue")) {
    o.fused_prologue = value != 0;
  } else if (!strcmp(key, "attn_heads_per_cta")) {
    o.attn_heads_per_cta = static_cast<int>(value);
  } else if (!strcmp(key, "attn_splits")) {
    o.attn_splits = static_cast<int>(value);
  } else if (!strcmp(key, "grouped_rep")) {
    o.grouped_rep = value != 0;
  } else if (!strcmp(key, "grouped_dynamic")) {
    o.grouped_dynamic = value != 0;
  } else if (!strcmp(key, "align_ctas")) {
    if (value < 0 || value > 8) return INFEROP_ERR_SHAPE;
    o.align_ctas = static_cast<int>(value);
  } else if (!strcmp(key, "quant_pdl")) {
    o.quant_pdl = value != 0;
  } else if (!strcmp(key, "gemm_pdl")) {
    o.gemm_pdl = value != 0;
  } else if (!strcmp(key, "gemm_ctas")) {
    if (value < 0 || value > 1024) return INFEROP_ERR_SHAPE;
    o.gemm_ctas = static_cast<int>(value);
  } else {
    return INFEROP_ERR_SHAPE;
  }
  return INFEROP_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// C++ drop-in wrappers (include/inferop/ops.h)
// ---------------------------------------------------------------------------
namespace inferop {

bool has_cuda() { return inferop_has_cuda() != 0; }
int device_count() { return inferop_device_count(); }
const char* device_name(int ordinal) { return inferop_device_name(ordinal); }
int device_sm_version(int ordinal) { return inferop_device_sm_version(ordinal); }

namespace {
void report(const char* op, int rc) {
  // shape / dtype problems follow the reference (silent or a contract line, printed by the
  // caller below); anything else is specific to this build and always reported
  if (rc != INFEROP_OK && rc != INFEROP_ERR_SHAPE && rc != INFEROP_ERR_DTYPE) {
    fprintf(stderr, "[inferop] %s: %s\n", op, inferop_status_string(rc));
  }
}
}  // namespace

void quant_fp8_per_token_group(void* q, void* scales, const void* x, dtype dt, int64_t rows,
                               int64_t cols, int group_size, void* stream) {
  report("quant_fp8_per_token_group",
         inferop_quant_fp8_per_token_group(q, scales, x, static_cast<int32_t>(dt), rows, cols,
                                           group_size, stream));
}

void dequant_fp8_per_token_group(void* x, dtype dt, const void* q, const void* scales,
                                 int64_t rows, int64_t cols, int group_size, void* stream) {
  report("dequant_fp8_per_token_group",
         inferop_dequant_fp8_per_token_group(x, static_cast<int32_t>(dt), q, scales, rows, cols,
                                             group_size, stream));
}

void w8a8_block_fp8_gemm(void* c, const void* a_q, const void* a_scales, const void* b_q,
                         const void* b_scales, int64_t m, int64_t n, int64_t k, int group_size,
                         int block_n, dtype out_dt, void* stream) {
  const int rc = inferop_w8a8_block_fp8_gemm(c, a_q, a_scales, b_q, b_scales, m, n, k, group_size,
                                             block_n, static_cast<int32_t>(out_dt), stream);
  if (rc == INFEROP_ERR_SHAPE) {
    fprintf(stderr,
            "[inferop] w8a8_block_fp8_gemm: requires group_size=128, block_n=128, K%%128==0, "
            "M>0, N>0 (got gs=%d bn=%d m=%lld n=%lld k=%lld)\n",
            group_size, block_n, static_cast<long long>(m), static_cast<long long>(n),
            static_cast<long long>(k));
  }
  report("w8a8_block_fp8_gemm", rc);
}

void topk_softmax(int32_t* topk_ids, void* topk_weights, const void* logits, int tokens,
                  int num_experts, int topk, bool renormalize, void* stream) {
  report("topk_softmax", inferop_topk_softmax(topk_ids, topk_weights, logits, tokens, num_experts, topk,
                                              renormalize ? 1 : 0, stream));
}

void rmsnorm(void* out, const void* in, const void* weight, dtype dt, int64_t rows, int64_t cols, float eps,
             void* stream) {
  report("rmsnorm", inferop_rmsnorm(out, in, weight, static_cast<int32_t>(dt), rows, cols, eps, stream));
}

void fused_add_rmsnorm(void* residual, void* out, const void* x, const void* weight, dtype dt, int64_t rows,
                       int64_t cols, float eps, void* stream) {
  report("fused_add_rmsnorm",
         inferop_fused_add_rmsnorm(residual, out, x, weight, static_cast<int32_t>(dt), rows, cols, eps, stream));
}

void rope_neox(void* qkv, const int64_t* positions, dtype dt, int64_t tokens, int heads, int head_dim,
               int rotary_dim, float base, float yarn_factor, void* stream) {
  report("rope_neox", inferop_rope_neox(qkv, positions, static_cast<int32_t>(dt), tokens, heads, head_dim,
                                        rotary_dim, base, yarn_factor, stream));
}

void paged_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache,
                       const int32_t* block_tables, const int32_t* seq_lens, dtype dt, int batch, int num_heads,
                       int num_kv_heads, int head_dim, int block_size, int max_blocks_per_seq, float scale,
                       void* stream) {
  report("paged_attn_decode",
         inferop_paged_attn_decode(out, q, k_cache, v_cache, block_tables, seq_lens, static_cast<int32_t>(dt), batch,
                                   num_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq, scale, stream));
}

void silu_and_mul(void* out, const void* gate_up, dtype dt, int64_t tokens, int64_t d, void* stream) {
  report("silu_and_mul", inferop_silu_and_mul(out, gate_up, static_cast<int32_t>(dt), tokens, d, stream));
}

}  // namespace inferop
