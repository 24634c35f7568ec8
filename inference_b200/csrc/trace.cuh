// Optional time stamps inside the GEMM kernels, for experiments: compiled out unless the
// translation unit is built with -DIB200_TRACE=1 (the shipped library is not).  A traced build
// records %globaltimer and clock64 at a few points of the first 64 K blocks of CTA 0 (pair 0)
// and exports ib200_trace_read_<tag>() to copy the record to the host.
#pragma once

#ifndef IB200_TRACE
#define IB200_TRACE 0
#endif

#if IB200_TRACE
#include <cuda_runtime.h>
#include <stdint.h>
#define IB200_TRACE_CAT2(a, b) a##b
#define IB200_TRACE_CAT(a, b) IB200_TRACE_CAT2(a, b)
static __device__ unsigned long long g_trace[2][4][64][4][2];   // [cta rank][role][K block][event][timer, clock]
static __device__ __forceinline__ void trace_at(uint32_t rank, int role, uint32_t it, int ev) {
  if (it < 64u) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g_trace[rank][role][it][ev][0] = t;
    g_trace[rank][role][it][ev][1] = static_cast<unsigned long long>(clock64());
  }
}
#define TRACE(rank, cond, role, it, ev) do { if (cond) trace_at(rank, role, it, ev); } while (0)
extern "C" __attribute__((visibility("default"))) int IB200_TRACE_CAT(ib200_trace_read_, IB200_TRACE_TAG)(void* host, size_t bytes) {
  return static_cast<int>(cudaMemcpyFromSymbol(host, g_trace, bytes < sizeof(g_trace) ? bytes : sizeof(g_trace)));
}
#else
#define TRACE(rank, cond, role, it, ev) do { } while (0)
#endif
