// Host-side construction of TMA tensor maps.  The driver's
// cuTensorMapEncodeTiled is reached through the runtime's driver-entry-point
// query, so the library links against the CUDA runtime only.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "internal.h"

namespace ib200 {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeFn>(sym);
    }
  });
  return fn;
}

}  // namespace

int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows,
                       uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols,
                       bool swizzle128) {
  EncodeFn fn = encode_fn();
  if (!fn) return INFEROP_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (pitch_bytes & 15u) != 0) {
    return INFEROP_ERR_POINTER;
  }
  const CUtensorMapDataType type = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                   : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const cuuint64_t dims[2] = {cols, rows};          // innermost first
  const cuuint64_t strides[1] = {pitch_bytes};      // byte stride of dimension 1
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r =
      fn(out, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
         CU_TENSOR_MAP_INTERLEAVE_NONE,
         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    note_cuda_error(cudaErrorInvalidValue);
    return INFEROP_ERR_CUDA;
  }
  return INFEROP_OK;
}

}  // namespace ib200
