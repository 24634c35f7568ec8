"""ctypes binding of libinferop_b200.so (the C ABI declared in include/inferop_b200.h).

The library is the only implementation: if it has not been built, importing
this module raises, and nothing falls back to torch or to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

OK = 0
ERR_SHAPE, ERR_DTYPE, ERR_POINTER, ERR_NO_DEVICE, ERR_ARCH, ERR_CUDA, ERR_LIMIT, ERR_DEVICE_WAIT = range(1, 9)

# every symbol include/inferop_b200.h declares: name -> (restype, argtypes)
_vp, _i32, _i64, _u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64
SIGNATURES = {
    "inferop_status_string": (C.c_char_p, [C.c_int]),
    "inferop_last_cuda_error": (C.c_int, []),
    "inferop_has_cuda": (C.c_int, []),
    "inferop_device_count": (C.c_int, []),
    "inferop_device_name": (C.c_char_p, [C.c_int]),
    "inferop_device_sm_version": (C.c_int, [C.c_int]),
    "inferop_quant_fp8_per_token_group": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _i64, _i32, _vp]),
    "inferop_dequant_fp8_per_token_group": (C.c_int, [_vp, _i32, _vp, _vp, _i64, _i64, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32,
                                              _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_fused_quant": (C.c_int, [_vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _i32, _i32,
                                                          _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_grouped": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.POINTER(_i64), _i64, _i64, _i64,
                                                      _i32, _i32, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_allgather": (C.c_int, [C.POINTER(_vp), _i32, _i32, _vp, _vp, _vp, _vp, _i64, _i64,
                                                        _i64, _i32, _i32, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_scatter": (C.c_int, [C.POINTER(_vp), _i32, _i32, _vp, _vp, _vp, _vp, _i64, _i64,
                                                      _i64, _i32, _i32, _vp]),
    "inferop_reduce_slots": (C.c_int, [_vp, _i32, _vp, _i32, _i64, _i64, _vp]),
    "inferop_w8a8_block_fp8_gemm_into": (C.c_int, [_vp, _i64, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32,
                                                   _vp]),
    "inferop_copy_2d_async": (C.c_int, [_vp, _i64, _vp, _i64, _i64, _i64, _vp]),
    "inferop_topk_softmax": (C.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "inferop_rmsnorm": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _i64, C.c_float, _vp]),
    "inferop_fused_add_rmsnorm": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i64, _i64, C.c_float, _vp]),
    "inferop_rmsnorm_quant": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i32, C.c_float, _vp]),
    "inferop_rope_neox": (C.c_int, [_vp, _vp, _i32, _i64, _i32, _i32, _i32, C.c_float, C.c_float, _vp]),
    "inferop_paged_attn_decode": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                            C.c_float, _vp]),
    "inferop_silu_and_mul": (C.c_int, [_vp, _vp, _i32, _i64, _i64, _vp]),
    "inferop_silu_and_mul_quant": (C.c_int, [_vp, _vp, _vp, _i32, _i64, _i64, _i32, _vp]),
    "inferop_moe_max_mtiles": (_i64, [_i64, _i32, _i32]),
    "inferop_moe_align": (C.c_int, [_vp, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "inferop_moe_scatter_quant": (C.c_int, [_vp, _vp, _vp, _i32, _vp, _i64, _i64, _i32, _i32, _vp]),
    "inferop_moe_permute_rows": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i32, _vp]),
    "inferop_moe_combine": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i64, _i64, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_grouped_tiles": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64,
                                                            _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_grouped_tiles_swiglu": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64,
                                                                   _i64, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "inferop_w8a8_block_fp8_gemm_fixed_scratch": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64,
                                                            _i32, _i32, _i32, _vp]),
    "inferop_device_status": (C.c_int, [C.POINTER(C.c_uint32), C.c_int]),
    "inferop_selftest_e4m3_cvt": (C.c_int, [_u64, _u64, C.POINTER(_u64)]),
    "inferop_selftest_quant_div": (C.c_int, [_i32, C.POINTER(_u64)]),
    "inferop_set_option": (C.c_int, [C.c_char_p, _i64]),
}


class InferopError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {status_string(status)} (status {status})")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m inference_b200.build` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def status_string(status: int) -> str:
    return lib.inferop_status_string(status).decode()


def check(status: int, what: str) -> None:
    if status != OK:
        raise InferopError(status, what)
