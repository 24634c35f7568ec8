"""The C-ABI library loads without a GPU and exports everything include/inferop_b200.h declares."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "inferop_b200.h")).read()
    return sorted(set(re.findall(r"INFEROP_API[^;(]*?\b(inferop_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path():
    syms = declared_symbols()
    for s in ("inferop_quant_fp8_per_token_group", "inferop_w8a8_block_fp8_gemm", "inferop_has_cuda"):
        assert s in syms


def test_library_exports_every_declared_symbol():
    from inference_b200 import _capi
    for s in declared_symbols():
        assert hasattr(_capi.lib, s), f"{s} declared but not exported"
        assert s in _capi.SIGNATURES, f"{s} has no ctypes signature"


def test_cpp_dropin_symbols_exported():
    # the C++ names of the reference's include/inferop/ops.h for this path
    from inference_b200.build import LIB_PATH
    lib = C.CDLL(LIB_PATH)
    for mangled in ("_ZN7inferop8has_cudaEv", "_ZN7inferop12device_countEv",
                    "_ZN7inferop25quant_fp8_per_token_groupEPvS0_PKvNS_5dtypeElliS0_",
                    "_ZN7inferop27dequant_fp8_per_token_groupEPvNS_5dtypeEPKvS3_lliS0_",
                    "_ZN7inferop19w8a8_block_fp8_gemmEPvPKvS2_S2_S2_llliiNS_5dtypeES0_"):
        assert hasattr(lib, mangled)


def test_argument_validation_needs_no_gpu():
    from inference_b200 import _capi
    lib = _capi.lib
    # shape / dtype / contract checks come before any device work
    assert lib.inferop_quant_fp8_per_token_group(1, 1, 1, 2, 4, 100, 128, None) == _capi.ERR_SHAPE
    assert lib.inferop_quant_fp8_per_token_group(1, 1, 1, 3, 4, 128, 128, None) == _capi.ERR_DTYPE
    assert lib.inferop_quant_fp8_per_token_group(None, 1, 1, 2, 4, 128, 128, None) == _capi.ERR_POINTER
    assert lib.inferop_rmsnorm(1, 1, 1, 2, 0, 128, 1e-6, None) == _capi.ERR_SHAPE
    assert lib.inferop_rmsnorm(1, 1, 1, 7, 4, 128, 1e-6, None) == _capi.ERR_DTYPE
    assert lib.inferop_fused_add_rmsnorm(1, None, 1, 1, 2, 4, 128, 1e-6, None) == _capi.ERR_POINTER
    assert lib.inferop_rope_neox(1, 1, 2, 4, 8, 128, 130, 10000.0, 1.0, None) == _capi.ERR_SHAPE
    assert lib.inferop_rope_neox(1, 1, 2, 4, 8, 128, 63, 10000.0, 1.0, None) == _capi.ERR_SHAPE
    assert lib.inferop_paged_attn_decode(16, 16, 16, 16, 16, 16, 2, 1, 8, 3, 128, 16, 4, 0.1, None) == _capi.ERR_SHAPE
    assert lib.inferop_paged_attn_decode(16, 16, 16, 16, 16, 16, 2, 1, 8, 4, 100, 16, 4, 0.1, None) == _capi.ERR_SHAPE
    assert lib.inferop_paged_attn_decode(16, 16, 24, 16, 16, 16, 2, 1, 8, 4, 128, 16, 4, 0.1, None) == _capi.ERR_POINTER
    assert lib.inferop_w8a8_block_fp8_gemm(1, 1, 1, 1, 1, 4, 4, 100, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert lib.inferop_w8a8_block_fp8_gemm(1, 1, 1, 1, 1, 4, 4, 128, 64, 128, 2, None) == _capi.ERR_SHAPE
    assert lib.inferop_w8a8_block_fp8_gemm(1, 1, 1, 1, 1, 0, 4, 128, 128, 128, 2, None) == _capi.ERR_SHAPE
    assert lib.inferop_w8a8_block_fp8_gemm(1, 1, 1, 1, 1, 4, 4, 128, 128, 128, 3, None) == _capi.ERR_DTYPE
    assert lib.inferop_set_option(b"no_such_key", 1) == _capi.ERR_SHAPE
    # the knobs of the grouped launches: accepted in range, refused out of range, defaults restored
    assert lib.inferop_set_option(b"align_ctas", 9) == _capi.ERR_SHAPE
    for key, values, default in ((b"align_ctas", (1, 8), 0), (b"grouped_rep", (0,), 1), (b"grouped_dynamic", (0,), 1)):
        for v in values:
            assert lib.inferop_set_option(key, v) == _capi.OK
        assert lib.inferop_set_option(key, default) == _capi.OK
    assert _capi.status_string(_capi.ERR_ARCH)


def test_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from inference_b200 import _capi, ops
    assert not ops.has_cuda() and ops.device_count() == 0
    assert ops.device_name(0) == "-" and ops.device_sm_version(0) == -1
    # a well-formed call must be refused, not served by some fallback
    rc = _capi.lib.inferop_w8a8_block_fp8_gemm(16, 16, 16, 16, 16, 4, 4, 128, 128, 128, 2, None)
    assert rc == _capi.ERR_NO_DEVICE
    rc = _capi.lib.inferop_quant_fp8_per_token_group(16, 16, 16, 2, 4, 128, 128, None)
    assert rc == _capi.ERR_NO_DEVICE


def test_host_half_converters_match_numpy():
    """include/inferop/common.h's fp16 helpers, compiled on the fly, against numpy's float16."""
    import subprocess
    import tempfile
    import numpy as np
    src = r'''
#include "inferop/common.h"
#include "inferop/fp8.h"
extern "C" void h2f(const uint16_t* h, float* f, long n){ for(long i=0;i<n;++i) f[i]=inferop::host_convert::half_to_float(h[i]); }
extern "C" void f2h(const float* f, uint16_t* h, long n){ for(long i=0;i<n;++i) h[i]=inferop::host_convert::float_to_half_rn(f[i]); }
extern "C" void f2b(const float* f, uint16_t* h, long n){ for(long i=0;i<n;++i) h[i]=inferop::host_convert::float_to_bf16_rn(f[i]); }
extern "C" void f2e(const float* f, uint8_t* h, long n){ for(long i=0;i<n;++i) h[i]=inferop::fp8::float_to_e4m3_rn_sat(f[i]); }
extern "C" void e2f(const uint8_t* h, float* f, long n){ for(long i=0;i<n;++i) f[i]=inferop::fp8::e4m3_to_float(h[i]); }
'''
    import oracle
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.cpp"), "w").write(src)
        so = os.path.join(d, "t.so")
        subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-I", os.path.join(ROOT, "include"),
                        os.path.join(d, "t.cpp"), "-o", so], check=True)
        lib = C.CDLL(so)
        h = np.arange(65536, dtype=np.uint16)
        f = np.empty(65536, np.float32)
        lib.h2f(h.ctypes.data_as(C.c_void_p), f.ctypes.data_as(C.c_void_p), C.c_long(65536))
        want = h.view(np.float16).astype(np.float32)
        nan = np.isnan(want)
        assert np.array_equal(np.isnan(f), nan) and np.array_equal(f[~nan].view(np.uint32), want[~nan].view(np.uint32))
        rng = np.random.default_rng(0)
        x = np.concatenate([rng.integers(0, 2 ** 32, 2_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32),
                            (rng.standard_normal(1_000_000) * 10.0 ** rng.uniform(-9, 6, 1_000_000)).astype(np.float32),
                            f[~nan], np.nextafter(f[~nan], np.float32(np.inf))])
        out = np.empty(x.size, np.uint16)
        lib.f2h(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_long(x.size))
        with np.errstate(over="ignore"):
            want = x.astype(np.float16).view(np.uint16)
        ok = ~np.isnan(x)
        assert np.array_equal(out[ok], want[ok])
        lib.f2b(x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_long(x.size))
        assert np.array_equal(out[ok], oracle.bf16_narrow(x)[ok])
        o8 = np.empty(x.size, np.uint8)
        lib.f2e(x.ctypes.data_as(C.c_void_p), o8.ctypes.data_as(C.c_void_p), C.c_long(x.size))
        assert np.array_equal(o8, oracle.e4m3_encode(x))
        b = np.arange(256, dtype=np.uint8)
        lib.e2f(b.ctypes.data_as(C.c_void_p), f.ctypes.data_as(C.c_void_p), C.c_long(256))
        assert np.array_equal(f[:256].view(np.uint32), oracle.e4m3_decode(b).view(np.uint32))


def test_reference_cuda_baseline_library_exports_its_two_entry_points():
    """oracle/_ref/libinferop_ref_cuda.so (the reference's CUDA kernels for this path, built from the
    reference tree by oracle/Makefile) is what bench.py times as the secondary GPU baseline."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libinferop_ref_cuda.so")
    if not os.path.exists(path):
        pytest.skip("not built here (needs the reference tree)")
    lib = ctypes.CDLL(path)
    for name in ("refcuda_quant_fp8_per_token_group", "refcuda_w8a8_block_fp8_gemm", "refcuda_rmsnorm",
                 "refcuda_rope_neox", "refcuda_paged_attn_decode"):
        assert hasattr(lib, name), name


def test_python_wrappers_reject_mistyped_or_misshaped_operands_before_the_c_call():
    """A wrong scale shape would make a kernel read out of bounds; ops.py refuses it on the host."""
    import torch
    from inference_b200 import ops
    m, n, k = 4, 256, 256
    aq = torch.zeros((m, k), dtype=torch.uint8)
    a_s = torch.zeros((m, k // 128))
    bq = torch.zeros((n, k), dtype=torch.uint8)
    bs = torch.zeros((n // 128, k // 128))
    ops._check_quantised(aq, a_s, bq, bs)
    for bad in [(aq.float(), a_s, bq, bs), (aq, a_s.double(), bq, bs), (aq, a_s[:, :1], bq, bs),
                (aq, a_s, bq, bs[:1]), (aq, a_s, bq[:, :128], bs), (aq[0], a_s, bq, bs)]:
        with pytest.raises((ValueError, ops.InferopError)):
            ops._check_quantised(*bad)
    ops._check_quantised(aq, a_s, bq.view(2, 128, k), bs.view(2, 1, k // 128), grouped=True)
    with pytest.raises(ValueError):
        ops._check_quantised(aq, a_s, bq.view(2, 128, k), bs, grouped=True)
    with pytest.raises(ValueError):      # CUDA tensors are required
        ops.w8a8_block_fp8_gemm(aq, a_s, bq, bs)
