"""The reference's own test programs for this path compile UNMODIFIED against this library's
headers and link against libinferop_b200.so: the C++ API is a drop-in (same names, signatures,
defaults).  Needs the reference tree, so it runs only where that is present; without a GPU the
programs execute their CPU-golden halves and skip the GPU halves at run time, exactly as they
do for the reference (tests/test_util.h:175-190)."""
import os
import subprocess

import pytest

from conftest import ROOT

# the reference tree: INFEROP_REFERENCE, else a directory "reference" beside this repository
REF = os.environ.get("INFEROP_REFERENCE", os.path.abspath(os.path.join(ROOT, "..", "reference")))
pytestmark = pytest.mark.skipif(not os.path.exists(os.path.join(REF, "tests", "test_gemm.cpp")),
                                reason="reference tree not present")


def _build(name, tmp_path):
    from inference_b200.build import LIB_DIR
    exe = str(tmp_path / name)
    cmd = ["g++", "-std=c++17", "-O2", "-DINFEROP_HAVE_CUDA", "-I", os.path.join(ROOT, "include"),
           "-I", REF, "-I", "/usr/local/cuda/include",
           os.path.join(REF, "tests", name + ".cpp"), os.path.join(REF, "reference", "reference.cpp"),
           "-L", LIB_DIR, "-linferop_b200", "-L", "/usr/local/cuda/lib64", "-lcudart",
           f"-Wl,-rpath,{LIB_DIR}", "-Wl,-rpath,/usr/local/cuda/lib64", "-o", exe]
    subprocess.run(cmd, check=True, capture_output=True, text=True)
    return exe


@pytest.mark.parametrize("name", ["test_fp8", "test_quant", "test_gemm", "test_topk", "test_silu_mul", "test_rmsnorm",
                                  "test_rope", "test_paged_attn"])
def test_reference_test_program_builds_and_its_cpu_half_passes(name, tmp_path):
    import torch
    exe = _build(name, tmp_path)
    if torch.cuda.is_available():
        pytest.skip("built; the GPU halves are exercised by the parity tests, not from here")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "0 failed" in r.stdout
