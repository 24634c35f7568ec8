"""inference_b200: B200 (sm_100a) implementation of inferop's blockwise-FP8 W8A8 path.

``ops`` mirrors the reference's operator interface over torch CUDA tensors;
everything computes in ``lib/libinferop_b200.so`` (hand-written CUDA behind the
C ABI of ``include/inferop_b200.h``).  Importing ``inference_b200.ops`` fails if
that library has not been built: there is no fallback.
"""
__all__ = ["ops", "build"]
