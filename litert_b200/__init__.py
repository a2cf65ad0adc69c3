"""litert_b200: B200 (sm_100a) kernels and delegate for LiteRT's quantized-inference hot path.

The compute lives in litert_b200/lib/liblitert_b200.so (CUDA, C ABI declared in include/litert_b200.h).
This package is the Python host mirror of that ABI; torch is used for device memory and streams only.
There is no CPU fallback: importing `ops` without the built library raises.
"""
__all__ = ["ops", "build"]
