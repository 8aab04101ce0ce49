"""denox_b200 — sm_100a dispatch backend for denox fp16 HWC U-Nets.

The product is `libdnxcu.so` (hand written CUDA kernels behind the C ABI of
`include/dnxcu.h`).  This package is the thin host-side mirror used by the
tests and the benchmark: ctypes bindings, seeded synthetic inputs and the two
network descriptions of the benchmark configurations.  It never computes on
the CPU: if the shared library is missing, importing `denox_b200.lib` raises.
"""
from . import rng, nets  # noqa: F401

__all__ = ["rng", "nets"]
