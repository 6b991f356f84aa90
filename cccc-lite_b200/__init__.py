"""B200 (sm_100a) quantized-weight linear for cccc: the host-side Python view of the library.

The directory name carries a hyphen, so it is loaded by path under the module name
`cccc_lite_b200` (see `load_package()` in __graft_entry__.py).  Everything that computes lives
in the CUDA library (csrc/); this package binds its C-ABI (capi) and, for the benchmark and the
tests, drives it with torch tensors that only hold device memory.
"""
from . import capi, hostapi  # noqa: F401
from .capi import (BFLOAT16, DOUBLE, FLOAT, FP4_E2M1, FP8_E4M3, FP8_E5M2, HALF, lib)  # noqa: F401
