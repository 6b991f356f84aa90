"""ctypes binding of the C harness over the C++ host layer (csrc/host/): the reference's own
Matrix / Cublas / GpuControl interface for the quantized-weight linear path."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcccc-b200-host.so")

MATRIX_NO_TRANS, MATRIX_TRANS = 0, 1

_vp, _i, _f = C.c_void_p, C.c_int, C.c_float
SYMBOLS = {
    "cccc_host_gpu_create": (_vp, [_i]),
    "cccc_host_gpu_destroy": (None, [_vp]),
    "cccc_host_gpu_sync": (None, [_vp]),
    "cccc_host_fused_calls": (_i, [_vp]),
    "cccc_host_fallback_calls": (_i, [_vp]),
    "cccc_host_matrix_view": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _f, _vp]),
    "cccc_host_matrix_new": (_vp, [_vp, _i, _i, _i, _i, _i]),
    "cccc_host_matrix_free": (None, [_vp]),
    "cccc_host_matrix_data": (_vp, [_vp]),
    "cccc_host_matrix_block_scale": (_vp, [_vp]),
    "cccc_host_matrix_quant_scale": (_f, [_vp]),
    "cccc_host_matrix_dtype": (_i, [_vp]),
    "cccc_host_matrix_quantize": (None, [_vp, _i]),
    "cccc_host_mul": (None, [_vp, _vp, _vp, _f, _f, _i, _i]),
    "cccc_host_mul_batched": (None, [_vp, _vp, _vp, _i, _i, _f, _f]),
    "cccc_host_gemm": (None, [_vp, _i, _i, _i, _i, _i, _f, _vp, _i, _i, _f, _vp, _i, _i, _f, _f, _vp, _i, _i, _vp, _vp]),
    "cccc_host_bin_open": (_vp, [C.c_char_p]),
    "cccc_host_bin_close": (None, [_vp]),
    "cccc_host_bin_has": (_i, [_vp, C.c_char_p]),
    "cccc_host_bin_bytes_read": (C.c_ulonglong, [_vp]),
    "cccc_host_bin_load_shard": (_i, [_vp, C.c_char_p, _i, _i, C.c_char, _i, _i, _vp, C.c_ulonglong, _vp, C.c_ulonglong,
                                      C.POINTER(C.c_float), C.POINTER(C.c_int), C.c_char_p, _i]),
    "cccc_host_bin_write": (_i, [C.c_char_p, _i, C.POINTER(C.c_char_p), C.POINTER(C.c_void_p), C.POINTER(C.c_ulonglong)]),
    "cccc_host_decode_create": (_vp, [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _f, _f, _f, C.c_char_p, _i]),
    "cccc_host_decode_destroy": (None, [_vp]),
    "cccc_host_decode_step": (_i, [_vp, _vp, _i, C.POINTER(C.c_int), C.POINTER(C.c_float)]),
    "cccc_host_decode_launches": (_i, [_vp]),
    "cccc_host_decode_weight_bytes": (C.c_ulonglong, [_vp]),
    "cccc_host_decode_buffer": (_vp, [_vp, C.c_char_p]),
}
_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python cccc-lite_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib
