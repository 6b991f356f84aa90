"""ctypes/numpy front end of the CPU oracle (oracle/cccc_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline leg of the benchmark may import this
module; the product library never does.  Each wrapper keeps the name and argument meaning
of the C function it calls; see that file for the reference lines each one follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libcccc_oracle.so")
_lib = None

# cccc::DataType (cccc/types.h:24-34)
FLOAT, DOUBLE, HALF, BFLOAT16, FP8_E4M3, FP8_E5M2, FP4_E2M1 = range(7)


def build(force: bool = False) -> str:
    """Compile the C oracle (and, if the reference tree is mounted, oracle/_ref)."""
    srcs = [os.path.join(_HERE, "cccc_oracle.c"), os.path.join(_HERE, "decode_ops_oracle.c")]
    if force or not os.path.exists(_LIB_PATH) or any(os.path.getmtime(_LIB_PATH) < os.path.getmtime(s) for s in srcs):
        subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        u8p, u16p, f32p = C.POINTER(C.c_uint8), C.POINTER(C.c_uint16), C.POINTER(C.c_float)
        L.oracle_e4m3_to_float.restype = C.c_float
        L.oracle_e4m3_to_float.argtypes = [C.c_uint8]
        L.oracle_e5m2_to_float.restype = C.c_float
        L.oracle_e5m2_to_float.argtypes = [C.c_uint8]
        L.oracle_float_to_e4m3.restype = C.c_uint8
        L.oracle_float_to_e4m3.argtypes = [C.c_float, C.c_float]
        L.oracle_float_to_e5m2.restype = C.c_uint8
        L.oracle_float_to_e5m2.argtypes = [C.c_float, C.c_float]
        L.oracle_fp4_nibble_to_float.restype = C.c_float
        L.oracle_fp4_nibble_to_float.argtypes = [C.c_uint8]
        L.oracle_float_to_fp4.restype = C.c_uint8
        L.oracle_float_to_fp4.argtypes = [C.c_float]
        L.oracle_float_to_bf16_rne.restype = C.c_uint16
        L.oracle_float_to_bf16_rne.argtypes = [C.c_float]
        L.oracle_float_to_bf16_trunc.restype = C.c_uint16
        L.oracle_float_to_bf16_trunc.argtypes = [C.c_float]
        L.oracle_fp8_to_bf16.argtypes = [u8p, C.c_int, u16p, C.c_size_t, C.c_float]
        L.oracle_fp8_to_float.argtypes = [u8p, C.c_int, f32p, C.c_size_t, C.c_float]
        L.oracle_float_to_fp8.argtypes = [f32p, u8p, C.c_int, C.c_size_t, C.c_float]
        L.oracle_fp4_to_bf16.argtypes = [u8p, u16p, C.c_size_t, C.c_float]
        L.oracle_fp4_packed_to_float.argtypes = [u8p, f32p, C.c_size_t, C.c_float]
        L.oracle_float_to_fp4_packed.argtypes = [f32p, u8p, C.c_size_t, C.c_float]
        L.oracle_fp4_blockscale_to_bf16.argtypes = [u8p, u8p, u16p, C.c_size_t, C.c_uint]
        L.oracle_float_to_fp4_blockscale.argtypes = [f32p, u8p, u8p, C.c_size_t, C.c_uint]
        L.oracle_float_to_bf16.argtypes = [f32p, u16p, C.c_size_t]
        L.oracle_linear_wq_bf16.argtypes = [C.c_int, u8p, u8p, C.c_float, u16p, u16p, f32p] + [C.c_size_t] * 7 + [
            C.c_float, C.c_float]
        L.oracle_cpu_path_dequant_sgemm.argtypes = [C.c_int, u8p, u8p, C.c_float, f32p, f32p, f32p] + [
            C.c_size_t] * 3 + [C.POINTER(C.c_double)] * 2
        L.oracle_num_threads.restype = C.c_int
        i32p = C.POINTER(C.c_int32)
        L.oracle_rms_norm_bf16.argtypes = [u16p, u16p, u16p, f32p, C.c_size_t, C.c_size_t, C.c_float]
        L.oracle_rope_bf16.argtypes = [u16p, u16p, u16p, u16p] + [C.c_size_t] * 4
        L.oracle_rope_tables_bf16.argtypes = [C.c_size_t, C.c_size_t, C.c_float, u16p, u16p]
        L.oracle_embed_bf16.argtypes = [i32p, u16p, u16p, C.c_size_t, C.c_size_t]
        L.oracle_silu_bf16.argtypes = [u16p, u16p, C.c_size_t]
        L.oracle_mul_bf16.argtypes = [u16p, u16p, u16p, C.c_size_t]
        L.oracle_add_bf16.argtypes = [u16p, u16p, u16p, C.c_size_t]
        L.oracle_kv_append_bf16.argtypes = [u16p, u16p] + [C.c_size_t] * 4
        L.oracle_attention_decode_bf16.argtypes = [u16p, u16p, u16p, u16p, f32p] + [C.c_size_t] * 5 + [i32p, C.c_float]
        _lib = L
    return _lib


def _p(a: np.ndarray | None, ct):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.POINTER(ct))


# ---- numpy helpers -----------------------------------------------------------------------

def bf16_bits_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(f: np.ndarray) -> np.ndarray:
    """RNE float32 -> bf16 bit patterns (the device rounding the path uses for operands)."""
    f = np.ascontiguousarray(f, dtype=np.float32)
    out = np.empty(f.shape, np.uint16)
    lib().oracle_float_to_bf16(_p(f.reshape(-1), C.c_float), _p(out.reshape(-1), C.c_uint16), f.size)
    return out


def fp8_to_bf16(src: np.ndarray, src_type: int, inv_scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.uint8)
    out = np.empty(src.shape, np.uint16)
    lib().oracle_fp8_to_bf16(_p(src.reshape(-1), C.c_uint8), src_type, _p(out.reshape(-1), C.c_uint16), src.size,
                             inv_scale)
    return out


def fp8_to_float(src: np.ndarray, src_type: int, inv_scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.uint8)
    out = np.empty(src.shape, np.float32)
    lib().oracle_fp8_to_float(_p(src.reshape(-1), C.c_uint8), src_type, _p(out.reshape(-1), C.c_float), src.size,
                              inv_scale)
    return out


def float_to_fp8(src: np.ndarray, dst_type: int, scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.float32)
    out = np.empty(src.shape, np.uint8)
    lib().oracle_float_to_fp8(_p(src.reshape(-1), C.c_float), _p(out.reshape(-1), C.c_uint8), dst_type, src.size,
                              scale)
    return out


def fp4_to_bf16(src: np.ndarray, n: int, inv_scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.uint8)
    out = np.empty(n, np.uint16)
    lib().oracle_fp4_to_bf16(_p(src.reshape(-1), C.c_uint8), _p(out, C.c_uint16), n, inv_scale)
    return out


def fp4_packed_to_float(src: np.ndarray, n: int, inv_scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.uint8)
    out = np.empty(n, np.float32)
    lib().oracle_fp4_packed_to_float(_p(src.reshape(-1), C.c_uint8), _p(out, C.c_float), n, inv_scale)
    return out


def float_to_fp4_packed(src: np.ndarray, scale: float) -> np.ndarray:
    src = np.ascontiguousarray(src, np.float32).reshape(-1)
    out = np.zeros((src.size + 1) // 2, np.uint8)
    lib().oracle_float_to_fp4_packed(_p(src, C.c_float), _p(out, C.c_uint8), src.size, scale)
    return out


def fp4_blockscale_to_bf16(nibbles: np.ndarray, scales: np.ndarray, n: int, block: int = 16) -> np.ndarray:
    nibbles = np.ascontiguousarray(nibbles, np.uint8).reshape(-1)
    scales = np.ascontiguousarray(scales, np.uint8).reshape(-1)
    out = np.empty(n, np.uint16)
    lib().oracle_fp4_blockscale_to_bf16(_p(nibbles, C.c_uint8), _p(scales, C.c_uint8), _p(out, C.c_uint16), n, block)
    return out


def float_to_fp4_blockscale(src: np.ndarray, block: int = 16):
    src = np.ascontiguousarray(src, np.float32).reshape(-1)
    nib = np.zeros((src.size + 1) // 2, np.uint8)
    sc = np.zeros((src.size + block - 1) // block, np.uint8)
    lib().oracle_float_to_fp4_blockscale(_p(src, C.c_float), _p(nib, C.c_uint8), _p(sc, C.c_uint8), src.size, block)
    return nib, sc


def linear_wq_bf16(w_type: int, W: np.ndarray, blk: np.ndarray | None, inv_scale: float, X: np.ndarray, N: int,
                   M: int, K: int, *, ldw: int | None = None, ldx: int | None = None, alpha: float = 1.0,
                   beta: float = 0.0, Y: np.ndarray | None = None, ldy_m: int | None = None, ldy_n: int = 1):
    """Y (bf16 bits, [M, ldy_m] by default) and the unrounded float32 [M, N] result."""
    ldw = K if ldw is None else ldw
    ldx = K if ldx is None else ldx
    ldy_m = N if ldy_m is None else ldy_m
    W = np.ascontiguousarray(W, np.uint8).reshape(-1)
    X = np.ascontiguousarray(X, np.uint16).reshape(-1)
    if Y is None:
        size = (M - 1) * ldy_m + (N - 1) * ldy_n + 1 if M and N else 0
        Y = np.zeros(size, np.uint16)
    else:
        Y = np.ascontiguousarray(Y, np.uint16).reshape(-1).copy()
    y32 = np.zeros((M, N), np.float32)
    blk_c = None if blk is None else np.ascontiguousarray(blk, np.uint8).reshape(-1)
    lib().oracle_linear_wq_bf16(w_type, _p(W, C.c_uint8), _p(blk_c, C.c_uint8), inv_scale, _p(X, C.c_uint16),
                                _p(Y, C.c_uint16), _p(y32.reshape(-1), C.c_float), N, M, K, ldw, ldx, ldy_m, ldy_n,
                                alpha, beta)
    return Y, y32


def quantise_activations_e4m3(X: np.ndarray, act_scale: float = 0.0):
    """BF16 bits -> (E4M3 bytes of the same shape, multiplier back) by the reference's W8A8 rules: act_scale > 0 is the
    static form (q = e4m3(x * (1 / act_scale)), multiplier act_scale, cccc/cublas_real.h:627-632); 0 the dynamic one
    (absmax by fmaxf, which skips NaN; q = e4m3(x * (448 / absmax)), multiplier absmax / 448; 1 and 1 for an all-zero
    tensor: cccc-cuda/cuda_functions.cu:2611-2657).  All arithmetic in float32 as there."""
    x = bf16_bits_to_f32(np.ascontiguousarray(X, np.uint16))
    if act_scale > 0.0:
        fwd, inv = np.float32(1.0) / np.float32(act_scale), np.float32(act_scale)
    else:
        mag = np.abs(x)
        a = np.float32(np.max(np.where(np.isnan(mag), np.float32(0.0), mag))) if mag.size else np.float32(0.0)
        fwd = np.float32(448.0) / a if a > 0 else np.float32(1.0)
        inv = a / np.float32(448.0) if a > 0 else np.float32(1.0)
    return float_to_fp8(x.reshape(-1), FP8_E4M3, float(fwd)).reshape(np.shape(X)), float(inv)


def linear_w8a8(W: np.ndarray, w_inv_scale: float, X: np.ndarray, N: int, M: int, K: int, *, act_scale: float = 0.0,
                alpha: float = 1.0):
    """The W8A8 linear (cccc/cublas_real.h:619-666): E4M3 weights [N, K] times the E4M3-quantised activations [M, K],
    both scales applied to the sums.  Returns (float64-accumulated float32 result [M, N], the quantised activations,
    the activations' multiplier back)."""
    q, inv = quantise_activations_e4m3(np.ascontiguousarray(X, np.uint16).reshape(M, K), act_scale)
    wf = fp8_to_float(np.ascontiguousarray(W, np.uint8).reshape(-1), FP8_E4M3, 1.0).reshape(N, K).astype(np.float64)
    xf = fp8_to_float(q.reshape(-1), FP8_E4M3, 1.0).reshape(M, K).astype(np.float64)
    y = (xf @ wf.T) * (float(alpha) * float(np.float32(w_inv_scale)) * float(np.float32(inv)))
    return y.astype(np.float32), q, inv


def cpu_path_dequant_sgemm(w_type: int, W: np.ndarray, blk: np.ndarray | None, inv_scale: float, Xf: np.ndarray,
                           N: int, M: int, K: int, wf: np.ndarray | None = None):
    """The reference's CPU form of the path (dequantise to float, then sgemm).  Returns
    (Y float32 [M, N], seconds in dequant, seconds in gemm)."""
    W = np.ascontiguousarray(W, np.uint8).reshape(-1)
    Xf = np.ascontiguousarray(Xf, np.float32).reshape(-1)
    if wf is None:
        wf = np.empty(N * K, np.float32)
    Y = np.empty((M, N), np.float32)
    td, tg = C.c_double(0), C.c_double(0)
    blk_c = None if blk is None else np.ascontiguousarray(blk, np.uint8).reshape(-1)
    lib().oracle_cpu_path_dequant_sgemm(w_type, _p(W, C.c_uint8), _p(blk_c, C.c_uint8), inv_scale, _p(Xf, C.c_float),
                                        _p(Y.reshape(-1), C.c_float), _p(wf, C.c_float), N, M, K, C.byref(td),
                                        C.byref(tg))
    return Y, td.value, tg.value


def num_threads() -> int:
    return int(lib().oracle_num_threads())


# ---- seeded synthetic inputs shared by tests, smoke and bench --------------------------------

def make_inputs(w_type: int, N: int, K: int, M: int, seed: int = 0, scaled: bool = False, w_std: float = 0.02):
    """Seeded inputs with the value distributions of the benchmark configurations:
    x ~ N(0,1) rounded to BF16 (RNE); W ~ N(0, w_std) quantised with the reference's own
    encoder rules (truncating FP8; block-16 FP4 with E4M3 scales).  `scaled` uses the
    per-tensor scale cccc computes (cccc/Matrix.cpp:344-346: fwd = maxval/absmax, stored
    multiplier = absmax/maxval) instead of 1.0."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(w_std)).astype(np.float32)
    x = rng.standard_normal((M, K), dtype=np.float32)
    X = f32_to_bf16_bits(x)
    blk = None
    inv_scale = 1.0
    if w_type == FP4_E2M1:
        Wq, blk = float_to_fp4_blockscale(w.reshape(-1), 16)
    else:
        fwd = 1.0
        if scaled:
            maxval = 448.0 if w_type == FP8_E4M3 else 57344.0
            absmax = float(np.abs(w).max())
            fwd = float(np.float32(maxval) / np.float32(absmax))
            inv_scale = float(np.float32(absmax) / np.float32(maxval))
        Wq = float_to_fp8(w, w_type, fwd).reshape(-1)
    return Wq, blk, inv_scale, X


# ---- the non-GEMM ops of the decode step (oracle/decode_ops_oracle.c) -----------------------------

def _u16(a):
    return np.ascontiguousarray(a, np.uint16)


def rms_norm_bf16(X: np.ndarray, scale: np.ndarray | None, eps: float = 1e-6) -> np.ndarray:
    """X: [outer, inner] BF16 bits; returns BF16 bits of the same shape."""
    X = _u16(X)
    outer, inner = int(np.prod(X.shape[:-1])), X.shape[-1]
    Y = np.empty_like(X)
    sc = None if scale is None else _u16(scale).reshape(-1)
    lib().oracle_rms_norm_bf16(_p(X.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16), _p(sc, C.c_uint16), None, outer,
                               inner, eps)
    return Y


def rope_tables_bf16(T: int, d_head: int, base: float):
    cos = np.empty((T, d_head // 2), np.uint16)
    sin = np.empty((T, d_head // 2), np.uint16)
    lib().oracle_rope_tables_bf16(T, d_head, base, _p(cos.reshape(-1), C.c_uint16), _p(sin.reshape(-1), C.c_uint16))
    return cos, sin


def rope_bf16(X: np.ndarray, cos: np.ndarray, sin: np.ndarray, pos_offset: int) -> np.ndarray:
    """X: [B, T, D] BF16 bits (B independent slices, T consecutive positions starting at pos_offset)."""
    X = _u16(X)
    B, T, D = X.shape
    Y = np.empty_like(X)
    lib().oracle_rope_bf16(_p(X.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16), _p(_u16(cos).reshape(-1), C.c_uint16),
                           _p(_u16(sin).reshape(-1), C.c_uint16), D, T, B, pos_offset)
    return Y


def embed_bf16(ids: np.ndarray, W: np.ndarray) -> np.ndarray:
    ids = np.ascontiguousarray(ids, np.int32).reshape(-1)
    W = _u16(W)
    Y = np.empty((ids.size, W.shape[1]), np.uint16)
    lib().oracle_embed_bf16(ids.ctypes.data_as(C.POINTER(C.c_int32)), _p(W.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16),
                            W.shape[1], ids.size)
    return Y


def silu_bf16(X: np.ndarray) -> np.ndarray:
    X = _u16(X)
    Y = np.empty_like(X)
    lib().oracle_silu_bf16(_p(X.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16), X.size)
    return Y


def mul_bf16(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    A, B = _u16(A), _u16(B)
    Y = np.empty_like(A)
    lib().oracle_mul_bf16(_p(A.reshape(-1), C.c_uint16), _p(B.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16), A.size)
    return Y


def add_bf16(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    A, B = _u16(A), _u16(B)
    Y = np.empty_like(A)
    lib().oracle_add_bf16(_p(A.reshape(-1), C.c_uint16), _p(B.reshape(-1), C.c_uint16), _p(Y.reshape(-1), C.c_uint16), A.size)
    return Y


def kv_append_bf16(x_new: np.ndarray, cache: np.ndarray, pos: int) -> None:
    """x_new: [n_heads, D]; cache: [n_heads, T_max, D], updated in place."""
    n_heads, T_max, D = cache.shape
    assert cache.dtype == np.uint16 and cache.flags["C_CONTIGUOUS"]
    lib().oracle_kv_append_bf16(_p(_u16(x_new).reshape(-1), C.c_uint16), _p(cache.reshape(-1), C.c_uint16), D, T_max, n_heads, pos)


def attention_decode_bf16(Q: np.ndarray, Kc: np.ndarray, Vc: np.ndarray, pos: np.ndarray, dk: float | None = None):
    """Q: [B, H, D]; caches: [B, Hkv, T_max, D]; pos: [B] newest valid row.  Returns (Y bits [B, H, D], y32)."""
    Q, Kc, Vc = _u16(Q), _u16(Kc), _u16(Vc)
    B, H, D = Q.shape
    _, Hkv, T_max, _ = Kc.shape
    pos = np.ascontiguousarray(pos, np.int32).reshape(-1)
    Y = np.empty_like(Q)
    y32 = np.empty(Q.shape, np.float32)
    lib().oracle_attention_decode_bf16(_p(Q.reshape(-1), C.c_uint16), _p(Kc.reshape(-1), C.c_uint16), _p(Vc.reshape(-1), C.c_uint16),
                                       _p(Y.reshape(-1), C.c_uint16), _p(y32.reshape(-1), C.c_float), B, H, Hkv, D, T_max,
                                       pos.ctypes.data_as(C.POINTER(C.c_int32)), float(D if dk is None else dk))
    return Y, y32
