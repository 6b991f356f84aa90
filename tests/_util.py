"""Helpers shared by the tests: package loading, device buffers, error metrics."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from __graft_entry__ import ROOT, load_package

REF_DIR = os.path.join(ROOT, "oracle", "_ref")

# north_star tolerance for GEMV/GEMM outputs against the FP32-accumulated reference output
MAX_REL = 1e-2
MIN_COS = 0.9999


def capi():
    return load_package().capi


def to_dev(a: np.ndarray):
    import torch

    if a.dtype == np.uint16:
        a = a.view(np.int16)
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def from_dev_u16(t) -> np.ndarray:
    return t.cpu().numpy().view(np.uint16)


def rel_cos(got: np.ndarray, ref: np.ndarray):
    """Max relative error (relative to max(|ref|, 1e-2*rms(ref)), which avoids 0/0) and cosine."""
    got = got.astype(np.float64).reshape(-1)
    ref = ref.astype(np.float64).reshape(-1)
    rms = np.sqrt(np.mean(ref ** 2)) if ref.size else 0.0
    denom = np.maximum(np.abs(ref), 1e-2 * rms + 1e-30)
    rel = float(np.max(np.abs(got - ref) / denom)) if ref.size else 0.0
    nn = np.linalg.norm(got) * np.linalg.norm(ref)
    cos = float(got @ ref / nn) if nn > 0 else 1.0
    return rel, cos


def assert_close(got: np.ndarray, ref: np.ndarray, what=""):
    assert np.all(np.isfinite(got)), what
    rel, cos = rel_cos(got, ref)
    assert rel <= MAX_REL and cos >= MIN_COS, (what, rel, cos)


def assert_close_rows(got: np.ndarray, ref: np.ndarray, what="", tol=MAX_REL):
    """The bar for outputs that pass through the reference's BF16 score / probability tensors (attention
    and everything downstream of it): |got - ref| <= tol * max(|ref|, rms of that output row) for every
    element, and cosine >= 0.9999 overall.  The floor is the row's rms, not a hundredth of it as for a
    single GEMM: a score whose exact value lies within FP32 summation error of a BF16 rounding boundary
    rounds either way depending on the summation order (cuBLAS's is not known), and one such flip moves
    every output of its head by up to 2^-8 * p_t * |v|, far above a hundredth of a near-zero output."""
    got = got.astype(np.float64).reshape(-1, got.shape[-1])
    ref = ref.astype(np.float64).reshape(-1, ref.shape[-1])
    assert np.all(np.isfinite(got)), what
    rms = np.sqrt(np.mean(ref ** 2, axis=1, keepdims=True)) + 1e-30
    rel = float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), rms)))
    _, cos = rel_cos(got, ref)
    assert rel <= tol and cos >= MIN_COS, (what, rel, cos)


def ref_cuda_lib():
    """The reference's own cuda_functions.cu built for sm_100a (oracle/_ref), or None."""
    path = os.path.join(REF_DIR, "libcccc-cuda-ref.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.cuda_convert.restype = C.c_int
    L.cuda_convert.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_uint, C.c_float]
    L.cuda_fp4_blockscale_to_bf16.restype = C.c_int
    L.cuda_fp4_blockscale_to_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint]
    L.cuda_float_to_fp4_blockscale.restype = C.c_int
    L.cuda_float_to_fp4_blockscale.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint]
    return L


def ref_gemm_lib(patched: bool = False):
    """The reference's Cublas::gemm dispatcher behind a C-ABI (oracle/_ref), or None.  patched: the same
    dispatcher compiled from the reference's header with the two call sites changed as the integration notes
    ask (oracle/patch_reference.py) and linked against cccc-cuda-b200 ahead of the reference's cccc-cuda."""
    path = os.path.join(REF_DIR, "libref_gpu_gemm_patched.so" if patched else "libref_gpu_gemm.so")
    if not os.path.exists(path):
        return None
    L = C.CDLL(path)
    L.ref_cublas_gemm.restype = C.c_int
    L.ref_cublas_gemm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int,
                                  C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int,
                                  C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    return L
