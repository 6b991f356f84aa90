"""ctypes binding of the C-ABI declared in include/cccc_cuda_b200.h.

The library is the product; this module only loads it and passes device pointers through.
There is no fallback: if the shared library is missing or a symbol is absent, loading fails.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcccc-cuda-b200.so")

# cccc::DataType (cccc/types.h:24-34)
FLOAT, DOUBLE, HALF, BFLOAT16, FP8_E4M3, FP8_E5M2, FP4_E2M1 = range(7)

PLAN_PLAIN, PLAN_DECODE, PLAN_PREFILL, PLAN_STREAM, PLAN_NATIVE = 0, 1, 2, 3, 4
FLAG_NO_STREAM = 0x800   # flags bit 11 of cuda_gemm_wq_bf16: the decode / prefill kernels even where the streaming kernel would be chosen
FLAG_STREAM = 7 << 8     # flags bits 8-10 = 7: the streaming kernel wherever it accepts the shape
FLAG_NATIVE = 0x1000     # flags bit 12: FP8 weights straight into the tensor cores (1..32 tokens) wherever the kernel accepts the shape
FLAG_NO_NATIVE = 0x2000  # flags bit 13: never that kernel
FLAG_NATIVE_FUSED = 0x4000  # flags bit 14: the FP8 native kernel splits the activations itself (up to 8 tokens)
FLAG_PDL = 1
FLAG_CHECKED = 2  # cuda_gemm_wq_bf16_static only
FLAG_OUT_F32 = 4  # Y is float32 (partial sums of a row-parallel shard)


def flag_prefill_variant(v):
    """flags bits 8-10 of cuda_gemm_wq_bf16: tile shape of the M > 32 path (0 = chosen by shape)."""
    return (int(v) & 7) << 8

_vp, _u, _f, _i = C.c_void_p, C.c_uint, C.c_float, C.c_int

# name -> (restype, argtypes): every symbol include/cccc_cuda_b200.h declares
SYMBOLS = {
    "cuda_convert": (_i, [_vp, _i, _vp, _i, _u, _f]),
    "cuda_fp4_blockscale_to_bf16": (_i, [_vp, _vp, _vp, _u, _u]),
    "cuda_float_to_fp4_blockscale": (_i, [_vp, _vp, _vp, _u, _u]),
    "cuda_check_error": (_i, [C.c_char_p]),
    "cuda_clear_last_error": (None, []),
    "cuda_gemm_wq_bf16": (_i, [_i, _vp, _vp, _f, _vp, _vp, _u, _u, _u, _u, _u, _u, _u, _f, _f, _vp, _u]),
    "cuda_gemm_wq_bf16_static": (_i, [_i, _vp, _vp, _f, _vp, _vp, _u, _u, _u, _u, _u, _u, _u, _f, _f, _vp, _u]),
    "cuda_gemm_wq_bf16_plan": (_i, [_i, _vp, _vp, _vp, _vp, _u, _u, _u, _u, _u, _u, _u]),
    "cuda_b200_allreduce_f32_to_bf16": (_i, [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), _vp, _vp, _vp, _u, _u, _i, _i,
                                             _vp, _u]),
    "cuda_b200_allreduce_recv_bytes": (C.c_ulonglong, [_i, _u]),
    "cuda_b200_allreduce_flag_bytes": (C.c_ulonglong, [_i]),
    "cuda_b200_allreduce_counter_bytes": (C.c_ulonglong, []),
    "cuda_gemm_wq_bf16_allreduce": (_i, [_i, _vp, _vp, _f, _vp, _vp, _u, _u, _u, _u, _u, _u, _u, _f, C.POINTER(C.c_ulonglong),
                                         C.POINTER(C.c_ulonglong), _vp, _u, _i, _i, _vp, _u]),
    "cuda_b200_fused_flag_bytes": (C.c_ulonglong, [_i]),
    "cuda_b200_fused_counter_bytes": (C.c_ulonglong, []),
    "cuda_argmax_bf16": (_i, [_vp, _u, _u, C.c_ulonglong, _vp, _vp, _vp]),
    "cuda_b200_launch_count": (C.c_ulonglong, []),
    "cuda_b200_version": (C.c_char_p, []),
}



class WqLinear(C.Structure):
    """cuda_wq_linear of include/cccc_cuda_b200.h."""
    _fields_ = [("W", C.c_void_p), ("blk_scales", C.c_void_p), ("Y", C.c_void_p), ("inv_scale", C.c_float),
                ("alpha", C.c_float), ("beta", C.c_float), ("N_out", C.c_uint), ("ldw", C.c_uint), ("ldy_m", C.c_uint),
                ("ldy_n", C.c_uint)]


SYMBOLS["cuda_gemm_wq_bf16_group"] = (_i, [_i, _u, C.POINTER(WqLinear), _vp, _u, _u, _u, _vp, _u])
SYMBOLS["cuda_gemm_w8a8_bf16"] = (_i, [_vp, _f, _vp, _f, _vp, _u, _u, _u, _u, _u, _u, _u, _f, _f, _vp, _u])
SYMBOLS["cuda_bf16_to_fp8e4m3_dynamic"] = (_i, [_vp, _vp, _u, _vp, _vp])
SYMBOLS["cuda_gemm_w8a8_bf16_group"] = (_i, [_u, C.POINTER(WqLinear), _vp, _f, _u, _u, _u, _vp, _u])
SYMBOLS["cuda_gemm_fp8_fp8"] = (_i, [_vp, _f, _vp, _f, _vp, _i, _u, _u, _u, _u, _u, _u, _u, _f, _f, _vp, _u])
SYMBOLS["cuda_add_fp8e4m3"] = (_i, [_vp, _vp, _vp, _u, _f, _f, _f])
SYMBOLS["cuda_addbias_fp8e4m3"] = (_i, [_vp, _vp, _vp, _u, _u, _u, _f, _f])
SYMBOLS["cuda_addbias_fp8e4m3_bf16bias"] = (_i, [_vp, _vp, _vp, _u, _u, _u, _f, _f])
SYMBOLS["cuda_silu_fp8e4m3"] = (_i, [_vp, _vp, _u])
SYMBOLS["cuda_elementmul_fp8e4m3"] = (_i, [_vp, _vp, _vp, _u, _f, _f])
SYMBOLS["cuda_embed_fwd_fp8_to_fp8"] = (_i, [_vp, _vp, _vp, _i, _i, _i, _f])
SYMBOLS["cuda_embed_fwd_bf16_to_fp8"] = (_i, [_vp, _vp, _vp, _i, _i, _i])



class AttnDecode(C.Structure):
    """cuda_attn_decode of include/cccc_cuda_b200.h."""
    _fields_ = [(n, C.c_void_p) for n in ("q", "k", "v", "q_norm", "k_norm", "cos_tab", "sin_tab", "k_cache", "v_cache", "pos", "out")] + [
        (n, C.c_uint) for n in ("ldq", "ldk", "ldv", "ldo", "B", "H", "Hkv", "head_dim", "T_max")] + [("epsilon", C.c_float), ("dk", C.c_float)]


SYMBOLS["cuda_rms_norm_bf16"] = (_i, [_vp, _vp, _vp, _vp, _vp, _u, _u, _f, _vp, _u])
SYMBOLS["cuda_rope_bf16"] = (_i, [_vp, _vp, _vp, _vp, _u, _u, _u, _u, _vp, _u])
SYMBOLS["cuda_embed_bf16"] = (_i, [_vp, _vp, _vp, _u, _u, _u, _vp, _u])
SYMBOLS["cuda_swiglu_bf16"] = (_i, [_vp, _vp, _vp, _u, _u, _u, _u, _u, _vp, _u])
SYMBOLS["cuda_attn_decode_bf16"] = (_i, [C.POINTER(AttnDecode), _vp, _u])



class DecodeInput(C.Structure):
    """cuda_decode_input of include/cccc_cuda_b200.h."""
    _fields_ = [("mode", C.c_int), ("x", C.c_void_p), ("ldx", C.c_uint), ("x2", C.c_void_p), ("ldx2", C.c_uint),
                ("norm_weight", C.c_void_p), ("epsilon", C.c_float)]


X_COPY, X_RMSNORM, X_SWIGLU = 0, 1, 2
SYMBOLS["cuda_decode_program_create"] = (_i, [C.POINTER(C.c_void_p), _i, _u])
SYMBOLS["cuda_decode_program_add_linears"] = (_i, [_vp, _u, C.POINTER(WqLinear), C.POINTER(DecodeInput), _u, _u])
SYMBOLS["cuda_decode_program_add_attention"] = (_i, [_vp, C.POINTER(AttnDecode)])
SYMBOLS["cuda_decode_program_finalize"] = (_i, [_vp])
SYMBOLS["cuda_decode_program_launch"] = (_i, [_vp, _vp])
SYMBOLS["cuda_decode_program_phases"] = (_u, [_vp])
SYMBOLS["cuda_decode_program_destroy"] = (None, [_vp])

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises if it has not been built (python cccc-lite_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            # not a fallback: the CUDA library is the only implementation; build it or fail
            import subprocess
            import sys

            subprocess.check_call([sys.executable, os.path.join(HERE, "build.py")])
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python cccc-lite_b200/build.py`")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)  # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def convert(src, src_type: int, dst, dst_type: int, n: int, scale: float = 1.0) -> int:
    return lib().cuda_convert(_ptr(src), src_type, _ptr(dst), dst_type, n, scale)


def fp4_blockscale_to_bf16(nibbles, scales, dst, n: int, block: int = 16) -> int:
    return lib().cuda_fp4_blockscale_to_bf16(_ptr(nibbles), _ptr(scales), _ptr(dst), n, block)


def float_to_fp4_blockscale(src, nibbles, scales, n: int, block: int = 16) -> int:
    return lib().cuda_float_to_fp4_blockscale(_ptr(src), _ptr(nibbles), _ptr(scales), n, block)


def check_error(label: str = "cuda") -> int:
    return lib().cuda_check_error(label.encode())


def gemm_wq_bf16(w_type: int, W, blk, inv_scale: float, X, Y, N: int, M: int, K: int, *, ldw: int | None = None,
                 ldx: int | None = None, ldy_m: int | None = None, ldy_n: int = 1, alpha: float = 1.0,
                 beta: float = 0.0, stream: int | None = None, flags: int = 0) -> int:
    """Asynchronous fused linear on `stream` (a raw cudaStream_t value; None = torch's current stream)."""
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_gemm_wq_bf16(w_type, _ptr(W), _ptr(blk), inv_scale, _ptr(X), _ptr(Y), N, M, K,
                                   K if ldw is None else ldw, K if ldx is None else ldx,
                                   N if ldy_m is None else ldy_m, ldy_n, alpha, beta, stream, flags)


def gemm_w8a8_bf16(W, w_inv_scale: float, X, act_scale: float, Y, N: int, M: int, K: int, *, ldw: int | None = None,
                   ldx: int | None = None, ldy_m: int | None = None, ldy_n: int = 1, alpha: float = 1.0, beta: float = 0.0,
                   stream: int | None = None, flags: int = 0) -> int:
    """W8A8 linear: E4M3 weights, BF16 activations quantised to E4M3 inside the call (act_scale > 0 static, 0 dynamic)."""
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_gemm_w8a8_bf16(_ptr(W), w_inv_scale, _ptr(X), act_scale, _ptr(Y), N, M, K, K if ldw is None else ldw,
                                     K if ldx is None else ldx, N if ldy_m is None else ldy_m, ldy_n, alpha, beta, stream, flags)


def gemm_w8a8_bf16_group(group, X, act_scale: float, M: int, K: int, *, ldx: int | None = None, stream: int | None = None,
                         flags: int = 0) -> int:
    """Up to three W8A8 linears sharing X (`group` from make_group) in one call: one quantisation, one launch."""
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_gemm_w8a8_bf16_group(len(group), group, _ptr(X), act_scale, M, K, K if ldx is None else ldx, stream, flags)


def bf16_to_fp8e4m3_dynamic(src, dst, n: int, absmax_tmp, inv_scale_out) -> int:
    return lib().cuda_bf16_to_fp8e4m3_dynamic(_ptr(src), _ptr(dst), n, _ptr(absmax_tmp), _ptr(inv_scale_out))


def gemm_wq_bf16_static(w_type: int, W, blk, inv_scale: float, X, Y, N: int, M: int, K: int, *, ldw: int | None = None,
                        ldx: int | None = None, ldy_m: int | None = None, ldy_n: int = 1, alpha: float = 1.0,
                        beta: float = 0.0, stream: int | None = None, flags: int = 0) -> int:
    """The allocation-free variant (fixed scratch inside the library, M <= 8); same arguments."""
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_gemm_wq_bf16_static(w_type, _ptr(W), _ptr(blk), inv_scale, _ptr(X), _ptr(Y), N, M, K,
                                          K if ldw is None else ldw, K if ldx is None else ldx,
                                          N if ldy_m is None else ldy_m, ldy_n, alpha, beta, stream, flags)


def make_group(linears, K: int):
    """A ctypes array of cuda_wq_linear from dicts with W, S (block scales or None), Y, N, and optional
    inv, alpha, beta, ldw, ldy_m, ldy_n.  Build it once and reuse it: it only holds pointers."""
    arr = (WqLinear * len(linears))()
    for a, L in zip(arr, linears):
        a.W = _ptr(L["W"])
        a.blk_scales = _ptr(L.get("S"))
        a.Y = _ptr(L["Y"])
        a.inv_scale = L.get("inv", 1.0)
        a.alpha = L.get("alpha", 1.0)
        a.beta = L.get("beta", 0.0)
        a.N_out = L["N"]
        a.ldw = L.get("ldw", K)
        a.ldy_m = L.get("ldy_m", L["N"])
        a.ldy_n = L.get("ldy_n", 1)
    return arr


def gemm_wq_bf16_group(w_type: int, group, X, M: int, K: int, *, ldx: int | None = None, stream: int | None = None,
                       flags: int = 0) -> int:
    """Several linears sharing the activations X in one call (`group` from make_group)."""
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_gemm_wq_bf16_group(w_type, len(group), group, _ptr(X), M, K, K if ldx is None else ldx, stream, flags)


def gemm_wq_bf16_plan(w_type: int, W, blk, X, Y, N: int, M: int, K: int, *, ldw=None, ldx=None, ldy_m=None,
                      ldy_n: int = 1) -> int:
    return lib().cuda_gemm_wq_bf16_plan(w_type, _ptr(W), _ptr(blk), _ptr(X), _ptr(Y), N, M, K,
                                        K if ldw is None else ldw, K if ldx is None else ldx,
                                        N if ldy_m is None else ldy_m, ldy_n)


class PushAllReduce:
    """The one-shot all-reduce over symmetric memory (cuda_b200_allreduce_f32_to_bf16).  Allocates the
    receive and flag areas with torch's symmetric memory, exchanges the mappings over `group`, and keeps
    the pointer arrays.  Every rank must construct it and then make the same calls."""

    def __init__(self, dist, group, rank: int, world: int, n_max: int, device):
        import torch
        import torch.distributed._symmetric_memory as symm_mem

        L = lib()
        self.rank, self.world, self.n_max = rank, world, n_max
        self.recv = symm_mem.empty(L.cuda_b200_allreduce_recv_bytes(world, n_max) // 4, dtype=torch.float32, device=device)
        self.flag = symm_mem.empty(L.cuda_b200_allreduce_flag_bytes(world) // 4, dtype=torch.int32, device=device)
        self.recv.zero_()
        self.flag.zero_()
        self.counters = torch.zeros(L.cuda_b200_allreduce_counter_bytes() // 4, dtype=torch.int32, device=device)
        hr = symm_mem.rendezvous(self.recv, group)
        hf = symm_mem.rendezvous(self.flag, group)
        self._handles = (hr, hf)
        self.recv_ptrs = (C.c_ulonglong * world)(*[int(p) for p in hr.buffer_ptrs])
        self.flag_ptrs = (C.c_ulonglong * world)(*[int(p) for p in hf.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)

    def __call__(self, partial, out, n: int, stream: int | None = None, flags: int = 0) -> int:
        if stream is None:
            import torch

            stream = torch.cuda.current_stream().cuda_stream
        return lib().cuda_b200_allreduce_f32_to_bf16(self.recv_ptrs, self.flag_ptrs, _ptr(self.counters), _ptr(partial), _ptr(out),
                                                     n, self.n_max, self.rank, self.world, stream, flags)


class FusedRowLinear:
    """The row-parallel linear with its all-reduce inside the kernel (cuda_gemm_wq_bf16_allreduce).
    Allocates the exchange areas with torch's symmetric memory and keeps the pointer arrays; every
    rank must construct it and then make the same calls."""

    def __init__(self, dist, group, rank: int, world: int, n_max: int, device):
        import torch
        import torch.distributed._symmetric_memory as symm_mem

        L = lib()
        self.rank, self.world, self.n_max = rank, world, n_max
        self.recv = symm_mem.empty(L.cuda_b200_allreduce_recv_bytes(world, n_max) // 4, dtype=torch.float32, device=device)
        self.flag = symm_mem.empty(L.cuda_b200_fused_flag_bytes(world) // 4, dtype=torch.int32, device=device)
        self.recv.zero_()
        self.flag.zero_()
        self.counters = torch.zeros(L.cuda_b200_fused_counter_bytes() // 4, dtype=torch.int32, device=device)
        hr = symm_mem.rendezvous(self.recv, group)
        hf = symm_mem.rendezvous(self.flag, group)
        self._handles = (hr, hf)
        self.recv_ptrs = (C.c_ulonglong * world)(*[int(p) for p in hr.buffer_ptrs])
        self.flag_ptrs = (C.c_ulonglong * world)(*[int(p) for p in hf.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)
        # From 9 tokens on the streaming tensor-core kernel is the faster linear; it has no exchange in its epilogue,
        # so those calls take the two-kernel form (FP32 partial sums, then the one-shot push all-reduce) on areas of
        # their own.
        self.push = PushAllReduce(dist, group, rank, world, n_max, device)
        self.partial = torch.zeros(n_max, dtype=torch.float32, device=device)

    def two_kernels(self, w_type: int, W, blk, inv_scale: float, X, Y, N: int, M: int, K: int, *, alpha: float = 1.0,
                    stream: int | None = None, flags: int = 0) -> int:
        """The same result as the fused call (sum over ranks in rank order, one BF16 rounding) as the linear with
        FP32 output followed by cuda_b200_allreduce_f32_to_bf16."""
        rc = gemm_wq_bf16(w_type, W, blk, inv_scale, X, self.partial, N, M, K, alpha=alpha, stream=stream, flags=flags | FLAG_OUT_F32)
        if rc != 0:
            return rc
        return self.push(self.partial, Y, M * N, stream=stream, flags=flags & 1)

    def __call__(self, w_type: int, W, blk, inv_scale: float, X, Y, N: int, M: int, K: int, *, ldw: int | None = None,
                 ldx: int | None = None, ldy_m: int | None = None, ldy_n: int = 1, alpha: float = 1.0,
                 stream: int | None = None, flags: int = 0) -> int:
        if stream is None:
            import torch

            stream = torch.cuda.current_stream().cuda_stream
        return lib().cuda_gemm_wq_bf16_allreduce(w_type, _ptr(W), _ptr(blk), inv_scale, _ptr(X), _ptr(Y), N, M, K,
                                                 K if ldw is None else ldw, K if ldx is None else ldx,
                                                 N if ldy_m is None else ldy_m, ldy_n, alpha, self.recv_ptrs, self.flag_ptrs,
                                                 _ptr(self.counters), self.n_max, self.rank, self.world, stream, flags)


def _stream(stream):
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    return stream


def rms_norm_bf16(X, Y, scale, rows: int, inner: int, eps: float = 1e-6, residual=None, sum_out=None, stream=None, flags: int = 0) -> int:
    return lib().cuda_rms_norm_bf16(_ptr(X), _ptr(residual), _ptr(sum_out), _ptr(Y), _ptr(scale), rows, inner, eps, _stream(stream), flags)


def rope_bf16(X, Y, cos_tab, sin_tab, D: int, T: int, B: int, pos_offset: int, stream=None, flags: int = 0) -> int:
    return lib().cuda_rope_bf16(_ptr(X), _ptr(Y), _ptr(cos_tab), _ptr(sin_tab), D, T, B, pos_offset, _stream(stream), flags)


def embed_bf16(ids, W, Y, D: int, n_tokens: int, vocab: int, stream=None, flags: int = 0) -> int:
    return lib().cuda_embed_bf16(_ptr(ids), _ptr(W), _ptr(Y), D, n_tokens, vocab, _stream(stream), flags)


def swiglu_bf16(gate, up, out, rows: int, cols: int, ld_gate=None, ld_up=None, ld_out=None, stream=None, flags: int = 0) -> int:
    return lib().cuda_swiglu_bf16(_ptr(gate), _ptr(up), _ptr(out), rows, cols, cols if ld_gate is None else ld_gate,
                                  cols if ld_up is None else ld_up, cols if ld_out is None else ld_out, _stream(stream), flags)


def make_attn_decode(*, q, k, v, k_cache, v_cache, pos, out, cos_tab, sin_tab, B: int, H: int, Hkv: int, head_dim: int, T_max: int,
                     q_norm=None, k_norm=None, ldq=None, ldk=None, ldv=None, ldo=None, eps: float = 1e-6, dk: float = 0.0):
    """A cuda_attn_decode filled from tensors (it only holds pointers: keep the tensors alive)."""
    a = AttnDecode()
    for name, t in (("q", q), ("k", k), ("v", v), ("q_norm", q_norm), ("k_norm", k_norm), ("cos_tab", cos_tab), ("sin_tab", sin_tab),
                    ("k_cache", k_cache), ("v_cache", v_cache), ("pos", pos), ("out", out)):
        setattr(a, name, _ptr(t))
    a.ldq = H * head_dim if ldq is None else ldq
    a.ldk = Hkv * head_dim if ldk is None else ldk
    a.ldv = Hkv * head_dim if ldv is None else ldv
    a.ldo = H * head_dim if ldo is None else ldo
    a.B, a.H, a.Hkv, a.head_dim, a.T_max, a.epsilon, a.dk = B, H, Hkv, head_dim, T_max, eps, dk
    return a


def attn_decode_bf16(desc, stream=None, flags: int = 0) -> int:
    return lib().cuda_attn_decode_bf16(C.byref(desc), _stream(stream), flags)


class DecodeProgram:
    """A recorded decode step that runs as one persistent kernel (cuda_decode_program_*)."""

    def __init__(self, w_type: int, M: int):
        self._h = C.c_void_p()
        rc = lib().cuda_decode_program_create(C.byref(self._h), w_type, M)
        if rc != 0:
            raise ValueError(f"cuda_decode_program_create: {rc}")
        self._keep = []

    def add_linears(self, group, K: int, x, *, mode: int = X_COPY, ldx: int | None = None, x2=None, ldx2: int | None = None,
                    norm_weight=None, eps: float = 1e-6, flags: int = 0) -> int:
        d = DecodeInput(mode, _ptr(x), K if ldx is None else ldx, _ptr(x2), K if ldx2 is None else ldx2, _ptr(norm_weight), eps)
        self._keep.append((group, x, x2, norm_weight))
        return lib().cuda_decode_program_add_linears(self._h, len(group), group, C.byref(d), K, flags)

    def add_attention(self, desc) -> int:
        self._keep.append(desc)
        return lib().cuda_decode_program_add_attention(self._h, C.byref(desc))

    def finalize(self) -> int:
        return lib().cuda_decode_program_finalize(self._h)

    def launch(self, stream=None) -> int:
        return lib().cuda_decode_program_launch(self._h, _stream(stream))

    @property
    def phases(self) -> int:
        return int(lib().cuda_decode_program_phases(self._h))

    def close(self):
        if self._h:
            lib().cuda_decode_program_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def argmax_bf16(logits, rows: int, cols: int, idx_out, val_out=None, ld: int | None = None, stream: int | None = None) -> int:
    if stream is None:
        import torch

        stream = torch.cuda.current_stream().cuda_stream
    return lib().cuda_argmax_bf16(_ptr(logits), rows, cols, cols if ld is None else ld, _ptr(idx_out), _ptr(val_out), stream)


def launch_count() -> int:
    return int(lib().cuda_b200_launch_count())


def version() -> str:
    return lib().cuda_b200_version().decode()
