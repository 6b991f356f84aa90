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
    "cccc_host_set_act_type": (None, [_vp, _i]),
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
    "cccc_host_gemm_typed": (None, [_vp, _i, _i, _i, _i, _i, _i, _f, _vp, _i, _vp, _i, _f, _vp, _i, _f, _i]),
    "cccc_host_sample": (_i, [C.POINTER(C.c_float), _i, _f, _i, _f, _f, C.POINTER(C.c_int), _i, C.POINTER(C.c_int), _i, C.c_uint]),
    "cccc_host_generate_canned": (_i, [C.POINTER(C.c_float), _i, _i, C.POINTER(C.c_int), _i, _i, C.POINTER(C.c_int), _f, _i, _f, _f,
                                       C.POINTER(C.c_int), _i, C.c_uint, _i, C.POINTER(C.c_int), _i, C.POINTER(C.c_int), _i,
                                       C.POINTER(C.c_int)]),
    "cccc_host_step_create": (_vp, [_vp, _vp, C.POINTER(C.c_int), _f, _f, _i, _i, C.c_char_p, _i]),
    "cccc_host_step_destroy": (None, [_vp]),
    "cccc_host_step_run": (_i, [_vp, C.POINTER(C.c_int), C.POINTER(C.c_int), _i, C.POINTER(C.c_int), C.POINTER(C.c_float), _vp]),
    "cccc_host_step_reset": (None, [_vp]),
    "cccc_host_step_use_program": (_i, [_vp, _i]),
    "cccc_host_step_info": (C.c_ulonglong, [_vp, _i]),
    "cccc_host_step_save": (_i, [_vp, C.c_char_p, C.c_char_p, _i]),
    "cccc_host_step_generate": (_i, [_vp, _i, C.POINTER(C.c_int), _i, C.POINTER(C.c_int), _f, _i, _f, _f, C.POINTER(C.c_int), _i, C.c_uint,
                                     _i, C.POINTER(C.c_int), _i, C.POINTER(C.c_int)]),
    "cccc_host_bin_write_quantised": (_i, [C.c_char_p, C.c_char_p, _i, _i, _i, _vp, C.c_ulonglong, _vp, C.c_ulonglong, _f]),
    "cccc_host_tp_combine_selftest": (_i, [_i, _i, C.POINTER(C.c_int), C.POINTER(C.c_float), C.POINTER(C.c_float), _vp, _i, C.POINTER(C.c_int),
                                           C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "cccc_host_tp_steps": (_i, [C.c_char_p, C.POINTER(C.c_int), _i, C.POINTER(C.c_int), _f, _f, C.POINTER(C.c_int), _i, C.POINTER(C.c_int),
                                C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_char_p, _i]),
    "cccc_host_tp_generate": (_i, [C.c_char_p, C.POINTER(C.c_int), _i, C.POINTER(C.c_int), _f, _f, C.POINTER(C.c_int), _i,
                                   C.POINTER(C.c_int), _f, _i, _f, _f, C.POINTER(C.c_int), _i, C.c_uint, _i, C.POINTER(C.c_int), _i,
                                   C.POINTER(C.c_int), C.c_char_p, _i]),
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


# ---- the generation side (csrc/host/generate.h, decode_step.h) ----

def _ints(values):
    values = [int(v) for v in values]
    return (C.c_int * max(1, len(values)))(*values), len(values)


def _sampler_args(sampler):
    s = dict(temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, banned_ids=())
    s.update(sampler or {})
    banned, nb = _ints(s["banned_ids"])
    return s["temperature"], s["top_k"], s["top_p"], s["repetition_penalty"], banned, nb


def _gen_ints(eos_ids=(), think_open_id=-1, think_close_id=-1, sys_n=0, turn_n=0, T=0, T_kv=0):
    """The generation settings as the flat int array the harness takes."""
    return _ints([len(eos_ids), *eos_ids, think_open_id, think_close_id, sys_n, turn_n, T, T_kv])[0]


def sample(logits, ctx_ids=(), seed=0, **sampler):
    """One token from a row of float logits: sample_logits of cccc-llm (cccc-llm/cccc-llm.cpp:181-343)."""
    import numpy as np

    l = np.ascontiguousarray(logits, dtype=np.float32)
    t, k, p, r, banned, nb = _sampler_args(sampler)
    ctx, nc = _ints(ctx_ids)
    return lib().cccc_host_sample(l.ctypes.data_as(C.POINTER(C.c_float)), l.size, t, k, p, r, banned, nb, ctx, nc, seed)


def generate_canned(table, ctx_ids, max_new, seed=0, sampler=None, **gen):
    """The generation loop over canned logits (step s of the model returns row s % len(table)).  Returns
    (generated ids, context after, trace of (token, pos) per model step, stats dict)."""
    import numpy as np

    tab = np.ascontiguousarray(table, dtype=np.float32)
    n_rows, V = tab.shape
    cap = len(ctx_ids) + max_new + 8
    ctx = (C.c_int * cap)(*[int(v) for v in ctx_ids])
    out = (C.c_int * max(1, max_new))()
    trace_cap = 8 * (len(ctx_ids) + max_new) + 64
    trace = (C.c_int * (2 * trace_cap))()
    stats = (C.c_int * 6)()
    t, k, p, r, banned, nb = _sampler_args(sampler)
    n = lib().cccc_host_generate_canned(tab.ctypes.data_as(C.POINTER(C.c_float)), n_rows, V, ctx, len(ctx_ids), cap, _gen_ints(**gen), t, k, p, r,
                                        banned, nb, seed, max_new, out, max_new, trace, trace_cap, stats)
    calls = min(stats[3], trace_cap)
    return (list(out[:n]), list(ctx[:min(stats[5], cap)]), [(trace[2 * i], trace[2 * i + 1]) for i in range(calls)],
            dict(rebuilds=stats[0], decode_steps=stats[1], prefill_tokens=stats[2], model_steps=stats[3], resets=stats[4]))


def model_ints(cfg, max_context, weight_data_type=-1):
    """cfg: an object with hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, layers, qk_norm (decode_model.ModelConfig)."""
    return _ints([cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.ffn, cfg.vocab, cfg.layers, int(cfg.qk_norm), max_context,
                  weight_data_type])[0]


class HostDecodeStep:
    """cccc::DecodeStep on one GPU: the whole decode step issued from C++ (weights from a container file)."""

    def __init__(self, gpu, binfile, cfg, max_context, max_batch=1, weight_data_type=-1, keep_host=False):
        err = C.create_string_buffer(512)
        self.cfg, self.max_batch = cfg, max_batch
        self.h = lib().cccc_host_step_create(gpu, binfile, model_ints(cfg, max_context, weight_data_type), cfg.rope_theta, cfg.eps, max_batch,
                                             int(keep_host), err, 512)
        if not self.h:
            raise RuntimeError("DecodeStep.load failed: " + err.value.decode())

    def step(self, ids, pos, want_logits=False):
        import numpy as np

        M = len(ids)
        a, _ = _ints(ids)
        b, _ = _ints(pos)
        nxt = (C.c_int * M)()
        best = (C.c_float * M)()
        logits = np.zeros((M, self.cfg.vocab), np.uint16) if want_logits else None
        rc = lib().cccc_host_step_run(self.h, a, b, M, nxt, best, logits.ctypes.data if want_logits else None)
        if rc != 0:
            raise RuntimeError(f"DecodeStep.step failed: {rc}")
        return list(nxt), list(best), logits

    def reset(self):
        lib().cccc_host_step_reset(self.h)

    def use_program(self, on=True):
        return bool(lib().cccc_host_step_use_program(self.h, int(on)))

    def info(self, what):
        return int(lib().cccc_host_step_info(self.h, what))

    def save(self, path):
        err = C.create_string_buffer(512)
        if lib().cccc_host_step_save(self.h, path.encode(), err, 512) != 0:
            raise RuntimeError(err.value.decode())

    def generate(self, ctx_ids, max_new, seed=0, sampler=None, **gen):
        ctx, nc = _ints(ctx_ids)
        out = (C.c_int * max(1, max_new))()
        stats = (C.c_int * 3)()
        t, k, p, r, banned, nb = _sampler_args(sampler)
        n = lib().cccc_host_step_generate(self.h, self.cfg.vocab, ctx, nc, _gen_ints(**gen), t, k, p, r, banned, nb, seed, max_new, out, max_new,
                                          stats)
        if n < 0:
            raise RuntimeError("a decode step failed")
        return list(out[:n]), dict(rebuilds=stats[0], decode_steps=stats[1], prefill_tokens=stats[2])

    def close(self):
        if self.h:
            lib().cccc_host_step_destroy(self.h)
            self.h = None


def tp_generate(path, devices, cfg, max_context, ctx_ids, max_new, seed=0, sampler=None, weight_data_type=-1, **gen):
    """Tensor-parallel generation in ONE process: a host thread, GpuControl and DecodeStep per device."""
    dev, world = _ints(devices)
    ctx, nc = _ints(ctx_ids)
    out = (C.c_int * max(1, max_new))()
    stats = (C.c_int * 3)()
    err = C.create_string_buffer(1024)
    t, k, p, r, banned, nb = _sampler_args(sampler)
    n = lib().cccc_host_tp_generate(path.encode(), dev, world, model_ints(cfg, max_context, weight_data_type), cfg.rope_theta, cfg.eps, ctx, nc,
                                    _gen_ints(**gen), t, k, p, r, banned, nb, seed, max_new, out, max_new, stats, err, 1024)
    if n == -2:
        raise RuntimeError("the ranks chose different tokens")
    if n < 0:
        raise RuntimeError("tensor-parallel generation failed: " + err.value.decode())
    return list(out[:n]), dict(rebuilds=stats[0], decode_steps=stats[1], prefill_tokens=stats[2])


def tp_steps(path, devices, cfg, max_context, tokens, weight_data_type=-1):
    """Feeds `tokens` at cache rows 0.. on the given devices (one process, a thread per device); returns
    (next ids [world][n], best logit [n], logits [n][vocab] float32)."""
    import numpy as np

    dev, world = _ints(devices)
    tok, n = _ints(tokens)
    nxt = (C.c_int * (world * n))()
    best = np.zeros(n, np.float32)
    logits = np.zeros((n, cfg.vocab), np.float32)
    err = C.create_string_buffer(1024)
    rc = lib().cccc_host_tp_steps(path.encode(), dev, world, model_ints(cfg, max_context, weight_data_type), cfg.rope_theta, cfg.eps, tok, n, nxt,
                                  best.ctypes.data_as(C.POINTER(C.c_float)), logits.ctypes.data_as(C.POINTER(C.c_float)), err, 1024)
    if rc != 0:
        raise RuntimeError(f"tensor-parallel steps failed ({rc}): " + err.value.decode())
    return np.array(list(nxt), np.int32).reshape(world, n), best, logits
