"""The ops between the linears of a decode layer (RMSNorm, RoPE, embedding gather, SwiGLU, attention over
the KV cache with q/k norm + RoPE + append in its prologue) through the C-ABI, against the CPU oracle
(oracle/decode_ops_oracle.c) and, for the three ops the reference implements as CUDA kernels of its own,
against the reference's cuda_rms_norm_fwd / cuda_rope_fwd / cuda_embed_fwd from oracle/_ref.

Bars.  Gather, append: bit-exact.  RMSNorm, RoPE: the arithmetic is the reference kernels' (same
summation order, same fused multiply-adds), so bit-exact against the reference's kernels on the device;
against the CPU oracle at most a rare one-unit difference in the last BF16 place is allowed, because the
device's rsqrt instruction is not IEEE's 1/sqrt.  SwiGLU: the same, for expf.  Attention: its sums run in
another order than cuBLAS's, so the bar is that of the GEMM outputs (1e-2, cosine >= 0.9999 against the
unrounded oracle output) with the element-wise error taken relative to max(|ref|, rms of the head's
output): see tests/_util.py:assert_close_rows for why the reference's BF16 score tensor asks for that."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close_rows, capi, from_dev_u16, ref_cuda_lib, to_dev

pytestmark = pytest.mark.gpu


def bf16_rand(rng, shape, std=1.0):
    return O.f32_to_bf16_bits((rng.standard_normal(shape) * std).astype(np.float32))


def ulp_diff(a, b):
    """Distance in BF16 code points (sign-magnitude order), uint16 arrays."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a) - key(b))


def assert_nearly_bit_equal(got, want, what, max_frac=2e-3):
    d = ulp_diff(got.reshape(-1), want.reshape(-1))
    assert d.max() <= 1, (what, int(d.max()))
    assert (d != 0).mean() <= max_frac, (what, float((d != 0).mean()))


@pytest.mark.parametrize("rows,inner", [(1, 4096), (4, 4096), (32, 4096), (3, 128), (40, 128), (2, 12288), (5, 1000)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rms_norm(rows, inner, with_residual):
    import torch

    c = capi()
    rng = np.random.default_rng(rows + inner)
    X = bf16_rand(rng, (rows, inner), 2.0)
    R = bf16_rand(rng, (rows, inner)) if with_residual else None
    w = O.f32_to_bf16_bits((1.0 + 0.02 * rng.standard_normal(inner)).astype(np.float32))
    dX, dW = to_dev(X), to_dev(w)
    dR = to_dev(R) if R is not None else None
    dS = torch.zeros(rows * inner, dtype=torch.int16, device="cuda") if R is not None else None
    dY = torch.zeros(rows * inner, dtype=torch.int16, device="cuda")
    assert c.rms_norm_bf16(dX, dY, dW, rows, inner, 1e-6, residual=dR, sum_out=dS) == 0 and c.check_error("rms") == 0
    xin = X
    if R is not None:
        xin = O.add_bf16(X, R)
        assert np.array_equal(from_dev_u16(dS).reshape(rows, inner), xin)   # the residual stream itself: exact
    want = O.rms_norm_bf16(xin, w, 1e-6)
    assert_nearly_bit_equal(from_dev_u16(dY).reshape(rows, inner), want, ("rms", rows, inner))
    L = ref_cuda_lib()
    if L is not None:
        # the reference's own kernel on the same device buffers: bit for bit
        L.cuda_rms_norm_fwd.restype = C.c_int
        L.cuda_rms_norm_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_uint, C.c_uint, C.c_float,
                                        C.c_float]
        dXin = to_dev(xin)
        ref = torch.zeros(rows * inner, dtype=torch.int16, device="cuda")
        inv = torch.zeros(rows, dtype=torch.float32, device="cuda")
        assert L.cuda_rms_norm_fwd(3, dXin.data_ptr(), ref.data_ptr(), dW.data_ptr(), 3, inv.data_ptr(), rows, inner, 1e-6, 1.0) == 0
        assert torch.equal(ref, dY), ("reference kernel", rows, inner)


@pytest.mark.parametrize("D,T,B,off", [(128, 1, 40, 4095), (128, 7, 3, 11), (64, 5, 2, 0), (128, 64, 8, 100)])
def test_rope(D, T, B, off):
    import torch

    c = capi()
    rng = np.random.default_rng(D + T + off)
    cos, sin = O.rope_tables_bf16(off + T, D, 1e6)
    X = bf16_rand(rng, (B, T, D))
    dX, dC, dS = to_dev(X), to_dev(cos), to_dev(sin)
    dY = torch.zeros(B * T * D, dtype=torch.int16, device="cuda")
    assert c.rope_bf16(dX, dY, dC, dS, D, T, B, off) == 0 and c.check_error("rope") == 0
    want = O.rope_bf16(X, cos, sin, off)
    assert np.array_equal(from_dev_u16(dY).reshape(B, T, D), want)
    L = ref_cuda_lib()
    if L is not None:
        L.cuda_rope_fwd.restype = C.c_int
        L.cuda_rope_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint, C.c_uint, C.c_uint]
        ref = torch.zeros(B * T * D, dtype=torch.int16, device="cuda")
        assert L.cuda_rope_fwd(3, dX.data_ptr(), ref.data_ptr(), dC.data_ptr(), dS.data_ptr(), D, T, B, off) == 0
        d = ulp_diff(from_dev_u16(ref), from_dev_u16(dY))
        # the same expression; which of the two products the reference's compiler fuses is its choice
        assert d.max() <= 1 and (d != 0).mean() < 1e-3, (int(d.max()), float((d != 0).mean()))


def test_embed_gather():
    import torch

    c = capi()
    rng = np.random.default_rng(3)
    V, D = 1000, 4096
    W = bf16_rand(rng, (V, D))
    ids = np.array([0, 999, 17, 17, 512], np.int32)
    dW = to_dev(W)
    dI = torch.from_numpy(ids).cuda()
    dY = torch.zeros(ids.size * D, dtype=torch.int16, device="cuda")
    assert c.embed_bf16(dI, dW, dY, D, ids.size, V) == 0 and c.check_error("embed") == 0
    assert np.array_equal(from_dev_u16(dY).reshape(-1, D), O.embed_bf16(ids, W))
    L = ref_cuda_lib()
    if L is not None:
        L.cuda_embed_fwd.restype = C.c_int
        L.cuda_embed_fwd.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]
        idf = torch.from_numpy(ids.astype(np.float32)).cuda()
        ref = torch.zeros(ids.size * D, dtype=torch.int16, device="cuda")
        assert L.cuda_embed_fwd(3, idf.data_ptr(), dW.data_ptr(), ref.data_ptr(), D, ids.size, 1, 1.0) == 0
        assert torch.equal(ref, dY)
    # an id outside the table gives zeros, not a wild read
    bad = torch.tensor([V + 5, -1], dtype=torch.int32, device="cuda")
    out = torch.ones(2 * D, dtype=torch.int16, device="cuda")
    assert c.embed_bf16(bad, dW, out, D, 2, V) == 0 and c.check_error("embed") == 0
    assert not out.any()


@pytest.mark.parametrize("rows,cols", [(1, 12288), (32, 14336), (3, 1000)])
def test_swiglu(rows, cols):
    import torch

    c = capi()
    rng = np.random.default_rng(cols)
    G, U = bf16_rand(rng, (rows, cols), 3.0), bf16_rand(rng, (rows, cols))
    dG, dU = to_dev(G), to_dev(U)
    dO = torch.zeros(rows * cols, dtype=torch.int16, device="cuda")
    assert c.swiglu_bf16(dG, dU, dO, rows, cols) == 0 and c.check_error("swiglu") == 0
    want = O.mul_bf16(O.silu_bf16(G), U)
    assert_nearly_bit_equal(from_dev_u16(dO).reshape(rows, cols), want, "swiglu")


def attention_case(B, H, Hkv, hd, T_max, pos, qk_norm, seed, strided=False):
    """Runs cuda_attn_decode_bf16 and the oracle's composition of the reference's ops on the same inputs."""
    import torch

    c = capi()
    rng = np.random.default_rng(seed)
    pos = np.asarray(pos, np.int32)
    q = bf16_rand(rng, (B, H * hd))
    k = bf16_rand(rng, (B, Hkv * hd))
    v = bf16_rand(rng, (B, Hkv * hd))
    Kc = bf16_rand(rng, (B, Hkv, T_max, hd))
    Vc = bf16_rand(rng, (B, Hkv, T_max, hd))
    qn = O.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)) if qk_norm else None
    kn = O.f32_to_bf16_bits((1.0 + 0.1 * rng.standard_normal(hd)).astype(np.float32)) if qk_norm else None
    cos, sin = O.rope_tables_bf16(int(pos.max()) + 1, hd, 1e6)

    # ---- oracle: the reference's op sequence ----
    Kc_o, Vc_o = Kc.copy(), Vc.copy()
    Qr = np.empty((B, H, hd), np.uint16)
    for b in range(B):
        qh = q[b].reshape(H, hd)
        kh = k[b].reshape(Hkv, hd)
        if qk_norm:
            qh = O.rms_norm_bf16(qh, qn, 1e-6)
            kh = O.rms_norm_bf16(kh, kn, 1e-6)
        Qr[b] = O.rope_bf16(qh.reshape(H, 1, hd), cos, sin, int(pos[b])).reshape(H, hd)
        kr = O.rope_bf16(kh.reshape(Hkv, 1, hd), cos, sin, int(pos[b])).reshape(Hkv, hd)
        if pos[b] < T_max:
            O.kv_append_bf16(kr, Kc_o[b], int(pos[b]))
            O.kv_append_bf16(v[b].reshape(Hkv, hd), Vc_o[b], int(pos[b]))
    Yo, y32 = O.attention_decode_bf16(Qr, Kc_o, Vc_o, pos)

    # ---- device ----
    if strided:    # q, k, v as slices of one row, as a fused qkv projection writes them
        ld = (H + 2 * Hkv) * hd
        qkv = np.zeros((B, ld), np.uint16)
        qkv[:, :H * hd], qkv[:, H * hd:(H + Hkv) * hd], qkv[:, (H + Hkv) * hd:] = q, k, v
        dqkv = to_dev(qkv)
        dq, dk, dv = dqkv.view(-1)[0:], dqkv.view(-1)[H * hd:], dqkv.view(-1)[(H + Hkv) * hd:]
        lds = dict(ldq=ld, ldk=ld, ldv=ld)
    else:
        dq, dk, dv = to_dev(q), to_dev(k), to_dev(v)
        lds = {}
    dK, dV = to_dev(Kc), to_dev(Vc)
    dpos = torch.from_numpy(pos).cuda()
    out = torch.full((B, H * hd), 0x7FC0, dtype=torch.int16, device="cuda")
    keep = [to_dev(cos), to_dev(sin), to_dev(qn) if qk_norm else None, to_dev(kn) if qk_norm else None]
    desc = c.make_attn_decode(q=dq, k=dk, v=dv, k_cache=dK, v_cache=dV, pos=dpos, out=out, cos_tab=keep[0], sin_tab=keep[1],
                              q_norm=keep[2], k_norm=keep[3], B=B, H=H, Hkv=Hkv, head_dim=hd, T_max=T_max, **lds)
    assert c.attn_decode_bf16(desc) == 0 and c.check_error("attn") == 0
    got = O.bf16_bits_to_f32(from_dev_u16(out)).reshape(B, H, hd)
    assert_close_rows(got, y32, ("attention", B, H, Hkv, hd, T_max, pos.tolist()))
    # the caches: only row pos of each (sequence, kv head) changed, and it holds the oracle's rotated key / the value
    gK, gV = from_dev_u16(dK).reshape(Kc.shape), from_dev_u16(dV).reshape(Vc.shape)
    assert np.array_equal(gV, Vc_o)
    assert_nearly_bit_equal(gK, Kc_o, "appended keys", max_frac=1e-4)
    untouched = np.ones(Kc.shape, bool)
    for b in range(B):
        if pos[b] < T_max:
            untouched[b, :, pos[b], :] = False
    assert np.array_equal(gK[untouched], Kc[untouched])
    return got


def test_attention_qwen3_shape_full_cache():
    """Benchmark configuration 5's attention: 32 query heads, 8 kv heads of 128, 4096 cached rows."""
    attention_case(1, 32, 8, 128, 4096, [4095], True, 0, strided=True)


@pytest.mark.parametrize("pos", [0, 1, 31, 32, 100, 1000, 2047])
def test_attention_positions(pos):
    attention_case(1, 8, 2, 128, 2048, [pos], True, pos)


def test_attention_batch_with_different_positions():
    attention_case(5, 32, 8, 128, 1024, [0, 17, 1023, 512, 300], True, 5)
    attention_case(32, 32, 8, 128, 512, list(range(100, 132)), False, 6)


@pytest.mark.parametrize("H,Hkv,hd", [(4, 4, 128), (8, 4, 128), (16, 2, 128), (8, 2, 64), (4, 4, 64), (16, 2, 64)])
def test_attention_head_layouts(H, Hkv, hd):
    attention_case(2, H, Hkv, hd, 777, [776, 300], H % 3 == 1, H + hd)


def test_attention_refuses_what_it_does_not_take():
    import torch

    c = capi()
    z = torch.zeros(4096, dtype=torch.int16, device="cuda")
    p = torch.zeros(1, dtype=torch.int32, device="cuda")
    ok = dict(q=z, k=z, v=z, k_cache=z, v_cache=z, pos=p, out=z, cos_tab=z, sin_tab=z, B=1, H=4, Hkv=4, head_dim=128, T_max=4)
    assert c.attn_decode_bf16(c.make_attn_decode(**{**ok, "head_dim": 96})) == -1
    assert c.attn_decode_bf16(c.make_attn_decode(**{**ok, "H": 12, "Hkv": 4})) == -1     # 3 query heads per kv head
    assert c.attn_decode_bf16(c.make_attn_decode(**{**ok, "H": 6, "Hkv": 4})) == -1
    assert c.attn_decode_bf16(c.make_attn_decode(**{**ok, "q": None})) == -1
    assert c.attn_decode_bf16(c.make_attn_decode(**{**ok, "B": 0})) == 0
    assert c.check_error("refused") == 0
