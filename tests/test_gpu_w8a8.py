"""W8A8: E4M3 weights times E4M3-quantised activations (the reference's mode with act_data_type = FP8_E4M3,
cccc/cublas_real.h:619-666).  The activation quantiser bit for bit against the reference's own kernels (compiled from
its cuda_functions.cu) and against the CPU oracle; the linear (tcgen05.mma kind::f8f6f4 on both operands as they are)
against the oracle at the GEMM bar (max relative error 1e-2 with the 1e-2 * rms floor, cosine >= 0.9999) and against
the reference's own dispatcher running its cublasLt FP8 x FP8 matmul on the same device buffers."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, ref_cuda_lib, ref_gemm_lib, to_dev

pytestmark = pytest.mark.gpu


def acts(rng, M, K, spread=0.0):
    x = rng.standard_normal((M, K)).astype(np.float32)
    if spread:
        x *= np.exp2(rng.integers(-spread, spread, (M, K))).astype(np.float32)
    return O.f32_to_bf16_bits(x)


@pytest.mark.parametrize("n", [1, 255, 4096, 100_003])
def test_dynamic_quantiser_matches_the_reference_s_kernels_and_the_oracle(n):
    import torch

    c = capi()
    rng = np.random.default_rng(n)
    X = acts(rng, 1, n, spread=6).reshape(-1)
    if n > 300:
        X[7] = 0x7FC0    # a NaN: fmaxf skips it in the absmax and the encoder writes 0x7F
    dX = to_dev(X)
    q = torch.zeros(n, dtype=torch.uint8, device="cuda")
    tmp = torch.full((1,), 7.0, dtype=torch.float32, device="cuda")
    inv = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert c.bf16_to_fp8e4m3_dynamic(dX, q, n, tmp, inv) == 0 and c.check_error("quant") == 0
    want_q, want_inv = O.quantise_activations_e4m3(X)
    assert np.array_equal(q.cpu().numpy(), want_q)
    assert np.float32(inv.item()) == np.float32(want_inv)
    R = ref_cuda_lib()
    if R is not None:
        R.cuda_bf16_to_fp8e4m3_dynamic.restype = C.c_int
        R.cuda_bf16_to_fp8e4m3_dynamic.argtypes = [C.c_void_p, C.c_void_p, C.c_uint, C.c_void_p, C.c_void_p]
        q2 = torch.zeros(n, dtype=torch.uint8, device="cuda")
        inv2 = torch.zeros(1, dtype=torch.float32, device="cuda")
        assert R.cuda_bf16_to_fp8e4m3_dynamic(dX.data_ptr(), q2.data_ptr(), n, tmp.data_ptr(), inv2.data_ptr()) == 0
        torch.cuda.synchronize()
        assert torch.equal(q, q2) and inv.item() == inv2.item()


def test_dynamic_quantiser_on_zeros():
    import torch

    c = capi()
    n = 512
    dX = torch.zeros(n, dtype=torch.int16, device="cuda")
    q = torch.full((n,), 9, dtype=torch.uint8, device="cuda")
    tmp = torch.zeros(1, dtype=torch.float32, device="cuda")
    inv = torch.zeros(1, dtype=torch.float32, device="cuda")
    assert c.bf16_to_fp8e4m3_dynamic(dX, q, n, tmp, inv) == 0 and c.check_error("quant") == 0
    assert int(q.max()) == 0 and inv.item() == 1.0


def run(W, w_inv, X, act_scale, N, M, K, Y0=None, **kw):
    import torch

    c = capi()
    dW, dX = to_dev(W), to_dev(X)
    f32 = bool(kw.get("flags", 0) & 4)
    ldy_m, ldy_n = kw.get("ldy_m", N), kw.get("ldy_n", 1)
    size = (M - 1) * ldy_m + (N - 1) * ldy_n + 1
    dY = to_dev(Y0) if Y0 is not None else torch.zeros(size, dtype=torch.float32 if f32 else torch.int16, device="cuda")
    before = c.launch_count()
    assert c.gemm_w8a8_bf16(dW, w_inv, dX, act_scale, dY, N, M, K, **kw) == 0 and c.check_error("w8a8") == 0
    # quantiser, linear; the dynamic scale of more than 16384 activations (or 32 tokens) takes an absmax launch of its own before them
    assert c.launch_count() - before == (3 if act_scale == 0 and (M * K > 16384 or M > 32) else 2)
    return dY.cpu().numpy() if f32 else from_dev_u16(dY)


@pytest.mark.parametrize("act_scale", [0.0, 0.0123])
@pytest.mark.parametrize("N,K,M", [(128, 128, 1), (256, 512, 2), (1000, 4096, 5), (4096, 4096, 16), (512, 2048, 17),
                                   (2500, 1024, 32), (6144, 4096, 1), (100, 28672, 3), (24576, 4096, 4)])
def test_w8a8_linear_matches_oracle(act_scale, N, K, M):
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=N + M, scaled=True)
    Y = run(W, w_inv, X, act_scale, N, M, K)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K, act_scale=act_scale)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (N, K, M, act_scale))


@pytest.mark.parametrize("fh", [1, 2, 3])
@pytest.mark.parametrize("act_scale", [0.0, 0.0123])
@pytest.mark.parametrize("N,K,M", [(256, 128, 33), (1000, 512, 100), (4096, 4096, 256), (1024, 2048, 300), (2500, 1024, 257),
                                   (100, 12288, 48), (4096, 4096, 64), (384, 256, 65), (6144, 4096, 1024), (24576, 1024, 2100)])
def test_w8a8_linear_above_32_tokens_matches_oracle(fh, act_scale, N, K, M):
    """More than 32 tokens: the CTA-pair kernels (flags bits 8-9: one tile of 256 or of 512 features per pair, or 3 = the
    persistent form that walks 256-feature tiles with two accumulators), ragged token and feature edges, TMA-stored
    tiles; 6144 x 4096 at 1024 and 24576 x 1024 at 2100 tokens give the persistent pairs several tiles each."""
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=N + M, scaled=True)
    Y = run(W, w_inv, X, act_scale, N, M, K, flags=fh << 8)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K, act_scale=act_scale)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (N, K, M, act_scale, fh))


@pytest.mark.parametrize("fh", [1, 2, 3])
def test_w8a8_above_32_tokens_float32_strides_and_accumulate(fh):
    """The element-by-element epilogue of the CTA-pair kernel: float32 output against float64 sums; transposed output with
    alpha and beta."""
    N, K, M = 700, 1024, 70
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=5, scaled=True)
    Yf = run(W, w_inv, X, 0.0, N, M, K, flags=4 | (fh << 8)).reshape(M, N)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K)
    rms = np.sqrt(np.mean(np.square(y32), axis=1, keepdims=True))
    assert np.max(np.abs(Yf - y32) / np.maximum(np.abs(y32), rms)) < 1e-5
    rng = np.random.default_rng(4)
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 3)).astype(np.float32))
    Y = run(W, w_inv, X, 0.0, N, M, K, Y0=Y0.copy(), alpha=0.25, beta=1.5, ldy_m=1, ldy_n=M + 3, flags=fh << 8)
    ya, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K, alpha=0.25)
    got = O.bf16_bits_to_f32(Y[:N * (M + 3)]).reshape(N, M + 3)
    want = ya.T + 1.5 * O.bf16_bits_to_f32(Y0)[:, :M]
    assert_close(got[:, :M].T.copy(), want.T.copy(), "alpha beta strides")
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])


@pytest.mark.parametrize("M", [4, 70])
def test_w8a8_static_scale_that_saturates(M):
    """A static activation scale below the data's range: about 7 % of the activations clamp to +-448 in the quantiser
    (and some fall into E4M3's subnormals), which the oracle's encoder models exactly."""
    N, K = 512, 1024
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=M, scaled=True)
    q, _ = O.quantise_activations_e4m3(X, act_scale=0.004)
    assert 0.02 < np.mean((q & 0x7F) == 0x7E) < 0.2
    Y = run(W, w_inv, X, 0.004, N, M, K)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K, act_scale=0.004)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, ("saturating", M))


def test_w8a8_float32_output_is_the_exact_sum():
    """FP8 x FP8 products are exact in FP32 and so are the sums of a few thousand of them at these magnitudes: the
    float32 output against the oracle's float64 sums."""
    N, K, M = 1024, 4096, 8
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=3, scaled=True)
    Yf = run(W, w_inv, X, 0.0, N, M, K, flags=4).reshape(M, N)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K)
    rms = np.sqrt(np.mean(np.square(y32), axis=1, keepdims=True))
    assert np.max(np.abs(Yf - y32) / np.maximum(np.abs(y32), rms)) < 1e-5


def test_w8a8_alpha_beta_and_strides():
    N, K, M = 200, 512, 20
    ldw, ldx = K + 256, K + 8
    rng = np.random.default_rng(3)
    Wd, _, w_inv, Xd = O.make_inputs(O.FP8_E4M3, N, ldw, M, seed=13, scaled=True)
    W = Wd.reshape(N, ldw)[:, :K].copy()
    X = np.zeros((M, ldx), np.uint16)
    X[:, :K] = Xd.reshape(M, ldw)[:, :K]
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 3)).astype(np.float32))
    Y = run(Wd, w_inv, X, 0.0, N, M, K, Y0=Y0.copy(), ldw=ldw, ldx=ldx, alpha=0.25, beta=1.5, ldy_m=1, ldy_n=M + 3)
    y32, _, _ = O.linear_w8a8(W, w_inv, X[:, :K].copy(), N, M, K, alpha=0.25)
    got = O.bf16_bits_to_f32(Y[:N * (M + 3)]).reshape(N, M + 3)
    want = y32.T + 1.5 * O.bf16_bits_to_f32(Y0)[:, :M]
    assert_close(got[:, :M].T.copy(), want.T.copy(), "alpha beta strides")
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])


def test_w8a8_refuses_what_it_does_not_serve():
    import torch

    c = capi()
    W = torch.zeros(256 * 256, dtype=torch.uint8, device="cuda")
    X = torch.zeros(64 * 256, dtype=torch.int16, device="cuda")
    Y = torch.zeros(64 * 256, dtype=torch.int16, device="cuda")
    assert c.gemm_w8a8_bf16(W, 1.0, X, 0.0, Y, 256, 33, 256) == 0 and c.check_error("33") == 0    # the CTA-pair kernel
    assert c.gemm_w8a8_bf16(W, 1.0, X, 0.0, Y, 256, 4, 192) == -1        # K % 128
    assert c.gemm_w8a8_bf16(W, 1.0, X, -1.0, Y, 256, 4, 256) == -1       # a negative activation scale
    assert c.gemm_w8a8_bf16(W, 1.0, X, 0.0, Y, 0, 4, 256) == 0           # nothing to do


@pytest.mark.parametrize("act_scale", [0.0, 0.02])
@pytest.mark.parametrize("M", [1, 8, 32, 48, 64, 300, 2048])
def test_w8a8_against_the_reference_s_own_dispatcher(act_scale, M):
    """cccc::Cublas::gemm's typed overload with the activation type set to FP8_E4M3 (cublasLt FP8 x FP8, both scale
    pointers) on the same device buffers."""
    import torch

    R = ref_gemm_lib()
    if R is None:
        pytest.skip("oracle/_ref/libref_gpu_gemm.so not built")
    R.ref_cublas_set_act_type.restype = C.c_int
    R.ref_cublas_set_act_type.argtypes = [C.c_int]
    c = capi()
    N, K = 4096, 4096
    W, _, w_inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=31 + M, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    ours = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    ref = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    assert c.gemm_w8a8_bf16(dW, w_inv, dX, act_scale, ours, N, M, K) == 0 and c.check_error("t") == 0
    R.ref_cublas_gemm_w8_typed.restype = C.c_int
    R.ref_cublas_gemm_w8_typed.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                           C.c_float, C.c_void_p, C.c_int, C.c_float, C.c_int, C.c_float]
    assert R.ref_cublas_set_act_type(O.FP8_E4M3) == 0
    try:
        # cccc's call: C(N x M, ldc N) = A^T (weight, lda K) * B (activations, ldb K), through the typed overload
        rc = R.ref_cublas_gemm_w8_typed(1, 0, N, M, K, 1.0, dW.data_ptr(), K, dX.data_ptr(), K, 0.0, ref.data_ptr(), N, w_inv,
                                        O.FP8_E4M3, act_scale)
    finally:
        R.ref_cublas_set_act_type(3)    # BFLOAT16 again: the library object is shared with other tests
    assert rc == 0
    a = O.bf16_bits_to_f32(from_dev_u16(ours)).reshape(M, N)
    b = O.bf16_bits_to_f32(from_dev_u16(ref)).reshape(M, N)
    y32, _, _ = O.linear_w8a8(W, w_inv, X, N, M, K, act_scale=act_scale)
    assert_close(b, y32, "the reference's W8A8 against the oracle")
    assert_close(a, b, "ours against the reference's W8A8")


def test_the_host_dispatcher_takes_w8a8_when_its_activation_type_says_so():
    """Matrix::mulBatched -> Cublas::gemm with setActDataType(FP8_E4M3), as cccc's MainProcess sets it for
    weight_data_type = fp8_e4m3 (cccc/MainProcess.cpp:398-409): the W8A8 linear; back to BFLOAT16: W8A16 again."""
    import torch

    from __graft_entry__ import load_package

    h = load_package().hostapi
    L = h.lib()
    g = L.cccc_host_gpu_create(0)
    assert g
    try:
        N, K, M = 512, 1024, 4
        W, _, inv, X = O.make_inputs(O.FP8_E4M3, N, K, M, seed=9, scaled=True)
        dW, dX = to_dev(W), to_dev(X)
        mW = L.cccc_host_matrix_view(g, dW.data_ptr(), K, N, 1, 1, O.FP8_E4M3, inv, None)
        mX = L.cccc_host_matrix_view(g, dX.data_ptr(), K, M, 1, 1, O.BFLOAT16, 1.0, None)
        outs = []
        for act in (O.FP8_E4M3, O.BFLOAT16):
            dY = torch.zeros(M * N, dtype=torch.int16, device="cuda")
            mY = L.cccc_host_matrix_view(g, dY.data_ptr(), N, M, 1, 1, O.BFLOAT16, 1.0, None)
            L.cccc_host_set_act_type(g, act)
            before = L.cccc_host_fused_calls(g)
            L.cccc_host_mul_batched(mW, mX, mY, h.MATRIX_TRANS, h.MATRIX_NO_TRANS, 1.0, 0.0)
            L.cccc_host_gpu_sync(g)
            assert L.cccc_host_fused_calls(g) == before + 1 and capi().check_error("host") == 0
            outs.append(O.bf16_bits_to_f32(from_dev_u16(dY)).reshape(M, N))
            L.cccc_host_matrix_free(mY)
        y8, _, _ = O.linear_w8a8(W, inv, X, N, M, K)
        _, y16 = O.linear_wq_bf16(O.FP8_E4M3, W, None, inv, X, N, M, K)
        assert_close(outs[0], y8, "host W8A8")
        assert_close(outs[1], y16, "host W8A16")
        assert not np.array_equal(outs[0], outs[1])    # the activations' quantisation is visible
        for m in (mW, mX):
            L.cccc_host_matrix_free(m)
    finally:
        L.cccc_host_set_act_type(g, O.BFLOAT16)
        L.cccc_host_gpu_destroy(g)


@pytest.mark.parametrize("n", [1000, 4096, 65536 + 16])
def test_fp8_elementwise_ops_match_the_reference_s_kernels(n):
    """add, silu, elementmul, addbias (E4M3 and BF16 bias) on E4M3 tensors: the same bytes as the reference's kernels
    (cccc-cuda/cuda_functions.cu:2446-2544), NaN bytes and saturation included; n = 1000 takes the one-byte path,
    the others sixteen bytes per thread."""
    import torch

    R = ref_cuda_lib()
    if R is None:
        pytest.skip("oracle/_ref/libcccc-cuda-ref.so not built")
    L = capi().lib()
    g = torch.Generator(device="cuda").manual_seed(n)
    A = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
    B = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
    R0 = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
    bias8 = torch.randint(0, 0x78, (64,), dtype=torch.uint8, device="cuda", generator=g)
    bias16 = torch.randn(64, device="cuda", generator=g).to(torch.bfloat16)
    sigs = {"cuda_add_fp8e4m3": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_float, C.c_float, C.c_float],
            "cuda_silu_fp8e4m3": [C.c_void_p, C.c_void_p, C.c_uint],
            "cuda_elementmul_fp8e4m3": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_float, C.c_float],
            "cuda_addbias_fp8e4m3": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint, C.c_uint, C.c_float, C.c_float],
            "cuda_addbias_fp8e4m3_bf16bias": [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_uint, C.c_uint, C.c_float, C.c_float]}
    for name, args in sigs.items():
        getattr(R, name).restype = C.c_int
        getattr(R, name).argtypes = args

    def both(name, build_args):
        outs = []
        for lib_ in (L, R):
            r = R0.clone()
            assert getattr(lib_, name)(*build_args(r)) == 0
            torch.cuda.synchronize()
            outs.append(r)
        assert torch.equal(outs[0], outs[1]), name
        return outs[0]

    for a, b, r in ((1.0, 1.0, 0.0), (0.5, -2.0, 1.0), (100.0, 100.0, 0.25)):
        both("cuda_add_fp8e4m3", lambda out: (A.data_ptr(), B.data_ptr(), out.data_ptr(), n, a, b, r))
    both("cuda_silu_fp8e4m3", lambda out: (A.data_ptr(), out.data_ptr(), n))
    for a, r in ((1.0, 0.0), (0.125, 1.0)):
        both("cuda_elementmul_fp8e4m3", lambda out: (A.data_ptr(), B.data_ptr(), out.data_ptr(), n, a, r))
    for size_mc, size_b in ((1, 64), (8, 50)):
        both("cuda_addbias_fp8e4m3", lambda out: (None, bias8.data_ptr(), out.data_ptr(), n, size_mc, size_b, 1.0, 1.0))
        both("cuda_addbias_fp8e4m3_bf16bias", lambda out: (None, bias16.data_ptr(), out.data_ptr(), n, size_mc, size_b, 0.5, 2.0))
    assert capi().check_error("fp8 ops") == 0


@pytest.mark.parametrize("D", [64, 100])
def test_fp8_embedding_variants_match_the_reference_s_kernels(D):
    """cuda_embed_fwd_fp8_to_fp8 (E4M3 table re-encoded to scale 1) and cuda_embed_fwd_bf16_to_fp8 (BF16 table encoded
    at scale 1), ids as floats: the same bytes as the reference's kernels (cccc-cuda/cuda_functions.cu:1615-1667);
    D = 100 takes the one-byte path."""
    import torch

    R = ref_cuda_lib()
    if R is None:
        pytest.skip("oracle/_ref/libcccc-cuda-ref.so not built")
    L = capi().lib()
    T, B, vocab = 7, 3, 50
    g = torch.Generator(device="cuda").manual_seed(D)
    ids = torch.randint(0, vocab, (B, T), device="cuda", generator=g).to(torch.float32)
    W8 = torch.randint(0, 256, (vocab, D), dtype=torch.uint8, device="cuda", generator=g)
    W16 = (torch.randn(vocab, D, device="cuda", generator=g) * 100).to(torch.bfloat16)
    for lib_ in (R,):
        lib_.cuda_embed_fwd_fp8_to_fp8.restype = C.c_int
        lib_.cuda_embed_fwd_fp8_to_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float]
        lib_.cuda_embed_fwd_bf16_to_fp8.restype = C.c_int
        lib_.cuda_embed_fwd_bf16_to_fp8.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    outs = []
    for lib_ in (L, R):
        y8 = torch.full((B, T, D), 0x55, dtype=torch.uint8, device="cuda")
        y16 = torch.full((B, T, D), 0x55, dtype=torch.uint8, device="cuda")
        assert lib_.cuda_embed_fwd_fp8_to_fp8(ids.data_ptr(), W8.data_ptr(), y8.data_ptr(), D, T, B, 0.37) == 0
        assert lib_.cuda_embed_fwd_bf16_to_fp8(ids.data_ptr(), W16.data_ptr(), y16.data_ptr(), D, T, B) == 0
        torch.cuda.synchronize()
        outs.append((y8, y16))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    assert capi().check_error("fp8 embed") == 0


@pytest.mark.parametrize("y_type", [3, 4])
@pytest.mark.parametrize("N,K,M", [(512, 1024, 1), (4096, 4096, 8), (1000, 2048, 32), (1000, 2048, 70), (2048, 1024, 512)])
def test_both_operands_e4m3_against_the_oracle_and_the_reference(y_type, N, K, M):
    """cuda_gemm_fp8_fp8: weights and activations E4M3 already, output BF16 (3) or E4M3 (4: the BF16 result re-encoded at
    scale 1).  Against float64 sums of the decoded operands, and against the reference's own overloads
    (cccc/cublas_real.h:754-834) through its dispatcher."""
    import torch

    c = capi()
    rng = np.random.default_rng(N + M + y_type)
    W, _, w_inv, _ = O.make_inputs(O.FP8_E4M3, N, K, M, seed=N + M, scaled=True)
    x_inv = 0.03125
    Xq = O.float_to_fp8(rng.standard_normal(M * K).astype(np.float32), O.FP8_E4M3, 1.0 / x_inv)
    wf = O.fp8_to_float(W, O.FP8_E4M3, 1.0).reshape(N, K).astype(np.float64)
    xf = O.fp8_to_float(Xq, O.FP8_E4M3, 1.0).reshape(M, K).astype(np.float64)
    y = ((xf @ wf.T) * (float(np.float32(w_inv)) * x_inv)).astype(np.float32)
    dW, dX = to_dev(W), to_dev(Xq)
    ours = torch.zeros(M * N, dtype=torch.int16 if y_type == 3 else torch.uint8, device="cuda")
    assert c.lib().cuda_gemm_fp8_fp8(dW.data_ptr(), w_inv, dX.data_ptr(), x_inv, ours.data_ptr(), y_type, N, M, K, K, K, N, 1, 1.0, 0.0, None, 0) == 0
    assert c.check_error("fp8 x fp8") == 0

    def check_bytes(got, want_bytes, what):
        # one E4M3 code is a 6-12 % step: sums that differ in their last bits may land on either side of a
        # truncation boundary, so a few bytes may differ by one code
        diff = np.abs(got.astype(np.int16) - want_bytes.astype(np.int16))
        assert diff.max() <= 1 and np.mean(diff != 0) < 2e-3, (what, int(diff.max()), float(np.mean(diff != 0)))

    if y_type == 3:
        assert_close(O.bf16_bits_to_f32(from_dev_u16(ours)).reshape(M, N), y, "oracle")
    else:
        want = O.float_to_fp8(O.bf16_bits_to_f32(O.f32_to_bf16_bits(y)).reshape(-1), O.FP8_E4M3, 1.0)
        check_bytes(ours.cpu().numpy(), want, "oracle")
    R = ref_gemm_lib()
    if R is None:
        return
    ref = torch.zeros(M * N, dtype=torch.int16 if y_type == 3 else torch.uint8, device="cuda")
    # cccc's call: C(N x M, ldc N) = A^T (weight, lda K) * B (activations, ldb K)
    rc = R.ref_cublas_gemm(1, 0, N, M, K, 1.0, dW.data_ptr(), O.FP8_E4M3, K, w_inv, dX.data_ptr(), O.FP8_E4M3, K, x_inv, 0.0,
                           ref.data_ptr(), y_type, N, 0.0, None, None)
    assert rc == 0
    if y_type == 3:
        assert_close(O.bf16_bits_to_f32(from_dev_u16(ours)).reshape(M, N), O.bf16_bits_to_f32(from_dev_u16(ref)).reshape(M, N), "reference")
    else:
        check_bytes(ours.cpu().numpy(), ref.cpu().numpy(), "reference")


@pytest.mark.parametrize("act_scale", [0.0, 0.04])
@pytest.mark.parametrize("M", [1, 12, 32, 130])
def test_w8a8_group_is_one_quantisation_and_one_launch_with_the_bits_of_separate_calls(act_scale, M):
    import torch

    c = capi()
    Ns, K = (512, 128, 160), 1024
    X = None
    items, host = [], []
    for j, N in enumerate(Ns):
        W, _, inv, Xj = O.make_inputs(O.FP8_E4M3, N, K, M, seed=3 + j, scaled=True)
        X = Xj if X is None else X
        host.append((W, inv, N))
        items.append(dict(W=to_dev(W), S=None, inv=inv, N=N, Y=torch.zeros(M * N, dtype=torch.int16, device="cuda"), alpha=1.0 + 0.5 * j, beta=0.0))
    dX = to_dev(X)
    before = c.launch_count()
    assert c.gemm_w8a8_bf16_group(c.make_group(items, K), dX, act_scale, M, K) == 0 and c.check_error("group") == 0
    assert c.launch_count() - before == (3 if act_scale == 0 and (M * K > 16384 or M > 32) else 2)
    for it, (W, inv, N) in zip(items, host):
        sep = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        assert c.gemm_w8a8_bf16(it["W"], inv, dX, act_scale, sep, N, M, K, alpha=it["alpha"]) == 0 and c.check_error("sep") == 0
        assert torch.equal(sep, it["Y"])
        y32, _, _ = O.linear_w8a8(W, inv, X, N, M, K, act_scale=act_scale, alpha=it["alpha"])
        assert_close(O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N), y32, ("oracle", M, N))


def test_e4m3_activations_read_in_place_or_copied_give_the_same_bits():
    """Above 32 tokens cuda_gemm_fp8_fp8 lets TMA read the E4M3 activations where they lie when their rows are 16-byte
    aligned; rows 8 bytes off are first moved into the workspace.  Same bits either way."""
    import torch

    c = capi()
    N, K, M = 640, 1024, 70
    rng = np.random.default_rng(2)
    W, _, w_inv, _ = O.make_inputs(O.FP8_E4M3, N, K, M, seed=1, scaled=True)
    Xq = O.float_to_fp8(rng.standard_normal(M * K).astype(np.float32), O.FP8_E4M3, 32.0).reshape(M, K)
    Xpad = np.zeros((M, K + 8), np.uint8)
    Xpad[:, :K] = Xq
    dW = to_dev(W)
    outs = []
    for X, ldx in ((Xq, K), (Xpad, K + 8)):
        dX = to_dev(X.reshape(-1))
        Y = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        before = c.launch_count()
        assert c.lib().cuda_gemm_fp8_fp8(dW.data_ptr(), w_inv, dX.data_ptr(), 0.03125, Y.data_ptr(), 3, N, M, K, K, ldx, N, 1, 1.0, 0.0, None, 0) == 0
        assert c.check_error("fp8 x fp8") == 0
        assert c.launch_count() - before == (1 if ldx == K else 2)
        outs.append(Y)
    assert torch.equal(outs[0], outs[1])
