"""The native-operand kernels: the quantised weight bytes go from HBM through TMA into shared memory and from there
into the tensor cores unchanged - FP8 (1 .. 32 tokens) into tcgen05.mma kind::f8f6f4, FP4 with its E4M3 block scales
(1 .. 32 tokens) into kind::mxf4nvf4 - and each BF16 activation row as three E5M2 rows (FP8) or seven E2M1 rows with
power-of-two block scales (FP4) whose sum it is.  A small kernel writes those rows (two launches); with flags bit 14
the FP8 kernel does it itself up to 8 tokens (one launch).
Forced through flags bit 12, so that every shape the kernels accept is checked, not only those the dispatcher gives them.
Against the CPU oracle at the GEMM bar (max relative error 1e-2 with the 1e-2 * rms floor, cosine >= 0.9999),
bit for bit on one-hot activations (where the output IS the dequantised weight), and bit for bit between runs
and between batch sizes."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, to_dev
from tests.test_gpu_onehot import all_positions, expected_bits, fp4_matrix, fp8_matrix, run_onehot

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3]
NATIVE = 0x1000
FUSED = 0x4000
FORMS = [0, FUSED]


def launches_of(wt, M, flags):
    """The split of the activations is a launch of its own unless the FP8 kernel was asked to do it itself (up to 8 tokens)."""
    return 1 if (wt != O.FP4_E2M1 and M <= 8 and (flags & FUSED)) else 2


def run(wt, W, inv, X, N, M, K, Y0=None, blk=None, **kw):
    import torch

    c = capi()
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    ldy_m, ldy_n = kw.get("ldy_m", N), kw.get("ldy_n", 1)
    size = (M - 1) * ldy_m + (N - 1) * ldy_n + 1
    f32 = bool(kw.get("flags", 0) & 4)
    if Y0 is not None:
        dY = to_dev(Y0)
    else:
        dY = torch.zeros(size, dtype=torch.float32 if f32 else torch.int16, device="cuda")
    kw["flags"] = kw.get("flags", 0) | NATIVE
    before = c.launch_count()
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, dY, N, M, K, **kw) == 0
    assert c.check_error("native") == 0
    assert c.launch_count() == before + launches_of(wt, M, kw["flags"])    # (the split of the activations, then) the linear
    return dY.cpu().numpy() if f32 else from_dev_u16(dY)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("N,K,M", [(128, 128, 1), (256, 512, 2), (384, 1024, 5), (200, 384, 6), (1000, 4096, 10), (512, 2048, 11),
                                   (4096, 4096, 16), (128, 12288, 17), (2500, 1024, 32), (6144, 4096, 1), (100, 28672, 3)])
def test_native_kernel_matches_oracle(wt, form, N, K, M):
    if form and M > 8:
        pytest.skip("the kernel splits the activations itself only up to 8 tokens")
    W, _, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=False)
    Y = run(wt, W, inv, X, N, M, K, flags=form)
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (wt, N, K, M))


@pytest.mark.parametrize("N,K,M", [(128, 256, 1), (256, 512, 2), (384, 1024, 3), (200, 768, 5), (1000, 4096, 6), (512, 2048, 8),
                                   (4096, 4096, 9), (128, 14336, 13), (6144, 4096, 1), (300, 1024, 7), (1000, 2048, 14),
                                   (640, 4096, 20), (2500, 1024, 32), (4096, 4096, 27)])
def test_native_fp4_kernel_matches_oracle(N, K, M):
    wt = O.FP4_E2M1
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=False)
    Y = run(wt, W, inv, X, N, M, K, blk=blk)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (wt, N, K, M))


def test_native_fp4_sums_stay_within_the_split_s_precision():
    """Seven E2M1 pieces hold an activation to 2^-16 of its 16-block's largest magnitude: the FP32 output stays within
    5e-5 (of the larger of |y| and the row's rms) of the oracle's float sums, two hundred times inside the GEMM bar."""
    wt, N, K, M = O.FP4_E2M1, 1024, 4096, 8
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=2, scaled=False)
    Yf = run(wt, W, inv, X, N, M, K, blk=blk, flags=4).reshape(M, N)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    rms = np.sqrt(np.mean(np.square(y32), axis=1, keepdims=True))
    assert np.max(np.abs(Yf - y32) / np.maximum(np.abs(y32), rms)) < 5e-5


def unsigned_scales(S):
    """The tensor cores read block scales as UNSIGNED E4M3 (the format of the reference's converter, whose scales are
    absmax / 6 >= 0); the sign bit that the generic matrix of the one-hot tests also exercises is outside that format."""
    return (S & 0x7F).astype(np.uint8)


@pytest.mark.parametrize("M", [1, 5, 9, 13, 14, 32])
def test_native_fp4_products_are_exact(M):
    N, K = 508, 512
    W, S = fp4_matrix(N, K)
    S = unsigned_scales(S)
    D = expected_bits(O.FP4_E2M1, W, S, 1.0, N, K)
    run_onehot(O.FP4_E2M1, W, S, 1.0, D, N, K, M, all_positions(K, M)[:40], flags=NATIVE)


@pytest.mark.parametrize("M", [3, 30])
def test_native_fp4_tiles_cut_across_ctas_are_exact(M):
    N, K = 200, 16384
    W, S = fp4_matrix(N, K)
    S = unsigned_scales(S)
    D = expected_bits(O.FP4_E2M1, W, S, 1.0, N, K)
    positions = np.random.default_rng(M).integers(0, K, (48, M))
    run_onehot(O.FP4_E2M1, W, S, 1.0, D, N, K, M, positions, flags=NATIVE)


def test_native_fp4_activations_of_very_different_magnitudes_and_non_finite_rows():
    wt, N, K, M = O.FP4_E2M1, 512, 1024, 4
    rng = np.random.default_rng(11)
    W, blk, inv, _ = O.make_inputs(wt, N, K, M, seed=5, scaled=False)
    x = rng.standard_normal((M, K)).astype(np.float32) * np.exp2(rng.integers(-6, 6, (M, K))).astype(np.float32)
    x[1] *= np.float32(2.0 ** -60)
    x[2] *= np.float32(2.0 ** 70)
    X = O.f32_to_bf16_bits(x).reshape(-1)
    Y = run(wt, W, inv, X, N, M, K, blk=blk, flags=4).reshape(M, N)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(Y, y32, ("range", wt))
    x[3, 17] = np.inf
    Y = run(wt, W, inv, O.f32_to_bf16_bits(x).reshape(-1), N, M, K, blk=blk, flags=4).reshape(M, N)
    assert np.isnan(Y[3]).all() and np.isfinite(Y[:3]).all()    # a row with an infinity or a NaN gives NaN outputs


@pytest.mark.parametrize("wt", WTS)
def test_native_float32_sums_are_those_of_fp32_accumulation(wt):
    """The FP32 output against the oracle's float sums: far inside the GEMM bar."""
    N, K, M = 1024, 4096, 8
    W, _, inv, X = O.make_inputs(wt, N, K, M, seed=2, scaled=False)
    Yf = run(wt, W, inv, X, N, M, K, flags=4).reshape(M, N)
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    rms = np.sqrt(np.mean(np.square(y32), axis=1, keepdims=True))
    assert np.max(np.abs(Yf - y32) / np.maximum(np.abs(y32), rms)) < 1e-5


@pytest.mark.parametrize("wt", WTS)
def test_native_activations_of_very_different_magnitudes(wt):
    """Rows whose elements span 2^40: what the split drops lies below 2^-31 of the row's largest magnitude."""
    N, K, M = 512, 1024, 4
    rng = np.random.default_rng(11)
    W, _, inv, _ = O.make_inputs(wt, N, K, M, seed=5, scaled=False)
    x = rng.standard_normal((M, K)).astype(np.float32) * np.exp2(rng.integers(-20, 20, (M, K))).astype(np.float32)
    x[1] *= np.float32(2.0 ** -60)    # a tiny row and a huge row: each token has its own power of two
    x[2] *= np.float32(2.0 ** 70)
    X = O.f32_to_bf16_bits(x).reshape(-1)
    Y = run(wt, W, inv, X, N, M, K, flags=4).reshape(M, N)
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    assert_close(Y, y32, ("range", wt))


@pytest.mark.parametrize("wt", WTS)
def test_native_alpha_beta_strides_and_output_modes(wt):
    N, K, M = 200, 512, 20
    ldw, ldx = K + 256, K + 8
    rng = np.random.default_rng(3)
    Wd, _, inv, Xd = O.make_inputs(wt, N, ldw, M, seed=13, scaled=False)
    X = np.zeros((M, ldx), np.uint16)
    X[:, :K] = Xd.reshape(M, ldw)[:, :K]
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 3)).astype(np.float32))
    kw = dict(ldw=ldw, ldx=ldx, alpha=0.25, beta=1.5, ldy_m=1, ldy_n=M + 3)
    Y = run(wt, Wd, 0.5, X, N, M, K, Y0=Y0.copy(), **kw)
    Yo, _ = O.linear_wq_bf16(wt, Wd, None, 0.5, X, N, M, K, Y=Y0, **kw)
    got = O.bf16_bits_to_f32(Y[:Yo.size]).reshape(N, M + 3)
    want = O.bf16_bits_to_f32(Yo).reshape(N, M + 3)
    assert_close(got[:, :M], want[:, :M], wt)
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])
    # residual epilogue: Y = bf16(bf16(W x) + Y)
    W, _, inv, X = O.make_inputs(wt, N, K, M, seed=4, scaled=False)
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    R0 = O.f32_to_bf16_bits(rng.standard_normal((M, N)).astype(np.float32))
    Yr = run(wt, W, inv, X, N, M, K, Y0=R0.copy().reshape(-1), beta=1.0, flags=8)
    prod = O.bf16_bits_to_f32(O.f32_to_bf16_bits(y32.astype(np.float32)))
    want = prod.reshape(M, N) + O.bf16_bits_to_f32(R0)
    assert_close(O.bf16_bits_to_f32(Yr).reshape(M, N), want, ("residual", wt))


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("inv", [1.0, 0.25])
@pytest.mark.parametrize("M,form", [(1, 0), (1, FUSED), (5, FUSED), (8, 0), (16, 0), (32, 0)])
def test_native_products_are_exact(wt, inv, M, form):
    N, K = 512, 512
    W = fp8_matrix(wt, N, K)
    D = expected_bits(wt, W, None, inv, N, K)
    run_onehot(wt, W, None, inv, D, N, K, M, all_positions(K, M)[:40], flags=NATIVE | form)


@pytest.mark.parametrize("wt", WTS)
def test_native_tiles_cut_across_ctas_are_exact(wt):
    """Few long rows: every feature tile is shared by many CTAs, whose partial tiles the last one adds."""
    N, K, M = 200, 16384, 3
    W = fp8_matrix(wt, N, K)
    D = expected_bits(wt, W, None, 1.0, N, K)
    positions = np.random.default_rng(M).integers(0, K, (48, M))
    run_onehot(wt, W, None, 1.0, D, N, K, M, positions, flags=NATIVE)


def test_a_scale_that_is_no_power_of_two_goes_to_the_dequantising_kernels():
    """The reference folds such a scale into the weights before their BF16 rounding; the native operands cannot."""
    wt, N, K, M = O.FP8_E5M2, 512, 512, 4
    W = fp8_matrix(wt, N, K)
    D = expected_bits(wt, W, None, 0.37, N, K)
    run_onehot(wt, W, None, 0.37, D, N, K, M, all_positions(K, M)[:8], flags=NATIVE)


@pytest.mark.parametrize("wt", WTS + [O.FP4_E2M1])
@pytest.mark.parametrize("M", [2, 12, 30])
def test_native_group_is_one_linear_launch(wt, M):

    from tests.test_gpu_group import build

    c = capi()
    Ns, K = (512, 128, 160), 1024
    items, host, X = build(wt, Ns, K, M, 3, (0.5, 1.0, 0.125))
    dX = to_dev(X)
    grp = c.make_group(items, K)
    before = c.launch_count()
    assert c.gemm_wq_bf16_group(wt, grp, dX, M, K, flags=NATIVE) == 0 and c.check_error("group") == 0
    assert c.launch_count() - before == launches_of(wt, M, NATIVE)
    for it, (W, blk, inv, N) in zip(items, host):
        got = O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N)
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        assert_close(got, y32, ("oracle", wt, M, N))


def test_same_bits_every_run_and_for_every_batch_size():
    """Parts of a tile are added in k order whoever arrives last, and a token's column does not depend on its
    neighbours: repeated calls and calls with more tokens give the same bits for a token."""
    wt, N, K = O.FP8_E5M2, 4096, 4096
    W, _, inv, X = O.make_inputs(wt, N, K, 32, seed=1, scaled=False)
    a = run(wt, W, inv, X, N, 32, K).reshape(32, N)
    for _ in range(3):
        assert np.array_equal(a, run(wt, W, inv, X, N, 32, K).reshape(32, N))
    for M in (1, 4, 9, 16):
        b = run(wt, W, inv, X[: M * K], N, M, K).reshape(M, N)
        assert np.array_equal(a[:M], b), M
    b = run(wt, W, inv, X[: 4 * K], N, 4, K, flags=FUSED).reshape(4, N)
    assert np.array_equal(a[:4], b)    # whichever kernel splits the activations


def test_the_dispatcher_takes_the_native_kernels_where_they_are_the_fastest():
    """Launches of whole tiles (between one and two 128-feature tiles per SM: gate+up) and lm_head-sized ones (FP8 256 MB,
    FP4 48 MB of weights); FP8 only from 3 tokens."""
    import torch

    c = capi()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    X = torch.zeros(32 * 4096, dtype=torch.int16, device="cuda")
    W = torch.zeros(16, dtype=torch.uint8, device="cuda")    # the plan query reads no memory
    Y = torch.zeros(16, dtype=torch.int16, device="cuda")
    plan = lambda wt, N, M: c.gemm_wq_bf16_plan(wt, W, W if wt == O.FP4_E2M1 else None, X, Y, N, M, 4096)
    assert plan(O.FP8_E5M2, 151936, 4) == c.PLAN_NATIVE and plan(O.FP8_E5M2, 151936, 32) == c.PLAN_NATIVE
    assert plan(O.FP8_E5M2, 151936, 1) == c.PLAN_DECODE and plan(O.FP8_E5M2, 12288, 4) == c.PLAN_DECODE
    assert plan(O.FP8_E5M2, 151936, 33) == c.PLAN_STREAM
    whole = 128 * (sms + sms // 2)    # one and a half tiles per SM
    assert plan(O.FP8_E5M2, whole, 3) == c.PLAN_NATIVE and plan(O.FP8_E5M2, whole, 32) == c.PLAN_NATIVE
    assert plan(O.FP8_E5M2, whole, 2) == c.PLAN_DECODE and plan(O.FP8_E5M2, 128 * sms, 4) == c.PLAN_DECODE
    assert plan(O.FP8_E5M2, 128 * (2 * sms + 1), 4) == c.PLAN_DECODE and plan(O.FP4_E2M1, whole, 1) == c.PLAN_NATIVE
    assert plan(O.FP4_E2M1, 28672, 1) == c.PLAN_NATIVE and plan(O.FP4_E2M1, 28672, 32) == c.PLAN_NATIVE
    assert plan(O.FP4_E2M1, 4096, 1) == c.PLAN_DECODE and plan(O.FP4_E2M1, 28672, 33) == c.PLAN_STREAM
