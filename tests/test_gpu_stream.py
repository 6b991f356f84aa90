"""The streaming tensor-core kernel (up to 128 tokens: tcgen05 UMMAs over weights dequantised on the fly, the k
range cut into a thread-block cluster whose partial tiles are summed through distributed shared memory), forced
through flags bits 8-10 = 7 so that every shape it accepts is checked, not only those the dispatcher gives it.
Against the CPU oracle at the GEMM bar (max relative error 1e-2 with the 1e-2 * rms floor, cosine >= 0.9999),
and bit for bit on one-hot activations, where the output IS the dequantised weight."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, to_dev
from tests.test_gpu_onehot import all_positions, expected_bits, fp4_matrix, fp8_matrix, run_onehot

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1]
STREAM = 7 << 8


def run(wt, W, blk, inv, X, N, M, K, Y0=None, **kw):
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
    kw["flags"] = kw.get("flags", 0) | STREAM
    before = c.launch_count()
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, dY, N, M, K, **kw) == 0
    assert c.check_error("stream") == 0 and c.launch_count() == before + 1
    return dY.cpu().numpy() if f32 else from_dev_u16(dY)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("N,K,M", [(128, 256, 1), (256, 512, 9), (384, 1024, 16), (200, 320, 17), (1000, 4096, 32), (512, 2048, 33),
                                   (4096, 4096, 48), (128, 12288, 64), (2500, 1024, 100), (1024, 4096, 128), (4096, 256, 5)])
def test_stream_kernel_matches_oracle(wt, N, K, M):
    if wt == O.FP4_E2M1 and K % 256:
        K = (K // 256 + 1) * 256       # the oracle's FP4 generator wants whole 256-element runs
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=True)
    Y = run(wt, W, blk, inv, X, N, M, K)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (wt, N, K, M))


@pytest.mark.parametrize("wt", WTS)
def test_stream_alpha_beta_strides_and_output_modes(wt):
    N, K, M = 200, 512, 20
    ldw, ldx = K + 256, K + 8
    rng = np.random.default_rng(3)
    Wd, blkd, inv, Xd = O.make_inputs(wt, N, ldw, M, seed=13, scaled=False)
    X = np.zeros((M, ldx), np.uint16)
    X[:, :K] = Xd.reshape(M, ldw)[:, :K]
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 3)).astype(np.float32))
    kw = dict(ldw=ldw, ldx=ldx, alpha=0.25, beta=1.5, ldy_m=1, ldy_n=M + 3)
    Y = run(wt, Wd, blkd, inv, X, N, M, K, Y0=Y0.copy(), **kw)
    Yo, _ = O.linear_wq_bf16(wt, Wd, blkd, inv, X, N, M, K, Y=Y0, **kw)
    got = O.bf16_bits_to_f32(Y[:Yo.size]).reshape(N, M + 3)
    want = O.bf16_bits_to_f32(Yo).reshape(N, M + 3)
    assert_close(got[:, :M], want[:, :M], wt)
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])
    # float32 output (the unrounded sums a row-parallel shard hands on)
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=4, scaled=True)
    Yf = run(wt, W, blk, inv, X, N, M, K, flags=4)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(Yf.reshape(M, N), y32, ("f32", wt))
    # residual epilogue: Y = bf16(bf16(W x) + Y)
    R0 = O.f32_to_bf16_bits(rng.standard_normal((M, N)).astype(np.float32))
    Yr = run(wt, W, blk, inv, X, N, M, K, Y0=R0.copy().reshape(-1), beta=1.0, flags=8)
    prod = O.bf16_bits_to_f32(O.f32_to_bf16_bits(y32.astype(np.float32)))
    want = prod.reshape(M, N) + O.bf16_bits_to_f32(R0)
    assert_close(O.bf16_bits_to_f32(Yr).reshape(M, N), want, ("residual", wt))


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3])
@pytest.mark.parametrize("inv", [1.0, 0.25, 0.37])
@pytest.mark.parametrize("M", [1, 16, 40, 128])
def test_stream_fp8_dequantises_bit_exactly(wt, inv, M):
    N, K = 512, 512
    W = fp8_matrix(wt, N, K)
    D = expected_bits(wt, W, None, inv, N, K)
    run_onehot(wt, W, None, inv, D, N, K, M, all_positions(K, M)[:40], flags=STREAM)


@pytest.mark.parametrize("M", [1, 16, 40, 128])
def test_stream_fp4_dequantises_bit_exactly(M):
    N, K = 508, 512
    W, S = fp4_matrix(N, K)
    D = expected_bits(O.FP4_E2M1, W, S, 1.0, N, K)
    run_onehot(O.FP4_E2M1, W, S, 1.0, D, N, K, M, all_positions(K, M)[:40], flags=STREAM)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("M", [1, 24])
def test_stream_cluster_slices_dequantise_bit_exactly(wt, M):
    """Few long rows: eight k slices per tile, combined through distributed shared memory."""
    N, K = 64, 16384
    if wt == O.FP4_E2M1:
        W, S = fp4_matrix(N, K)
    else:
        W, S = fp8_matrix(wt, N, K), None
    inv = 0.37 if wt != O.FP4_E2M1 else 1.0
    D = expected_bits(wt, W, S, inv, N, K)
    positions = np.random.default_rng(M).integers(0, K, (48, M))
    run_onehot(wt, W, S, inv, D, N, K, M, positions, flags=STREAM)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("M", [4, 40])
def test_stream_group_is_one_launch(wt, M):
    import torch

    from tests.test_gpu_group import build

    c = capi()
    Ns, K = (512, 128, 160), 1024
    items, host, X = build(wt, Ns, K, M, 3, (0.37, 1.0, 0.011))
    dX = to_dev(X)
    grp = c.make_group(items, K)
    before = c.launch_count()
    assert c.gemm_wq_bf16_group(wt, grp, dX, M, K, flags=STREAM) == 0 and c.check_error("group") == 0
    assert c.launch_count() - before == 1
    for it, (W, blk, inv, N) in zip(items, host):
        got = O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N)
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        assert_close(got, y32, ("oracle", wt, M, N))


def test_same_bits_every_run():
    """The slices are summed in slice order, so a repeated call gives the same bits."""
    import torch

    wt, N, K, M = O.FP8_E5M2, 4096, 4096, 24
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=1, scaled=True)
    a = run(wt, W, blk, inv, X, N, M, K)
    for _ in range(3):
        assert np.array_equal(a, run(wt, W, blk, inv, X, N, M, K))
