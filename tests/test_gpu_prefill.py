"""The prefill-side linear (M > 32 tokens, tcgen05/TMEM kernel) through the C-ABI against the CPU
oracle and the reference's own GPU path.  Tolerance as stated for GEMM outputs: max relative error
1e-2 and cosine >= 0.9999 against the FP32-accumulated reference output."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, ref_gemm_lib, to_dev

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1]


def run(wt, W, blk, inv, X, N, M, K, **kw):
    import torch

    c = capi()
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    ldy_m = kw.get("ldy_m", N)
    ldy_n = kw.get("ldy_n", 1)
    y0 = kw.pop("Y0", None)
    size = (M - 1) * ldy_m + (N - 1) * ldy_n + 1
    dY = to_dev(y0) if y0 is not None else torch.zeros(size, dtype=torch.int16, device="cuda")
    plan = c.gemm_wq_bf16_plan(wt, dW, dB, dX, dY, N, M, K, ldw=kw.get("ldw"), ldx=kw.get("ldx"))
    if plan == c.PLAN_STREAM:
        plan = c.PLAN_PREFILL    # up to 128 tokens the dispatcher prefers the streaming kernel; this file tests the prefill kernel
    kw["flags"] = kw.get("flags", 0) | c.FLAG_NO_STREAM
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, dY, N, M, K, **kw) == 0
    assert c.check_error("prefill") == 0
    return from_dev_u16(dY), plan


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("N,K,M", [(128, 64, 33), (128, 256, 64), (256, 512, 256), (384, 1024, 300), (200, 320, 257),
                                   (1024, 4096, 512), (15300, 128, 600), (2500, 8192, 300)])
def test_prefill_small_shapes_match_oracle(wt, N, K, M):
    c = capi()
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=True)
    Y, plan = run(wt, W, blk, inv, X, N, M, K)
    assert plan == c.PLAN_PREFILL
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (wt, N, K, M))


@pytest.mark.parametrize("wt", WTS)
def test_prefill_alpha_beta_and_strides(wt):
    N, K, M = 200, 256, 70
    ldw, ldx = K + 256, K + 8
    rng = np.random.default_rng(3)
    Wd, blkd, inv, Xd = O.make_inputs(wt, N, ldw, M, seed=13, scaled=False)
    X = np.zeros((M, ldx), np.uint16)
    X[:, :K] = Xd.reshape(M, ldw)[:, :K]
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 3)).astype(np.float32))
    kw = dict(ldw=ldw, ldx=ldx, alpha=0.25, beta=1.5, ldy_m=1, ldy_n=M + 3)
    Y, plan = run(wt, Wd, blkd, inv, X, N, M, K, Y0=Y0.copy(), **kw)
    assert plan == capi().PLAN_PREFILL
    Yo, _ = O.linear_wq_bf16(wt, Wd, blkd, inv, X, N, M, K, Y=Y0, **kw)
    got = O.bf16_bits_to_f32(Y[:Yo.size]).reshape(N, M + 3)
    want = O.bf16_bits_to_f32(Yo).reshape(N, M + 3)
    assert_close(got[:, :M], want[:, :M], wt)
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])


@pytest.mark.parametrize("wt", WTS)
def test_prefill_config4_shape_against_reference_gpu_path(wt):
    """Benchmark configuration 4 (M=2048 tokens) on the q projection shape, against the reference's own
    dequantise-then-cuBLAS path on the same buffers, plus an oracle check on a row subset."""
    import torch

    R = ref_gemm_lib()
    c = capi()
    N, K, M = 4096, 4096, 2048
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=41, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    ours = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    assert c.gemm_wq_bf16_plan(wt, dW, dB, dX, ours, N, M, K) == c.PLAN_PREFILL
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, ours, N, M, K) == 0 and c.check_error("t") == 0
    a = O.bf16_bits_to_f32(from_dev_u16(ours)).reshape(M, N)
    rows = np.arange(0, N, 97)
    toks = np.arange(0, M, 61)
    Wsub = (W.reshape(N, K // 2) if wt == O.FP4_E2M1 else W.reshape(N, K))[rows]
    bsub = blk.reshape(N, K // 16)[rows] if blk is not None else None
    _, y32 = O.linear_wq_bf16(wt, Wsub.reshape(-1), bsub, inv, X.reshape(M, K)[toks], rows.size, toks.size, K)
    assert_close(a[np.ix_(toks, rows)], y32, "oracle subset")
    if R is None:
        pytest.skip("oracle/_ref/libref_gpu_gemm.so not built")
    ref = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    rc = R.ref_cublas_gemm(1, 0, N, M, K, 1.0, dW.data_ptr(), wt, K, inv, dX.data_ptr(), 3, K, 1.0, 0.0, ref.data_ptr(), 3, N,
                           0.0, dB.data_ptr() if dB is not None else None, None)
    assert rc == 0
    assert_close(a, O.bf16_bits_to_f32(from_dev_u16(ref)).reshape(M, N), "reference gpu path")


VARIANTS = [1, 2, 3, 4, 5, 6]    # one CTA per tile: 128x128, 128x256, 256x256; CTA pairs: 256x256, 512x256, 256x512


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("N,K,M", [(128, 64, 33), (300, 256, 300), (520, 512, 700), (1000, 1024, 513)])
def test_prefill_every_tile_shape_matches_oracle(wt, variant, N, K, M):
    """Ragged feature and token counts (tiles partly or wholly past the edges) in every tile shape,
    BF16 output written by the TMA-store epilogue."""
    c = capi()
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M + variant, scaled=True)
    Y, plan = run(wt, W, blk, inv, X, N, M, K, flags=c.flag_prefill_variant(variant))
    assert plan == c.PLAN_PREFILL
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(Y).reshape(M, N), y32, (wt, variant, N, K, M))


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("wt", WTS)
def test_prefill_every_tile_shape_direct_epilogue(wt, variant):
    """alpha/beta accumulate into a transposed, padded Y and float32 output: the epilogue that
    stores from registers instead of through TMA."""
    import torch

    c = capi()
    N, K, M = 300, 256, 290
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=77 + variant, scaled=False)
    rng = np.random.default_rng(5)
    Y0 = O.f32_to_bf16_bits(rng.standard_normal((N, M + 5)).astype(np.float32))
    kw = dict(alpha=0.5, beta=-1.25, ldy_m=1, ldy_n=M + 5)
    Y, _ = run(wt, W, blk, inv, X, N, M, K, Y0=Y0.copy(), flags=c.flag_prefill_variant(variant), **kw)
    Yo, _ = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, Y=Y0, **kw)
    got = O.bf16_bits_to_f32(Y[:Yo.size]).reshape(N, M + 5)
    want = O.bf16_bits_to_f32(Yo).reshape(N, M + 5)
    assert_close(got[:, :M], want[:, :M], (wt, variant))
    assert np.array_equal(got[:, M:], O.bf16_bits_to_f32(Y0)[:, M:])
    # float32 output (flags bit 2), against the oracle's unrounded sums
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    y = torch.zeros(M * N, dtype=torch.float32, device="cuda")
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, y, N, M, K, flags=c.FLAG_OUT_F32 | c.flag_prefill_variant(variant)) == 0
    assert c.check_error("f32") == 0
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(y.cpu().numpy().reshape(M, N), y32, (wt, variant, "f32"))


@pytest.mark.parametrize("wt", WTS)
def test_prefill_tile_shapes_agree_bit_for_bit(wt):
    """At the token count of benchmark configuration 4 every tile shape accumulates the same products in the same
    k order in FP32, so the BF16 outputs are identical; the default choice is one of them."""
    import torch

    c = capi()
    N, K, M = 1536, 4096, 2048
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=9, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    outs = []
    for variant in [0] + VARIANTS:
        y = torch.full((M * N,), 0x7FC0, dtype=torch.int16, device="cuda")
        assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, y, N, M, K, flags=c.flag_prefill_variant(variant)) == 0
        assert c.check_error("v") == 0
        outs.append(from_dev_u16(y))
    for variant, y in zip(VARIANTS, outs[1:]):
        assert np.array_equal(y, outs[0]), variant
    rows = np.arange(0, N, 53)
    toks = np.arange(0, M, 67)
    Wsub = (W.reshape(N, K // 2) if wt == O.FP4_E2M1 else W.reshape(N, K))[rows]
    bsub = blk.reshape(N, K // 16)[rows] if blk is not None else None
    _, y32 = O.linear_wq_bf16(wt, Wsub.reshape(-1), bsub, inv, X.reshape(M, K)[toks], rows.size, toks.size, K)
    assert_close(O.bf16_bits_to_f32(outs[0]).reshape(M, N)[np.ix_(toks, rows)], y32, "oracle subset")


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
@pytest.mark.parametrize("pad", [8, 3])
@pytest.mark.parametrize("variant", [0, 1, 4, 6])
def test_prefill_padded_output_rows_keep_their_padding(wt, pad, variant):
    """Y with a row stride larger than N: a multiple of 8 elements keeps the TMA-store epilogue (the
    store must clip at N, not at the stride), any other stride takes the register epilogue; the padding
    columns are never written in either."""
    import torch

    c = capi()
    N, K, M = 520, 256, 300
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=17 + pad + variant, scaled=True)
    ld = N + pad
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    y = torch.full((M * ld,), 0x4140, dtype=torch.int16, device="cuda")    # bf16 12.0 everywhere
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, y, N, M, K, ldy_m=ld, flags=c.flag_prefill_variant(variant)) == 0
    assert c.check_error("padded") == 0
    got = O.bf16_bits_to_f32(from_dev_u16(y)).reshape(M, ld)
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(got[:, :N], y32, (wt, pad, variant))
    assert np.all(got[:, N:] == 12.0)
