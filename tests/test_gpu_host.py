"""The C++ host layer (Matrix::mul / mulBatched / quantizeWeights, Cublas::gemm, GpuControl) driven
the way cccc drives it, against the CPU oracle and the direct C-ABI call."""
import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, to_dev

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1]


@pytest.fixture(scope="module")
def host():
    h = load_package().hostapi
    L = h.lib()
    g = L.cccc_host_gpu_create(0)
    assert g
    yield h, L, g
    L.cccc_host_gpu_destroy(g)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("M", [1, 7, 64])
def test_mul_batched_is_the_llm_linear(host, wt, M):
    """batchedMul(W, X, 1, 0) of the generated model scripts: W (K, N_out, 1, 1), X (K, M, 1, 1),
    Y (N_out, M, 1, 1), ta = TRANS (cccc/Matrix.cpp:1162-1208)."""
    import torch

    h, L, g = host
    c = capi()
    N, K = 512, 1024
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=M, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    dY = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    mW = L.cccc_host_matrix_view(g, dW.data_ptr(), K, N, 1, 1, wt, inv, dB.data_ptr() if dB is not None else None)
    mX = L.cccc_host_matrix_view(g, dX.data_ptr(), K, M, 1, 1, O.BFLOAT16, 1.0, None)
    mY = L.cccc_host_matrix_view(g, dY.data_ptr(), N, M, 1, 1, O.BFLOAT16, 1.0, None)
    before = L.cccc_host_fused_calls(g)
    L.cccc_host_mul_batched(mW, mX, mY, h.MATRIX_TRANS, h.MATRIX_NO_TRANS, 1.0, 0.0)
    L.cccc_host_gpu_sync(g)
    assert L.cccc_host_fused_calls(g) == before + 1 and c.check_error("host") == 0
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    got = O.bf16_bits_to_f32(from_dev_u16(dY)).reshape(M, N)
    assert_close(got, y32, (wt, M))
    direct = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, direct, N, M, K) == 0 and c.check_error("direct") == 0
    assert torch.equal(direct, dY)
    for m in (mW, mX, mY):
        L.cccc_host_matrix_free(m)


@pytest.mark.parametrize("wt", WTS)
def test_mul_weight_as_second_operand(host, wt):
    """Matrix::mul with the weight as B: R (tokens x N_out) = X^T-stored activations times W."""
    import torch

    h, L, g = host
    N, K, M = 320, 512, 5
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=3, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    r0 = O.f32_to_bf16_bits(np.random.default_rng(1).standard_normal((N, M)).astype(np.float32))
    dR = to_dev(r0)
    # mul() reads row_ and number_: a (K,1,1,M) activation matrix and a (K,1,1,N) weight
    mX = L.cccc_host_matrix_view(g, dX.data_ptr(), K, 1, 1, M, O.BFLOAT16, 1.0, None)
    mW = L.cccc_host_matrix_view(g, dW.data_ptr(), K, 1, 1, N, wt, inv, dB.data_ptr() if dB is not None else None)
    mR = L.cccc_host_matrix_view(g, dR.data_ptr(), M, 1, 1, N, O.BFLOAT16, 1.0, None)
    before = L.cccc_host_fused_calls(g)
    L.cccc_host_mul(mX, mW, mR, 0.5, 2.0, h.MATRIX_TRANS, h.MATRIX_NO_TRANS)
    L.cccc_host_gpu_sync(g)
    assert L.cccc_host_fused_calls(g) == before + 1
    Yo, _ = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=0.5, beta=2.0, Y=r0, ldy_m=1, ldy_n=M)
    assert_close(O.bf16_bits_to_f32(from_dev_u16(dR)), O.bf16_bits_to_f32(Yo), wt)
    for m in (mX, mW, mR):
        L.cccc_host_matrix_free(m)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
def test_layouts_the_fused_kernel_does_not_take_fall_back_like_the_reference(host, wt):
    """Weight stored with K strided (op(A) = A): dequantise into the workspace, then cuBLAS."""
    import torch

    h, L, g = host
    N, K, M = 256, 512, 4
    # a [K, N] row-major quantised weight, i.e. (N x K) column-major with lda = N
    Wt, blkt, inv, X = O.make_inputs(wt, K, N, M, seed=8, scaled=True)
    X = O.f32_to_bf16_bits(np.random.default_rng(2).standard_normal((M, K)).astype(np.float32))
    if wt == O.FP4_E2M1:
        wd = O.bf16_bits_to_f32(O.fp4_blockscale_to_bf16(Wt, blkt, K * N, 16)).reshape(K, N)
    else:
        wd = O.bf16_bits_to_f32(O.fp8_to_bf16(Wt, wt, inv)).reshape(K, N)
    ref = O.bf16_bits_to_f32(X).astype(np.float64) @ wd.astype(np.float64)      # [M, N]
    dW, dX = to_dev(Wt), to_dev(X)
    dB = to_dev(blkt) if blkt is not None else None
    dC = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    before = L.cccc_host_fallback_calls(g)
    # C (N x M, ldc N) = A (N x K, lda N, no trans) * B (K x M, ldb K)
    L.cccc_host_gemm(g, h.MATRIX_NO_TRANS, h.MATRIX_NO_TRANS, N, M, K, 1.0, dW.data_ptr(), wt, N, inv, dX.data_ptr(), O.BFLOAT16,
                     K, 1.0, 0.0, dC.data_ptr(), O.BFLOAT16, N, dB.data_ptr() if dB is not None else None, None)
    L.cccc_host_gpu_sync(g)
    assert L.cccc_host_fallback_calls(g) == before + 1
    assert_close(O.bf16_bits_to_f32(from_dev_u16(dC)).reshape(M, N), ref, wt)


def test_mul_batched_with_two_batches_offsets_the_block_scales(host):
    import torch

    h, L, g = host
    N, K, M = 128, 256, 3
    parts = [O.make_inputs(O.FP4_E2M1, N, K, M, seed=s) for s in (11, 12)]
    W = np.concatenate([p[0] for p in parts])
    blk = np.concatenate([p[1] for p in parts])
    X = np.concatenate([p[3].reshape(-1) for p in parts])
    dW, dB, dX = to_dev(W), to_dev(blk), to_dev(X)
    dY = torch.zeros(2 * M * N, dtype=torch.int16, device="cuda")
    mW = L.cccc_host_matrix_view(g, dW.data_ptr(), K, N, 1, 2, O.FP4_E2M1, 1.0, dB.data_ptr())
    mX = L.cccc_host_matrix_view(g, dX.data_ptr(), K, M, 1, 2, O.BFLOAT16, 1.0, None)
    mY = L.cccc_host_matrix_view(g, dY.data_ptr(), N, M, 1, 2, O.BFLOAT16, 1.0, None)
    L.cccc_host_mul_batched(mW, mX, mY, h.MATRIX_TRANS, h.MATRIX_NO_TRANS, 1.0, 0.0)
    L.cccc_host_gpu_sync(g)
    got = O.bf16_bits_to_f32(from_dev_u16(dY)).reshape(2, M, N)
    for b, p in enumerate(parts):
        _, y32 = O.linear_wq_bf16(O.FP4_E2M1, p[0], p[1], 1.0, p[3], N, M, K)
        assert_close(got[b], y32, b)


@pytest.mark.parametrize("target", WTS)
def test_quantize_weights_follows_the_reference_rules(host, target):
    """Matrix::quantizeWeights (cccc/Matrix.cpp:301-355), then the quantised matrix in a linear."""
    import torch

    h, L, g = host
    N, K = 192, 256
    w = (np.random.default_rng(4).standard_normal(N * K) * 0.02).astype(np.float32)
    m = L.cccc_host_matrix_new(g, K, N, 1, 1, O.FLOAT)
    torch.cuda.synchronize()
    import ctypes

    dptr = L.cccc_host_matrix_data(m)
    src = torch.from_numpy(w).cuda()
    ctypes.CDLL("libcudart.so").cudaMemcpy(ctypes.c_void_p(dptr), ctypes.c_void_p(src.data_ptr()), ctypes.c_size_t(w.nbytes), 3)
    L.cccc_host_matrix_quantize(m, target)
    assert L.cccc_host_matrix_dtype(m) == target
    n_bytes = N * K // 2 if target == O.FP4_E2M1 else N * K
    out = torch.zeros(n_bytes, dtype=torch.uint8, device="cuda")
    ctypes.CDLL("libcudart.so").cudaMemcpy(ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(L.cccc_host_matrix_data(m)),
                                           ctypes.c_size_t(n_bytes), 3)
    q = out.cpu().numpy()
    if target == O.FP4_E2M1:
        nib, sc = O.float_to_fp4_blockscale(w, 16)
        scd = torch.zeros(N * K // 16, dtype=torch.uint8, device="cuda")
        ctypes.CDLL("libcudart.so").cudaMemcpy(ctypes.c_void_p(scd.data_ptr()), ctypes.c_void_p(L.cccc_host_matrix_block_scale(m)),
                                               ctypes.c_size_t(N * K // 16), 3)
        assert np.array_equal(q, nib) and np.array_equal(scd.cpu().numpy(), sc)
    else:
        maxval = np.float32(448.0 if target == O.FP8_E4M3 else 57344.0)
        absmax = np.float32(np.abs(w).max())
        assert np.array_equal(q, O.float_to_fp8(w, target, float(maxval / absmax)))
        assert np.float32(L.cccc_host_matrix_quant_scale(m)) == np.float32(absmax / maxval)
    L.cccc_host_matrix_free(m)


@pytest.mark.parametrize("wt", WTS[:2])
@pytest.mark.parametrize("weight_is_a", [1, 0])
def test_typed_gemm_overloads(host, wt, weight_is_a):
    """Cublas::gemm(uint8_t* A, bfloat16* B -> bfloat16* C) and its mirror (cccc/cublas_real.h:599-685, 688-752):
    the same linear as the type-erased dispatcher gives, served by the fused kernel."""
    import torch

    h, L, g = host
    c = capi()
    N, K, M = 384, 512, 6
    W, _, inv, X = O.make_inputs(wt, N, K, M, seed=21 + wt, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    got = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    before = L.cccc_host_fused_calls(g)
    if weight_is_a:
        # C (N_out x tokens, ldc = N_out) = W^T X
        L.cccc_host_gemm_typed(g, 1, h.MATRIX_TRANS, h.MATRIX_NO_TRANS, N, M, K, 1.0, dW.data_ptr(), K, dX.data_ptr(), K, 0.0,
                               got.data_ptr(), N, inv, wt)
    else:
        # C (tokens x N_out, ldc = tokens) = X^T W
        L.cccc_host_gemm_typed(g, 0, h.MATRIX_TRANS, h.MATRIX_NO_TRANS, M, N, K, 1.0, dX.data_ptr(), K, dW.data_ptr(), K, 0.0,
                               got.data_ptr(), M, inv, wt)
    L.cccc_host_gpu_sync(g)
    assert L.cccc_host_fused_calls(g) == before + 1 and c.check_error("typed") == 0
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    out = O.bf16_bits_to_f32(from_dev_u16(got))
    out = out.reshape(M, N) if weight_is_a else out.reshape(N, M).T
    assert_close(out, y32, ("typed", wt, weight_is_a))
