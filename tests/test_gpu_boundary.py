"""The drop-in boundary, compiled and run: the reference's own Cublas::gemm (cccc/cublas_real.h), built from the
reference's header with the two call sites of its W8A16 / W4A16 BF16 branches changed the way a maintainer would
change them (oracle/patch_reference.py; :943 weight as A, :1066 weight as B), linked against this library ahead of
the reference's cccc-cuda.  A call through that dispatcher must land in cuda_gemm_wq_bf16: the bits of the direct
call, no dequantised copy of the weight in the dispatcher's workspace, and the reference's own branch still there
for the operand orders the fused kernel does not take."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, ref_gemm_lib, to_dev

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1]


@pytest.fixture(scope="module")
def libs():
    P, R = ref_gemm_lib(patched=True), ref_gemm_lib()
    if P is None or R is None:
        pytest.skip("oracle/_ref holds no built reference dispatcher")
    return P, R


def call(Lib, ta, tb, M, N, K, A, typeA, lda, invA, B, typeB, ldb, invB, C, ldc, blkA=None, blkB=None, alpha=1.0, beta=0.0):
    return Lib.ref_cublas_gemm(ta, tb, M, N, K, alpha, A.data_ptr(), typeA, lda, invA, B.data_ptr(), typeB, ldb, invB, beta, C.data_ptr(), 3, ldc,
                               0.0, blkA.data_ptr() if blkA is not None else None, blkB.data_ptr() if blkB is not None else None)


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("M", [1, 8, 100, 300])
def test_the_patched_dispatcher_lands_in_the_fused_kernel_weight_as_a(libs, wt, M):
    """batchedMul(W, X): C (N_out x tokens, ldc = N_out) = W^T (K x N_out) X (K x tokens)."""
    import torch

    P, R = libs
    c = capi()
    N, K = 1024, 2048
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=M + wt, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    got = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    direct = torch.zeros_like(got)
    before = c.launch_count()
    assert call(P, 1, 0, N, M, K, dW, wt, K, inv, dX, 3, K, 1.0, got, N, blkA=dB) == 0
    launches = c.launch_count() - before
    assert launches >= 1 and (M > 32 or launches == 1)    # decode: exactly one launch, no separate dequantisation kernel
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, direct, N, M, K) == 0 and c.check_error("direct") == 0
    assert torch.equal(got, direct)
    # and it is the reference's result: the unpatched dispatcher (its dequantise + cublasGemmEx) on the same buffers
    ref = torch.zeros_like(got)
    assert call(R, 1, 0, N, M, K, dW, wt, K, inv, dX, 3, K, 1.0, ref, N, blkA=dB) == 0
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(from_dev_u16(got)).reshape(M, N), y32, ("patched", wt, M))
    assert_close(O.bf16_bits_to_f32(from_dev_u16(ref)).reshape(M, N), y32, ("reference", wt, M))


@pytest.mark.parametrize("wt", WTS)
def test_weight_as_b_and_beta(libs, wt):
    """The mirrored operand order (:1066): C (tokens x N_out, ldc = tokens) = X^T W, with alpha and beta."""
    import torch

    P, R = libs
    c = capi()
    N, K, M = 512, 1024, 5
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=3 + wt, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    y0 = O.f32_to_bf16_bits(np.random.default_rng(1).standard_normal(M * N).astype(np.float32))
    got, ref = to_dev(y0), to_dev(y0)
    before = c.launch_count()
    assert call(P, 1, 0, M, N, K, dX, 3, K, 1.0, dW, wt, K, inv, got, M, blkB=dB, alpha=0.5, beta=1.0) == 0
    assert c.launch_count() == before + 1
    assert call(R, 1, 0, M, N, K, dX, 3, K, 1.0, dW, wt, K, inv, ref, M, blkB=dB, alpha=0.5, beta=1.0) == 0
    direct = to_dev(y0)
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, direct, N, M, K, ldy_m=1, ldy_n=M, alpha=0.5, beta=1.0) == 0 and c.check_error("direct") == 0
    assert torch.equal(got, direct)
    a = O.bf16_bits_to_f32(from_dev_u16(got)).reshape(N, M)
    b = O.bf16_bits_to_f32(from_dev_u16(ref)).reshape(N, M)
    assert_close(a, b, ("weight as B", wt))


def test_no_dequantised_weight_in_the_dispatcher_workspace(libs):
    """The reference's branch grows its workspace to the whole weight in BF16 (ensureWS, :946); the patched call
    leaves device memory where it was.  256 MB of FP8 weight would need 512 MB there."""
    import torch

    P, R = libs
    c = capi()
    N, K, M = 32768, 8192, 1
    wt = O.FP8_E5M2
    dW = torch.randint(0, 120, (N * K,), dtype=torch.uint8, device="cuda")
    dX = to_dev(O.f32_to_bf16_bits(np.random.default_rng(2).standard_normal(M * K).astype(np.float32)))
    got, ref = (torch.zeros(M * N, dtype=torch.int16, device="cuda") for _ in range(2))
    assert c.gemm_wq_bf16(wt, dW, None, 1.0, dX, got, N, M, K) == 0 and c.check_error("warm") == 0    # the library's own workspace exists
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    assert call(P, 1, 0, N, M, K, dW, wt, K, 2.0 ** -8, dX, 3, K, 1.0, got, N) == 0
    free1 = torch.cuda.mem_get_info()[0]
    assert free0 - free1 < (64 << 20)
    assert call(R, 1, 0, N, M, K, dW, wt, K, 2.0 ** -8, dX, 3, K, 1.0, ref, N) == 0
    free2 = torch.cuda.mem_get_info()[0]
    assert free1 - free2 >= N * K * 2 - (64 << 20)
    a, b = O.bf16_bits_to_f32(from_dev_u16(got)), O.bf16_bits_to_f32(from_dev_u16(ref))
    assert_close(a.reshape(M, N), b.reshape(M, N).astype(np.float64), "patched vs reference at 256 MB")


def test_operand_orders_the_fused_kernel_does_not_take_keep_the_reference_branch(libs):
    """Weight stored with the output feature contiguous (TransA = NO_TRANS): the inserted block steps aside and the
    reference's dequantise + cuBLAS branch runs, served by this library's cuda_convert."""
    import torch

    P, R = libs
    c = capi()
    N, K, M = 256, 512, 4
    wt = O.FP8_E4M3
    W, _, inv, X = O.make_inputs(wt, N, K, M, seed=8, scaled=True)
    Wt = np.ascontiguousarray(W.reshape(N, K).T).reshape(-1)          # (N_out x K) column-major, lda = N_out
    dW, dX = to_dev(Wt), to_dev(X)
    got, ref = (torch.zeros(M * N, dtype=torch.int16, device="cuda") for _ in range(2))
    assert call(P, 0, 0, N, M, K, dW, wt, N, inv, dX, 3, K, 1.0, got, N) == 0
    assert call(R, 0, 0, N, M, K, dW, wt, N, inv, dX, 3, K, 1.0, ref, N) == 0
    _, y32 = O.linear_wq_bf16(wt, W, None, inv, X, N, M, K)
    assert_close(O.bf16_bits_to_f32(from_dev_u16(got)).reshape(M, N), y32, "fallback branch")
    assert torch.equal(got, ref)       # the same cuBLAS call on the same dequantised BF16 weight
