"""cuda_gemm_wq_bf16_static: the linear for callers that may not allocate (hosts with a fixed
device-memory plan that hand the library no allocator, latency-critical loops that may not block
on one).  Its scratch is a fixed array
inside the library.  The test calls it through the C-ABI twice in a row per shape and requires the
output of the regular entry point, on shapes that use the split-k exchange (which is what needs the
scratch) and on shapes that do not; it also checks that sizes beyond the fixed scratch are refused.
Collected last, so that a run stopping at the first failure has already run everything else."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, to_dev

pytestmark = pytest.mark.gpu

# (N, K, M): few long row blocks -> split-k exchange through the scratch; the others -> whole row blocks
SHAPES = [(64, 16384, 1), (96, 8192, 5), (64, 16384, 8), (4096, 4096, 1), (1000, 2304, 7)]


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1])
@pytest.mark.parametrize("N,K,M", SHAPES)
def test_static_scratch_entry_matches_regular_entry(wt, N, K, M):
    import torch

    c = capi()
    if wt == O.FP4_E2M1 and K % 256:
        pytest.skip("FP4 TMA path needs K % 256 == 0")
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    want = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    assert c.gemm_wq_bf16(wt, dW, dB, inv, dX, want, N, M, K) == 0 and c.check_error("regular") == 0
    ref = O.bf16_bits_to_f32(from_dev_u16(want))
    for call in range(2):  # two calls in a row share the array
        got = torch.full((M * N,), 0x7FC0, dtype=torch.int16, device="cuda")
        rc = c.gemm_wq_bf16_static(wt, dW, dB, inv, dX, got, N, M, K, flags=c.FLAG_CHECKED)
        assert rc == 0, (call, rc)
        out = O.bf16_bits_to_f32(from_dev_u16(got))
        assert_close(out, ref, (wt, N, K, M, call))
        # same kernel, same schedule, same summation order: the bits agree as well
        assert torch.equal(got, want), (wt, N, K, M, call)
    # and against the CPU oracle, once
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    assert_close(out.reshape(M, N), y32, "oracle")


def test_static_scratch_entry_unchecked_and_alpha_beta():
    import torch

    c = capi()
    N, K, M = 64, 16384, 3
    W, blk, inv, X = O.make_inputs(O.FP8_E5M2, N, K, M, seed=9, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    y0 = torch.randn(M * N, device="cuda").to(torch.bfloat16)
    a, b = y0.clone(), y0.clone()
    assert c.gemm_wq_bf16(O.FP8_E5M2, dW, None, inv, dX, a, N, M, K, alpha=0.5, beta=-1.0) == 0
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, b, N, M, K, alpha=0.5, beta=-1.0) == 0
    # cuda_check_error covers pending CUDA errors and the regular workspace; the fixed array's own
    # status word is only looked at by checked calls, so the result itself is what is compared here
    assert c.check_error("after the unchecked static call") == 0
    assert torch.equal(a, b)


def test_static_scratch_entry_allocates_nothing():
    """The property the entry point exists for: free device memory does not move across its calls."""
    import torch

    c = capi()
    N, K, M = 64, 16384, 4
    W, blk, inv, X = O.make_inputs(O.FP8_E5M2, N, K, M, seed=2, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    y = torch.zeros(M * N, dtype=torch.int16, device="cuda")
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, N, M, K, flags=c.FLAG_CHECKED) == 0  # set-up call
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(8):
        assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, N, M, K) == 0
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, N, M, K, flags=c.FLAG_CHECKED) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)


_ALONE = r"""
import sys
sys.path.insert(0, {root!r})
import numpy as np, torch
from __graft_entry__ import load_package
from oracle import oracle as O
from tests._util import assert_close, to_dev, from_dev_u16
c = load_package().capi
for wt, (N, K, M) in ((O.FP8_E5M2, (64, 16384, 8)), (O.FP4_E2M1, (96, 8192, 5)), (O.FP8_E4M3, (4096, 4096, 1))):
    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + M, scaled=True)
    dW, dX = to_dev(W), to_dev(X)
    dB = to_dev(blk) if blk is not None else None
    _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    for call in range(2):
        got = torch.full((M * N,), 0x7FC0, dtype=torch.int16, device="cuda")
        assert c.gemm_wq_bf16_static(wt, dW, dB, inv, dX, got, N, M, K, flags=c.FLAG_CHECKED) == 0
        assert_close(O.bf16_bits_to_f32(from_dev_u16(got)).reshape(M, N), y32, (wt, call))
print("STATIC-ALONE-OK")
"""


def test_static_scratch_entry_alone_in_a_fresh_process():
    """A process that never calls the regular entry point (so the regular workspace is never created)
    gets the oracle's result from the allocation-free one."""
    import subprocess
    import sys

    from __graft_entry__ import ROOT

    r = subprocess.run([sys.executable, "-c", _ALONE.format(root=ROOT)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "STATIC-ALONE-OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])


def test_static_scratch_entry_refuses_what_it_cannot_hold(capfd):
    import torch

    c = capi()
    N, K = 256, 1024
    W, blk, inv, X = O.make_inputs(O.FP8_E5M2, N, K, 9, seed=1)
    dW, dX = to_dev(W), to_dev(X)
    y = torch.zeros(9 * N, dtype=torch.int16, device="cuda")
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, N, 9, K) == -1       # more than 8 tokens
    assert "at most 8 tokens" in capfd.readouterr().err
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, N, 2, K - 24) == -1  # K % 64 != 0
    assert "use cuda_gemm_wq_bf16" in capfd.readouterr().err
    assert c.gemm_wq_bf16_static(O.BFLOAT16, dW, None, inv, dX, y, N, 2, K) == -1
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, None, None, inv, dX, y, N, 2, K) == -1
    assert c.gemm_wq_bf16_static(O.FP8_E5M2, dW, None, inv, dX, y, 0, 2, K) == 0
    assert not y.any() and c.check_error("refused") == 0
