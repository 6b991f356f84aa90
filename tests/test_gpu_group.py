"""cuda_gemm_wq_bf16_group: several linears that share the activations (q/k/v, gate/up) in one call.
The result must be that of separate cuda_gemm_wq_bf16 calls, whatever path the group takes."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, from_dev_u16, to_dev

pytestmark = pytest.mark.gpu

WTS = [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1]


def build(wt, Ns, K, M, seed, scales):
    import torch

    items, host = [], []
    X = None
    for j, N in enumerate(Ns):
        W, blk, inv, Xj = O.make_inputs(wt, N, K, M, seed=seed + j, scaled=False)
        if X is None:
            X = Xj
        inv = scales[j % len(scales)] if wt != O.FP4_E2M1 else 1.0
        host.append((W, blk, inv, N))
        items.append(dict(W=to_dev(W), S=to_dev(blk) if blk is not None else None, inv=inv, N=N,
                          Y=torch.zeros(M * N, dtype=torch.int16, device="cuda"), alpha=1.0 + 0.5 * j, beta=0.0))
    return items, host, X


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("M", [1, 5, 20])
@pytest.mark.parametrize("scales", [(1.0, 0.5, 2.0), (0.37, 1.0, 0.011)])
def test_group_of_three_is_one_launch_and_matches_separate_calls(wt, M, scales):
    import torch

    c = capi()
    Ns, K = (512, 128, 160), 1024
    items, host, X = build(wt, Ns, K, M, 3, scales)
    dX = to_dev(X)
    grp = c.make_group(items, K)
    before = c.launch_count()
    assert c.gemm_wq_bf16_group(wt, grp, dX, M, K) == 0 and c.check_error("group") == 0
    assert c.launch_count() - before == 1
    for it, (W, blk, inv, N) in zip(items, host):
        sep = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        assert c.gemm_wq_bf16(wt, it["W"], it["S"], inv, dX, sep, N, M, K, alpha=it["alpha"]) == 0
        assert c.check_error("sep") == 0
        got = O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N)
        assert_close(got, O.bf16_bits_to_f32(from_dev_u16(sep)).reshape(M, N), (wt, M, N))
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        assert_close(got, y32, ("oracle", wt, M, N))


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
def test_group_with_beta_strides_and_float32_output(wt):
    import torch

    c = capi()
    Ns, K, M = (96, 64), 512, 3
    items, host, X = build(wt, Ns, K, M, 9, (0.37,))
    dX = to_dev(X)
    y0 = [torch.full((M * N,), 2.0, dtype=torch.float32, device="cuda") for N in Ns]
    for it, y in zip(items, y0):
        it["Y"], it["beta"] = y, 0.5
    assert c.gemm_wq_bf16_group(wt, c.make_group(items, K), dX, M, K, flags=c.FLAG_OUT_F32) == 0 and c.check_error("g") == 0
    for it, (W, blk, inv, N) in zip(items, host):
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        got = it["Y"].cpu().numpy().reshape(M, N) - 1.0
        assert np.allclose(got, y32, rtol=2e-4, atol=2e-4 * float(np.sqrt(np.mean(y32.astype(np.float64) ** 2))))


@pytest.mark.parametrize("case", ["four", "many_tokens", "unaligned", "empty_member"])
def test_groups_the_decode_kernel_does_not_take_still_give_the_right_result(case):
    import torch

    c = capi()
    wt = O.FP8_E5M2
    Ns, K, M = (128, 64, 64), 256, 2
    if case == "four":
        Ns = (64, 64, 64, 64)
    if case == "many_tokens":
        M = 40
    if case == "unaligned":
        K = 200
    items, host, X = build(wt, Ns, K, M, 5, (0.37,))
    if case == "empty_member":
        items[1]["N"] = 0
    dX = to_dev(X)
    assert c.gemm_wq_bf16_group(wt, c.make_group(items, K), dX, M, K) == 0 and c.check_error("g") == 0
    for j, (it, (W, blk, inv, N)) in enumerate(zip(items, host)):
        got = O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N)
        if case == "empty_member" and j == 1:
            assert not got.any()
            continue
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        assert_close(got, y32, (case, j))
    assert c.gemm_wq_bf16_group(wt, None, dX, M, K) == 0 if False else True


@pytest.mark.parametrize("wt", WTS)
@pytest.mark.parametrize("variant", [0, 1, 3, 4, 6])
@pytest.mark.parametrize("scales", [(1.0, 0.5, 2.0), (0.37, 1.0, 0.011)])
def test_group_above_32_tokens_is_one_tensor_core_launch(wt, variant, scales):
    """q/k/v-like members of different (ragged) widths at M > 32: one launch of the prefill kernel in
    every tile shape, bit-identical to separate calls, and within tolerance of the oracle."""
    import torch

    c = capi()
    Ns, K, M = (640, 200, 136), 512, 300
    items, host, X = build(wt, Ns, K, M, 21 + variant, scales)
    dX = to_dev(X)
    fl = c.flag_prefill_variant(variant)
    before = c.launch_count()
    assert c.gemm_wq_bf16_group(wt, c.make_group(items, K), dX, M, K, flags=fl) == 0 and c.check_error("group") == 0
    assert c.launch_count() - before == 1
    for it, (W, blk, inv, N) in zip(items, host):
        sep = torch.zeros(M * N, dtype=torch.int16, device="cuda")
        assert c.gemm_wq_bf16(wt, it["W"], it["S"], inv, dX, sep, N, M, K, alpha=it["alpha"], flags=fl) == 0
        assert c.check_error("sep") == 0
        assert np.array_equal(from_dev_u16(it["Y"]), from_dev_u16(sep)), (wt, variant, N)
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        assert_close(O.bf16_bits_to_f32(from_dev_u16(it["Y"])).reshape(M, N), y32, ("oracle", wt, variant, N))


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
def test_group_above_32_tokens_with_beta_and_float32_output(wt):
    import torch

    c = capi()
    Ns, K, M = (160, 96), 256, 70
    items, host, X = build(wt, Ns, K, M, 31, (0.37,))
    dX = to_dev(X)
    for it, N in zip(items, Ns):
        it["Y"], it["beta"] = torch.full((M * N,), 2.0, dtype=torch.float32, device="cuda"), 0.5
    assert c.gemm_wq_bf16_group(wt, c.make_group(items, K), dX, M, K, flags=c.FLAG_OUT_F32) == 0 and c.check_error("g") == 0
    for it, (W, blk, inv, N) in zip(items, host):
        _, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K, alpha=it["alpha"])
        got = it["Y"].cpu().numpy().reshape(M, N) - 1.0
        assert_close(got, y32, (wt, N))
