"""The benchmark configurations at their own shapes, through the C-ABI.

Configuration 2: Qwen3-8B W8A16 decode linears (q/o 4096x4096, k/v 1024x4096, gate/up 12288x4096, down
4096x12288, lm_head 151936x4096) at M in {1, 4, 16, 32}.  Configuration 3: Llama-3.1-8B W4A16 decode
linears (FP4 block 16 with E4M3 scales; gate/up 14336x4096, down 4096x14336, lm_head 128256x4096) at
M in {1, 8, 32}.  Configuration 4: M = 2048 tokens through every configuration-2 projection and through
the two grouped calls (q+k+v, gate+up) that the benchmark times.

Weights ~ N(0, 0.02) are drawn and quantised ON THE DEVICE with this library's quantisers (which other
tests pin bit for bit to the reference's), because the CPU oracle would take minutes on 6e8 elements.
Every output is then checked twice: against the CPU oracle on a subset of rows (and tokens) whose
weight bytes are copied back, and, for all rows, against a float32 matmul of the library's own
bit-exact dequantisation.  Tolerance for GEMV/GEMM outputs: max relative error 1e-2, cosine >= 0.9999."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close, capi, to_dev

pytestmark = pytest.mark.gpu

QWEN = {"q_o": (4096, 4096), "k_v": (1024, 4096), "gate_up": (12288, 4096), "down": (4096, 12288)}
LLAMA = {"q_o": (4096, 4096), "k_v": (1024, 4096), "gate_up": (14336, 4096), "down": (4096, 14336)}


def device_weight(wt, N, K, seed, scaled=True):
    """N(0, 0.02) weights quantised on the device with the reference's rules (cccc/Matrix.cpp:301-355):
    returns (bytes, block scales or None, dequant multiplier)."""
    import torch

    c = capi()
    g = torch.Generator(device="cuda").manual_seed(seed)
    n = N * K
    step = 1 << 27
    if wt == O.FP4_E2M1:
        nib = torch.empty(n // 2, dtype=torch.uint8, device="cuda")
        sc = torch.empty(n // 16, dtype=torch.uint8, device="cuda")
        for b in range(0, n, step):
            e = min(n, b + step)
            w = torch.randn(e - b, device="cuda", generator=g) * 0.02
            assert c.float_to_fp4_blockscale(w, nib[b // 2:], sc[b // 16:], e - b, 16) == 0
        return nib, sc, 1.0
    w8 = torch.empty(n, dtype=torch.uint8, device="cuda")
    maxval = 448.0 if wt == O.FP8_E4M3 else 57344.0
    absmax = 0.02 * 5.5  # a fixed bound instead of the tensor's own maximum: one pass, same value range
    fwd = float(np.float32(maxval) / np.float32(absmax)) if scaled else 1.0
    inv = float(np.float32(absmax) / np.float32(maxval)) if scaled else 1.0
    for b in range(0, n, step):
        e = min(n, b + step)
        w = (torch.randn(e - b, device="cuda", generator=g) * 0.02).clamp_(-absmax, absmax)
        assert c.convert(w, c.FLOAT, w8[b:], wt, e - b, fwd) == 0
    return w8, None, inv


def device_acts(M, K, seed):
    import torch

    g = torch.Generator(device="cuda").manual_seed(1000 + seed)
    return torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)


def dequantised(wt, W, S, inv, N, K):
    """The library's standalone dequantisation (bit-equal to the reference's kernels, tests/test_gpu_convert.py)."""
    import torch

    c = capi()
    out = torch.empty(N * K, dtype=torch.bfloat16, device="cuda")
    step = 1 << 28
    for b in range(0, N * K, step):
        e = min(N * K, b + step)
        if wt == O.FP4_E2M1:
            assert c.fp4_blockscale_to_bf16(W[b // 2:], S[b // 16:], out[b:], e - b, 16) == 0
        else:
            assert c.convert(W[b:], wt, out[b:], c.BFLOAT16, e - b, inv) == 0
    return out.view(N, K)


def check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, rows, toks=None, alpha=1.0):
    """CPU oracle on the chosen output features (and tokens): their weight rows are copied back."""
    import torch

    ridx = torch.from_numpy(rows).cuda()
    wb = K // 2 if wt == O.FP4_E2M1 else K
    Wsub = W.view(N, wb)[ridx].cpu().numpy()
    Ssub = S.view(N, K // 16)[ridx].cpu().numpy() if S is not None else None
    Xh = X.view(torch.int16).cpu().numpy().view(np.uint16).reshape(M, K)
    Yh = Y.float().cpu().numpy().reshape(M, N)
    if toks is not None:
        Xh, Yh = Xh[toks], Yh[toks]
    _, y32 = O.linear_wq_bf16(wt, Wsub.reshape(-1), None if Ssub is None else Ssub.reshape(-1), inv, Xh, rows.size, Xh.shape[0], K,
                              alpha=alpha)
    assert_close(Yh[:, rows], y32, ("oracle subset", wt, N, K, M))


def check_all_rows(wt, W, S, inv, X, Y, N, M, K, alpha=1.0):
    """Every output against float32 x (bit-exact dequantised weights), in slabs of output features."""
    import torch

    step = max(1, (1 << 26) // K)
    Xf = X.float()
    for b in range(0, N, step):
        e = min(N, b + step)
        wb = K // 2 if wt == O.FP4_E2M1 else K
        Wd = dequantised(wt, W.view(N, wb)[b:e].reshape(-1), None if S is None else S.view(N, K // 16)[b:e].reshape(-1), inv, e - b, K)
        ref = (Xf @ Wd.float().t()) * alpha
        assert_close(Y.view(M, N)[:, b:e].float().cpu().numpy(), ref.cpu().numpy(), ("all rows", wt, N, K, M, b))


def subset(N, count, seed):
    rng = np.random.default_rng(seed)
    edge = min(48, N // 2)
    return np.unique(np.concatenate([np.arange(edge), np.arange(N - edge, N), rng.integers(0, N, count)]))


def native_by_default(wt, M, Ns, K):
    """The dispatcher's rule for the native-operand kernels: launches of whole tiles (between one and two 128-feature
    tiles per SM) and lm_head-sized ones (FP8 256 MB, FP4 48 MB of weights), up to 32 tokens, FP8 only from 3."""
    import torch

    sms = torch.cuda.get_device_properties(0).multi_processor_count
    tiles = sum((n + 127) // 128 for n in Ns)
    elems = sum(Ns) * K
    if M > 32 or (wt != O.FP4_E2M1 and M < 3):
        return False
    if sms < tiles <= 2 * sms and not (wt == O.FP4_E2M1 and M > 13):
        return True
    return elems // 2 >= 48 << 20 if wt == O.FP4_E2M1 else elems >= 256 << 20


def is_pow2(x):
    m, _ = np.frexp(x)
    return m == 0.5


def run_one(wt, N, K, M, seed, plan):
    import torch

    c = capi()
    if 9 <= M <= 128:
        plan = c.PLAN_STREAM    # the streaming tensor-core kernel takes these shapes from 9 to 128 tokens
    if native_by_default(wt, M, [N], K):
        plan = c.PLAN_NATIVE
    W, S, inv = device_weight(wt, N, K, seed)
    X = device_acts(M, K, seed)
    Y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert c.gemm_wq_bf16_plan(wt, W, S, X, Y, N, M, K) == plan
    assert c.gemm_wq_bf16(wt, W, S, inv, X, Y, N, M, K) == 0 and c.check_error("config") == 0
    return W, S, inv, X, Y


@pytest.mark.parametrize("M", [1, 4, 16, 32])
@pytest.mark.parametrize("name", list(QWEN))
def test_config2_qwen3_w8a16_decode_linears(name, M):
    N, K = QWEN[name]
    wt = O.FP8_E5M2
    W, S, inv, X, Y = run_one(wt, N, K, M, 7 * N + K + M, capi().PLAN_DECODE)
    check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, subset(N, 400, M))
    check_all_rows(wt, W, S, inv, X, Y, N, M, K)


@pytest.mark.parametrize("M", [1, 32])
def test_config2_qwen3_lm_head(M):
    N, K = 151936, 4096
    wt = O.FP8_E5M2
    W, S, inv, X, Y = run_one(wt, N, K, M, 5 + M, capi().PLAN_DECODE)
    check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, subset(N, 1200, M))
    check_all_rows(wt, W, S, inv, X, Y, N, M, K)


@pytest.mark.parametrize("M", [1, 8, 32])
@pytest.mark.parametrize("name", list(LLAMA))
def test_config3_llama_w4a16_decode_linears(name, M):
    N, K = LLAMA[name]
    wt = O.FP4_E2M1
    W, S, inv, X, Y = run_one(wt, N, K, M, 3 * N + K + M, capi().PLAN_DECODE)
    check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, subset(N, 400, M))
    check_all_rows(wt, W, S, inv, X, Y, N, M, K)


@pytest.mark.parametrize("M", [1, 8, 32])
def test_config3_llama_lm_head(M):
    N, K = 128256, 4096
    wt = O.FP4_E2M1
    W, S, inv, X, Y = run_one(wt, N, K, M, 11 + M, capi().PLAN_DECODE)
    check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, subset(N, 1200, M))
    check_all_rows(wt, W, S, inv, X, Y, N, M, K)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
@pytest.mark.parametrize("name", list(QWEN))
def test_config4_prefill_every_projection(wt, name):
    N, K = QWEN[name]
    M = 2048
    W, S, inv, X, Y = run_one(wt, N, K, M, N + 3 * K, capi().PLAN_PREFILL)
    toks = np.unique(np.concatenate([np.arange(0, M, 67), [M - 1]]))
    check_against_oracle_subset(wt, W, S, inv, X, Y, N, M, K, subset(N, 200, 4), toks)
    check_all_rows(wt, W, S, inv, X, Y, N, M, K)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
@pytest.mark.parametrize("members", [("q_o", "k_v", "k_v"), ("gate_up", "gate_up")])
@pytest.mark.parametrize("M", [1, 32, 2048])
def test_grouped_calls_of_the_benchmark(wt, members, M):
    """q+k+v and gate+up as one cuda_gemm_wq_bf16_group call each, as bench.py issues them: decode at
    M = 1 and 32, prefill (configuration 4) at M = 2048."""
    import torch

    c = capi()
    K = 4096
    X = device_acts(M, K, 77 + M)
    items = []
    for j, name in enumerate(members):
        N = QWEN[name][0]
        W, S, inv = device_weight(wt, N, K, 100 * j + N + M)
        items.append(dict(W=W, S=S, inv=inv, N=N, Y=torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda"),
                          alpha=1.0 + 0.25 * j))
    before = c.launch_count()
    assert c.gemm_wq_bf16_group(wt, c.make_group(items, K), X, M, K) == 0 and c.check_error("group") == 0
    # one launch for the group; before a native-operand kernel the split of the activations is a launch of its own
    # (an FP8 scale that is no power of two keeps the kernels that dequantise)
    native = native_by_default(wt, M, [it["N"] for it in items], K) and (wt == O.FP4_E2M1 or all(is_pow2(it["inv"]) for it in items))
    assert c.launch_count() - before == (2 if native else 1)
    toks = None if M <= 32 else np.unique(np.concatenate([np.arange(0, M, 131), [M - 1]]))
    for it in items:
        check_against_oracle_subset(wt, it["W"], it["S"], it["inv"], X, it["Y"], it["N"], M, K, subset(it["N"], 150, M), toks,
                                    alpha=it["alpha"])
        check_all_rows(wt, it["W"], it["S"], it["inv"], X, it["Y"], it["N"], M, K, alpha=it["alpha"])
