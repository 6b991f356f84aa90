"""'Dequantised weights bit-exact' on the path that ships: inside the fused kernels.

The fused decode and prefill kernels dequantise with other instructions than the standalone
conversions (byte permutes and hardware converts, the FP4 exponent-insertion trick).  A one-hot
activation row makes their result observable: with X[m, :] = 1.0 at one position k_m and 0 elsewhere,
alpha = 1 and beta = 0,

    Y[m, n] = bf16( dq(W[n, k_m]) * 1.0 + zeros ) = dq(W[n, k_m])

so every output must equal the oracle's dequantised BF16 weight (cccc-cuda/cuda_functions.cu:2756-2771
for FP8, :2926-2939 for FP4 block scale) BIT FOR BIT.  Covered: all 256 FP8 bytes that are finite x
{scale 1.0, a power of two, 0.37}; all 16 nibbles x all 254 non-NaN E4M3 block-scale bytes; every
position of k; every decode tile configuration (M <= 2, <= 8, <= 16, <= 32), the split-k schedule, and
the six prefill tile shapes.  Only the sign of a zero is not compared: a -0 weight times 1.0 added to
the +0 accumulator gives +0 in any FP32 accumulation, in the reference's cuBLAS call as well.

Inf and NaN weight bytes are kept out of these matrices (Inf x 0 = NaN would spill over a whole row) and
have their own test: a NaN byte gives a NaN output row here, where the reference's integer rounding trick
turns the NaN into -0 - the one documented difference."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import capi, to_dev

pytestmark = pytest.mark.gpu

ONE = 0x3F80  # bf16 1.0


def finite_bytes(wt):
    b = np.arange(256, dtype=np.uint8)
    if wt == O.FP8_E5M2:
        return b[(b & 0x7C) != 0x7C]
    return b[(b & 0x7F) != 0x7F]


def fp8_matrix(wt, N, K):
    """Row n, column k holds finite byte number (n + 7k) of the type: every byte meets every k position."""
    fb = finite_bytes(wt)
    n = np.arange(N)[:, None]
    k = np.arange(K)[None, :]
    return fb[(n + 7 * k) % fb.size].astype(np.uint8)


def fp4_matrix(N, K):
    """Row n uses block-scale byte number n of the 254 non-NaN ones (shifted along k so that a row meets
    several), nibble (k + n) & 15."""
    sb = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], np.uint8)
    n = np.arange(N)[:, None]
    k = np.arange(K)[None, :]
    nib = ((k + n) & 15).astype(np.uint8)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    blocks = np.arange(K // 16)[None, :]
    scales = sb[(n + 3 * blocks) % sb.size].astype(np.uint8)
    return packed, scales


def expected_bits(wt, W, S, inv, N, K):
    if wt == O.FP4_E2M1:
        return O.fp4_blockscale_to_bf16(W.reshape(-1), S.reshape(-1), N * K, 16).reshape(N, K)
    return O.fp8_to_bf16(W.reshape(-1), wt, inv).reshape(N, K)


def same_up_to_zero_sign(got, want):
    """uint16 BF16 patterns equal, where +0 and -0 count as equal."""
    g = got.astype(np.uint16).copy()
    w = want.astype(np.uint16).copy()
    g[g == 0x8000] = 0
    w[w == 0x8000] = 0
    return g == w


def run_onehot(wt, W, S, inv, D, N, K, M, positions, flags=0):
    """One launch per set of positions (one position per token); returns the number of outputs compared."""
    import torch

    c = capi()
    dW = to_dev(W.reshape(-1))
    dS = to_dev(S.reshape(-1)) if S is not None else None
    dD = torch.from_numpy(D.view(np.int16)).cuda()           # [N, K] expected bits
    total = 0
    for ks in positions:
        ks = np.asarray(ks, dtype=np.int64)
        assert ks.size == M
        X = torch.zeros(M, K, dtype=torch.int16, device="cuda")
        kt = torch.from_numpy(ks).cuda()
        X[torch.arange(M, device="cuda"), kt] = ONE
        Y = torch.full((M, N), 0x7FC0, dtype=torch.int16, device="cuda")
        assert c.gemm_wq_bf16(wt, dW, dS, inv, X, Y, N, M, K, flags=flags) == 0
        want = dD[:, kt].t().contiguous()
        g = torch.where(Y == -32768, torch.zeros_like(Y), Y)   # 0x8000 as int16
        w = torch.where(want == -32768, torch.zeros_like(want), want)
        if not torch.equal(g, w):
            bad = (g != w).nonzero()[:5].cpu().numpy()
            m, n = bad[0]
            raise AssertionError((wt, inv, M, "first mismatches (token, feature)", bad.tolist(), "k", int(ks[m]),
                                  "got", hex(int(Y[m, n]) & 0xFFFF), "want", hex(int(want[m, n]) & 0xFFFF)))
        total += M * N
    assert c.check_error("one-hot") == 0
    return total


def all_positions(K, M, stride=37):
    """Sets of M positions that together cover every k of [0, K)."""
    order = (np.arange(K) * stride) % K
    assert np.unique(order).size == K
    pad = (-K) % M
    order = np.concatenate([order, order[:pad]])
    return order.reshape(-1, M)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3])
@pytest.mark.parametrize("inv", [1.0, 0.25, 0.37])
@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_fp8_decode_kernels_dequantise_bit_exactly(wt, inv, M):
    N, K = 512, 512
    W = fp8_matrix(wt, N, K)
    D = expected_bits(wt, W, None, inv, N, K)
    assert c_plan(wt, W, None, N, M, K) == (capi().PLAN_DECODE if M <= 8 else capi().PLAN_STREAM)
    run_onehot(wt, W, None, inv, D, N, K, M, all_positions(K, M), flags=capi().FLAG_NO_STREAM)


@pytest.mark.parametrize("M", [1, 8, 16, 32])
def test_fp4_decode_kernels_dequantise_bit_exactly(M):
    N, K = 508, 512     # 508 = 2 x 254: every non-NaN scale byte twice, with different nibbles
    W, S = fp4_matrix(N, K)
    D = expected_bits(O.FP4_E2M1, W, S, 1.0, N, K)
    assert c_plan(O.FP4_E2M1, W, S, N, M, K) == (capi().PLAN_DECODE if M <= 8 else capi().PLAN_STREAM)
    run_onehot(O.FP4_E2M1, W, S, 1.0, D, N, K, M, all_positions(K, M), flags=capi().FLAG_NO_STREAM)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1])
@pytest.mark.parametrize("M", [1, 8])
def test_split_k_schedule_dequantises_bit_exactly(wt, M):
    """Few long rows: the k range is split between CTAs and combined through the workspace."""
    N, K = 64, 16384
    if wt == O.FP4_E2M1:
        W, S = fp4_matrix(N, K)
    else:
        W, S = fp8_matrix(wt, N, K), None
    inv = 0.37 if wt != O.FP4_E2M1 else 1.0
    D = expected_bits(wt, W, S, inv, N, K)
    rng = np.random.default_rng(M)
    positions = rng.integers(0, K, (48, M))
    run_onehot(wt, W, S, inv, D, N, K, M, positions)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1])
@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("M", [64, 2048])
def test_prefill_kernels_dequantise_bit_exactly(wt, variant, M):
    c = capi()
    N, K = 512, 512
    if wt == O.FP4_E2M1:
        N = 508
        W, S = fp4_matrix(N, K)
    else:
        W, S = fp8_matrix(wt, N, K), None
    for inv in ((1.0,) if wt == O.FP4_E2M1 else (1.0, 0.25, 0.37)):
        D = expected_bits(wt, W, S, inv, N, K)
        assert c_plan(wt, W, S, N, M, K) == (c.PLAN_STREAM if M <= 128 else c.PLAN_PREFILL)    # a tile-shape flag keeps the prefill kernel
        # M tokens cover every k position M / K times over
        positions = [(np.arange(M) * 37 + 11) % K]
        run_onehot(wt, W, S, inv, D, N, K, M, positions, flags=c.flag_prefill_variant(variant))


@pytest.mark.parametrize("wt,inv", [(O.FP8_E5M2, 1.0), (O.FP8_E5M2, 0.25), (O.FP8_E5M2, 0.37), (O.FP8_E4M3, 1.0), (O.FP8_E4M3, 0.37),
                                    (O.FP4_E2M1, 1.0)])
@pytest.mark.parametrize("M", [1, 2])
def test_decode_program_dequantises_bit_exactly(wt, inv, M):
    """The persistent decode-program kernel has k steps of its own (CUDA-core FMAs for weights without a
    per-weight multiplier, tensor-core steps otherwise): the same one-hot check, every k position."""
    import torch

    c = capi()
    N, K = (508, 512) if wt == O.FP4_E2M1 else (512, 512)
    if wt == O.FP4_E2M1:
        W, S = fp4_matrix(N, K)
    else:
        W, S = fp8_matrix(wt, N, K), None
    D = expected_bits(wt, W, S, inv, N, K)
    dW = to_dev(W.reshape(-1))
    dS = to_dev(S.reshape(-1)) if S is not None else None
    dD = torch.from_numpy(D.view(np.int16)).cuda()
    X = torch.zeros(M, K, dtype=torch.int16, device="cuda")
    Y = torch.zeros(M, N, dtype=torch.int16, device="cuda")
    grp = c.make_group([dict(W=dW, S=dS, inv=inv, N=N, Y=Y)], K)
    prog = c.DecodeProgram(wt, M)
    assert prog.add_linears(grp, K, X) == 0 and prog.finalize() == 0
    for ks in all_positions(K, M):
        kt = torch.from_numpy(np.asarray(ks, np.int64)).cuda()
        X.zero_()
        X[torch.arange(M, device="cuda"), kt] = ONE
        Y.fill_(0x7FC0)
        assert prog.launch() == 0
        want = dD[:, kt].t().contiguous()
        g = torch.where(Y == -32768, torch.zeros_like(Y), Y)
        w = torch.where(want == -32768, torch.zeros_like(want), want)
        assert torch.equal(g, w), (wt, inv, M, ks.tolist())
    assert c.check_error("program one-hot") == 0
    prog.close()


def c_plan(wt, W, S, N, M, K):
    import torch

    c = capi()
    X = torch.zeros(M, K, dtype=torch.int16, device="cuda")
    return c.gemm_wq_bf16_plan(wt, to_dev(W.reshape(-1)), to_dev(S.reshape(-1)) if S is not None else None, X, None, N, M, K)


@pytest.mark.parametrize("wt,nan_byte", [(O.FP8_E5M2, 0x7E), (O.FP8_E4M3, 0x7F)])
@pytest.mark.parametrize("M", [1, 32, 64])
def test_nan_weight_byte_gives_a_nan_row(wt, nan_byte, M):
    """The documented difference: the fused kernels round with the hardware conversion, so a NaN weight
    byte makes its output feature NaN for every token (the reference's integer rounding trick wraps the
    NaN to -0 instead, cuda_functions.cu:2761-2764; its own quantisers never emit NaN bytes).  Rows
    without a NaN byte are unaffected."""
    import torch

    c = capi()
    N, K = 128, 512
    W = fp8_matrix(wt, N, K)
    W[5, 77] = nan_byte
    W[100, 300] = nan_byte | 0x80
    X = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    Y = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    assert c.gemm_wq_bf16(wt, to_dev(W.reshape(-1)), None, 0.37, X, Y, N, M, K) == 0 and c.check_error("nan") == 0
    y = Y.float().cpu().numpy()
    assert np.all(np.isnan(y[:, 5])) and np.all(np.isnan(y[:, 100]))
    rest = np.delete(y, [5, 100], axis=1)
    assert np.all(np.isfinite(rest))
    Wc = np.delete(W, [5, 100], axis=0)
    Xh = X.view(torch.int16).cpu().numpy().view(np.uint16)
    _, y32 = O.linear_wq_bf16(wt, Wc.reshape(-1), None, 0.37, Xh, N - 2, M, K)
    from tests._util import assert_close

    assert_close(rest, y32, "rows without NaN bytes")
