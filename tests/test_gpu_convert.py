"""cuda_convert and the FP4 block-scale pair on the GPU: bit-exact against the CPU oracle and,
where oracle/_ref holds it, against the reference's own cuda_functions.cu built for sm_100a."""
import numpy as np
import pytest

from oracle import oracle as O
from tests._util import capi, from_dev_u16, ref_cuda_lib, to_dev

pytestmark = pytest.mark.gpu


def _rand_bytes(n, seed):
    rng = np.random.default_rng(seed)
    b = rng.integers(0, 256, size=n, dtype=np.uint8)
    b[:256] = np.arange(256, dtype=np.uint8)  # every code point, NaN/Inf included
    return b


@pytest.mark.parametrize("n", [1, 15, 16, 257, 4096 + 3, 1 << 20])
@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3])
def test_fp8_to_bf16_bit_exact(wt, n):
    import torch

    c = capi()
    src = _rand_bytes(max(n, 256), 1)[:n] if n < 256 else _rand_bytes(n, 1)
    for scale in (1.0, 0.37, 2.0 ** -7):
        d_src = to_dev(src)
        d_dst = torch.zeros(n + 8, dtype=torch.int16, device="cuda")
        assert c.convert(d_src, wt, d_dst, c.BFLOAT16, n, scale) == 0
        got = from_dev_u16(d_dst)
        assert np.array_equal(got[:n], O.fp8_to_bf16(src, wt, scale)), (wt, n, scale)
        assert not got[n:].any(), "wrote past n"


def test_fp8_to_bf16_unaligned_pointers():
    import torch

    c = capi()
    n = 1000
    src = _rand_bytes(n + 3, 2)
    d_src = to_dev(src)
    d_dst = torch.zeros(n + 4, dtype=torch.int16, device="cuda")
    assert c.convert(d_src.data_ptr() + 3, c.FP8_E5M2, d_dst.data_ptr() + 2, c.BFLOAT16, n, 0.5) == 0
    assert np.array_equal(from_dev_u16(d_dst)[1:n + 1], O.fp8_to_bf16(src[3:], O.FP8_E5M2, 0.5))


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP8_E4M3])
def test_float_fp8_both_ways(wt):
    import torch

    c = capi()
    rng = np.random.default_rng(5)
    f = np.concatenate([rng.standard_normal(5000) * s for s in (1e-6, 1e-3, 1.0, 300.0, 1e5)]).astype(np.float32)
    f[:4] = [np.inf, -np.inf, np.nan, -0.0]
    d_f = to_dev(f)
    d_q = torch.zeros(f.size, dtype=torch.uint8, device="cuda")
    assert c.convert(d_f, c.FLOAT, d_q, wt, f.size, 1.7) == 0
    q = d_q.cpu().numpy()
    assert np.array_equal(q, O.float_to_fp8(f, wt, 1.7))
    d_back = torch.zeros(f.size, dtype=torch.float32, device="cuda")
    assert c.convert(d_q, wt, d_back, c.FLOAT, f.size, 0.25) == 0
    want = O.fp8_to_float(q, wt, 0.25)
    got = d_back.cpu().numpy()
    fin = np.isfinite(want)
    assert np.array_equal(got[fin], want[fin]) and np.array_equal(np.isnan(got), np.isnan(want))


def test_fp4_per_tensor_and_packing():
    import torch

    c = capi()
    rng = np.random.default_rng(6)
    f = (rng.standard_normal(4097) * 2.5).astype(np.float32)
    d_f = to_dev(f)
    d_q = torch.zeros((f.size + 1) // 2, dtype=torch.uint8, device="cuda")
    assert c.convert(d_f, c.FLOAT, d_q, c.FP4_E2M1, f.size, 1.3) == 0
    q = d_q.cpu().numpy()
    assert np.array_equal(q, O.float_to_fp4_packed(f, 1.3))
    d_h = torch.zeros(f.size, dtype=torch.int16, device="cuda")
    assert c.convert(d_q, c.FP4_E2M1, d_h, c.BFLOAT16, f.size, 0.013) == 0
    assert np.array_equal(from_dev_u16(d_h), O.fp4_to_bf16(q, f.size, 0.013))
    d_f2 = torch.zeros(f.size, dtype=torch.float32, device="cuda")
    assert c.convert(d_q, c.FP4_E2M1, d_f2, c.FLOAT, f.size, 0.013) == 0
    assert np.array_equal(d_f2.cpu().numpy(), O.fp4_packed_to_float(q, f.size, 0.013))


@pytest.mark.parametrize("n", [16, 37, 16 * 1000, 16 * 4096 + 5])
def test_fp4_blockscale_both_ways(n):
    import torch

    c = capi()
    rng = np.random.default_rng(7)
    f = (rng.standard_normal(n) * 0.02).astype(np.float32)
    f[:16] = 0
    d_f = to_dev(f)
    d_nib = torch.zeros((n + 1) // 2, dtype=torch.uint8, device="cuda")
    d_sc = torch.zeros((n + 15) // 16, dtype=torch.uint8, device="cuda")
    assert c.float_to_fp4_blockscale(d_f, d_nib, d_sc, n, 16) == 0
    nib, sc = O.float_to_fp4_blockscale(f, 16)
    assert np.array_equal(d_nib.cpu().numpy(), nib) and np.array_equal(d_sc.cpu().numpy(), sc)
    d_h = torch.zeros(n, dtype=torch.int16, device="cuda")
    assert c.fp4_blockscale_to_bf16(d_nib, d_sc, d_h, n, 16) == 0
    assert np.array_equal(from_dev_u16(d_h), O.fp4_blockscale_to_bf16(nib, sc, n, 16))
    # every scale byte, NaN code points included, and a block size other than 16
    sc_all = np.arange(256, dtype=np.uint8)
    nib_all = _rand_bytes(256 * 4, 8)
    d_h2 = torch.zeros(256 * 8, dtype=torch.int16, device="cuda")
    assert c.fp4_blockscale_to_bf16(to_dev(nib_all), to_dev(sc_all), d_h2, 256 * 8, 8) == 0
    assert np.array_equal(from_dev_u16(d_h2), O.fp4_blockscale_to_bf16(nib_all, sc_all, 256 * 8, 8))


def test_plain_casts_and_table_holes():
    import torch

    c = capi()
    rng = np.random.default_rng(9)
    f = (rng.standard_normal(3001) * 3).astype(np.float32)
    t = torch.from_numpy(f).cuda()
    out_bf = torch.zeros(f.size, dtype=torch.bfloat16, device="cuda")
    assert c.convert(t, c.FLOAT, out_bf, c.BFLOAT16, f.size, 1.0) == 0
    assert torch.equal(out_bf, t.to(torch.bfloat16))
    out_f = torch.zeros(f.size, dtype=torch.float32, device="cuda")
    assert c.convert(out_bf, c.BFLOAT16, out_f, c.FLOAT, f.size, 1.0) == 0
    assert torch.equal(out_f, out_bf.float())
    h = t.half()
    assert c.convert(h, c.HALF, out_f, c.FLOAT, f.size, 1.0) == 0
    assert torch.equal(out_f, h.float())
    assert c.convert(h, c.HALF, out_bf, c.BFLOAT16, f.size, 1.0) == 0
    assert torch.equal(out_bf, h.float().to(torch.bfloat16))
    out_h = torch.zeros(f.size, dtype=torch.float16, device="cuda")
    assert c.convert(out_bf, c.BFLOAT16, out_h, c.HALF, f.size, 1.0) == 0
    assert torch.equal(out_h, out_bf.float().half())
    # same type, scale 1: copies n BYTES (reference behaviour)
    a = torch.arange(64, dtype=torch.uint8, device="cuda")
    b = torch.zeros(64, dtype=torch.uint8, device="cuda")
    assert c.convert(a, c.FP8_E5M2, b, c.FP8_E5M2, 40, 1.0) == 0
    assert torch.equal(b[:40], a[:40]) and not b[40:].any()
    # unsupported pairs -> -1, as the reference's table
    assert c.convert(a, c.DOUBLE, b, c.FLOAT, 4, 1.0) == -1
    assert c.convert(a, c.FP8_E5M2, b, c.FP8_E4M3, 4, 1.0) == -1
    assert c.convert(a, 9, b, c.FLOAT, 4, 1.0) == -1


def test_against_reference_cuda_kernels():
    """Same device buffers through the reference's own kernels (oracle/_ref) and ours."""
    import torch

    R = ref_cuda_lib()
    if R is None:
        pytest.skip("oracle/_ref/libcccc-cuda-ref.so not built")
    c = capi()
    n = 1 << 16
    src = _rand_bytes(n, 11)
    d_src = to_dev(src)
    for wt in (c.FP8_E5M2, c.FP8_E4M3):
        for scale in (1.0, 0.0123):
            a = torch.zeros(n, dtype=torch.int16, device="cuda")
            b = torch.zeros(n, dtype=torch.int16, device="cuda")
            assert R.cuda_convert(d_src.data_ptr(), wt, a.data_ptr(), c.BFLOAT16, n, scale) == 0
            assert c.convert(d_src, wt, b, c.BFLOAT16, n, scale) == 0
            assert torch.equal(a, b), (wt, scale)
    # FP4 per-tensor and block-scale dequant, all scale bytes
    a = torch.zeros(2 * n, dtype=torch.int16, device="cuda")
    b = torch.zeros(2 * n, dtype=torch.int16, device="cuda")
    assert R.cuda_convert(d_src.data_ptr(), c.FP4_E2M1, a.data_ptr(), c.BFLOAT16, 2 * n, 0.37) == 0
    assert c.convert(d_src, c.FP4_E2M1, b, c.BFLOAT16, 2 * n, 0.37) == 0
    assert torch.equal(a, b)
    sc = to_dev(_rand_bytes(2 * n // 16, 12))
    assert R.cuda_fp4_blockscale_to_bf16(d_src.data_ptr(), sc.data_ptr(), a.data_ptr(), 2 * n, 16) == 0
    assert c.fp4_blockscale_to_bf16(d_src, sc, b, 2 * n, 16) == 0
    assert torch.equal(a, b)
    # quantisers
    f = (torch.randn(n, device="cuda") * 0.02).float()
    f[:3] = torch.tensor([float("nan"), float("inf"), -float("inf")], device="cuda")
    for wt in (c.FP8_E5M2, c.FP8_E4M3):
        qa = torch.zeros(n, dtype=torch.uint8, device="cuda")
        qb = torch.zeros(n, dtype=torch.uint8, device="cuda")
        assert R.cuda_convert(f.data_ptr(), c.FLOAT, qa.data_ptr(), wt, n, 2000.0) == 0
        assert c.convert(f, c.FLOAT, qb, wt, n, 2000.0) == 0
        assert torch.equal(qa, qb)
    f[:3] = 0
    na, nb = (torch.zeros(n // 2, dtype=torch.uint8, device="cuda") for _ in range(2))
    sa, sb = (torch.zeros(n // 16, dtype=torch.uint8, device="cuda") for _ in range(2))
    assert R.cuda_float_to_fp4_blockscale(f.data_ptr(), na.data_ptr(), sa.data_ptr(), n, 16) == 0
    assert c.float_to_fp4_blockscale(f, nb, sb, n, 16) == 0
    assert torch.equal(na, nb) and torch.equal(sa, sb)
