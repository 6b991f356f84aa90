"""The C++ decode-linears driver (weights from the converter's container, grouped launches, one CUDA
graph per token, token chosen on the device) and the device arg-max."""
import ctypes as C
import math
import struct

import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle as O
from tests._util import capi, to_dev
from tests.test_loader_cpu import write_container

pytestmark = pytest.mark.gpu


def test_argmax_first_maximum_nan_and_strides():
    import torch

    c = capi()
    rows, cols, ld = 5, 151936, 151936 + 8
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(rows, ld, device="cuda", generator=g).to(torch.bfloat16)
    x[0, 777] = 50.0
    x[0, 90000] = 50.0            # tie: the first one wins
    x[1, :] = float("nan")        # only NaN: -1
    x[2, 5] = float("nan")
    x[2, 6] = 40.0
    x[3, :cols] = -float("inf")
    x[3, cols - 1] = -1e30
    x[4, cols:] = 100.0           # beyond cols: must be ignored
    idx = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    val = torch.zeros(rows, dtype=torch.float32, device="cuda")
    assert c.argmax_bf16(x, rows, cols, idx, val, ld=ld) == 0 and c.check_error("argmax") == 0
    got = idx.cpu().tolist()
    assert got[0] == 777 and got[1] == -1 and got[2] == 6 and got[3] == cols - 1
    assert got[4] == int(torch.argmax(x[4, :cols].float()).item())
    assert val[0].item() == 50.0 and val[2].item() == 40.0
    assert c.argmax_bf16(x, 0, cols, idx, val) == 0 and c.argmax_bf16(None, 1, cols, idx, val) == -1


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
def test_decode_driver_matches_the_same_chain_issued_by_hand(tmp_path, wt):
    import torch

    h = load_package().hostapi
    L = h.lib()
    c = capi()
    hidden, q_dim, kv_dim, ffn, vocab, layers, M = 256, 256, 64, 512, 1024, 2, 3
    sfx = "fp8_e5m2" if wt == O.FP8_E5M2 else "fp4_e2m1"
    entries, host = {"data_type": sfx.encode()}, {}
    shapes = {"W_q": (q_dim, hidden), "W_k": (kv_dim, hidden), "W_v": (kv_dim, hidden), "W_o": (hidden, q_dim),
              "W_gate": (ffn, hidden), "W_up": (ffn, hidden), "W_down": (hidden, ffn)}
    seed = 0
    names = [f"{k}_{i}" for i in range(layers) for k in shapes] + ["W_lm_head"]
    for name in names:
        N, K = (vocab, hidden) if name == "W_lm_head" else shapes[name.rsplit("_", 1)[0]]
        seed += 1
        W, blk, inv, _ = O.make_inputs(wt, N, K, 1, seed=seed, scaled=True)
        entries[f"weight_{sfx}_{name}"] = W.tobytes()
        if blk is not None:
            entries[f"blockscale_{name}"] = blk.tobytes()
        else:
            entries[f"scale_{name}"] = struct.pack("<f", inv)
        host[name] = (W, blk, inv, N, K)
    path = str(tmp_path / "model.bin")
    write_container(path, entries)

    g = L.cccc_host_gpu_create(0)
    f = L.cccc_host_bin_open(path.encode())
    assert g and f
    alphas = [1.0 / (0.02 * math.sqrt(hidden)), 1.0 / (0.02 * math.sqrt(hidden)), 1.0 / (0.02 * math.sqrt(ffn)), 1.0]
    err = C.create_string_buffer(256)
    d = L.cccc_host_decode_create(g, f, hidden, q_dim, kv_dim, ffn, vocab, layers, 8, *alphas, err, 256)
    assert d, err.value
    assert L.cccc_host_decode_weight_bytes(d) == sum(len(v) for k, v in entries.items() if k.startswith(("weight_", "blockscale_")))
    x = O.f32_to_bf16_bits(np.random.default_rng(3).standard_normal((M, hidden)).astype(np.float32))
    ids = (C.c_int * M)()
    vals = (C.c_float * M)()
    for _ in range(3):    # first call records the graph, the others replay it
        assert L.cccc_host_decode_step(d, x.ctypes.data, M, ids, vals) == 0
    assert L.cccc_host_decode_launches(d) == layers * 4 + 2

    # the same chain by hand through the C-ABI (q -> o -> gate -> down per layer, then lm_head)
    def lin(name, src, alpha):
        W, blk, inv, N, K = host[name]
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        assert c.gemm_wq_bf16(wt, to_dev(W), to_dev(blk) if blk is not None else None, inv, src, out, N, M, K, alpha=alpha) == 0
        return out

    cur = to_dev(x).view(torch.bfloat16).view(M, hidden)
    for i in range(layers):
        q = lin(f"W_q_{i}", cur, alphas[0])
        o = lin(f"W_o_{i}", q, alphas[0])
        gate = lin(f"W_gate_{i}", o, alphas[1])
        cur = lin(f"W_down_{i}", gate, alphas[2])
    logits = lin("W_lm_head", cur, alphas[3])
    assert c.check_error("chain") == 0
    want = torch.argmax(logits.float(), dim=1).cpu().tolist()
    got = list(ids)
    top = logits.float().max(dim=1).values.cpu().numpy()
    # the driver's grouped launches and the hand-issued ones run the same kernels on the same data
    assert got == want, (got, want)
    assert np.allclose(np.array(list(vals)), top, rtol=1e-2)
    # the device buffer of the logits is reachable for the hooks of a full decode step
    lp = L.cccc_host_decode_buffer(d, b"logits")
    assert lp
    L.cccc_host_decode_destroy(d)
    L.cccc_host_bin_close(f)
    L.cccc_host_gpu_destroy(g)
