"""Tensor-parallel shard logic on CPU: shard arithmetic, and two gloo ranks that each compute
their shard of a linear with the CPU oracle and combine the results (all-gather for column
shards, all-reduce for row shards); the combined result must equal the unsharded linear."""
import os
import socket
import sys

import numpy as np
import pytest

from __graft_entry__ import ROOT, load_package
from oracle import oracle as O


def tp():
    load_package()
    import importlib

    return importlib.import_module("cccc_lite_b200.tp")


def test_shard_arithmetic():
    T = tp()
    for wt in (O.FP8_E5M2, O.FP4_E2M1):
        per = 2 if wt == O.FP4_E2M1 else 1
        N, K = 1024, 4096
        for world in (1, 2, 4, 8):
            cover = np.zeros(N * K // per, np.int32)
            cover_r = np.zeros(N * K // per, np.int32)
            for r in range(world):
                c = T.column_shard(N, K, world, r)
                assert (c.N, c.K) == (N // world, K)
                rng = T.weight_byte_ranges(c, N, K, wt)
                assert len(rng) == 1 and rng[0] == (r * N // world * K // per, N // world * K // per)
                cover[rng[0][0]:rng[0][0] + rng[0][1]] += 1
                s = T.row_shard(N, K, world, r, wt)
                assert (s.N, s.K) == (N, K // world) and s.K % T.k_alignment(wt) == 0
                rr = T.weight_byte_ranges(s, N, K, wt)
                assert len(rr) == N
                for o, ln in rr:
                    cover_r[o:o + ln] += 1
                if wt == O.FP4_E2M1:
                    for (o, ln), (so, sl) in zip(rr, T.scale_byte_ranges(s, N, K)):
                        assert so * 8 == o and sl * 8 == ln  # 16 elements: 8 nibble bytes, 1 scale byte
            assert (cover == 1).all() and (cover_r == 1).all()
    # the shapes of the benchmark divide over 8 ranks; bad splits are refused
    for K in (4096, 12288, 14336):
        assert T.row_shard(4096, K, 8, 7, O.FP4_E2M1).k1 == K
    with pytest.raises(ValueError):
        T.row_shard(64, 4096 + 64, 8, 0, O.FP8_E5M2)
    with pytest.raises(ValueError):
        T.column_shard(1001, 64, 2, 0)


def _worker(rank, world, port, wt, kind, q):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T = tp()
        N, K, M = 96, 1024, 3
        W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=5, scaled=True)
        s = T.make_shard(kind, N, K, world, rank, wt)
        Ws, bs = T.slice_weight(W, blk, s, N, K, wt)
        Xs = T.slice_activation(X.reshape(M, K), s)
        _, y32 = O.linear_wq_bf16(wt, Ws, bs, inv, Xs, s.N, M, s.K)
        full = T.combine(kind, torch.from_numpy(y32.copy()), dist, world).numpy()
        _, ref = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
        ok = np.allclose(full, ref, rtol=1e-5, atol=1e-6) and full.shape == (M, N)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["col", "row"])
@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
def test_two_gloo_ranks_match_unsharded(wt, kind):
    import torch.multiprocessing as mp

    O.lib()  # build once, before forking workers
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, wt, kind, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_in_process_rank_combines(world):
    """cccc::TensorParallel (one host thread per rank, no device): every rank gets the largest logit's id with the
    lowest rank winning a tie and all-NaN shards (id -1) ignored, the largest absmax, and the gathered row of logits in
    rank order; the barrier is reused over many rounds."""
    import ctypes as C

    from __graft_entry__ import load_package
    from oracle import oracle as O

    L = load_package().hostapi.lib()
    per = 5
    rng = np.random.default_rng(world)
    ids = rng.integers(0, 1000, world).astype(np.int32)
    vals = rng.standard_normal(world).astype(np.float32)
    vals[world - 1] = vals.max() + 1.0            # the last rank wins ...
    vals[0] = vals[world - 1]                     # ... but rank 0 ties with it: the lowest rank takes it
    if world > 2:
        ids[1] = -1                               # a shard of only NaN never wins
        vals[1] = 1e30
    absmax = np.abs(rng.standard_normal(world)).astype(np.float32)
    shards = O.f32_to_bf16_bits(rng.standard_normal(world * per).astype(np.float32))
    out_ids = np.zeros(world, np.int32)
    out_best = np.zeros(world, np.float32)
    out_abs = np.zeros(world, np.float32)
    full = np.zeros((world, world * per), np.float32)
    p = lambda a, t: a.ctypes.data_as(C.POINTER(t))
    bad = L.cccc_host_tp_combine_selftest(world, 200, p(ids, C.c_int), p(vals, C.c_float), p(absmax, C.c_float), shards.ctypes.data, per,
                                          p(out_ids, C.c_int), p(out_best, C.c_float), p(out_abs, C.c_float), p(full, C.c_float))
    assert bad == 0
    assert np.all(out_ids == ids[0]) and np.all(out_best == vals[0])
    assert np.all(out_abs == absmax.max())
    want = O.bf16_bits_to_f32(shards)
    for r in range(world):
        assert np.array_equal(full[r], want)
