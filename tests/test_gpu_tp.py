"""Tensor-parallel linears on 2, 4 and 8 GPUs (NCCL for the plumbing): each rank runs its shard through
the C-ABI, shards are combined with all-gather / all-reduce, and the result must equal the unsharded
(CPU oracle) result within the stated tolerance (max relative error 1e-2, cosine >= 0.9999).  The
fused linear + all-reduce must give the bits of the two separate calls, also when calls of different
shapes follow each other on one exchange area with nothing in between.  Each world size needs that
many GPUs and is skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest

from __graft_entry__ import ROOT

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import importlib

        from __graft_entry__ import load_package
        from oracle import oracle as O
        from tests._util import rel_cos

        capi = load_package().capi
        T = importlib.import_module("cccc_lite_b200.tp")
        results = []
        for wt in (O.FP8_E5M2, O.FP4_E2M1):
            for kind, N, K in (("col", 1024, 4096), ("row", 4096, 2048), ("col", 4096, 1024)):
                for M in (1, 8):
                    W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=N + K + M, scaled=True)
                    s = T.make_shard(kind, N, K, world, rank, wt)
                    Ws, bs = T.slice_weight(W, blk, s, N, K, wt)
                    Xs = T.slice_activation(X.reshape(M, K), s)
                    dW = torch.from_numpy(Ws).cuda()
                    dB = torch.from_numpy(bs).cuda() if bs is not None else None
                    dX = torch.from_numpy(Xs.view(np.int16)).cuda()
                    # row-parallel shards hand FP32 partial sums to the all-reduce (rounded to BF16 once, after)
                    f32 = kind == "row"
                    part = torch.zeros(M, s.N, dtype=torch.float32 if f32 else torch.bfloat16, device="cuda")
                    assert capi.gemm_wq_bf16(wt, dW, dB, inv, dX, part, s.N, M, s.K, flags=capi.FLAG_OUT_F32 if f32 else 0) == 0
                    assert capi.check_error("tp") == 0
                    full = T.combine(kind, part, dist, world).to(torch.bfloat16)
                    _, ref = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
                    rel, cos = rel_cos(full.float().cpu().numpy(), ref)
                    results.append((wt, kind, N, K, M, rel <= 1e-2 and cos >= 0.9999 and tuple(full.shape) == (M, N), rel, cos))
        # the one-shot push all-reduce against NCCL's sum, several calls in a row (both buffer sets)
        n_max = 8 * 4096
        ar = capi.PushAllReduce(dist, dist.group.WORLD, rank, world, n_max, torch.device("cuda", rank))
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        for call, n in enumerate((4096, 8 * 4096, 4096, 1024, 4096)):
            part = torch.randn(n, device="cuda", generator=g, dtype=torch.float32)
            want = part.clone()
            dist.all_reduce(want)
            out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
            assert ar(part, out, n) == 0 and capi.check_error("push") == 0
            results.append(("push", call, n, 0, 0, bool(torch.equal(out, want.to(torch.bfloat16))), 0.0, 1.0))
        # the row-parallel linear with the all-reduce inside the kernel: bit-identical to the two
        # separate calls, several calls in a row (both buffer sets, whole-row-block and split-k schedules)
        fused = capi.FusedRowLinear(dist, dist.group.WORLD, rank, world, n_max, torch.device("cuda", rank))
        for wt in (O.FP8_E5M2, O.FP4_E2M1):
            for N, K, M in ((4096, 4096, 1), (4096, 12288, 8), (256, 16384, 4), (1000, 2048, 20), (4096, 4096, 1)):
                W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=3 * N + K + M, scaled=True)
                s = T.make_shard("row", N, K, world, rank, wt)
                Ws, bs = T.slice_weight(W, blk, s, N, K, wt)
                Xs = T.slice_activation(X.reshape(M, K), s)
                dW = torch.from_numpy(Ws).cuda()
                dB = torch.from_numpy(bs).cuda() if bs is not None else None
                dX = torch.from_numpy(Xs.view(np.int16)).cuda()
                part = torch.zeros(M * N, dtype=torch.float32, device="cuda")
                two = torch.zeros(M * N, dtype=torch.bfloat16, device="cuda")
                assert capi.gemm_wq_bf16(wt, dW, dB, inv, dX, part, N, M, s.K, flags=capi.FLAG_OUT_F32 | capi.FLAG_NO_STREAM) == 0
                assert ar(part, two, M * N) == 0 and capi.check_error("two") == 0
                one = torch.full((M * N,), float("nan"), dtype=torch.bfloat16, device="cuda")
                rc = fused(wt, dW, dB, inv, dX, one, N, M, s.K)
                ok = rc == 0 and capi.check_error("fused") == 0 and bool(torch.equal(one.view(torch.int16), two.view(torch.int16)))
                _, ref = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
                rel, cos = rel_cos(one.float().cpu().numpy().reshape(M, N), ref)
                results.append(("fused", wt, N, K, M, ok and rel <= 1e-2 and cos >= 0.9999, rel, cos))
        # calls of different shapes back to back on ONE exchange area, no host synchronisation and no
        # other collective in between: row-block counts and tile heights change from call to call
        # (4096 features in 32-row blocks, 256 in 32-row blocks, 20 tokens in 64-row blocks), which
        # is what the per-area call counter exists for.  Expected bits come from the two-kernel form.
        wt = O.FP8_E5M2
        mixed = [(4096, 4096, 1), (256, 4096, 4), (4096, 4096, 1), (1000, 2048, 20), (4096, 4096, 1), (256, 4096, 4),
                 (512, 4096, 32)]
        prepared = []
        for N, K, M in mixed:
            W, blk, inv, X = O.make_inputs(wt, N, K, M, seed=5 * N + K + M, scaled=True)
            s = T.make_shard("row", N, K, world, rank, wt)
            Ws, bs = T.slice_weight(W, blk, s, N, K, wt)
            Xs = T.slice_activation(X.reshape(M, K), s)
            dW = torch.from_numpy(Ws).cuda()
            dX = torch.from_numpy(Xs.view(np.int16)).cuda()
            part = torch.zeros(M * N, dtype=torch.float32, device="cuda")
            two = torch.zeros(M * N, dtype=torch.bfloat16, device="cuda")
            assert capi.gemm_wq_bf16(wt, dW, None, inv, dX, part, N, M, s.K, flags=capi.FLAG_OUT_F32 | capi.FLAG_NO_STREAM) == 0
            assert ar(part, two, M * N) == 0 and capi.check_error("two") == 0
            prepared.append((dW, dX, inv, N, M, s.K, two))
        for rep in range(3):    # an odd number of calls per pass: every pass starts on the other slot set
            outs = []
            for dW, dX, inv, N, M, Ks, two in prepared:
                one = torch.full((M * N,), float("nan"), dtype=torch.bfloat16, device="cuda")
                assert fused(wt, dW, None, inv, dX, one, N, M, Ks, flags=capi.FLAG_PDL) == 0
                outs.append(one)
            ok = capi.check_error("mixed") == 0
            for (dW, dX, inv, N, M, Ks, two), one in zip(prepared, outs):
                results.append(("fused-mixed", rep, N, Ks, M, ok and bool(torch.equal(one.view(torch.int16), two.view(torch.int16))),
                                0.0, 1.0))
        # ---- the whole decode step, tensor parallel, against the unsharded oracle chain ----
        dm = importlib.import_module("cccc_lite_b200.decode_model")
        from tests.test_gpu_decode_model import make_model, oracle_step

        cfg = dm.ModelConfig(hidden=1024, n_heads=16, n_kv_heads=8, head_dim=128, ffn=2048, vocab=4096, layers=2, rope_theta=1e4)
        Tctx = 32
        # two sequences (fused exchange inside the decode kernel), and twelve (from 9 tokens on the row-parallel linears
        # are the streaming kernel with FP32 output followed by the push all-reduce)
        for wt, Mb in ((O.FP8_E5M2, 2), (O.FP4_E2M1, 2), (O.FP8_E5M2, 12)):
            w = make_model(wt, cfg, seed=11 + wt)
            cos, sin = O.rope_tables_bf16(Tctx, cfg.head_dim, cfg.rope_theta)

            def shard_lin(L3, kind, N, K):
                W, blk, inv = L3
                s = T.make_shard(kind, N, K, world, rank, wt)
                Ws, bs = T.slice_weight(W, blk, s, N, K, wt)
                return torch.from_numpy(Ws).cuda(), (torch.from_numpy(bs).cuda() if bs is not None else None), inv

            def dev16(a):
                return torch.from_numpy(a.view(np.int16)).cuda()

            dw = dict(emb=dev16(w["emb"]), final_norm=dev16(w["final_norm"]), lm_head=shard_lin(w["lm_head"], "col", cfg.vocab, cfg.hidden),
                      layers=[])
            for L in w["layers"]:
                d = dict(q=shard_lin(L["q"], "col", cfg.q_dim, cfg.hidden), k=shard_lin(L["k"], "col", cfg.kv_dim, cfg.hidden),
                         v=shard_lin(L["v"], "col", cfg.kv_dim, cfg.hidden), o=shard_lin(L["o"], "row", cfg.hidden, cfg.q_dim),
                         gate=shard_lin(L["gate"], "col", cfg.ffn, cfg.hidden), up=shard_lin(L["up"], "col", cfg.ffn, cfg.hidden),
                         down=shard_lin(L["down"], "row", cfg.hidden, cfg.ffn))
                d.update({k: dev16(L[k]) for k in ("attn_norm", "ffn_norm", "q_norm", "k_norm")})
                dw["layers"].append(d)
            model = dm.DecodeModel(capi, torch, cfg, wt, dw, dev16(cos), dev16(sin), Mb, Tctx, torch.device("cuda", rank), world=world,
                                   rank=rank, fused_row_linear=fused, dist=dist)
            Kc = [np.zeros((Mb, cfg.n_kv_heads, Tctx, cfg.head_dim), np.uint16) for _ in range(cfg.layers)]
            Vc = [np.zeros((Mb, cfg.n_kv_heads, Tctx, cfg.head_dim), np.uint16) for _ in range(cfg.layers)]
            pos = np.zeros(Mb, np.int32)
            ids = ((np.arange(Mb) * 997 + 3) % cfg.vocab).astype(np.int32)
            for step in range(3):
                want = oracle_step(wt, cfg, w, ids, pos, Kc, Vc, cos, sin)
                model.ids.copy_(torch.from_numpy(ids))
                model.pos.copy_(torch.from_numpy(pos))
                model.step(Mb)
                ok = capi.check_error("tp step") == 0
                parts = [torch.empty_like(model.logits) for _ in range(world)]
                dist.all_gather(parts, model.logits)
                got = torch.cat(parts, dim=1)[:Mb].float().cpu().numpy()
                rms = np.sqrt(np.mean(want.astype(np.float64) ** 2, axis=1, keepdims=True))
                rel = float(np.max(np.abs(got - want) / np.maximum(np.abs(want), rms)))
                _, cos_sim = rel_cos(got, want)
                best = model.ids[:Mb].cpu().numpy()
                same_choice = all(best[b] == int(np.argmax(got[b])) for b in range(Mb))
                results.append(("tp-decode-step", wt, step, 0, Mb, ok and rel <= 3e-2 and cos_sim >= 0.9999 and same_choice, rel, cos_sim))
                ids = np.argmax(want, axis=1).astype(np.int32)
                pos = pos + 1
        # a shape the fused kernel does not take is refused, not mangled
        results.append(("fused-refuses", 0, 0, 0, 0, fused(O.FP8_E5M2, dW, dB, inv, dX, one, 64, 40, 64) == -1, 0.0, 1.0))
        q.put((rank, results))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shards_match_unsharded(world):
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, results in out:
        bad = [r for r in results if not r[5]]
        assert not bad, (rank, bad)
