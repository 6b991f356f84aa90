"""A whole decode step (embedding, layers of RMSNorm / q+k+v / attention / o + residual / RMSNorm /
gate+up / SwiGLU / down + residual, final norm, lm_head, arg-max) issued through the C-ABI by
cccc_lite_b200.decode_model.DecodeModel, against the same step composed from the CPU oracle's
restatements of the reference's ops (the op sequence of scripts/convert_weights.py:488-584, 688).

Several tokens are decoded in a row, so the KV cache the later ones read is the one the earlier ones
wrote.  Bar: the logits against the oracle's unrounded logits with tests/_util.py:assert_close_rows
(every op in the chain was checked on its own at its own bar; what is left here is the rare last-place
flip of an intermediate BF16 tensor and what the later layers make of it), the caches within one BF16
unit in the last place, and the chosen token equal whenever the oracle's best logit leads by more than
the tolerance."""
import importlib

import numpy as np
import pytest

from oracle import oracle as O
from tests._util import assert_close_rows, capi, from_dev_u16, to_dev

pytestmark = pytest.mark.gpu


def make_model(wt, cfg, seed):
    rng = np.random.default_rng(seed)

    def lin(N, K):
        W, blk, inv, _ = O.make_inputs(wt, N, K, 1, seed=int(rng.integers(1 << 30)), scaled=True, w_std=1.0 / np.sqrt(K))
        return W, blk, inv

    def norm(n):
        return O.f32_to_bf16_bits((1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32))

    layers = []
    for _ in range(cfg.layers):
        layers.append(dict(q=lin(cfg.q_dim, cfg.hidden), k=lin(cfg.kv_dim, cfg.hidden), v=lin(cfg.kv_dim, cfg.hidden),
                           o=lin(cfg.hidden, cfg.q_dim), gate=lin(cfg.ffn, cfg.hidden), up=lin(cfg.ffn, cfg.hidden),
                           down=lin(cfg.hidden, cfg.ffn), attn_norm=norm(cfg.hidden), ffn_norm=norm(cfg.hidden),
                           q_norm=norm(cfg.head_dim) if cfg.qk_norm else None, k_norm=norm(cfg.head_dim) if cfg.qk_norm else None))
    emb = O.f32_to_bf16_bits(rng.standard_normal((cfg.vocab, cfg.hidden)).astype(np.float32))
    return dict(layers=layers, emb=emb, final_norm=norm(cfg.hidden), lm_head=lin(cfg.vocab, cfg.hidden))


def oracle_linear(wt, L, X, N, M, K):
    W, blk, inv = L
    Y, y32 = O.linear_wq_bf16(wt, W, blk, inv, X, N, M, K)
    return Y.reshape(M, N), y32


def oracle_step(wt, cfg, w, ids, pos, Kc, Vc, cos, sin):
    """One step for M sequences; Kc / Vc: per layer [M, Hkv, T, hd] uint16, updated in place."""
    M = ids.size
    x = O.embed_bf16(ids, w["emb"])
    for i, L in enumerate(w["layers"]):
        xn = O.rms_norm_bf16(x, L["attn_norm"], cfg.eps)
        q, _ = oracle_linear(wt, L["q"], xn, cfg.q_dim, M, cfg.hidden)
        k, _ = oracle_linear(wt, L["k"], xn, cfg.kv_dim, M, cfg.hidden)
        v, _ = oracle_linear(wt, L["v"], xn, cfg.kv_dim, M, cfg.hidden)
        Qr = np.empty((M, cfg.n_heads, cfg.head_dim), np.uint16)
        for b in range(M):
            qh, kh = q[b].reshape(cfg.n_heads, cfg.head_dim), k[b].reshape(cfg.n_kv_heads, cfg.head_dim)
            if cfg.qk_norm:
                qh, kh = O.rms_norm_bf16(qh, L["q_norm"], cfg.eps), O.rms_norm_bf16(kh, L["k_norm"], cfg.eps)
            Qr[b] = O.rope_bf16(qh.reshape(cfg.n_heads, 1, -1), cos, sin, int(pos[b])).reshape(cfg.n_heads, -1)
            kr = O.rope_bf16(kh.reshape(cfg.n_kv_heads, 1, -1), cos, sin, int(pos[b])).reshape(cfg.n_kv_heads, -1)
            O.kv_append_bf16(kr, Kc[i][b], int(pos[b]))
            O.kv_append_bf16(v[b].reshape(cfg.n_kv_heads, -1), Vc[i][b], int(pos[b]))
        att, _ = O.attention_decode_bf16(Qr, Kc[i], Vc[i], pos)
        o, _ = oracle_linear(wt, L["o"], att.reshape(M, cfg.q_dim), cfg.hidden, M, cfg.q_dim)
        x = O.add_bf16(x, o)
        xn = O.rms_norm_bf16(x, L["ffn_norm"], cfg.eps)
        g, _ = oracle_linear(wt, L["gate"], xn, cfg.ffn, M, cfg.hidden)
        u, _ = oracle_linear(wt, L["up"], xn, cfg.ffn, M, cfg.hidden)
        h = O.mul_bf16(O.silu_bf16(g), u)
        d, _ = oracle_linear(wt, L["down"], h, cfg.hidden, M, cfg.ffn)
        x = O.add_bf16(x, d)
    xn = O.rms_norm_bf16(x, w["final_norm"], cfg.eps)
    _, logits32 = oracle_linear(wt, w["lm_head"], xn, cfg.vocab, M, cfg.hidden)
    return logits32


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
@pytest.mark.parametrize("M,qk_norm", [(1, True), (3, False)])
def test_decode_steps_match_the_oracle_chain(wt, M, qk_norm):
    import torch

    c = capi()
    dm = importlib.import_module("cccc_lite_b200.decode_model")
    cfg = dm.ModelConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=2, rope_theta=1e4,
                         qk_norm=qk_norm)
    T = 64
    w = make_model(wt, cfg, seed=wt * 10 + M)
    cos, sin = O.rope_tables_bf16(T, cfg.head_dim, cfg.rope_theta)

    def dev_lin(L):
        W, blk, inv = L
        return to_dev(W), (to_dev(blk) if blk is not None else None), inv

    dw = dict(emb=to_dev(w["emb"]), final_norm=to_dev(w["final_norm"]), lm_head=dev_lin(w["lm_head"]), layers=[])
    for L in w["layers"]:
        d = {k: dev_lin(L[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")}
        d.update({k: (to_dev(L[k]) if L[k] is not None else None) for k in ("attn_norm", "ffn_norm", "q_norm", "k_norm")})
        dw["layers"].append(d)
    model = dm.DecodeModel(c, torch, cfg, wt, dw, to_dev(cos), to_dev(sin), M, T, torch.device("cuda"))

    rng = np.random.default_rng(M)
    Kc = [np.zeros((M, cfg.n_kv_heads, T, cfg.head_dim), np.uint16) for _ in range(cfg.layers)]
    Vc = [np.zeros((M, cfg.n_kv_heads, T, cfg.head_dim), np.uint16) for _ in range(cfg.layers)]
    pos = np.arange(M, dtype=np.int32) * 0            # every sequence starts empty
    ids = rng.integers(0, cfg.vocab, M).astype(np.int32)
    for step in range(5):
        want = oracle_step(wt, cfg, w, ids, pos, Kc, Vc, cos, sin)
        model.ids.copy_(torch.from_numpy(ids))
        model.pos.copy_(torch.from_numpy(pos))
        n = model.step(M)
        assert n == 8 * cfg.layers + 4 and c.check_error("step") == 0
        got = model.logits[:M].float().cpu().numpy()
        assert_close_rows(got, want, ("logits", wt, M, step))
        best = model.ids[:M].cpu().numpy()
        for b in range(M):
            order = np.argsort(want[b])
            margin = want[b, order[-1]] - want[b, order[-2]]
            if margin > 2e-2 * np.sqrt(np.mean(want[b] ** 2)):
                assert best[b] == order[-1], (step, b)
        for i in range(cfg.layers):
            gk = from_dev_u16(model.k_cache[i].view(torch.int16)).reshape(Kc[i].shape)
            gv = from_dev_u16(model.v_cache[i].view(torch.int16)).reshape(Vc[i].shape)
            kd = np.abs(O.bf16_bits_to_f32(gk) - O.bf16_bits_to_f32(Kc[i]))
            vd = np.abs(O.bf16_bits_to_f32(gv) - O.bf16_bits_to_f32(Vc[i]))
            assert kd.max() <= 0.05 and vd.max() <= 0.05, (step, i, float(kd.max()), float(vd.max()))
        # next token: the oracle's choice, so both sides keep decoding the same sequence
        ids = np.argmax(want, axis=1).astype(np.int32)
        pos = pos + 1


def test_step_launch_count_and_graph_replay():
    """The step is capturable: a CUDA graph of it replays to the same logits."""
    import torch

    c = capi()
    dm = importlib.import_module("cccc_lite_b200.decode_model")
    cfg = dm.ModelConfig(hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024, vocab=2048, layers=2, rope_theta=1e4)
    wt = O.FP8_E5M2
    w = make_model(wt, cfg, seed=3)
    cos, sin = O.rope_tables_bf16(32, cfg.head_dim, cfg.rope_theta)

    def dev_lin(L):
        W, blk, inv = L
        return to_dev(W), (to_dev(blk) if blk is not None else None), inv

    dw = dict(emb=to_dev(w["emb"]), final_norm=to_dev(w["final_norm"]), lm_head=dev_lin(w["lm_head"]), layers=[])
    for L in w["layers"]:
        d = {k: dev_lin(L[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")}
        d.update({k: to_dev(L[k]) for k in ("attn_norm", "ffn_norm", "q_norm", "k_norm")})
        dw["layers"].append(d)
    model = dm.DecodeModel(c, torch, cfg, wt, dw, to_dev(cos), to_dev(sin), 2, 32, torch.device("cuda"))
    start = torch.tensor([5, 9], dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        model.ids.copy_(start)
        model.pos.fill_(3)
        model.step(2)
        stream.synchronize()
        eager = model.logits.clone()
        g = torch.cuda.CUDAGraph()
        model.ids.copy_(start)
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            model.step(2)
        model.ids.copy_(start)
        g.replay()
        stream.synchronize()
    assert c.check_error("graph") == 0
    assert torch.equal(eager, model.logits)
