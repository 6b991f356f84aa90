"""The decode step and the generation loop driven from C++ (csrc/host/decode_step.cpp, generate.cpp): weights from
a container file as scripts/convert_weights.py names them, every launch issued by cccc::DecodeStep, tokens chosen
by cccc::Generator.  Checked against the Python-issued step (cccc_lite_b200.decode_model.DecodeModel, itself held
to the CPU oracle in tests/test_gpu_decode_model.py): the two issue the same launches on the same bytes, so logits
and tokens must agree bit for bit.

Tensor parallel runs inside ONE process here (a host thread and a GpuControl per device, peer access between the
devices); its logits are held to the one-GPU step at the whole-step bar of tests/test_gpu_decode_model.py."""
import importlib
import struct

import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle as O
from tests._util import assert_close_rows, capi, to_dev
from tests.test_gpu_decode_model import STEP_TOL, make_model
from tests.test_loader_cpu import write_container

pytestmark = pytest.mark.gpu

SUFFIX = {O.FP8_E5M2: "fp8_e5m2", O.FP8_E4M3: "fp8_e4m3", O.FP4_E2M1: "fp4_e2m1"}
T = 64


def small_cfg(qk_norm=True, layers=2, hidden=512, heads=4, kv=2, ffn=1024, vocab=2048):
    dm = importlib.import_module("cccc_lite_b200.decode_model")
    return dm.ModelConfig(hidden=hidden, n_heads=heads, n_kv_heads=kv, head_dim=128, ffn=ffn, vocab=vocab, layers=layers, rope_theta=1e4,
                          qk_norm=qk_norm)


def container_entries(wt, cfg, w):
    """The model under the converter's names (scripts/convert_weights.py:145-166, 200)."""
    e = {}

    def lin(name, L):
        W, blk, inv = L
        e[f"weight_{SUFFIX[wt]}_{name}"] = W.tobytes()
        if wt == O.FP4_E2M1:
            e[f"blockscale_{name}"] = blk.tobytes()
        else:
            e[f"scale_{name}"] = struct.pack("<f", inv)

    for i, L in enumerate(w["layers"]):
        for k in ("q", "k", "v", "o", "gate", "up", "down"):
            lin(f"W_{k}_{i}", L[k])
        e[f"weight_bf16_W_rms_attn_{i}"] = L["attn_norm"].tobytes()
        e[f"weight_bf16_W_rms_ffn_{i}"] = L["ffn_norm"].tobytes()
        if cfg.qk_norm:
            e[f"weight_bf16_W_qnorm_{i}"] = L["q_norm"].tobytes()
            e[f"weight_bf16_W_knorm_{i}"] = L["k_norm"].tobytes()
    lin("W_lm_head", w["lm_head"])
    e["weight_bf16_W_emb"] = w["emb"].tobytes()
    e["weight_bf16_W_rms_final"] = w["final_norm"].tobytes()
    return e


def python_model(wt, cfg, w, M):
    import torch

    c = capi()
    dm = importlib.import_module("cccc_lite_b200.decode_model")
    cos, sin = O.rope_tables_bf16(T, cfg.head_dim, cfg.rope_theta)

    def dev_lin(L):
        W, blk, inv = L
        return to_dev(W), (to_dev(blk) if blk is not None else None), inv

    dw = dict(emb=to_dev(w["emb"]), final_norm=to_dev(w["final_norm"]), lm_head=dev_lin(w["lm_head"]), layers=[])
    for L in w["layers"]:
        d = {k: dev_lin(L[k]) for k in ("q", "k", "v", "o", "gate", "up", "down")}
        d.update({k: (to_dev(L[k]) if L[k] is not None else None) for k in ("attn_norm", "ffn_norm", "q_norm", "k_norm")})
        dw["layers"].append(d)
    return dm.DecodeModel(c, torch, cfg, wt, dw, to_dev(cos), to_dev(sin), M, T, torch.device("cuda"))


@pytest.fixture(scope="module")
def host():
    h = load_package().hostapi
    L = h.lib()
    g = L.cccc_host_gpu_create(0)
    assert g
    yield h, L, g
    L.cccc_host_gpu_destroy(g)


@pytest.mark.parametrize("wt", [O.FP8_E5M2, O.FP4_E2M1])
@pytest.mark.parametrize("M,qk_norm", [(1, True), (3, False)])
def test_cpp_step_is_the_python_issued_step(host, tmp_path, wt, M, qk_norm):
    import torch

    h, L, g = host
    cfg = small_cfg(qk_norm)
    w = make_model(wt, cfg, seed=wt * 7 + M)
    path = str(tmp_path / "model.bin")
    write_container(path, container_entries(wt, cfg, w))
    f = L.cccc_host_bin_open(path.encode())
    step = h.HostDecodeStep(g, f, cfg, T, max_batch=M)
    assert step.info(0) == 8 * cfg.layers + 4 and step.info(3) == wt and step.info(2) == 0
    model = python_model(wt, cfg, w, M)
    rng = np.random.default_rng(M)
    ids = [int(v) for v in rng.integers(0, cfg.vocab, M)]
    for s in range(6):
        pos = [s] * M
        model.ids.copy_(torch.tensor(ids, dtype=torch.int32))
        model.pos.copy_(torch.tensor(pos, dtype=torch.int32))
        model.step(M)
        torch.cuda.synchronize()
        want_logits = model.logits[:M].view(torch.int16).cpu().numpy().view(np.uint16)
        want_ids = model.ids[:M].cpu().tolist()
        nxt, best, logits = step.step(ids, pos, want_logits=True)
        assert np.array_equal(logits, want_logits), s
        assert nxt == want_ids
        assert best == [float(v) for v in model.best[:M].cpu()]
        ids = nxt
    # a reset cache gives the first step's result again
    step.reset()
    first = step.step([5] * M, [0] * M, want_logits=True)
    step.reset()
    again = step.step([5] * M, [0] * M, want_logits=True)
    assert first[0] == again[0] and np.array_equal(first[2], again[2])
    step.close()
    L.cccc_host_bin_close(f)


@pytest.mark.parametrize("target", [O.FP8_E5M2, O.FP8_E4M3, O.FP4_E2M1])
def test_unquantised_checkpoints_are_quantised_on_load_and_saved_as_a_cache(host, tmp_path, target):
    """BF16 / float tensors + weight_data_type (cccc/Net.cpp:1142-1233): the loaded model is the one the oracle's
    quantiser gives, and the cache file it writes loads to the same model without quantising again."""
    h, L, g = host
    cfg = small_cfg(True, layers=1)
    rng = np.random.default_rng(target)
    names = [(f"W_{k}_0", n, kk) for k, n, kk in (("q", cfg.q_dim, cfg.hidden), ("k", cfg.kv_dim, cfg.hidden), ("v", cfg.kv_dim, cfg.hidden),
                                                   ("o", cfg.hidden, cfg.q_dim), ("gate", cfg.ffn, cfg.hidden), ("up", cfg.ffn, cfg.hidden),
                                                   ("down", cfg.hidden, cfg.ffn))] + [("W_lm_head", cfg.vocab, cfg.hidden)]
    raw, pre = {}, {}
    for j, (name, N, K) in enumerate(names):
        wf = (rng.standard_normal(N * K) / np.sqrt(K)).astype(np.float32)
        bits = O.f32_to_bf16_bits(wf)
        wf = O.bf16_bits_to_f32(bits)                     # the checkpoint's values
        if j % 2:
            raw[f"weight_float_{name}"] = wf.tobytes()      # a float checkpoint holding BF16-exact values
        else:
            raw[f"weight_bf16_{name}"] = bits.tobytes()
        if target == O.FP4_E2M1:
            nib, sc = O.float_to_fp4_blockscale(wf, 16)
            pre[f"weight_{SUFFIX[target]}_{name}"] = nib.tobytes()
            pre[f"blockscale_{name}"] = sc.tobytes()
        else:
            maxval = np.float32(448.0 if target == O.FP8_E4M3 else 57344.0)
            absmax = np.float32(np.abs(wf).max())
            pre[f"weight_{SUFFIX[target]}_{name}"] = O.float_to_fp8(wf, target, float(maxval / absmax)).tobytes()
            pre[f"scale_{name}"] = struct.pack("<f", float(absmax / maxval))
    norm = lambda n: O.f32_to_bf16_bits((1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)).tobytes()
    common = {"weight_bf16_W_rms_attn_0": norm(cfg.hidden), "weight_bf16_W_rms_ffn_0": norm(cfg.hidden), "weight_bf16_W_qnorm_0": norm(128),
              "weight_bf16_W_knorm_0": norm(128), "weight_bf16_W_rms_final": norm(cfg.hidden),
              "weight_bf16_W_emb": O.f32_to_bf16_bits(rng.standard_normal(cfg.vocab * cfg.hidden).astype(np.float32)).tobytes()}
    p_raw, p_pre, p_cache = (str(tmp_path / n) for n in ("raw.bin", "pre.bin", "cache.bin"))
    write_container(p_raw, {**raw, **common})
    write_container(p_pre, {**pre, **common})

    def run(path, **kw):
        f = L.cccc_host_bin_open(path.encode())
        step = h.HostDecodeStep(g, f, cfg, T, **kw)
        out, ids = [], [3]
        for s in range(4):
            nxt, best, logits = step.step(ids, [s], want_logits=True)
            out.append((nxt, logits.copy()))
            ids = nxt
        return step, f, out

    s_raw, f_raw, got = run(p_raw, weight_data_type=target, keep_host=True)
    assert s_raw.info(2) == 8 and s_raw.info(3) == target
    s_pre, f_pre, want = run(p_pre)
    assert s_pre.info(2) == 0
    for (a, la), (b, lb) in zip(got, want):
        assert a == b and np.array_equal(la, lb)
    s_raw.save(p_cache)
    s_cache, f_cache, again = run(p_cache)
    assert s_cache.info(2) == 0
    for (a, la), (b, lb) in zip(again, want):
        assert a == b and np.array_equal(la, lb)
    # the cache file holds the reference's named-weight keys
    for name, _, _ in names:
        assert L.cccc_host_bin_has(f_cache, f"weight_{SUFFIX[target]}_{name}".encode())
        assert L.cccc_host_bin_has(f_cache, (f"blockscale_{name}" if target == O.FP4_E2M1 else f"scale_{name}").encode())
    # without a target type an unquantised checkpoint is refused, loudly
    f2 = L.cccc_host_bin_open(p_raw.encode())
    with pytest.raises(RuntimeError, match="not quantised"):
        h.HostDecodeStep(g, f2, cfg, T)
    L.cccc_host_bin_close(f2)
    for s, f in ((s_raw, f_raw), (s_pre, f_pre), (s_cache, f_cache)):
        s.close()
        L.cccc_host_bin_close(f)


def test_generate_runs_the_reference_loop_over_the_step(host, tmp_path):
    """Generator over DecodeStep: greedy tokens are those of stepping by hand; a small cache forces a rebuild; a
    sampling run asks for the logits and stays inside top-k."""
    h, L, g = host
    wt = O.FP8_E5M2
    cfg = small_cfg(True)
    w = make_model(wt, cfg, seed=99)
    path = str(tmp_path / "model.bin")
    write_container(path, container_entries(wt, cfg, w))
    f = L.cccc_host_bin_open(path.encode())
    step = h.HostDecodeStep(g, f, cfg, T)
    prompt = [11, 12, 13, 14, 15]
    # by hand: prompt rows 0-4, then feed each chosen token at the next row
    nxt = None
    for i, t in enumerate(prompt):
        nxt, _, _ = step.step([t], [i])
    by_hand, pos = [], len(prompt)
    for _ in range(10):
        by_hand.append(nxt[0])
        nxt, _, _ = step.step([nxt[0]], [pos])
        pos += 1
    got, stats = step.generate(prompt, 10, T=32, T_kv=T)
    assert got == by_hand and stats == dict(rebuilds=0, decode_steps=10, prefill_tokens=5)
    # EOS stops the loop and is not emitted
    got_eos, _ = step.generate(prompt, 10, eos_ids=[by_hand[4]], T=32, T_kv=T)
    assert got_eos == by_hand[:by_hand.index(by_hand[4])]
    # a cache of 12 rows fills up: the loop rebuilds it from [system | turn | tail] and carries on
    got_small, stats_small = step.generate(prompt, 20, sys_n=2, turn_n=2, T=8, T_kv=12)
    assert stats_small["rebuilds"] >= 1 and got_small[:7] == by_hand[:7]
    # sampling: the same seed gives the same tokens, another seed others
    a, _ = step.generate(prompt, 12, seed=3, sampler=dict(temperature=1.0, top_k=20), T=32, T_kv=T)
    b, _ = step.generate(prompt, 12, seed=3, sampler=dict(temperature=1.0, top_k=20), T=32, T_kv=T)
    c, _ = step.generate(prompt, 12, seed=4, sampler=dict(temperature=1.0, top_k=20), T=32, T_kv=T)
    assert a == b and a != c and a != by_hand[:12]
    step.close()
    L.cccc_host_bin_close(f)


def test_decode_program_behind_the_cpp_step(host, tmp_path):
    """useProgram: the same tokens from one persistent kernel per step (3 launches) as from 8 launches per layer."""
    h, L, g = host
    wt = O.FP8_E5M2
    cfg = small_cfg(True, layers=3, heads=8, kv=2)    # the program's attention takes 4 query heads per kv head
    w = make_model(wt, cfg, seed=5)
    path = str(tmp_path / "model.bin")
    write_container(path, container_entries(wt, cfg, w))
    f = L.cccc_host_bin_open(path.encode())
    step = h.HostDecodeStep(g, f, cfg, T)
    seq = [int(v) for v in np.random.default_rng(1).integers(0, cfg.vocab, 24)]
    ref = [step.step([t], [i], want_logits=True) for i, t in enumerate(seq)]
    assert step.info(1) == 8 * cfg.layers + 4
    step.reset()
    assert step.use_program(True)
    got = [step.step([t], [i], want_logits=True) for i, t in enumerate(seq)]
    assert step.info(1) == 3
    same = []
    for (n0, b0, l0), (n1, b1, l1) in zip(ref, got):
        a, b = O.bf16_bits_to_f32(l1), O.bf16_bits_to_f32(l0)
        assert_close_rows(a, b, "program vs launches", tol=STEP_TOL)
        same.append(float((l0 == l1).mean()))
    assert np.median(same) > 0.98
    step.close()
    L.cccc_host_bin_close(f)


def _devices():
    import torch

    return torch.cuda.device_count()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("wt,raw", [(O.FP8_E5M2, False), (O.FP4_E2M1, False), (O.FP8_E4M3, True)])
def test_tensor_parallel_in_one_process(host, tmp_path, world, wt, raw):
    """`world` host threads, one GpuControl each, peer access set up in C++ (no torch.distributed): the sharded step's
    logits against the one-GPU step's, the combined arg-max against the gathered logits, and the generation loop
    agreeing on every rank.  raw: float checkpoint quantised per shard while loading, with the tensor's absmax
    combined across the ranks, against the same checkpoint quantised whole on one GPU."""
    if _devices() < world:
        pytest.skip(f"needs {world} GPUs")
    h, L, g = host
    cfg = small_cfg(True, layers=2, hidden=2048, heads=16, kv=8, ffn=4096, vocab=4096)   # K / world stays a multiple of 256 up to 8 ranks
    kw = {}
    if raw:
        rng = np.random.default_rng(12)
        e = {}
        for i in range(cfg.layers):
            for k, n, kk in (("q", cfg.q_dim, cfg.hidden), ("k", cfg.kv_dim, cfg.hidden), ("v", cfg.kv_dim, cfg.hidden), ("o", cfg.hidden, cfg.q_dim),
                             ("gate", cfg.ffn, cfg.hidden), ("up", cfg.ffn, cfg.hidden), ("down", cfg.hidden, cfg.ffn)):
                e[f"weight_float_W_{k}_{i}"] = (rng.standard_normal(n * kk) / np.sqrt(kk)).astype(np.float32).tobytes()
            for k, n in (("rms_attn", cfg.hidden), ("rms_ffn", cfg.hidden), ("qnorm", 128), ("knorm", 128)):
                e[f"weight_bf16_W_{k}_{i}"] = O.f32_to_bf16_bits((1.0 + 0.05 * rng.standard_normal(n)).astype(np.float32)).tobytes()
        e["weight_float_W_lm_head"] = (rng.standard_normal(cfg.vocab * cfg.hidden) / np.sqrt(cfg.hidden)).astype(np.float32).tobytes()
        e["weight_bf16_W_emb"] = O.f32_to_bf16_bits(rng.standard_normal(cfg.vocab * cfg.hidden).astype(np.float32)).tobytes()
        e["weight_bf16_W_rms_final"] = O.f32_to_bf16_bits(np.ones(cfg.hidden, np.float32)).tobytes()
        kw = dict(weight_data_type=wt)
    else:
        e = container_entries(wt, cfg, make_model(wt, cfg, seed=world))
    path = str(tmp_path / "model.bin")
    write_container(path, e)
    tokens = [int(v) for v in np.random.default_rng(world).integers(0, cfg.vocab, 6)]
    f = L.cccc_host_bin_open(path.encode())
    one = h.HostDecodeStep(g, f, cfg, T, **kw)
    want = [one.step([t], [i], want_logits=True) for i, t in enumerate(tokens)]
    nxt, best, logits = h.tp_steps(path, list(range(world)), cfg, T, tokens, **kw)
    for i, (n1, b1, l1) in enumerate(want):
        ref = O.bf16_bits_to_f32(l1)[0]
        assert_close_rows(logits[i:i + 1], ref[None, :], ("tp logits", world, i), tol=STEP_TOL)
        # every rank holds the same winner, which is the first maximum of the gathered row
        assert len(set(int(v) for v in nxt[:, i])) == 1
        assert int(nxt[0, i]) == int(np.argmax(logits[i])) and best[i] == logits[i].max()
    got, stats = h.tp_generate(path, list(range(world)), cfg, T, tokens, 8, T=32, T_kv=T, **kw)
    assert len(got) == 8 and stats["decode_steps"] == 8
    # sampling needs the whole row of logits on every rank: the ranks must still agree (tp_generate raises otherwise)
    got_s, _ = h.tp_generate(path, list(range(world)), cfg, T, tokens, 8, seed=2, sampler=dict(temperature=0.8, top_k=10), T=32, T_kv=T, **kw)
    assert len(got_s) == 8
    one.close()
    L.cccc_host_bin_close(f)
