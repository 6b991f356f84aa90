"""The C++ sampler and generation loop (csrc/host/generate.cpp) against an independent Python restatement of
cccc-llm's sample_logits and run_generate (cccc-llm/cccc-llm.cpp:181-343, 347-577).  CPU only: the model is a
table of canned logits.

The multinomial draw is checked exactly: std::mt19937(seed) is numpy's RandomState(seed) generator (the same
init_genrand seeding), and libstdc++'s uniform_real_distribution<float> takes one 32-bit output, as
float32(raw) / 2^32, stepping down to the float below 1 when that rounds to 1."""
import numpy as np
import pytest

from __graft_entry__ import load_package


def H():
    return load_package().hostapi


def mt_uniform_float(seed):
    rs = np.random.RandomState(seed)
    st = rs.get_state()
    bg = np.random.MT19937()
    bg.state = {"bit_generator": "MT19937", "state": {"key": st[1], "pos": st[2]}}
    raw = int(bg.random_raw())
    r = np.float32(np.float32(raw) / np.float32(4294967296.0))
    return np.nextafter(np.float32(1), np.float32(0)) if r >= 1 else r


def py_sample(logits, ctx=(), seed=0, temperature=0.0, top_k=0, top_p=1.0, repetition_penalty=1.0, banned_ids=()):
    """sample_logits, op for op, in float32."""
    f = np.float32
    l = np.array(logits, dtype=np.float32)
    V = l.size
    for i in banned_ids:
        if 0 <= i < V:
            l[i] = f(-1e30)
    if repetition_penalty != 1.0 and len(ctx):
        for i in list(ctx)[-512:]:
            if 0 <= i < V:
                l[i] = l[i] / f(repetition_penalty) if l[i] > 0 else l[i] * f(repetition_penalty)
    if temperature <= 0:
        return int(np.argmax(l))
    l = (l / f(temperature)).astype(np.float32)
    if 0 < top_k < V:
        thr = np.sort(l)[::-1][top_k - 1]
        l[l < thr] = f(-1e30)
    e = np.exp((l - l.max()).astype(np.float32)).astype(np.float32)
    s = f(0)
    for v in e:
        s = f(s + v)
    p = (e / s).astype(np.float32) if s > 0 else e
    if top_p < 1.0:
        order = sorted(range(V), key=lambda i: (p[i], i), reverse=True)
        cum, cutting = f(0), False
        for i in order:
            if cutting:
                p[i] = 0
                continue
            cum = f(cum + p[i])
            if cum > f(top_p):
                cutting = True
        s = f(0)
        for v in p:
            s = f(s + v)
        if s > 0:
            p = (p / s).astype(np.float32)
    r = mt_uniform_float(seed)
    cum = f(0)
    for i in range(V):
        cum = f(cum + p[i])
        if r <= cum:
            return i
    return V - 1


def test_greedy_is_the_first_maximum_after_bans_and_penalty():
    h = H()
    l = np.array([0.5, 3.0, -1.0, 3.0, 2.9], np.float32)
    assert h.sample(l) == 1
    assert h.sample(l, banned_ids=[1]) == 3
    assert h.sample(l, banned_ids=[1, 3, 99, -4]) == 4
    # the penalty divides positive logits and multiplies negative ones, for tokens of the last 512 context ids
    assert h.sample(l, ctx_ids=[1, 3], repetition_penalty=1.5) == 4
    assert h.sample(np.array([-1.0, -1.2], np.float32), ctx_ids=[0], repetition_penalty=1.5) == 1
    old = [1] + [0] * 512       # token 1 is 513 back: out of the window
    assert h.sample(l, ctx_ids=old, repetition_penalty=100.0) == 1
    assert h.sample(l, ctx_ids=old[1:] + [1], repetition_penalty=100.0) == 3


@pytest.mark.parametrize("cfg", [dict(temperature=1.0), dict(temperature=0.7, top_k=5), dict(temperature=1.3, top_p=0.8),
                                 dict(temperature=0.9, top_k=8, top_p=0.6, repetition_penalty=1.2, banned_ids=[2, 7])])
def test_sampler_matches_the_restatement_draw_for_draw(cfg):
    h = H()
    rng = np.random.default_rng(11)
    V = 40
    ctx = [int(v) for v in rng.integers(0, V, 30)]
    seen = set()
    for seed in range(150):
        l = (3.0 * rng.standard_normal(V)).astype(np.float32)
        got = h.sample(l, ctx_ids=ctx, seed=seed, **cfg)
        assert got == py_sample(l, ctx, seed, **cfg), (seed, cfg)
        seen.add(got)
        if cfg.get("top_k"):
            kth = np.sort(l)[::-1][cfg["top_k"] - 1] if "repetition_penalty" not in cfg else None
            if kth is not None:
                assert l[got] >= kth
        assert got not in cfg.get("banned_ids", ())
    assert len(seen) > 3       # it does sample


def test_top_k_one_and_tiny_top_p_are_greedy():
    h = H()
    rng = np.random.default_rng(3)
    for seed in range(20):
        l = rng.standard_normal(64).astype(np.float32)
        assert h.sample(l, seed=seed, temperature=1.0, top_k=1) == int(np.argmax(l))
        assert h.sample(l, seed=seed, temperature=1.0, top_p=1e-6) == int(np.argmax(l))


# ---- the generation loop ----

def py_generate(table, ctx, max_new, eos_ids=(), think_open_id=-1, think_close_id=-1, sys_n=0, turn_n=0, T=0, T_kv=0):
    """run_generate with greedy sampling over canned logits; returns (generated, ctx, trace, stats)."""
    ctx = list(ctx)
    calls, trace = [0], []
    stats = dict(rebuilds=0, decode_steps=0, prefill_tokens=0, resets=0)

    def model(token, pos):
        trace.append((token, pos))
        row = table[calls[0] % len(table)]
        calls[0] += 1
        return int(np.argmax(row))

    def prefill(tokens):
        stats["resets"] += 1
        nxt = 0
        for i, t in enumerate(tokens):
            nxt = model(t, i)
            stats["prefill_tokens"] += 1
        return nxt

    out = []
    n = min(len(ctx), T)
    nxt = prefill(ctx[len(ctx) - n:])
    pos, ctx_at_start, depth = n, len(ctx), 0
    for _ in range(max_new):
        if nxt in eos_ids:
            break
        ctx.append(nxt)
        out.append(nxt)
        if think_open_id >= 0 and nxt == think_open_id:
            depth += 1
        elif think_close_id >= 0 and nxt == think_close_id and depth > 0:
            depth -= 1
        if T_kv > 0 and pos >= T_kv:
            stats["rebuilds"] += 1
            if stats["rebuilds"] > 4:
                break
            anchor = sys_n + turn_n
            gen_so_far = len(ctx) - ctx_at_start
            max_rebuild = min(T, T_kv // 2)
            if max_rebuild <= anchor:
                max_rebuild = anchor + 1
            max_tail = max_rebuild - anchor
            x = [0] * max(T, max_rebuild + 1)
            for i in range(min(sys_n, T)):
                x[i] = ctx[i]
            for i in range(turn_n):
                if sys_n + i < T:
                    x[sys_n + i] = ctx[sys_n + i]
            if depth > 0 and think_open_id >= 0:
                x[anchor] = think_open_id
                tail = min(gen_so_far, max_tail - 1)
                for i in range(tail):
                    x[anchor + 1 + i] = ctx[len(ctx) - tail + i]
                tail_n = 1 + tail
            else:
                tail = max(0, min(ctx_at_start - anchor, max_tail))
                for i in range(tail):
                    x[anchor + i] = ctx[ctx_at_start - tail + i]
                tail_n = tail
            rebuild_n = anchor + tail_n
            nxt = prefill(x[:rebuild_n])
            pos = rebuild_n
            del ctx[rebuild_n:]
            ctx_at_start = rebuild_n
            continue
        nxt = model(nxt, pos)
        pos += 1
        stats["decode_steps"] += 1
    stats["model_steps"] = calls[0]
    return out, ctx, trace, stats


def canned(V, rows, seed, force=None):
    rng = np.random.default_rng(seed)
    t = rng.standard_normal((rows, V)).astype(np.float32)
    for r, tok in (force or {}).items():
        t[r, tok] = 50.0
    return t


def test_prefill_then_decode_until_eos():
    h = H()
    V, ctx = 32, [3, 4, 5, 6, 7]
    table = canned(V, 23, 1, force={4 + 9: 31})    # the 10th sampled token is EOS (31): prefill uses rows 0-4
    gen = dict(eos_ids=[31], T=16, T_kv=64)
    got = h.generate_canned(table, ctx, 50, **gen)
    want = py_generate(table, ctx, 50, **gen)
    assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
    assert len(got[0]) == 9 and got[3]["rebuilds"] == 0 and got[3]["prefill_tokens"] == 5 and got[3]["resets"] == 1
    # rows go to cache positions 0.., the decode steps continue from the prompt's length
    assert [p for _, p in got[2]] == list(range(5 + 9))
    assert [t for t, _ in got[2][:5]] == ctx and [t for t, _ in got[2][5:]] == got[0]


def test_only_the_last_T_tokens_are_prefilled_and_max_new_bounds_the_loop():
    h = H()
    V, ctx = 16, list(range(1, 13))
    table = canned(V, 7, 2)
    gen = dict(T=8, T_kv=1000)
    out, ctx_after, trace, stats = h.generate_canned(table, ctx, 6, **gen)
    assert (out, ctx_after, trace) == py_generate(table, ctx, 6, **gen)[:3]
    assert [t for t, _ in trace[:8]] == ctx[-8:] and stats["prefill_tokens"] == 8 and len(out) == 6
    assert ctx_after == ctx + out


@pytest.mark.parametrize("thinking", [False, True])
def test_a_full_cache_is_rebuilt_from_system_turn_and_tail(thinking):
    h = H()
    V = 64
    sys_n, turn_n = 3, 4
    ctx = list(range(10, 10 + sys_n)) + list(range(20, 20 + turn_n)) + [30, 31, 32]     # system | turn | earlier tool results
    force = {len(ctx) - 1: 60} if thinking else {}    # the first sampled token opens a thinking block
    table = canned(V - 4, 41, 4)
    table = np.concatenate([table, np.full((41, 4), -40.0, np.float32)], axis=1)        # ids 60-63 only when forced
    for r, tok in force.items():
        table[r, tok] = 50.0
    gen = dict(eos_ids=[63], think_open_id=60, think_close_id=61, sys_n=sys_n, turn_n=turn_n, T=16, T_kv=24)
    got = h.generate_canned(table, ctx, 40, **gen)
    want = py_generate(table, ctx, 40, **gen)
    assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
    for k in ("rebuilds", "decode_steps", "prefill_tokens", "model_steps", "resets"):
        assert got[3][k] == want[3][k], k
    assert got[3]["rebuilds"] >= 1 and got[3]["resets"] == 1 + min(got[3]["rebuilds"], 4)
    # after the first rebuild the cache holds [system | turn | marker? | tail], at most min(T, T_kv / 2) rows
    start = next(i for i, (_, p) in enumerate(got[2]) if p == 0 and i > 0)
    rows = []
    for t, p in got[2][start:]:
        if p != len(rows):
            break
        rows.append(t)
    # the rebuilt rows are followed by decode steps at the next positions: cut at min(T, T_kv / 2)
    rows = rows[:12]
    assert rows[:sys_n + turn_n] == ctx[:sys_n + turn_n]
    if thinking:
        assert rows[sys_n + turn_n] == 60
    else:
        assert rows[sys_n + turn_n:sys_n + turn_n + 3] == [30, 31, 32]


def test_the_rebuild_limit_stops_the_loop():
    h = H()
    V = 16
    table = canned(V, 13, 9)
    gen = dict(sys_n=2, turn_n=2, T=8, T_kv=8)
    got = h.generate_canned(table, [1, 2, 3, 4, 5], 500, **gen)
    want = py_generate(table, [1, 2, 3, 4, 5], 500, **gen)
    assert got[0] == want[0] and got[1] == want[1] and got[2] == want[2]
    assert got[3]["rebuilds"] == 5 and len(got[0]) < 500


def test_sampling_in_the_loop_uses_the_logits_and_the_context():
    h = H()
    V = 24
    table = canned(V, 17, 6)
    a = h.generate_canned(table, [1, 2, 3], 12, seed=5, sampler=dict(temperature=1.0, top_k=6), T=8, T_kv=100)
    b = h.generate_canned(table, [1, 2, 3], 12, seed=5, sampler=dict(temperature=1.0, top_k=6), T=8, T_kv=100)
    c = h.generate_canned(table, [1, 2, 3], 12, seed=6, sampler=dict(temperature=1.0, top_k=6), T=8, T_kv=100)
    assert a[0] == b[0] and a[0] != c[0]
    for step, tok in enumerate(a[0]):
        row = table[(2 + step) % 17]           # prefill used rows 0-2; token `step` is sampled from row 2 + step
        assert row[tok] >= np.sort(row)[::-1][5]
    # banned ids never come out, even as the arg-max
    forced = canned(V, 5, 7, force={r: 9 for r in range(5)})
    d = h.generate_canned(forced, [1], 8, sampler=dict(banned_ids=[9]), T=4, T_kv=100)
    assert 9 not in d[0] and len(d[0]) == 8
