"""Benchmark of the quantized-weight linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--wtype e5m2|fp4] [--impl reference]

Headline workload (N=1): the linears of one decode token of a Qwen3-8B-shaped model with FP8_E5M2
weights and BF16 activations: 36 layers x (q 4096<-4096, k 1024<-4096, v 1024<-4096, o 4096<-4096,
gate 12288<-4096, up 12288<-4096, down 4096<-12288) plus lm_head 151936<-4096, batch M tokens
(default 1).  A step is one pass over all 253 linears through the library's C-ABI: q,k,v and
gate,up of a layer, which read the same activations, as one cuda_gemm_wq_bf16_group call each, the
others as cuda_gemm_wq_bf16.  7.57 GB of distinct weights are resident in HBM, so every step streams
far more than the L2 holds.  The metric is algorithmic bytes per second (weights + scales +
activations in + out, each counted once per linear).

Next to the headline, rank 0 of a 1-GPU run reports (outside the timed regions): the same chain at
M = 4, 16, 32 (`decode_by_m`), the Llama-3.1-8B FP4 block-scale chain at M = 1, 8, 32 (`fp4`), the
prefill GEMMs at M = 2048 (`prefill`), the reference's own GPU path and cuBLAS BF16 on the same
shapes (`ref_gpu`), and the reference's CPU path on a bounded sample (`cpu_baseline`).  At every N,
`decode_step` is the whole decode step of the 36-layer model (RMSNorm, q/k norm, RoPE, attention over
a 4096-row BF16 KV cache, SwiGLU, residuals, lm_head, arg-max) at batch 1, 8 and 32 in tokens per second.

With N>1 (launched under torchrun, one rank per GPU) the same token is computed tensor-parallel:
q/k/v/gate/up/lm_head split by output feature, o/down split by input feature with the all-reduce fused
into their kernel, logits all-gathered; `value` stays whole-job bytes of the unsharded model per second.

`--impl reference` times the reference's CPU form of the path (its types.h decode to float, then
OpenBLAS sgemm) on all host cores, each step a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import glob
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

QWEN = dict(HIDDEN=4096, QDIM=4096, KVDIM=1024, FFN=12288, VOCAB=151936, LAYERS=36, HEADS=32, KVHEADS=8, HD=128, THETA=1e6, QKNORM=True)
LLAMA = dict(HIDDEN=4096, QDIM=4096, KVDIM=1024, FFN=14336, VOCAB=128256, LAYERS=32, HEADS=32, KVHEADS=8, HD=128, THETA=5e5, QKNORM=False)
W_STD = 0.02
CONTEXT = 4096


def model_dims(wtype: str, layers: int | None = None):
    m = LLAMA if wtype == "fp4" else QWEN
    d = [m["HIDDEN"], m["QDIM"], m["KVDIM"], m["FFN"], m["VOCAB"], m["LAYERS"]]
    if layers:
        d[5] = layers
    return tuple(d)


def layer_linears(dims):
    """(name, N_out, K, source buffer, kind) for one layer; kind: col = split N, row = split K."""
    hidden, qdim, kvdim, ffn, _, _ = dims
    return [
        ("q", qdim, hidden, "x", "col"), ("k", kvdim, hidden, "x", "col"), ("v", kvdim, hidden, "x", "col"),
        ("o", hidden, qdim, "q", "row"), ("gate", ffn, hidden, "o", "col"), ("up", ffn, hidden, "o", "col"),
        ("down", hidden, ffn, "gate", "row"),
    ]


def algorithmic_bytes(N, K, M, wtype):
    w = N * K // 2 + N * K // 16 if wtype == "fp4" else N * K
    return w + 2 * M * K + 2 * M * N


def step_bytes(dims, M, wtype):
    total = 0
    for _, N, K, _, _ in layer_linears(dims):
        total += algorithmic_bytes(N, K, M, wtype)
    return total * dims[5] + algorithmic_bytes(dims[4], dims[0], M, wtype)


def workload_config(args, dims, world):
    """What is measured, as both arms (this library and the reference's CPU path) describe it."""
    M = args.tokens
    return {
        "workload": f"{'llama-3.1-8b w4a16' if args.wtype == 'fp4' else 'qwen3-8b w8a16'} decode linears: "
                    f"{dims[5]} layers x (q,k,v,o,gate,up,down) + lm_head, M={M}",
        "tokens": M, "wtype": args.wtype, "bytes_per_step": step_bytes(dims, M, args.wtype),
        "l2": "7.5 GB of distinct weights per step (> L2)", "parallelism": f"tp{world}",
        "weights": "seeded 1 MiB byte blocks per linear, tiled to the linear's size (same bytes in both arms)",
    }


# ---- seeded weight bytes, identical on the host and on the device ----------------------------------
BLOCK = 1 << 20


def weight_blocks(wtype: str, layer: int, name: str, rank: int = 0):
    """The 1 MiB block of weight bytes (and, FP4, of block-scale bytes) that a linear's buffers repeat.
    E5M2: exponent field 5..10 (magnitudes of N(0, 0.02) weights), random mantissa and sign.  FP4: uniform
    nibbles, E4M3 scale bytes 1..7.  Kernel time does not depend on the values; parity is the tests' job."""
    import numpy as np

    seed = 1000003 * (layer + 1) + 7919 * (sum(ord(ch) for ch in name)) + rank
    rng = np.random.default_rng(seed)
    if wtype == "fp4":
        return rng.integers(0, 256, BLOCK, dtype=np.uint8), rng.integers(1, 8, BLOCK, dtype=np.uint8)
    e = (rng.integers(5, 11, BLOCK, dtype=np.uint8) << 2) | rng.integers(0, 4, BLOCK, dtype=np.uint8)
    return (e | (rng.integers(0, 2, BLOCK, dtype=np.uint8) << 7)).astype(np.uint8), None


def tiled_host(block, nbytes):
    import numpy as np

    return np.resize(block, nbytes)


def tiled_dev(torch, block, nbytes, dev):
    t = torch.from_numpy(block).to(dev)
    reps = (nbytes + t.numel() - 1) // t.numel()
    return t.repeat(reps)[:nbytes].contiguous() if reps > 1 else t[:nbytes].contiguous()


# ---- clocks ------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi SM clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
                 str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            time.sleep(0.25)    # let the first samples arrive before the timed region starts
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append((time.time(), parts))

    def stop(self, t_begin=None, t_end=None):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, s in self.samples:
            if t_begin is not None and not (t_begin <= ts <= t_end + 0.05):
                continue
            try:
                clocks.append(float(s[1]))
                mx = float(s[2])
            except ValueError:
                continue
            for name, val in zip(names, s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        med = clocks[len(clocks) // 2] if clocks else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(clocks)}


# ---- the GPU arm ----------------------------------------------------------------------------------
def build_model(torch, capi, dims, M, wtype, rank, world, dev):
    """The model's linears in the quantised byte format, resident in HBM, plus the chain's buffers."""
    hidden, qdim, kvdim, ffn, vocab, layers = dims
    wt = capi.FP4_E2M1 if wtype == "fp4" else capi.FP8_E5M2

    def weight(layer, name, N, K):
        wb, sb = weight_blocks(wtype, layer, name, rank)
        if wtype == "fp4":
            return tiled_dev(torch, wb, N * K // 2, dev), tiled_dev(torch, sb, N * K // 16, dev), 1.0
        return tiled_dev(torch, wb, N * K, dev), None, 1.0

    def shard(N, K, kind):
        if world == 1:
            return N, K
        return (N // world, K) if kind == "col" else (N, K // world)

    lin = []
    for i in range(layers):
        for name, N, K, src, kind in layer_linears(dims):
            n, k = shard(N, K, kind)
            W, S, inv = weight(i, name, n, k)
            lin.append(dict(name=name, N=n, K=k, W=W, S=S, inv=inv, src=src, kind=kind, fullN=N, fullK=K))
    n, k = shard(vocab, hidden, "col")
    W, S, inv = weight(layers, "lm_head", n, k)
    lin.append(dict(name="lm_head", N=n, K=k, W=W, S=S, inv=inv, src="x", kind="col", fullN=vocab, fullK=hidden))
    return wt, lin, chain_buffers(torch, dims, M, world, dev)


def chain_buffers(torch, dims, M, world, dev):
    hidden, qdim, kvdim, ffn, vocab, _ = dims
    z = lambda *s, dt=torch.bfloat16: torch.zeros(*s, dtype=dt, device=dev)
    bufs = {"x": z(M, hidden), "q": z(M, qdim // world), "k": z(M, kvdim // world), "v": z(M, kvdim // world), "o": z(M, hidden),
            "gate": z(M, ffn // world), "up": z(M, ffn // world), "logits": z(M, vocab // world),
            "logits_all": z(world, M, vocab // world), "partial": z(M, hidden, dt=torch.float32)}
    bufs["down"] = bufs["x"]    # the layer chain: "down" of a layer is the next layer's "x"
    return bufs


def plan_step(capi, lin, bufs, M, world, grouped):
    """The launches of one token: consecutive linears that read the same buffer (q,k,v; gate,up) become
    one grouped call when `grouped`; row-parallel linears stay alone (their partial sums are reduced)."""
    calls, i = [], 0
    while i < len(lin):
        L = lin[i]
        row_parallel = world > 1 and L["kind"] == "row"
        members = [L]
        if grouped and not row_parallel:
            while (i + len(members) < len(lin) and len(members) < 3 and lin[i + len(members)]["src"] == L["src"]
                   and lin[i + len(members)]["K"] == L["K"] and lin[i + len(members)]["name"] != "lm_head"
                   and not (world > 1 and lin[i + len(members)]["kind"] == "row") and L["name"] != "lm_head"):
                members.append(lin[i + len(members)])
        src = bufs["x"] if L["name"] == "lm_head" else bufs[L["src"]]
        items = []
        for Lm in members:
            dst = bufs["logits"] if Lm["name"] == "lm_head" else bufs[Lm["name"]]
            out = bufs["partial"] if row_parallel else dst
            items.append(dict(W=Lm["W"], S=Lm["S"], inv=Lm["inv"], Y=out, N=Lm["N"], alpha=1.0 / (W_STD * math.sqrt(Lm["fullK"]))))
        calls.append(dict(items=items, group=capi.make_group(items, L["K"]), src=src, K=L["K"], row_parallel=row_parallel,
                          dst=bufs["logits"] if L["name"] == "lm_head" else bufs[L["name"]], name=L["name"]))
        i += len(members)
    return calls


def run_step(torch, dist, capi, wt, calls, bufs, M, world, flags):
    """One token's linears.  alpha keeps activation magnitudes steady through the random layers.
    With more than one rank, row-parallel linears (o, down) write FP32 partial sums, which are
    all-reduced and rounded to BF16 once; the logits are all-gathered.  Returns the number of kernels the library
    launched (its own counter: a call is one kernel, or two where the activations are split by a kernel of their own)."""
    launched_before = capi.launch_count()
    for c in calls:
        fused = bufs.get("fused_row_linear") if c["row_parallel"] else None
        if fused is not None:
            # the row-parallel linear and its all-reduce as one kernel
            it = c["items"][0]
            rc = fused(wt, it["W"], it["S"], it["inv"], c["src"], c["dst"], it["N"], M, c["K"], alpha=it["alpha"], flags=flags)
            if rc != 0:
                raise RuntimeError(f"fused linear {c['name']} failed: {rc}")
            continue
        if len(c["items"]) == 1:
            it = c["items"][0]
            rc = capi.gemm_wq_bf16(wt, it["W"], it["S"], it["inv"], c["src"], it["Y"], it["N"], M, c["K"], alpha=it["alpha"],
                                   flags=flags | (capi.FLAG_OUT_F32 if c["row_parallel"] else 0))
        else:
            rc = capi.gemm_wq_bf16_group(wt, c["group"], c["src"], M, c["K"], flags=flags)
        if rc != 0:
            raise RuntimeError(f"linear {c['name']} failed: {rc}")
        if c["row_parallel"]:
            ar = bufs.get("push_allreduce")
            if ar is not None:
                if ar(bufs["partial"], c["dst"], bufs["partial"].numel(), flags=flags & 1) != 0:
                    raise RuntimeError("cuda_b200_allreduce_f32_to_bf16 failed")
            else:
                dist.all_reduce(bufs["partial"])
                c["dst"].copy_(bufs["partial"])
    if world > 1:
        dist.all_gather_into_tensor(bufs["logits_all"], bufs["logits"])
    return capi.launch_count() - launched_before


def build_chain_program(capi, wt, calls, M):
    """The same chain recorded as a decode program: one persistent kernel per token
    (cuda_decode_program_*).  Raises ValueError where the program kernel does not take the chain."""
    prog = capi.DecodeProgram(wt, M)
    for c in calls:
        if prog.add_linears(c["group"], c["K"], c["src"], mode=capi.X_COPY) != 0:
            prog.close()
            raise ValueError(f"decode program does not take linear {c['name']}")
    if prog.finalize() != 0:
        prog.close()
        raise ValueError("decode program: finalize failed")
    return prog


def start_watchdog(seconds: float):
    """A benchmark must never occupy a GPU indefinitely: if the process is still alive after `seconds`,
    say so on stdout and leave."""
    def fire():
        print(json.dumps({"error": f"bench.py watchdog: no result after {seconds:.0f} s", "rank": os.environ.get("RANK", "0")}),
              flush=True)
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def traffic_ratio():
    """DRAM bytes / algorithmic bytes of the decode kernel, read from the ncu summary under profiles/
    (a line `traffic_ratio: <x>`), so that it moves with the capture; None if the summary is absent."""
    try:
        for line in open(os.path.join(ROOT, "profiles", "gemv_wq_kernel_qwen3_decode_m1.md")):
            if line.strip().startswith("traffic_ratio:"):
                return float(line.split(":", 1)[1].split()[0])
    except Exception:
        pass
    return None


def time_chain(torch, capi, wt, lin, dims, M, wtype, flags, reps, dev, stream):
    """The linears-only chain at M tokens on one GPU: CUDA-graph replay, CUDA events.  Returns a report."""
    bufs = chain_buffers(torch, dims, M, 1, dev)
    calls = plan_step(capi, lin, bufs, M, 1, True)
    with torch.cuda.stream(stream):
        bufs["x"].normal_()
        n = run_step(torch, None, capi, wt, calls, bufs, M, 1, flags)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            run_step(torch, None, capi, wt, calls, bufs, M, 1, flags)
        for _ in range(5):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    b = step_bytes(dims, M, wtype)
    peak = float(load_peaks().get("hbm_gbs", 6650.0))
    gbs = b / ms / 1e6
    return {"tokens": M, "ms_per_step": round(ms, 4), "gbs": round(gbs, 1), "frac": round(gbs / peak, 4), "launches_per_step": n,
            "linears_tok_per_s": round(M / ms * 1e3, 1)}


def time_w8a8_chain(torch, capi, lin, dims, M, flags, reps, dev, stream, act_scale):
    """The same chain of linears in the reference's W8A8 mode: the weight bytes read as E4M3, the BF16 activations
    quantised to E4M3 inside each call (act_scale > 0: static scale; 0: dynamic absmax); q,k,v and gate,up of a layer as one
    cuda_gemm_w8a8_bf16_group call each, the others as cuda_gemm_w8a8_bf16 (145 calls).  CUDA-graph replay, CUDA events."""
    bufs = chain_buffers(torch, dims, M, 1, dev)
    calls = plan_step(capi, lin, bufs, M, 1, True)

    def step():
        before = capi.launch_count()
        for c in calls:
            it = c["items"][0]
            if len(c["items"]) > 1:
                rc = capi.gemm_w8a8_bf16_group(c["group"], c["src"], act_scale, M, c["K"], flags=flags & 1)
            else:
                rc = capi.gemm_w8a8_bf16(it["W"], it["inv"], c["src"], act_scale, it["Y"], it["N"], M, c["K"], alpha=it["alpha"], flags=flags & 1)
            if rc != 0:
                raise RuntimeError(f"w8a8 linear {c['name']} failed: {rc}")
        return capi.launch_count() - before

    with torch.cuda.stream(stream):
        bufs["x"].normal_()
        n = step()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            step()
        for _ in range(5):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
    ms = e0.elapsed_time(e1) / reps
    b = step_bytes(dims, M, "e5m2")
    peak = float(load_peaks().get("hbm_gbs", 6650.0))
    gbs = b / ms / 1e6
    return {"tokens": M, "act_scale": "static" if act_scale > 0 else "dynamic", "ms_per_step": round(ms, 4), "gbs": round(gbs, 1),
            "frac": round(gbs / peak, 4), "launches_per_step": n, "linears_tok_per_s": round(M / ms * 1e3, 1)}


def decode_step_model(torch, capi, dm, dims, wt, lin, world, rank, M_max, dev, bufs):
    """The whole-model decode step (configuration 5) around the chain's weights: norms, embedding table, RoPE
    tables (cccc/NetCifa.cpp:431-475), and a BF16 KV cache of CONTEXT rows per sequence filled with N(0,1)."""
    m = QWEN
    cfg = dm.ModelConfig(m["HIDDEN"], m["HEADS"], m["KVHEADS"], m["HD"], m["FFN"], m["VOCAB"], dims[5], m["THETA"], m["QKNORM"])
    ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=dev)
    layers = []
    for i in range(dims[5]):
        L = {nm: (lin[i * 7 + j]["W"], lin[i * 7 + j]["S"], lin[i * 7 + j]["inv"]) for j, nm in enumerate(("q", "k", "v", "o", "gate", "up", "down"))}
        L.update(attn_norm=ones(cfg.hidden), ffn_norm=ones(cfg.hidden), q_norm=ones(cfg.head_dim), k_norm=ones(cfg.head_dim))
        layers.append(L)
    g = torch.Generator(device=dev).manual_seed(5)
    emb = torch.randn(cfg.vocab, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
    w = dict(layers=layers, emb=emb, final_norm=ones(cfg.hidden), lm_head=(lin[-1]["W"], lin[-1]["S"], lin[-1]["inv"]))
    half = cfg.head_dim // 2
    t = torch.arange(CONTEXT, dtype=torch.float32).unsqueeze(1)
    inv_freq = torch.pow(torch.tensor(cfg.rope_theta, dtype=torch.float32), -2.0 * torch.arange(half, dtype=torch.float32) / cfg.head_dim)
    ang = t * inv_freq.unsqueeze(0)
    trunc = lambda x: (x.contiguous().view(torch.int32) >> 16).to(torch.int16).view(torch.bfloat16).to(dev)    # host bfloat16(float) truncates
    model = dm.DecodeModel(capi, torch, cfg, wt, w, trunc(torch.cos(ang)), trunc(torch.sin(ang)), M_max, CONTEXT, dev, world=world,
                           rank=rank, fused_row_linear=bufs.get("fused_row_linear"))
    for kc, vc in zip(model.k_cache, model.v_cache):
        kc.normal_(generator=g)
        vc.normal_(generator=g)
    return model


def time_decode_step(torch, dist, capi, model, dims, M, wtype, flags, reps, dev, stream, world, program=False):
    """Batch-M decode steps with every sequence's cache full (the new token goes to row CONTEXT-1 and
    attention reads CONTEXT rows): CUDA-graph replay (or, program=True, the recorded decode program: embedding,
    one persistent kernel, arg-max), CUDA events, max over ranks."""
    with torch.cuda.stream(stream):
        model.pos.fill_(CONTEXT - 1)
        model.ids.copy_(torch.arange(model.B, dtype=torch.int32, device=dev) % 1000)
        if program:
            model.build_program(M)
            n = model.step_program(M)
            stream.synchronize()

            class Direct:
                def replay(self):
                    model.step_program(M)
            g = Direct()
        else:
            launched_before = capi.launch_count()
            model.step(M, flags)
            n = capi.launch_count() - launched_before
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                model.step(M, flags)
        for _ in range(3):
            g.replay()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        stream.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            tt = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
    b = step_bytes(dims, M, wtype) + model.kv_bytes_full(M, CONTEXT)
    peak = float(load_peaks().get("hbm_gbs", 6650.0))
    gbs = b / ms / 1e6
    return {"batch": M, "context": CONTEXT, "ms_per_step": round(ms, 4), "tok_per_s": round(M / ms * 1e3, 1), "launches_per_step": n,
            "bytes_per_step": b, "kv_bytes_per_step": model.kv_bytes_full(M, CONTEXT), "gbs": round(gbs, 1),
            "frac_of_hbm_peak_per_gpu": round(gbs / world / peak, 4)}


def gpu_arm(args):
    import torch

    from __graft_entry__ import load_package

    pkg = load_package()
    capi = pkg.capi
    capi.lib()
    import importlib

    dm = importlib.import_module("cccc_lite_b200.decode_model")
    watchdog = start_watchdog(args.watchdog)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        import datetime

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=120))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    M = args.tokens
    dims = model_dims(args.wtype, args.layers)
    wt, lin, bufs = build_model(torch, capi, dims, M, args.wtype, rank, world, dev)
    calls = plan_step(capi, lin, bufs, M, world, bool(args.group))
    allreduce = "none"
    if world > 1:
        allreduce = "nccl"
        if args.ar in ("push", "fused"):
            try:
                n_max = max(M, 32) * dims[0]
                if args.ar == "fused":
                    bufs["fused_row_linear"] = capi.FusedRowLinear(dist, dist.group.WORLD, rank, world, n_max, dev)
                else:
                    bufs["push_allreduce"] = capi.PushAllReduce(dist, dist.group.WORLD, rank, world, n_max, dev)
                allreduce = args.ar
            except Exception as e:  # no symmetric memory on this system: NCCL does the exchange
                if rank == 0:
                    print(f"peer-memory all-reduce unavailable ({type(e).__name__}: {e}); using NCCL", file=sys.stderr, flush=True)
        ok = torch.tensor([1 if allreduce != "nccl" else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            bufs.pop("push_allreduce", None)
            bufs.pop("fused_row_linear", None)
            allreduce = "nccl"
    flags = capi.FLAG_PDL if args.pdl else 0

    x_host = torch.randn(M, dims[0]).to(torch.bfloat16).pin_memory()
    logits_host = torch.empty(world, M, dims[4] // world, dtype=torch.bfloat16).pin_memory()
    stream = torch.cuda.Stream(device=dev)
    bytes_per_step = step_bytes(dims, M, args.wtype)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    prog = None
    if world == 1 and M <= 2 and args.program:
        try:
            prog = build_chain_program(capi, wt, calls, M)
        except ValueError as e:
            print(f"decode program not used: {e}", file=sys.stderr, flush=True)

    with torch.cuda.stream(stream):
        bufs["x"].copy_(x_host, non_blocking=True)
        launches_per_step = run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)  # first call: workspace
        stream.synchronize()
        assert capi.check_error("bench warmup") == 0
        graph = None
        if prog is not None:
            launches_per_step = 1
        elif not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            bufs["x"].copy_(x_host, non_blocking=True)
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)

        def one_step():
            if prog is not None:
                if prog.launch(stream.cuda_stream) != 0:
                    raise RuntimeError("decode program launch failed")
            elif graph is not None:
                graph.replay()
            else:
                run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)

        # ---- device-resident arm ----
        for _ in range(args.warmup):
            bufs["x"].copy_(x_host, non_blocking=True)
            one_step()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        t_begin = time.time()
        e0.record(stream)
        for _ in range(args.steps):
            one_step()
        e1.record(stream)
        barrier()
        t_end = time.time()
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

        # ---- end to end: host activations in, host logits out, every step ----
        src_logits = bufs["logits_all"] if world > 1 else bufs["logits"]
        for _ in range(max(1, min(args.warmup, 5))):
            bufs["x"].copy_(x_host, non_blocking=True)
            one_step()
            logits_host.view(-1)[:src_logits.numel()].copy_(src_logits.view(-1), non_blocking=True)
        barrier()
        e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2.record(stream)
        for _ in range(args.steps):
            bufs["x"].copy_(x_host, non_blocking=True)
            one_step()
            logits_host.view(-1)[:src_logits.numel()].copy_(src_logits.view(-1), non_blocking=True)
            stream.synchronize()  # the caller reads the logits before it can issue the next token
        e3.record(stream)
        barrier()
        ms_e2e = max_over_ranks(e2.elapsed_time(e3))
        assert capi.check_error("bench") == 0

        # ---- outside the timed regions: the fused exchange against the two-kernel form, bit for bit ----
        exchange_check = None
        if world > 1 and "fused_row_linear" in bufs:
            try:
                bufs["x"].copy_(x_host, non_blocking=True)
                run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)
                stream.synchronize()
                fused_logits = src_logits.clone()
                fused = bufs.pop("fused_row_linear")
                bufs["push_allreduce"] = capi.PushAllReduce(dist, dist.group.WORLD, rank, world, M * dims[0], dev)
                bufs["x"].copy_(x_host, non_blocking=True)
                run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)
                stream.synchronize()
                same = torch.tensor([1 if torch.equal(fused_logits, src_logits) else 0], device=dev)
                dist.all_reduce(same, op=dist.ReduceOp.MIN)
                bufs.pop("push_allreduce", None)
                bufs["fused_row_linear"] = fused
                exchange_check = "logits identical to the two-kernel form on every rank" if int(same.item()) == 1 else "MISMATCH"
                assert capi.check_error("exchange check") == 0
            except Exception as e:  # the check must not cost the measurement
                exchange_check = f"not run ({type(e).__name__}: {e})"

    ms_per_step = ms / args.steps
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9
    e2e_value = bytes_per_step / (ms_e2e / args.steps * 1e-3) / 1e9
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    per_gpu = value / world
    ratio = traffic_ratio()
    alg_per_launch = bytes_per_step / launches_per_step / world
    out = {
        "metric": "decode_linear_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x fp8_e5m2 -> f32 acc" if args.wtype != "fp4"
        else "bf16 x fp4_e2m1(block16,e4m3 scales) -> f32 acc", "data": "synthetic",
        "config": workload_config(args, dims, world),
        "run": {"path": "decode program: the 145 grouped linears of a token as ONE persistent kernel (cuda_decode_program_*)" if prog is not None
                else "one launch per grouped linear (cuda_gemm_wq_bf16 / _group)", "cuda_graph": graph is not None, "pdl": bool(args.pdl), "grouped_qkv_gateup": bool(args.group), "allreduce": allreduce,
                "exchange_check": exchange_check if world > 1 else None, "timed_region_s": round(ms / 1e3, 3),
                "linears_tok_per_s": round(M / (ms_per_step * 1e-3), 1)},
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": src_logits.numel() * 2, "linears_tok_per_s": round(M / (ms_e2e / args.steps * 1e-3), 1)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(per_gpu / peak, 4), "traffic": int(round(alg_per_launch * ratio)) if ratio else None,
                     "traffic_source": "ncu dram__bytes_read+write of one layer's launches over their algorithmic bytes "
                                       f"(traffic_ratio {ratio} in profiles/gemv_wq_kernel_qwen3_decode_m1.md), scaled to this step's bytes per launch",
                     "algorithmic_bytes_per_launch": int(round(alg_per_launch)), "peak_source": peak_src,
                     "kernel": "decode_program_kernel" if prog is not None else "gemv_wq_kernel", "launches_per_step": launches_per_step,
                     "avg_launch_us": round(ms_per_step * 1e3 / launches_per_step, 3)},
        "clocks": clocks,
    }

    # ---- the whole decode step (configuration 5), at every N ----
    if not args.no_decode_step and args.wtype != "fp4" and M == 1:
        graph = None
        try:
            with torch.cuda.stream(stream):
                model = decode_step_model(torch, capi, dm, dims, wt, lin, world, rank, 32, dev, bufs)
            steps = {}
            for mb in (1, 8, 32):
                steps[f"batch{mb}"] = time_decode_step(torch, dist, capi, model, dims, mb, args.wtype, flags, {1: 30, 8: 16}.get(mb, 8), dev, stream,
                                                       world)
            if world == 1:
                for mb in (1, 2):
                    try:
                        steps[f"batch{mb}_program"] = time_decode_step(torch, dist, capi, model, dims, mb, args.wtype, flags, 30, dev, stream, world,
                                                                       program=True)
                    except ValueError as e:
                        steps[f"batch{mb}_program"] = {"unavailable": str(e)}
            assert capi.check_error("decode step") == 0
            steps["note"] = ("36-layer Qwen3-8B-shaped decode step: embedding, RMSNorm, q/k norm + RoPE + cache append + attention over "
                             f"{CONTEXT} BF16 rows, o + residual, RMSNorm, gate/up, SwiGLU, down + residual, final norm, lm_head, arg-max; "
                             "bytes = linears + K and V rows read")
            out["decode_step"] = steps
            out["gpu_launches"] += sum(v.get("launches_per_step", 0) for k, v in steps.items() if k.startswith("batch"))
            del model
        except Exception as e:
            out["decode_step"] = {"error": f"{type(e).__name__}: {e}"}
    if rank == 0 and world == 1:
        graph = None
        if not args.no_extras and args.wtype != "fp4" and M == 1:
            if prog is not None:
                out["run"]["by_launches"] = time_chain(torch, capi, wt, lin, dims, 1, args.wtype, flags, 40, dev, stream)
            out["decode_by_m"] = [time_chain(torch, capi, wt, lin, dims, m, args.wtype, flags, 40, dev, stream) for m in (4, 16, 32)]
            try:
                out["w8a8"] = {"workload": "the same 253 linears in the W8A8 mode (weight bytes read as E4M3, activations quantised to E4M3 "
                                           "inside each call), grouped like the headline (145 calls)",
                               "by_m": [time_w8a8_chain(torch, capi, lin, dims, m, flags, 40, dev, stream, a) for m, a in ((1, 0.05), (1, 0.0), (32, 0.05))]}
            except Exception as e:
                out["w8a8"] = {"error": f"{type(e).__name__}: {e}"}
            try:
                out["ref_gpu"] = ref_gpu_probe(torch, capi, dims, dev)
            except Exception as e:
                out["ref_gpu"] = {"error": f"{type(e).__name__}: {e}"}
            del lin, calls, bufs
            torch.cuda.empty_cache()
            ldims = model_dims("fp4", args.layers)
            wt4, lin4, _ = build_model(torch, capi, ldims, 1, "fp4", 0, 1, dev)
            out["fp4"] = {"workload": "llama-3.1-8b w4a16 decode linears (FP4 block 16, E4M3 scales): 32 layers + lm_head",
                          "by_m": [time_chain(torch, capi, wt4, lin4, ldims, m, "fp4", flags, 40, dev, stream) for m in (1, 8, 32)]}
            del lin4
            torch.cuda.empty_cache()
        if not args.no_prefill:
            out["prefill"] = prefill_probe(torch, capi, dims, args.wtype, dev, peaks)
            out["gpu_launches"] += out["prefill"]["launches"]
        assert capi.check_error("extras") == 0
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(args, budget_s=12.0)
        print(json.dumps(out), flush=True)
    watchdog.cancel()
    if world > 1:
        # Leave in an orderly way but without tearing NCCL down under a captured graph, which has
        # been seen to block: drop the graph, drain the device, meet the other ranks, exit.
        graph = None
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        os._exit(0)


def prefill_probe(torch, capi, dims, wtype, dev, peaks):
    """The prefill configuration (config 4) in brief: M=2048 tokens through one layer's seven linears (tcgen05 kernels),
    q/k/v and gate/up as grouped calls on their shared input, timed with CUDA events; reported next to
    the decode line as TFLOP/s of 2*M*N*K."""
    M = 2048
    wt = capi.FP4_E2M1 if wtype == "fp4" else capi.FP8_E5M2
    g = torch.Generator(device=dev).manual_seed(7)
    calls = []    # (K, X, group, n_members)
    flops = 0.0
    by_input = {}
    for name, N, K, _, _ in layer_linears(dims):
        key = "attn_in" if name in ("q", "k", "v") else ("mlp_in" if name in ("gate", "up") else name)
        by_input.setdefault(key, (K, []))[1].append(N)
    for key, (K, Ns) in by_input.items():
        X = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        members = []
        for N in Ns:
            nb = N * K // 2 if wtype == "fp4" else N * K
            W = torch.randint(0, 120, (nb,), dtype=torch.uint8, device=dev, generator=g)
            S = torch.randint(1, 8, (N * K // 16,), dtype=torch.uint8, device=dev, generator=g) if wtype == "fp4" else None
            members.append(dict(W=W, S=S, Y=torch.zeros(M, N, dtype=torch.bfloat16, device=dev), N=N, inv=0.37))
            flops += 2.0 * M * N * K
        calls.append((K, X, capi.make_group(members, K), members))

    def layer():
        for K, X, grp, _ in calls:
            if capi.gemm_wq_bf16_group(wt, grp, X, M, K) != 0:
                raise RuntimeError("prefill linear failed")

    before = capi.launch_count()
    for _ in range(3):
        layer()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record()
    for _ in range(reps):
        layer()
    e1.record()
    torch.cuda.synchronize(dev)
    launches = capi.launch_count() - before
    if capi.check_error("prefill probe") != 0:
        raise RuntimeError("prefill probe failed")
    ms = e0.elapsed_time(e1) / reps
    tf = flops / ms / 1e9
    peak = float(peaks.get("bf16_tflops", 1590.0))
    out = {"workload": "one layer's seven linears as four calls (q+k+v, o, gate+up, down), M=2048 tokens", "ms_per_layer": round(ms, 4),
           "tflops": round(tf, 1), "peak_tflops": peak, "frac": round(tf / peak, 4),
           "peak_source": "measured" if "bf16_tflops" in peaks else "fallback",
           "kernel": "gemm_wq_prefill_pair_kernel (tcgen05, cta_group::2)", "launches": launches}
    if wtype != "fp4":
        # the same four calls in the W8A8 mode: the weight bytes read as E4M3, the activations quantised to E4M3 inside each
        # call (static scale, then dynamic), E4M3 x E4M3 on the tensor cores; no FP8 peak is measured on this pool, so TFLOP/s only
        w8 = {}
        for label, act_scale in (("static", 0.05), ("dynamic", 0.0)):
            def layer8():
                for K, X, grp, _ in calls:
                    if capi.gemm_w8a8_bf16_group(grp, X, act_scale, M, K) != 0:
                        raise RuntimeError("W8A8 prefill linear failed")
            before = capi.launch_count()
            for _ in range(3):
                layer8()
            torch.cuda.synchronize(dev)
            e0.record()
            for _ in range(reps):
                layer8()
            e1.record()
            torch.cuda.synchronize(dev)
            if capi.check_error("W8A8 prefill probe") != 0:
                raise RuntimeError("W8A8 prefill probe failed")
            ms8 = e0.elapsed_time(e1) / reps
            w8[label] = {"ms_per_layer": round(ms8, 4), "tflops": round(flops / ms8 / 1e9, 1)}
            out["launches"] += capi.launch_count() - before
        w8["kernel"] = "gemm_w8a8_pair_kernel (tcgen05 kind::f8f6f4, cta_group::2), quantiser included"
        out["w8a8"] = w8
    return out


def ref_gpu_probe(torch, capi, dims, dev):
    """The kernel-to-beat on the same GPU: the reference's own Cublas::gemm (cccc/cublas_real.h:943-964:
    dequantise the whole weight to BF16, cublasGemmEx, two device synchronisations), built unmodified
    into oracle/_ref/libref_gpu_gemm.so, on one layer's seven linears at M = 1 and M = 2048; next to it
    plain cuBLAS BF16 (torch.matmul) on weights dequantised beforehand, and this library on the same
    buffers.  L2-cold: three distinct weight sets are cycled."""
    path = os.path.join(ROOT, "oracle", "_ref", "libref_gpu_gemm.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_gpu_gemm.so not built (reference tree absent at build time)"}
    R = C.CDLL(path)
    R.ref_cublas_gemm.restype = C.c_int
    R.ref_cublas_gemm.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p,
                                  C.c_int, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    wt = capi.FP8_E5M2
    shapes = [(N, K) for _, N, K, _, _ in layer_linears(dims)]
    sets = []
    for s in range(3):
        ws = []
        for j, (N, K) in enumerate(shapes):
            wb, _ = weight_blocks("e5m2", 100 + s, f"ref{j}")
            W = tiled_dev(torch, wb, N * K, dev)
            Wd = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
            assert capi.convert(W, wt, Wd, capi.BFLOAT16, N * K, 0.37) == 0
            ws.append((W, Wd))
        sets.append(ws)
    report = {}
    for M in (1, 2048):
        X = {K: torch.randn(M, K, device=dev).to(torch.bfloat16) for _, K in shapes}
        Y = {N: torch.zeros(M, N, dtype=torch.bfloat16, device=dev) for N, _ in shapes}
        flops = sum(2.0 * M * N * K for N, K in shapes)
        nbytes = sum(algorithmic_bytes(N, K, M, "e5m2") for N, K in shapes)

        def ref_layer(ws):
            for (N, K), (W, _) in zip(shapes, ws):
                # cccc's call: C(N x M, ldc N) = A^T (weight, lda K) * B (activations, ldb K)
                if R.ref_cublas_gemm(1, 0, N, M, K, 1.0, W.data_ptr(), wt, K, 0.37, X[K].data_ptr(), 3, K, 1.0, 0.0, Y[N].data_ptr(), 3, N, 0.0,
                                     None, None) != 0:
                    raise RuntimeError("reference gemm failed")

        def cublas_layer(ws):
            for (N, K), (_, Wd) in zip(shapes, ws):
                torch.matmul(X[K], Wd.t(), out=Y[N])

        def ours_layer(ws):
            for (N, K), (W, _) in zip(shapes, ws):
                if capi.gemm_wq_bf16(wt, W, None, 0.37, X[K], Y[N], N, M, K) != 0:
                    raise RuntimeError("linear failed")

        res = {}
        for name, fn in (("reference_cublas_gemm", ref_layer), ("cublas_bf16_predequantised", cublas_layer), ("this_library", ours_layer)):
            fn(sets[0])
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 6
            e0.record()
            for r in range(reps):
                fn(sets[r % 3])
            e1.record()
            torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1) / reps
            res[name] = {"ms_per_layer": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 2)}
        report[f"M{M}"] = res
    report["note"] = ("one Qwen3-8B layer's seven linears issued one by one (no grouping, no graph) on L2-cold weights, per-tensor scale 0.37; "
                      "gbs = algorithmic bytes of the quantised linear / time; the reference path includes its dequantisation and device syncs")
    return report


# ---- the CPU arm -------------------------------------------------------------------------------------
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class CpuPath:
    """The reference's CPU form of the path: its own types.h decode into float (oracle/_ref/libref_cpu_path.so,
    built from the reference tree) then OpenBLAS sgemm as cccc/cblas_real.h:332-335 calls it; kind "reference".
    Where that library is absent (no reference tree at build time) or no OpenBLAS is found, the oracle's C
    restatement of the same two steps is used; kind "port"."""

    def __init__(self):
        import numpy as np

        self.np = np
        self.threads = host_threads()
        os.environ["OMP_NUM_THREADS"] = str(self.threads)    # a launcher may have set 1: this arm uses every core
        self.kind, self.blas = "port", "oracle dot loop"
        self.L = None
        path = os.path.join(ROOT, "oracle", "_ref", "libref_cpu_path.so")
        if os.path.exists(path):
            try:
                L = C.CDLL(path)
                L.ref_cpu_dequant.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p, C.c_size_t]
                L.ref_cpu_sgemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
                L.ref_cpu_set_threads(self.threads)
                for pat, prefix in (("scipy.libs/libscipy_openblas-*.so", b"scipy_"), ("opencv_python_headless.libs/libopenblas*.so", b"")):
                    hits = []
                    for sp in sys.path:
                        hits += glob.glob(os.path.join(sp, pat))
                    if hits and L.ref_cpu_blas_init(hits[0].encode(), prefix, self.threads) == 0:
                        self.L, self.kind, self.blas = L, "reference", f"OpenBLAS cblas_sgemm ({os.path.basename(hits[0])})"
                        break
            except OSError:
                self.L = None
        if self.L is None:
            from oracle import oracle as O

            self.O = O
            self.threads = O.num_threads()

    def linear(self, wt, W, S, inv, Xf, N, M, K, wf):
        """Returns (seconds in dequant, seconds in sgemm)."""
        np = self.np
        if self.L is None:
            _, td, tg = self.O.cpu_path_dequant_sgemm(wt, W, S, inv, Xf, N, M, K, wf=wf[:N * K])
            return td, tg
        Y = np.empty((M, N), np.float32)
        vp = lambda a: None if a is None else a.ctypes.data_as(C.c_void_p)
        t0 = time.perf_counter()
        self.L.ref_cpu_dequant(wt, vp(W), vp(S), inv, vp(wf), N * K)
        t1 = time.perf_counter()
        if self.L.ref_cpu_sgemm(vp(wf), vp(Xf), vp(Y), N, M, K) != 0:
            raise RuntimeError("no BLAS")
        return t1 - t0, time.perf_counter() - t1


def cpu_sample(args, dims):
    """A 1/layers sample of the token: one layer's seven linears plus vocab/layers rows of lm_head, with
    the GPU arm's weight bytes (layer 0's blocks)."""
    import numpy as np

    M = args.tokens
    wt = 6 if args.wtype == "fp4" else 5
    lins = []
    for name, N, K, _, _ in layer_linears(dims):
        lins.append((name, 0, N, K))
    lins.append(("lm_head", dims[5], max(16, dims[4] // dims[5] // 16 * 16), dims[0]))
    mats = []
    for name, layer, N, K in lins:
        wb, sb = weight_blocks(args.wtype, layer, name)
        if args.wtype == "fp4":
            mats.append((N, K, tiled_host(wb, N * K // 2), tiled_host(sb, N * K // 16)))
        else:
            mats.append((N, K, tiled_host(wb, N * K), None))
    rng = np.random.default_rng(0)
    xs = {K: rng.standard_normal((M, K)).astype(np.float32) for _, K, _, _ in mats}
    wf = np.empty(max(N * K for N, K, _, _ in mats), np.float32)
    nbytes = sum(algorithmic_bytes(N, K, M, args.wtype) for N, K, _, _ in mats)
    return wt, mats, xs, wf, nbytes


def cpu_baseline(args, budget_s: float, path: CpuPath | None = None):
    """The reference's CPU path on a bounded sample: 1/36-of-a-token samples until the budget is used."""
    dims = model_dims(args.wtype, args.layers)
    path = path or CpuPath()
    wt, mats, xs, wf, nbytes = cpu_sample(args, dims)
    t_deq = t_gemm = 0.0
    n = 0
    t0 = time.perf_counter()
    while n == 0 or (time.perf_counter() - t0 < budget_s and n < dims[5]):
        for N, K, W, S in mats:
            td, tg = path.linear(wt, W, S, 1.0, xs[K], N, args.tokens, K, wf)
            t_deq += td
            t_gemm += tg
        n += 1
    el = t_deq + t_gemm
    return {"value": round(n * nbytes / el / 1e9, 3), "unit": "GB/s", "cores": path.threads, "kind": path.kind, "blas": path.blas,
            "sample": f"{n} x (one layer's 7 linears + 1/{dims[5]} of lm_head) = {n}/{dims[5]} of a token, M={args.tokens}; "
                      f"decode to float {t_deq:.2f} s + sgemm {t_gemm:.2f} s",
            "ms_per_sample": round(el / n * 1e3, 2)}


def reference_arm(args):
    """Rank 0 only.  Each step is a bounded sample of the GPU arm's workload (1/36 of a token: one layer's
    seven linears and 1/36 of lm_head's rows, the same weight bytes), timed on all host cores; value is the
    sample's algorithmic bytes over its own wall time, ms_per_step the sample's real time."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    dims = model_dims(args.wtype, args.layers)
    path = CpuPath()
    wt, mats, xs, wf, nbytes = cpu_sample(args, dims)
    times = []
    t_deq = t_gemm = 0.0
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        d = g = 0.0
        for N, K, W, S in mats:
            td, tg = path.linear(wt, W, S, 1.0, xs[K], N, args.tokens, K, wf)
            d += td
            g += tg
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
            t_deq += d
            t_gemm += g
    sec = sum(times) / len(times)
    value = nbytes / sec / 1e9
    sample = (f"each step = one layer's 7 linears + 1/{dims[5]} of lm_head's rows ({nbytes} algorithmic bytes, 1/{dims[5]} of a token), "
              f"M={args.tokens}; decode to float {t_deq / len(times) * 1e3:.1f} ms + sgemm {t_gemm / len(times) * 1e3:.1f} ms per step")
    out = {
        "impl": "reference", "metric": "decode_linear_hbm_gbs", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 (weights decoded to float) sgemm", "data": "synthetic",
        "config": workload_config(args, dims, world),
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": path.threads, "kind": path.kind, "blas": path.blas, "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=1)
    ap.add_argument("--wtype", default="e5m2", choices=["e5m2", "fp4"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--ar", default="fused", choices=["fused", "push", "nccl"],
                    help="exchange of row-parallel partial sums (N>1): inside the linear's kernel, a separate push kernel, or NCCL")
    ap.add_argument("--group", type=int, default=1, help="1: q,k,v and gate,up of a layer go through cuda_gemm_wq_bf16_group")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (small cases for profiling)")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip decode_by_m, fp4 and ref_gpu")
    ap.add_argument("--no-decode-step", action="store_true")
    ap.add_argument("--program", action="store_true",
                    help="headline chain through cuda_decode_program_* (one persistent kernel per token) instead of launch by launch")
    ap.add_argument("--watchdog", type=float, default=540.0, help="seconds after which a stuck run exits by itself")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
