"""Benchmark of the quantized-weight linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens M] [--wtype e5m2|fp4] [--impl reference]

Workload (N=1): the linears of one decode token of a Qwen3-8B-shaped model with FP8_E5M2 weights
and BF16 activations: 36 layers x (q 4096<-4096, k 1024<-4096, v 1024<-4096, o 4096<-4096,
gate 12288<-4096, up 12288<-4096, down 4096<-12288) plus lm_head 151936<-4096, batch M tokens
(default 1).  A step is one pass over all 253 linears through the library's C-ABI: q,k,v and
gate,up of a layer, which read the same activations, as one cuda_gemm_wq_bf16_group call each
(--group 0: every linear its own cuda_gemm_wq_bf16 call), the others as cuda_gemm_wq_bf16.
7.57 GB of distinct weights are resident in HBM, so every step streams far more than the L2 holds.  The metric is algorithmic bytes per second (weights + scales +
activations in + out, each counted once per linear).

With N>1 (launched under torchrun, one rank per GPU) the same token is computed tensor-parallel:
q/k/v/gate/up/lm_head split by output feature, o/down split by input feature with an NCCL
all-reduce, logits all-gathered; `value` stays whole-job bytes of the unsharded model per second.

`--impl reference` times the CPU form of the path (dequantise to float, then sgemm) on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HIDDEN, QDIM, KVDIM, FFN, VOCAB, LAYERS = 4096, 4096, 1024, 12288, 151936, 36
LLAMA = dict(HIDDEN=4096, QDIM=4096, KVDIM=1024, FFN=14336, VOCAB=128256, LAYERS=32)
W_STD = 0.02
# DRAM bytes / algorithmic bytes of the decode kernel, from the ncu capture summarised under profiles/
# (q+k+v 25.220 + o 16.832 + gate+up 100.731 + down 50.400 MB read and written against 193.07 MB)
NCU_TRAFFIC_RATIO = 1.0006


def model_dims(wtype: str, layers: int | None = None):
    if wtype == "fp4":
        d = [LLAMA["HIDDEN"], LLAMA["QDIM"], LLAMA["KVDIM"], LLAMA["FFN"], LLAMA["VOCAB"], LLAMA["LAYERS"]]
    else:
        d = [HIDDEN, QDIM, KVDIM, FFN, VOCAB, LAYERS]
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
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
                 str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
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
    """Random weights of the model's shapes, already in the quantised byte format, resident in HBM.
    E5M2 bytes drawn so that values look like N(0, 0.02) magnitudes (exponent field 5..10), FP4
    nibbles uniform with E4M3 block scales near 0.0067: the kernels' time does not depend on the
    values, and parity is the tests' job."""
    hidden, qdim, kvdim, ffn, vocab, layers = dims
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    wt = capi.FP4_E2M1 if wtype == "fp4" else capi.FP8_E5M2

    def weight(N, K):
        if wtype == "fp4":
            nib = torch.randint(0, 256, (N * K // 2,), dtype=torch.uint8, device=dev, generator=g)
            sc = torch.randint(1, 8, (N * K // 16,), dtype=torch.uint8, device=dev, generator=g)  # subnormal E4M3
            return nib, sc, 1.0
        e = torch.randint(5, 11, (N * K,), dtype=torch.uint8, device=dev, generator=g) << 2
        e |= torch.randint(0, 4, (N * K,), dtype=torch.uint8, device=dev, generator=g)
        e |= torch.randint(0, 2, (N * K,), dtype=torch.uint8, device=dev, generator=g) << 7
        return e, None, 1.0

    def shard(N, K, kind):
        if world == 1:
            return N, K
        return (N // world, K) if kind == "col" else (N, K // world)

    lin = []
    for _ in range(layers):
        for name, N, K, src, kind in layer_linears(dims):
            n, k = shard(N, K, kind)
            W, S, inv = weight(n, k)
            lin.append(dict(name=name, N=n, K=k, W=W, S=S, inv=inv, src=src, kind=kind, fullN=N, fullK=K))
    n, k = shard(vocab, hidden, "col")
    W, S, inv = weight(n, k)
    lin.append(dict(name="lm_head", N=n, K=k, W=W, S=S, inv=inv, src="x", kind="col", fullN=vocab, fullK=hidden))
    bufs = {
        "x": torch.zeros(M, hidden, dtype=torch.bfloat16, device=dev),
        "q": torch.zeros(M, qdim // world, dtype=torch.bfloat16, device=dev),
        "k": torch.zeros(M, kvdim // world, dtype=torch.bfloat16, device=dev),
        "v": torch.zeros(M, kvdim // world, dtype=torch.bfloat16, device=dev),
        "o": torch.zeros(M, hidden, dtype=torch.bfloat16, device=dev),
        "gate": torch.zeros(M, ffn // world, dtype=torch.bfloat16, device=dev),
        "up": torch.zeros(M, ffn // world, dtype=torch.bfloat16, device=dev),
        "down": torch.zeros(M, hidden, dtype=torch.bfloat16, device=dev),
        "logits": torch.zeros(M, vocab // world, dtype=torch.bfloat16, device=dev),
        "logits_all": torch.zeros(world, M, vocab // world, dtype=torch.bfloat16, device=dev),
        "partial": torch.zeros(M, hidden, dtype=torch.float32, device=dev),
    }
    return wt, lin, bufs


def plan_step(capi, lin, bufs, M, world, grouped):
    """The launches of one token: consecutive linears that read the same buffer (q,k,v; gate,up) become
    one grouped call when `grouped`; row-parallel linears stay alone (their partial sums are reduced)."""
    import math

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
    all-reduced and rounded to BF16 once; the logits are all-gathered."""
    n_launch = 0
    for c in calls:
        fused = bufs.get("fused_row_linear") if c["row_parallel"] else None
        if fused is not None:
            # the row-parallel linear and its all-reduce as one kernel
            it = c["items"][0]
            rc = fused(wt, it["W"], it["S"], it["inv"], c["src"], c["dst"], it["N"], M, c["K"], alpha=it["alpha"], flags=flags)
            if rc != 0:
                raise RuntimeError(f"fused linear {c['name']} failed: {rc}")
            n_launch += 1
            continue
        if len(c["items"]) == 1:
            it = c["items"][0]
            rc = capi.gemm_wq_bf16(wt, it["W"], it["S"], it["inv"], c["src"], it["Y"], it["N"], M, c["K"], alpha=it["alpha"],
                                   flags=flags | (capi.FLAG_OUT_F32 if c["row_parallel"] else 0))
        else:
            rc = capi.gemm_wq_bf16_group(wt, c["group"], c["src"], M, c["K"], flags=flags)
        if rc != 0:
            raise RuntimeError(f"linear {c['name']} failed: {rc}")
        n_launch += 1
        if c["row_parallel"]:
            ar = bufs.get("push_allreduce")
            if ar is not None:
                if ar(bufs["partial"], c["dst"], bufs["partial"].numel(), flags=flags & 1) != 0:
                    raise RuntimeError("cuda_b200_allreduce_f32_to_bf16 failed")
                n_launch += 1
            else:
                dist.all_reduce(bufs["partial"])
                c["dst"].copy_(bufs["partial"])
    if world > 1:
        dist.all_gather_into_tensor(bufs["logits_all"], bufs["logits"])
    return n_launch


def start_watchdog(seconds: float):
    """A benchmark must never hang a GPU box: if the process is still alive after `seconds`, say so
    on stdout and leave."""
    def fire():
        print(json.dumps({"error": f"bench.py watchdog: no result after {seconds:.0f} s", "rank": os.environ.get("RANK", "0")}),
              flush=True)
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


def gpu_arm(args):
    import torch

    from __graft_entry__ import load_package

    capi = load_package().capi
    capi.lib()
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
    # the layer chain: "down" of a layer is the next layer's "x"
    bufs["down"] = bufs["x"]
    calls = plan_step(capi, lin, bufs, M, world, bool(args.group))
    allreduce = "none"
    if world > 1:
        allreduce = "nccl"
        if args.ar in ("push", "fused"):
            try:
                if args.ar == "fused":
                    bufs["fused_row_linear"] = capi.FusedRowLinear(dist, dist.group.WORLD, rank, world, M * dims[0], dev)
                else:
                    bufs["push_allreduce"] = capi.PushAllReduce(dist, dist.group.WORLD, rank, world, M * dims[0], dev)
                allreduce = args.ar
            except Exception as e:  # symmetric memory not available on this box: NCCL does the exchange
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

    with torch.cuda.stream(stream):
        bufs["x"].copy_(x_host, non_blocking=True)
        launches_per_step = run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)  # first call: workspace
        stream.synchronize()
        assert capi.check_error("bench warmup") == 0
        graph = None
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            bufs["x"].copy_(x_host, non_blocking=True)
            with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                run_step(torch, dist, capi, wt, calls, bufs, M, world, flags)

        def one_step():
            if graph is not None:
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
        e0.record(stream)
        for _ in range(args.steps):
            one_step()
        e1.record(stream)
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        clocks = sampler.stop() if rank == 0 else None

        # ---- end to end: host activations in, host logits out, every step ----
        src_logits = bufs["logits_all"] if world > 1 else bufs["logits"]
        for _ in range(max(1, args.warmup // 2)):
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
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    per_gpu = value / world
    out = {
        "metric": "decode_linear_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x fp8_e5m2 -> f32 acc" if args.wtype != "fp4"
        else "bf16 x fp4_e2m1(block16,e4m3 scales) -> f32 acc", "data": "synthetic",
        "config": {
            "workload": f"{'llama-3.1-8b w4a16' if args.wtype == 'fp4' else 'qwen3-8b w8a16'} decode linears: "
                        f"{dims[5]} layers x (q,k,v,o,gate,up,down) + lm_head, M={M}",
            "tokens": M, "bytes_per_step": bytes_per_step, "l2": "7.5 GB of distinct weights per step (> L2)",
            "cuda_graph": graph is not None, "pdl": bool(args.pdl), "grouped_qkv_gateup": bool(args.group), "allreduce": allreduce, "exchange_check": exchange_check if world > 1 else None, "parallelism": f"tp{world}",
            "tok_per_s": round(M / (ms_per_step * 1e-3), 1),
        },
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                "d2h_bytes_per_step": src_logits.numel() * 2, "tok_per_s": round(M / (ms_e2e / args.steps * 1e-3), 1)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(per_gpu, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(per_gpu / peak, 4), "traffic": int(round(bytes_per_step * NCU_TRAFFIC_RATIO / launches_per_step / world)),
                     "traffic_source": "ncu dram__bytes_read+write of one layer's launches (profiles/gemv_wq_kernel_qwen3_decode_m1.md), "
                                       "1.0006 x algorithmic, scaled to this step's bytes per launch",
                     "algorithmic_bytes_per_launch": int(round(bytes_per_step / launches_per_step / world)), "peak_source": peak_src,
                     "kernel": "gemv_wq_kernel", "launches_per_step": launches_per_step,
                     "avg_launch_us": round(ms_per_step * 1e3 / launches_per_step, 3)},
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_prefill:
        graph = None
        out["prefill"] = prefill_probe(torch, capi, dims, args.wtype, dev, peaks)
        out["gpu_launches"] += out["prefill"]["launches"]
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
    return {"workload": "one layer's seven linears as four calls (q+k+v, o, gate+up, down), M=2048 tokens", "ms_per_layer": round(ms, 4),
            "tflops": round(tf, 1), "peak_tflops": peak, "frac": round(tf / peak, 4),
            "peak_source": "measured" if "bf16_tflops" in peaks else "fallback",
            "kernel": "gemm_wq_prefill_pair_kernel (tcgen05, cta_group::2)", "launches": launches}


# ---- the CPU arm -------------------------------------------------------------------------------------
def cpu_baseline(args, budget_s: float):
    """The CPU form of the path (dequantise to float, then sgemm; oracle port) on a bounded sample:
    whole layers of the same workload until the time budget is used."""
    import numpy as np

    from oracle import oracle as O

    dims = model_dims(args.wtype, args.layers)
    M = args.tokens
    wt = O.FP4_E2M1 if args.wtype == "fp4" else O.FP8_E5M2
    rng = np.random.default_rng(0)
    shapes = [(N, K) for _, N, K, _, _ in layer_linears(dims)]
    mats = {}
    for N, K in set(shapes):
        if wt == O.FP4_E2M1:
            mats[(N, K)] = (rng.integers(0, 256, N * K // 2, dtype=np.uint8), rng.integers(1, 8, N * K // 16, dtype=np.uint8))
        else:
            mats[(N, K)] = (rng.integers(0x14, 0x2C, N * K, dtype=np.uint8), None)
    wf = np.empty(max(N * K for N, K in shapes), np.float32)
    xs = {K: rng.standard_normal((M, K)).astype(np.float32) for _, K in shapes}
    done_bytes, t_deq, t_gemm, layers = 0, 0.0, 0.0, 0
    t0 = time.perf_counter()
    while layers == 0 or (time.perf_counter() - t0 < budget_s and layers < dims[5]):
        for N, K in shapes:
            W, S = mats[(N, K)]
            _, td, tg = O.cpu_path_dequant_sgemm(wt, W, S, 1.0, xs[K], N, M, K, wf=wf[:N * K])
            t_deq += td
            t_gemm += tg
            done_bytes += algorithmic_bytes(N, K, M, args.wtype)
        layers += 1
    el = t_deq + t_gemm
    return {"value": round(done_bytes / el / 1e9, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{layers} of {dims[5]} layers (7 linears each), M={M}; dequant {t_deq:.2f} s + sgemm {t_gemm:.2f} s",
            "ms_per_layer": round(el / max(layers, 1) * 1e3, 2)}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    dims = model_dims(args.wtype, args.layers)
    M = args.tokens
    # each "step" is a bounded sample: one layer's seven linears
    per_step_budget = 1.0
    vals = []
    for i in range(args.warmup + args.steps):
        cb = cpu_baseline(args, budget_s=per_step_budget * 0.0 + 1e-9)  # exactly one layer per step
        if i >= args.warmup:
            vals.append(cb)
    value = sum(v["value"] for v in vals) / len(vals)
    ms_layer = sum(v["ms_per_layer"] for v in vals) / len(vals)
    bytes_per_step = step_bytes(dims, M, args.wtype)
    out = {
        "impl": "reference", "metric": "decode_linear_hbm_gbs", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(bytes_per_step / (value * 1e9) * 1e3, 2), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 (dequantised) sgemm", "data": "synthetic",
        "config": {"workload": f"{'llama-3.1-8b w4a16' if args.wtype == 'fp4' else 'qwen3-8b w8a16'} decode linears: "
                               f"{dims[5]} layers x (q,k,v,o,gate,up,down) + lm_head, M={M}", "tokens": M,
                   "bytes_per_step": bytes_per_step,
                   "note": "each timed step is one layer's seven linears on the host cores; ms_per_step is scaled to the whole token"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": vals[0]["cores"], "kind": "port",
                         "sample": f"one layer (7 linears) per step, {ms_layer:.1f} ms per layer"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
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
    ap.add_argument("--watchdog", type=float, default=420.0, help="seconds after which a stuck run exits by itself")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()
