"""One decode step of a cccc LLM (the layer scripts/convert_weights.py:488-584 generates) issued through
the C-ABI: every linear is a fused quantized-weight kernel, everything between them is one of the
decode ops of include/cccc_cuda_b200.h.  Device tensors come from the caller (torch is only the
allocator and, with several ranks, the NCCL plumbing); this module holds pointers and issues launches,
nothing is computed in Python.

Per layer, 8 launches (the reference issues about 40 ops, each with a device synchronisation):
    rms_norm -> q+k+v (one grouped launch into one [M, (H + 2 Hkv) hd] buffer) -> attention (q/k norm, RoPE,
    cache append, softmax(K q) V) -> o -> rms_norm -> gate+up (one grouped launch) -> swiglu -> down
then the final norm, lm_head and the device arg-max.  The two residual adds of a layer ride along: on
one GPU in the epilogue of o and down (flags bit 3 of cuda_gemm_wq_bf16), with several ranks in the
RMSNorm that follows (its `residual` input), because there o and down end in the fused all-reduce.

Tensor parallel (world > 1, one process per GPU): each rank is given ITS shard of every linear (q, k, v,
gate, up, lm_head by output feature; o, down by input feature) and keeps the KV cache of its own kv heads;
norm weights, tables and the embedding are replicated.  o and down run cuda_gemm_wq_bf16_allreduce; the
per-rank arg-max winners are combined with one small all-gather.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class ModelConfig:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    layers: int
    rope_theta: float = 1e6
    qk_norm: bool = True
    eps: float = 1e-6

    @property
    def q_dim(self):
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self):
        return self.n_kv_heads * self.head_dim


QWEN3_8B = ModelConfig(4096, 32, 8, 128, 12288, 151936, 36, 1e6, True)
LLAMA31_8B = ModelConfig(4096, 32, 8, 128, 14336, 128256, 32, 5e5, False)


class DecodeModel:
    """weights: dict with
         "emb" [vocab, hidden] bf16, "final_norm" [hidden] bf16, "lm_head" (W, S, inv),
         "layers": list of dicts with "q","k","v","o","gate","up","down" -> (W, S, inv) quantised tensors
         (S = FP4 block scales or None, inv = per-tensor dequant multiplier; with world > 1 this rank's shard)
         and "attn_norm", "ffn_norm" [hidden], "q_norm", "k_norm" [head_dim] (or None) bf16;
       cos_tab / sin_tab: [max_context, head_dim/2] bf16 (cccc/NetCifa.cpp:431-475);
       fused_row_linear: a capi.FusedRowLinear (world > 1) whose areas hold max_batch * hidden floats."""

    def __init__(self, capi, torch, cfg: ModelConfig, w_type: int, weights: dict, cos_tab, sin_tab, max_batch: int, max_context: int,
                 device, world: int = 1, rank: int = 0, fused_row_linear=None, dist=None):
        self.c, self.torch, self.cfg, self.wt, self.w = capi, torch, cfg, w_type, weights
        self.B, self.T = max_batch, max_context
        self.cos, self.sin = cos_tab, sin_tab
        self.world, self.rank, self.fused, self.dist = world, rank, fused_row_linear, dist
        if world > 1 and (cfg.n_kv_heads % world or cfg.ffn % world or cfg.vocab % world or fused_row_linear is None):
            raise ValueError("tensor parallel needs kv heads, ffn and vocab divisible by the ranks and a FusedRowLinear")
        if world > 1 and dist is None:
            import torch.distributed as dist_mod

            self.dist = dist_mod
        bf = dict(dtype=torch.bfloat16, device=device)
        c = cfg
        self.H, self.Hkv = c.n_heads // world, c.n_kv_heads // world
        self.q_loc, self.kv_loc, self.ffn_loc, self.vocab_loc = self.H * c.head_dim, self.Hkv * c.head_dim, c.ffn // world, c.vocab // world
        self.qkv_ld = self.q_loc + 2 * self.kv_loc
        self.ids = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self.best = torch.zeros(max_batch, dtype=torch.float32, device=device)
        self.pos = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self.x = torch.zeros(max_batch, c.hidden, **bf)        # the residual stream
        self.xn = torch.zeros(max_batch, c.hidden, **bf)
        self.tmp = torch.zeros(max_batch, c.hidden, **bf)      # a row-parallel linear's output before the residual add
        self.qkv = torch.zeros(max_batch, self.qkv_ld, **bf)
        self.att = torch.zeros(max_batch, self.q_loc, **bf)
        self.gu = torch.zeros(max_batch, 2 * self.ffn_loc, **bf)
        self.h = torch.zeros(max_batch, self.ffn_loc, **bf)
        self.logits = torch.zeros(max_batch, self.vocab_loc, **bf)
        if world > 1:
            self.cand = torch.zeros(max_batch, 2, dtype=torch.float32, device=device)           # (best logit, its global id)
            self.cand_all = torch.zeros(world, max_batch, 2, dtype=torch.float32, device=device)
        self.k_cache = [torch.zeros(max_batch, self.Hkv, max_context, c.head_dim, **bf) for _ in range(c.layers)]
        self.v_cache = [torch.zeros(max_batch, self.Hkv, max_context, c.head_dim, **bf) for _ in range(c.layers)]
        self._plans = {}

    # ---- launch descriptors, built once per batch size (they only hold pointers) ----
    def _plan(self, M: int):
        if M in self._plans:
            return self._plans[M]
        c, C = self.cfg, self.c
        esz = 2
        plan = []
        for i, L in enumerate(self.w["layers"]):
            qkv_items = []
            off = 0
            for name, n in (("q", self.q_loc), ("k", self.kv_loc), ("v", self.kv_loc)):
                W, S, inv = L[name]
                qkv_items.append(dict(W=W, S=S, inv=inv, N=n, Y=self.qkv.data_ptr() + off * esz, ldy_m=self.qkv_ld))
                off += n
            gu_items = []
            for j, name in enumerate(("gate", "up")):
                W, S, inv = L[name]
                gu_items.append(dict(W=W, S=S, inv=inv, N=self.ffn_loc, Y=self.gu.data_ptr() + j * self.ffn_loc * esz, ldy_m=2 * self.ffn_loc))
            attn = C.make_attn_decode(q=self.qkv.data_ptr(), k=self.qkv.data_ptr() + self.q_loc * esz,
                                      v=self.qkv.data_ptr() + (self.q_loc + self.kv_loc) * esz, k_cache=self.k_cache[i],
                                      v_cache=self.v_cache[i], pos=self.pos, out=self.att, cos_tab=self.cos, sin_tab=self.sin,
                                      q_norm=L.get("q_norm"), k_norm=L.get("k_norm"), B=M, H=self.H, Hkv=self.Hkv, head_dim=c.head_dim,
                                      T_max=self.T, ldq=self.qkv_ld, ldk=self.qkv_ld, ldv=self.qkv_ld, eps=c.eps)
            plan.append(dict(qkv=C.make_group(qkv_items, c.hidden), gu=C.make_group(gu_items, c.hidden), attn=attn, L=L,
                             keep=(qkv_items, gu_items)))
        self._plans[M] = plan
        return plan

    def step(self, M: int, flags: int = 1, from_ids: bool = True) -> int:
        """Issues one decode step for M sequences on torch's current stream; returns the number of launches.
        Inputs: self.ids (token ids) when from_ids, else self.x (embedded tokens); self.pos (row each token
        is appended at).  Outputs: self.logits (this rank's vocabulary shard), and self.ids / self.best =
        arg-max token (global id, the same on every rank) and its logit."""
        c, C, wt = self.cfg, self.c, self.wt
        tp = self.world > 1
        RES = 8  # flags bit 3 of cuda_gemm_wq_bf16: Y = bf16(bf16(W x) + Y), the reference's residual add
        n = 0

        def ok(rc, what):
            if rc != 0:
                raise RuntimeError(f"{what} failed: {rc}")
            return 1

        def row_linear(L3, src, K_loc, what):
            """o / down: on one GPU straight into the residual stream; with several ranks the fused
            linear + all-reduce into self.tmp, which the next RMSNorm adds to the stream."""
            W, S, inv = L3
            if tp:
                if M >= 9 and (M * c.hidden) % 4 == 0:
                    # the streaming tensor-core kernel + the push all-reduce: faster than the fused decode kernel from 9 tokens on
                    return ok(self.fused.two_kernels(wt, W, S, inv, src, self.tmp, c.hidden, M, K_loc, flags=flags), what) + 1
                return ok(self.fused(wt, W, S, inv, src, self.tmp, c.hidden, M, K_loc, flags=flags), what)
            return ok(C.gemm_wq_bf16(wt, W, S, inv, src, self.x, c.hidden, M, K_loc, beta=1.0, flags=flags | RES), what)

        def norm(scale, pending):
            """RMSNorm of the stream into self.xn; `pending`: self.tmp still has to be added to the stream."""
            if pending:
                return ok(C.rms_norm_bf16(self.x, self.xn, scale, M, c.hidden, c.eps, residual=self.tmp, sum_out=self.x, flags=flags), "rms_norm")
            return ok(C.rms_norm_bf16(self.x, self.xn, scale, M, c.hidden, c.eps, flags=flags), "rms_norm")

        if from_ids:
            n += ok(C.embed_bf16(self.ids, self.w["emb"], self.x, c.hidden, M, c.vocab, flags=flags), "embed")
        pending = False
        for i, P in enumerate(self._plan(M)):
            L = P["L"]
            n += norm(L["attn_norm"], pending)
            n += ok(C.gemm_wq_bf16_group(wt, P["qkv"], self.xn, M, c.hidden, flags=flags), "qkv")
            n += ok(C.attn_decode_bf16(P["attn"], flags=flags), "attention")
            n += row_linear(L["o"], self.att, self.q_loc, "o")
            n += norm(L["ffn_norm"], tp)
            n += ok(C.gemm_wq_bf16_group(wt, P["gu"], self.xn, M, c.hidden, flags=flags), "gate+up")
            n += ok(C.swiglu_bf16(self.gu, self.gu.data_ptr() + self.ffn_loc * 2, self.h, M, self.ffn_loc, 2 * self.ffn_loc, 2 * self.ffn_loc,
                                  self.ffn_loc, flags=flags), "swiglu")
            n += row_linear(L["down"], self.h, self.ffn_loc, "down")
            pending = tp
        n += norm(self.w["final_norm"], pending)
        W, S, inv = self.w["lm_head"]
        n += ok(C.gemm_wq_bf16(wt, W, S, inv, self.xn, self.logits, self.vocab_loc, M, c.hidden, flags=flags), "lm_head")
        n += ok(C.argmax_bf16(self.logits, M, self.vocab_loc, self.ids, self.best), "argmax")
        if tp:
            # every rank's winner (logit, global id) to every rank; the largest logit wins, the lowest rank on a tie
            t = self.torch
            self.cand[:M, 0] = self.best[:M]
            self.cand[:M, 1] = (self.ids[:M] + self.rank * self.vocab_loc).to(t.float32)
            self.dist.all_gather_into_tensor(self.cand_all, self.cand)
            vals = self.cand_all[:, :M, 0]
            top = vals.max(dim=0).values
            first = (vals == top.unsqueeze(0)).to(t.int32).argmax(dim=0)
            self.best[:M] = top
            self.ids[:M] = self.cand_all[:, :M, 1].gather(0, first.unsqueeze(0)).squeeze(0).to(t.int32)
        return n

    # ---- the same step as ONE persistent kernel (cuda_decode_program_*), one GPU, M <= 2 ----
    def build_program(self, M: int):
        """Records the step's layers, final norm and lm_head as a decode program; embedding and arg-max stay
        separate launches around it.  Raises ValueError where the program kernel does not take the model."""
        if self.world > 1:
            raise ValueError("the decode program runs on one GPU")
        c, C = self.cfg, self.c
        prog = C.DecodeProgram(self.wt, M)
        RES = 8

        def ok(rc, what):
            if rc != 0:
                prog.close()
                raise ValueError(f"decode program: {what} not taken ({rc})")

        groups = []
        for P in self._plan(M):
            L = P["L"]
            ok(prog.add_linears(P["qkv"], c.hidden, self.x, mode=C.X_RMSNORM, norm_weight=L["attn_norm"], eps=c.eps), "q+k+v")
            ok(prog.add_attention(P["attn"]), "attention")
            W, S, inv = L["o"]
            go = C.make_group([dict(W=W, S=S, inv=inv, N=c.hidden, Y=self.x, beta=1.0)], self.q_loc)
            ok(prog.add_linears(go, self.q_loc, self.att, mode=C.X_COPY, flags=RES), "o")
            # gate and up as one paired phase whose epilogue writes swiglu(gate, up) straight into self.h
            (Wg, Sg, ig), (Wu, Su, iu) = L["gate"], L["up"]
            gp = C.make_group([dict(W=Wg, S=Sg, inv=ig, N=self.ffn_loc, Y=self.h), dict(W=Wu, S=Su, inv=iu, N=self.ffn_loc, Y=self.h)], c.hidden)
            ok(prog.add_linears(gp, c.hidden, self.x, mode=C.X_RMSNORM, norm_weight=L["ffn_norm"], eps=c.eps, flags=16), "gate+up")
            W, S, inv = L["down"]
            gd = C.make_group([dict(W=W, S=S, inv=inv, N=c.hidden, Y=self.x, beta=1.0)], self.ffn_loc)
            ok(prog.add_linears(gd, self.ffn_loc, self.h, mode=C.X_COPY, flags=RES), "down")
            groups += [go, gp, gd]
        W, S, inv = self.w["lm_head"]
        gh = C.make_group([dict(W=W, S=S, inv=inv, N=self.vocab_loc, Y=self.logits)], c.hidden)
        ok(prog.add_linears(gh, c.hidden, self.x, mode=C.X_RMSNORM, norm_weight=self.w["final_norm"], eps=c.eps), "lm_head")
        ok(prog.finalize(), "finalize")
        self._programs = getattr(self, "_programs", {})
        self._programs[M] = (prog, groups, gh)
        return prog

    def step_program(self, M: int, from_ids: bool = True) -> int:
        """One decode step through the recorded program: embedding, ONE kernel, arg-max.  Same inputs and
        outputs as step()."""
        c, C = self.cfg, self.c
        prog = self._programs[M][0]
        n = 0
        if from_ids:
            if C.embed_bf16(self.ids, self.w["emb"], self.x, c.hidden, M, c.vocab) != 0:
                raise RuntimeError("embed failed")
            n += 1
        if prog.launch() != 0:
            raise RuntimeError("decode program launch failed")
        if C.argmax_bf16(self.logits, M, self.vocab_loc, self.ids, self.best) != 0:
            raise RuntimeError("argmax failed")
        return n + 2

    def kv_bytes_full(self, M: int, context: int) -> int:
        """Bytes of K and V rows a step of the WHOLE model (all ranks) reads when every sequence has `context` cached rows."""
        c = self.cfg
        return 2 * c.layers * M * c.n_kv_heads * context * c.head_dim * 2
