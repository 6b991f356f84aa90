"""Tensor-parallel sharding of the quantized-weight linears (host logic).

The reference has no tensor parallelism (its only multi-GPU mode is data-parallel training,
cccc/MainProcess.cpp:583-591, switched off in "lite"); correctness of a sharded linear is therefore
equality with the unsharded one.  Shards follow the Megatron split of a transformer layer:

  column-parallel (q, k, v, gate, up, lm_head): rank r owns output features [r*N/P, (r+1)*N/P).
      W is [N, K] with K contiguous (cccc's (K, N) column-major bytes), so the shard is ONE
      contiguous byte range of the blob, and so are its FP4 block scales.
  row-parallel (o, down): rank r owns input features [r*K/P, (r+1)*K/P) of every output row: N
      strided runs.  K/P must keep whole FP4 scale blocks (16) and, for the TMA kernels, whole k
      steps (64 elements FP8, 256 FP4).  Partial sums are added with an all-reduce.

A per-tensor FP8 scale is shared by all shards unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

FP8_E4M3, FP8_E5M2, FP4_E2M1 = 4, 5, 6


@dataclass(frozen=True)
class Shard:
    kind: str   # "col" or "row"
    n0: int
    n1: int
    k0: int
    k1: int

    @property
    def N(self) -> int:
        return self.n1 - self.n0

    @property
    def K(self) -> int:
        return self.k1 - self.k0


def k_alignment(w_type: int) -> int:
    """Granularity a row-parallel split of K must keep (whole TMA k steps, whole scale blocks)."""
    return 256 if w_type == FP4_E2M1 else 64


def column_shard(N: int, K: int, world: int, rank: int) -> Shard:
    if N % world:
        raise ValueError(f"N={N} does not divide over {world} ranks")
    n = N // world
    return Shard("col", rank * n, (rank + 1) * n, 0, K)


def row_shard(N: int, K: int, world: int, rank: int, w_type: int) -> Shard:
    a = k_alignment(w_type)
    if K % (world * a):
        raise ValueError(f"K={K} does not divide over {world} ranks in multiples of {a}")
    k = K // world
    return Shard("row", 0, N, rank * k, (rank + 1) * k)


def make_shard(kind: str, N: int, K: int, world: int, rank: int, w_type: int) -> Shard:
    return column_shard(N, K, world, rank) if kind == "col" else row_shard(N, K, world, rank, w_type)


def weight_byte_ranges(s: Shard, N: int, K: int, w_type: int):
    """(offset, length) byte ranges of the weight blob [N, K] that the shard reads, in order.
    Column shards: one range.  Row shards: one run per output row."""
    per = 2 if w_type == FP4_E2M1 else 1  # elements per byte
    if s.kind == "col":
        return [(s.n0 * K // per, s.N * K // per)]
    return [((n * K + s.k0) // per, s.K // per) for n in range(s.n0, s.n1)]


def scale_byte_ranges(s: Shard, N: int, K: int):
    """The same for the FP4 block scales (one E4M3 byte per 16 elements of the flat buffer)."""
    if s.kind == "col":
        return [(s.n0 * K // 16, s.N * K // 16)]
    return [((n * K + s.k0) // 16, s.K // 16) for n in range(s.n0, s.n1)]


def _gather(blob: np.ndarray, ranges) -> np.ndarray:
    if len(ranges) == 1:
        o, ln = ranges[0]
        return np.ascontiguousarray(blob[o:o + ln])
    return np.concatenate([blob[o:o + ln] for o, ln in ranges])


def slice_weight(W: np.ndarray, blk: np.ndarray | None, s: Shard, N: int, K: int, w_type: int):
    """The shard's compact [s.N, s.K] weight bytes (and block scales) cut out of the full blob."""
    W = np.ascontiguousarray(W, np.uint8).reshape(-1)
    Ws = _gather(W, weight_byte_ranges(s, N, K, w_type))
    bs = None
    if blk is not None:
        bs = _gather(np.ascontiguousarray(blk, np.uint8).reshape(-1), scale_byte_ranges(s, N, K))
    return Ws, bs


def slice_activation(X: np.ndarray, s: Shard) -> np.ndarray:
    """Row-parallel linears read only their K range of the activations."""
    return np.ascontiguousarray(X[:, s.k0:s.k1]) if s.kind == "row" else X


def combine(kind: str, partial, dist, world: int):
    """Column shards: concatenate features (all-gather).  Row shards: add partial sums (all-reduce).
    `partial` is a torch tensor [M, n_local]; returns the full [M, N] tensor on every rank."""
    import torch

    if world == 1:
        return partial
    if kind == "row":
        dist.all_reduce(partial)
        return partial
    parts = [torch.empty_like(partial) for _ in range(world)]
    dist.all_gather(parts, partial.contiguous())
    return torch.cat(parts, dim=1)
