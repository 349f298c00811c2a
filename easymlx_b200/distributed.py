"""Multi-GPU layout of the paged-attention path: one process per GPU, sequences partitioned across ranks.

Sequences are independent (an output row depends only on its own sequence's pages), so every rank owns the
pages, tables and queries of its sequences and runs the single-GPU path unchanged; there is no collective on
the data path.  Only two helpers talk to ``torch.distributed``: ``gather_packed_outputs`` (reassemble the
packed output in the original batch order, used by parity checks and by callers that need the whole batch on
every rank) and ``all_gather_heads`` (KV-head sharding of one long-context batch: every rank computes the
query heads of its KV heads and the slices are all-gathered over NCCL).  The reference has no counterpart:
its only multi-device code is a replicated lock-step control plane
(``inference/esurge/distributed/``) and the page-to-shard arithmetic of ``core/dp_sharding.py:51-73``.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


def partition_by_sequence(query_lens, kv_lens, world: int, token_weight: float = 64.0) -> list[np.ndarray]:
    """Greedy longest-first assignment of sequences to ranks.  The load of a sequence is its attended KV
    tokens plus ``token_weight`` per new token (write + per-row work); ties keep batch order.  Returns, per
    rank, the sorted indices of its sequences."""
    q = np.asarray(query_lens, dtype=np.int64)
    kv = np.asarray(kv_lens, dtype=np.int64)
    if q.shape != kv.shape:
        raise ValueError("query_lens and kv_lens must have the same length")
    if world <= 0:
        raise ValueError("world must be positive")
    cost = kv + token_weight * q
    order = np.argsort(-cost, kind="stable")
    load = np.zeros(world)
    parts: list[list[int]] = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))
        parts[r].append(int(i))
        load[r] += float(cost[i])
    return [np.asarray(sorted(p), dtype=np.int64) for p in parts]


def local_token_index(query_lens, seqs: np.ndarray) -> np.ndarray:
    """Positions, in the packed global batch, of the tokens of ``seqs`` (in that order)."""
    q = np.asarray(query_lens, dtype=np.int64)
    starts = np.concatenate([[0], np.cumsum(q)])
    if len(seqs) == 0:
        return np.zeros(0, dtype=np.int64)
    return np.concatenate([np.arange(starts[s], starts[s + 1]) for s in seqs]).astype(np.int64)


def gather_packed_outputs(local_out: torch.Tensor, query_lens, parts: list[np.ndarray], group=None) -> torch.Tensor:
    """All ranks contribute the output rows of their sequences; every rank receives the packed
    ``[T, Hq, D]`` output in the original batch order."""
    world = dist.get_world_size(group)
    total = int(np.sum(query_lens))
    counts = [int(len(local_token_index(query_lens, p))) for p in parts]
    width = max(counts) if counts else 0
    padded = local_out.new_zeros((width,) + tuple(local_out.shape[1:]))
    padded[: local_out.shape[0]] = local_out
    gathered = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(gathered, padded, group=group)
    out = local_out.new_zeros((total,) + tuple(local_out.shape[1:]))
    for r in range(world):
        idx = torch.as_tensor(local_token_index(query_lens, parts[r]), device=local_out.device)
        out[idx] = gathered[r][: counts[r]]
    return out


def all_gather_heads(local_out: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """KV-head sharding: ``local_out[T, Hq/world, D]`` of every rank -> ``[T, Hq, D]`` (rank r holds query heads
    ``[r*Hq/world, (r+1)*Hq/world)``)."""
    world = dist.get_world_size(group)
    t, h, d = local_out.shape
    buf = out if out is not None else local_out.new_empty((world, t, h, d))
    dist.all_gather_into_tensor(buf.view(world * t, h, d), local_out.contiguous(), group=group)
    return buf.permute(1, 0, 2, 3).reshape(t, world * h, d)


__all__ = ("all_gather_heads", "gather_packed_outputs", "local_token_index", "partition_by_sequence")
