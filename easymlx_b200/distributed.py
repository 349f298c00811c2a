"""Multi-GPU layout of the paged-attention path: one process per GPU, sequences partitioned across ranks.

Sequences are independent (an output row depends only on its own sequence's pages), so every rank owns the
pages, tables and queries of its sequences and runs the single-GPU path unchanged; there is no collective on
the data path.  Only two helpers talk to ``torch.distributed``: ``gather_packed_outputs`` (reassemble the
packed output in the original batch order, used by parity checks and by callers that need the whole batch on
every rank) and ``all_gather_heads`` (KV-head sharding of one long-context batch: every rank computes the
query heads of its KV heads and the slices are all-gathered over NCCL).  ``PeerGather`` removes that collective:
the attention kernels store every finished row straight into the full output buffer of every rank through
peer-mapped memory and exchange flags (``emlx_attn_decode_gather``).  The reference has no counterpart:
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


PEER_FLAG_BYTES = 512      # EMLX_PEER_FLAG_BYTES
PEER_HANDLE_BYTES = 64     # EMLX_PEER_HANDLE_BYTES
MAX_PEERS = 8              # EMLX_MAX_PEERS


class _DevicePointer:
    """Lets ``torch.as_tensor`` wrap device memory that this module allocated itself."""

    def __init__(self, ptr: int, shape: tuple[int, ...], typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}


class GatherTarget:
    """The buffers a gathering attention call writes: this rank's flag block and full ``[T, Hq, D]`` output, and the
    table of every rank's buffers as mapped into this process (``emlx_gather_init``).

    ``GatherTarget.local(...)`` builds it from plain device tensors that live in this process (one GPU playing
    every rank in turn, for tests); ``PeerGather`` builds it from buffers shared between the processes of a node."""

    def __init__(self, flag_block: int, out_ptrs: list[int], flag_ptrs: list[int], rank: int, total_q_heads: int,
                 head_offset: int, out: torch.Tensor, poll_limit: int = 0, keep=()):
        import ctypes as C

        from . import _native as nv

        world = len(out_ptrs)
        self.flag_block, self.rank, self.world = int(flag_block), int(rank), world
        self.total_q_heads, self.head_offset = int(total_q_heads), int(head_offset)
        self.out = out                      # this rank's full output, [T_max, total_q_heads, D]
        self._keep = keep
        outs = (C.c_void_p * world)(*out_ptrs)
        flags = (C.c_void_p * world)(*flag_ptrs)
        nv.check(nv.lib().emlx_gather_init(C.c_void_p(self.flag_block), outs, flags, world, rank, int(poll_limit),
                                           nv.stream_ptr(out.device)))

    @classmethod
    def local(cls, outs: list[torch.Tensor], flags: list[torch.Tensor], rank: int, head_offset: int,
              poll_limit: int = 0) -> "GatherTarget":
        return cls(flags[rank].data_ptr(), [o.data_ptr() for o in outs], [f.data_ptr() for f in flags], rank,
                   int(outs[rank].shape[1]), head_offset, outs[rank], poll_limit, keep=(outs, flags))


class PeerGather:
    """KV-head sharding without the all-gather: one buffer per rank (flag block + full ``[T_max, Hq, D]`` output) in
    memory the other ranks of the node map (``emlx_peer_buffer_create`` / ``_open``, handles exchanged with
    ``all_gather_object``).  ``target`` is what ``AttentionCall(..., gather=...)`` takes; ``output(T)`` is the
    gathered result of the last call.  Every rank must make the same calls; what reads ``output`` must be queued on
    the calling stream before the next call."""

    def __init__(self, max_tokens: int, total_q_heads: int, head_dim: int, dtype: torch.dtype, device, group=None,
                 poll_limit: int = 0):
        import ctypes as C

        from . import _native as nv

        lib = nv.lib()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks")
        if total_q_heads % self.world:
            raise ValueError("total_q_heads must divide by the number of ranks")
        self.device = torch.device(device)
        item = torch.empty((), dtype=dtype).element_size()
        out_bytes = max_tokens * total_q_heads * head_dim * item
        self._bytes = PEER_FLAG_BYTES + out_bytes
        self._own, self._mapped = 0, []
        with torch.cuda.device(self.device):
            # every step that can fail is followed by an exchange of what happened, so that the ranks fail together
            # instead of leaving one another in a collective
            ptr, handle = C.c_void_p(), (C.c_ubyte * PEER_HANDLE_BYTES)()
            rc = lib.emlx_peer_buffer_create(self._bytes, C.byref(ptr), handle)
            mine = bytes(handle) if rc == nv.EMLX_OK else nv.last_error()
            self._own = int(ptr.value or 0) if rc == nv.EMLX_OK else 0
            handles: list = [None] * self.world
            dist.all_gather_object(handles, mine, group=group)
            bases, problem = [], next((h for h in handles if isinstance(h, str)), None)
            if problem is None:
                for r in range(self.world):
                    if r == self.rank:
                        bases.append(self._own)
                        continue
                    p = C.c_void_p()
                    buf = (C.c_ubyte * PEER_HANDLE_BYTES).from_buffer_copy(handles[r])
                    if lib.emlx_peer_buffer_open(buf, C.byref(p)) != nv.EMLX_OK:
                        problem = nv.last_error()
                        break
                    self._mapped.append(int(p.value))
                    bases.append(int(p.value))
            problems: list = [None] * self.world
            dist.all_gather_object(problems, problem, group=group)
            problem = next((x for x in problems if x), None)
            if problem is not None:
                for p in self._mapped:
                    lib.emlx_peer_buffer_close(p)
                if self._own:
                    lib.emlx_peer_buffer_free(self._own)
                self._own, self._mapped = 0, []
                raise RuntimeError(f"peer-mapped buffers are not available: {problem}")
            typestr = {torch.float16: "<f2", torch.bfloat16: "<u2"}[dtype]
            full = torch.as_tensor(_DevicePointer(self._own + PEER_FLAG_BYTES, (max_tokens, total_q_heads, head_dim), typestr),
                                   device=self.device)
            if dtype == torch.bfloat16:
                full = full.view(torch.bfloat16)
            self.target = GatherTarget(self._own, [b + PEER_FLAG_BYTES for b in bases], bases, self.rank, total_q_heads,
                                       self.rank * (total_q_heads // self.world), full, poll_limit)
            torch.cuda.synchronize(self.device)
        dist.barrier(group=group)   # every rank's table is in place before anyone's first call

    def output(self, tokens: int) -> torch.Tensor:
        return self.target.out[:tokens]

    def close(self) -> None:
        """Unmaps the other ranks' buffers and frees this rank's (after a barrier: nobody may still be storing)."""
        from . import _native as nv

        lib = nv.lib()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for p in self._mapped:
            lib.emlx_peer_buffer_close(p)
        self._mapped = []
        dist.barrier(group=self.group)
        if self._own:
            lib.emlx_peer_buffer_free(self._own)
            self._own = 0


__all__ = ("GatherTarget", "PeerGather", "all_gather_heads", "gather_packed_outputs", "local_token_index", "partition_by_sequence")
