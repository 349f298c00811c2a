"""Paged KV cache on CUDA tensors.

Host-side mirror of easymlx ``caching/paged/cache.py``: ``PageCacheView``
(``:499-1306``), ``PageCacheConfig`` / ``PageCache`` (``:1309-1445``),
``build_query_start_loc`` (``:1448-1465``) and ``PageMetadata`` (``:1468-1543``) keep
their names, arguments and return values.  The index arithmetic and the scatter of
``concatenate_to_cache`` run in two CUDA kernels (``emlx_build_metadata``,
``emlx_kv_write``) instead of host loops and fancy-index assignments; nothing here
synchronises with the device.

Storage modes: ``float16`` / ``bfloat16`` / ``float32`` pools in the reference layout
``[num_blocks, block_size, num_kv_heads, head_dim]``, and affine group-64 pools with 8 or
4 bits (``cache_dtype="affine8" | "affine4"`` or ``cache_bits=8 | 4``), which the reference
does not have.  Its ``fp8`` and ``turboquant`` modes are not provided.
"""

from __future__ import annotations

import math
import os
import typing as tp
from collections import OrderedDict
from dataclasses import dataclass, field

import torch

from ... import _native as nv

_CHECK = os.environ.get("EASYMLX_B200_CHECK", "0") not in ("", "0")
QUANT_GROUP = 64
_FUSED_STEP_MAX_SEQS = 2048  # batch size up to which emlx_kv_write_step serves a batch in one launch

def wide_units_geometry(num_q_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    """Head geometry the 128-row (tcgen05) kernel can run: a GQA group that divides 128 and head_dim 64 or 128."""
    if num_kv_heads <= 0 or num_q_heads % num_kv_heads:
        return False
    group = num_q_heads // num_kv_heads
    return head_dim in (64, 128) and group <= 128 and 128 % group == 0


_TORCH_DTYPES = {
    "float16": torch.float16, "half": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
    "torch.float16": torch.float16, "torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32,
}


def _resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    name = getattr(dtype, "__name__", None) or str(dtype)
    return _TORCH_DTYPES.get(name.replace("numpy.", "").replace("<class '", "").replace("'>", ""), torch.float16)


def _resolve_bits(cache_dtype: str | None, cache_bits: int | None) -> int:
    """0 for a float pool, 8 or 4 for an affine pool."""
    mode = str(cache_dtype or "auto").lower()
    if mode in ("fp8",) or mode.startswith("turboquant"):
        raise NotImplementedError(f"cache_dtype={cache_dtype!r} is not provided; use float16/bfloat16/float32 or affine8/affine4")
    if mode in ("affine", "affine8", "int8", "q8"):
        bits = 8 if mode != "affine" else int(cache_bits or 8)
    elif mode in ("affine4", "int4", "q4"):
        bits = 4
    else:
        return 0
    if bits not in (4, 8):
        raise ValueError("affine KV supports 8 or 4 bits")
    return bits


class _DeviceIntCache:
    """Small LRU of host integer tuples already uploaded (the reference keeps an LRU of 64 start-location
    arrays for the same reason, ``inference/esurge/runners/model_runner.py:559-570``)."""

    def __init__(self, capacity: int = 64):
        self.capacity = capacity
        self.items: OrderedDict = OrderedDict()

    def get(self, values: tuple[int, ...], device) -> torch.Tensor:
        key = (values, str(device))
        hit = self.items.get(key)
        if hit is not None:
            self.items.move_to_end(key)
            return hit
        t = torch.tensor(values, dtype=torch.int32).pin_memory().to(device, non_blocking=True) if values else \
            torch.zeros(0, dtype=torch.int32, device=device)
        self.items[key] = t
        if len(self.items) > self.capacity:
            self.items.popitem(last=False)
        return t


_uploaded = _DeviceIntCache()


def build_query_start_loc(query_lens: tp.Iterable[int], device=None) -> torch.Tensor:
    """``[0, q0, q0+q1, ...]`` as int32 (host prefix sum, like the reference; the packed-batch path
    builds the same array on the GPU inside ``concatenate_to_cache``)."""
    offsets = [0]
    for n in query_lens:
        offsets.append(offsets[-1] + int(n))
    return torch.tensor(offsets, dtype=torch.int32, device=device)


@dataclass
class PageMetadata:
    """Kernel-agnostic paged-attention metadata; same fields as the reference's dataclass."""

    query_start_loc: tp.Any
    block_tables: tp.Any | None = None
    kv_lens: tp.Any | None = None
    block_size: int | None = None
    sliding_window: int | None = None
    is_single_token_decode: bool = False
    slot_ids: tuple[int, ...] | None = None
    # filled by concatenate_to_cache: upper bound of query tokens per sequence known on the host (0 = unknown)
    max_query_len: int = field(default=0, compare=False)
    # filled by concatenate_to_cache: the distinct query lengths of the batch when the host knows them; lets the
    # attention call skip the kernels of row classes the batch does not contain
    query_len_set: tuple[int, ...] | None = field(default=None, compare=False)
    # filled by concatenate_to_cache: sequences of the batch with more than 16 query rows (tokens x GQA group), when the
    # host knows the lengths; over an affine pool those rows then go to the tcgen05 kernel through expanded pages
    long_seqs: int = field(default=0, compare=False)
    # attention work list built on the GPU together with the metadata: (buffer, num_q_heads, sliding_window, plan_flags)
    plan: tp.Any | None = field(default=None, compare=False)
    # optional host hint from the runner: length of the longest scheduled sequence after this step (0 = unknown);
    # a length-dependent rotary embedding (longrope) picks its table from it without reading the device
    max_kv_len: int = field(default=0, compare=False)

    def with_cache_state(self, *, block_tables, kv_lens, block_size: int) -> "PageMetadata":
        return PageMetadata(
            query_start_loc=self.query_start_loc, block_tables=block_tables, kv_lens=kv_lens,
            block_size=int(block_size), sliding_window=self.sliding_window,
            is_single_token_decode=self.is_single_token_decode, slot_ids=self.slot_ids,
            max_query_len=self.max_query_len, plan=self.plan, query_len_set=self.query_len_set,
            long_seqs=self.long_seqs,
        )

    def with_sliding_window(self, sliding_window: int | None) -> "PageMetadata":
        return PageMetadata(
            query_start_loc=self.query_start_loc, block_tables=self.block_tables, kv_lens=self.kv_lens,
            block_size=self.block_size, sliding_window=sliding_window,
            is_single_token_decode=self.is_single_token_decode, slot_ids=self.slot_ids,
            max_query_len=self.max_query_len, query_len_set=self.query_len_set, long_seqs=self.long_seqs,
        )


def expanded_page_hint(query_lens, group: int) -> int:
    """Number of sequences with more than 16 query rows, or 0 when expanding their pages does not pay.

    The hint sizes the scratch of the expanded-page route of an affine pool.  The route pays off for prefill chunks
    (hundreds of rows re-read their context once per 32-row unit otherwise); for rows of a few dozen (speculative-
    decoding verification) expanding every page costs more than it saves (measured on a spec-verify batch over an
    8-bit pool: 1.15 ms on the 32-row units, 1.48 ms through expanded pages), so the hint is only given when those
    sequences average at least 64 rows.  ``query_lens`` unknown on the host (``None``) gives 0.
    """
    if query_lens is None:
        return 0
    long_rows = [q * group for q in query_lens if q * group > 16]
    return len(long_rows) if long_rows and sum(long_rows) >= 64 * len(long_rows) else 0


class PageCacheView:
    """Block-table based KV cache backed by CUDA tensors.

    ``key_cache`` / ``value_cache``: ``[num_blocks, block_size, num_kv_heads, head_dim]`` for float pools.
    Affine pools (``cache_bits`` 8 or 4) hold bytes instead: keys ``[NB, bs, Hkv, D*bits/8]``, values
    ``[NB, Hkv, D, bs*bits/8]`` and fp16 ``k_scales/k_biases/v_scales/v_biases [NB, Hkv, bs, D/64]``.
    ``block_tables [num_seqs, blocks_per_seq]`` and ``kv_lens [num_seqs]`` are int32; the runner writes
    them directly, as it does in the reference (``inference/esurge/runners/model_runner.py:1127-1131``).
    """

    def __init__(self, *, key_cache, value_cache, block_tables, kv_lens, block_size: int, num_kv_heads: int,
                 head_dim: int, page_key_cache=None, page_value_cache=None, page_vec_size: int | None = None,
                 cache_dtype_is_fp8: bool = False, k_scales=None, v_scales=None, k_biases=None, v_biases=None,
                 cache_bits: int = 0) -> None:
        if cache_dtype_is_fp8:
            raise NotImplementedError("fp8 KV pools are not provided")
        if page_key_cache is not None or page_value_cache is not None:
            raise NotImplementedError("the packed side caches of the PageAttention runtime are not provided")
        self.key_cache, self.value_cache = key_cache, value_cache
        self.block_tables, self.kv_lens = block_tables, kv_lens
        self.block_size, self.num_kv_heads, self.head_dim = int(block_size), int(num_kv_heads), int(head_dim)
        self.page_key_cache = self.page_value_cache = None
        self.page_vec_size = 0
        self.cache_dtype_is_fp8 = False
        self.k_scales, self.v_scales, self.k_biases, self.v_biases = k_scales, v_scales, k_biases, v_biases
        self.cache_bits = int(cache_bits)
        self._status: torch.Tensor | None = None
        self._ticket: torch.Tensor | None = None
        self._validate_shape()

    # ------------------------------------------------------------------ geometry
    @property
    def cache(self) -> "PageCacheView":
        return self

    @property
    def blocks_per_seq(self) -> int:
        return int(self.block_tables.shape[1])

    @property
    def num_seqs(self) -> int:
        return int(self.block_tables.shape[0])

    @property
    def max_seq_len(self) -> int:
        return self.blocks_per_seq * self.block_size

    @property
    def num_blocks(self) -> int:
        return int(self.key_cache.shape[0])

    @property
    def is_affine(self) -> bool:
        return self.cache_bits in (4, 8)

    @property
    def status(self) -> torch.Tensor:
        """Device word the kernels OR their validation bits into (see ``check``)."""
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=self.key_cache.device)
        return self._status

    @property
    def ticket(self) -> torch.Tensor:
        """Arrival counter of the fused decode step (zero between launches; the kernel resets it)."""
        if self._ticket is None:
            self._ticket = torch.zeros(1, dtype=torch.int32, device=self.key_cache.device)
        return self._ticket

    def check(self) -> None:
        """Synchronise and raise if any kernel that used this cache flagged a bad slot / page / overflow."""
        rc = nv.lib().emlx_read_status(nv.ptr(self.status), nv.stream_ptr(self.key_cache.device))
        if rc != nv.EMLX_OK:
            self.status.zero_()  # report once
        nv.check(rc)

    def _validate_shape(self) -> None:
        if self.block_tables.ndim != 2:
            raise ValueError("block_tables must be rank-2: [num_seqs, blocks_per_seq]")
        if self.kv_lens.ndim != 1:
            raise ValueError("kv_lens must be rank-1: [num_seqs]")
        if self.key_cache.ndim != 4 or self.value_cache.ndim != 4:
            raise ValueError("key_cache/value_cache must be rank-4.")
        num_seqs, blocks_per_seq = self.block_tables.shape
        if self.kv_lens.shape[0] != num_seqs:
            raise ValueError("kv_lens length must match block_tables first dimension.")
        nb, bs, hkv, d = self.key_cache.shape[0], self.block_size, self.num_kv_heads, self.head_dim
        if self.is_affine:
            bits = self.cache_bits
            if d % QUANT_GROUP or bs % 8:
                raise ValueError("affine KV needs head_dim % 64 == 0 and block_size % 8 == 0")
            if tuple(self.key_cache.shape) != (nb, bs, hkv, d * bits // 8) or self.key_cache.dtype != torch.uint8:
                raise ValueError("affine key_cache must be uint8 [num_blocks, block_size, num_kv_heads, head_dim*bits/8]")
            if tuple(self.value_cache.shape) != (nb, hkv, d, bs * bits // 8) or self.value_cache.dtype != torch.uint8:
                raise ValueError("affine value_cache must be uint8 [num_blocks, num_kv_heads, head_dim, block_size*bits/8]")
            for t in (self.k_scales, self.k_biases, self.v_scales, self.v_biases):
                if t is None or tuple(t.shape) != (nb, hkv, bs, d // QUANT_GROUP) or t.dtype != torch.float16:
                    raise ValueError("affine scale/bias must be float16 [num_blocks, num_kv_heads, block_size, head_dim/64]")
        else:
            if self.key_cache.shape != self.value_cache.shape:
                raise ValueError("key_cache and value_cache must have the same shape.")
            if self.key_cache.shape[1] != bs:
                raise ValueError("key_cache block size does not match block_size.")
            if self.key_cache.shape[2] != hkv:
                raise ValueError("key_cache num_kv_heads does not match configured value.")
            if self.key_cache.shape[3] != d:
                raise ValueError("key_cache head_dim does not match configured value.")

    # ------------------------------------------------------------------ allocation
    @classmethod
    def init(cls, *, num_seqs: int, max_seq_len: int, num_kv_heads: int, head_dim: int, block_size: int = 16,
             dtype=torch.float16, cache_dtype: str | None = None, cache_bits: int | None = None,
             device=None, num_blocks: int | None = None) -> "PageCacheView":
        """Zeroed pool with the reference's contiguous table: slot ``i`` owns pages
        ``[i*blocks_per_seq, (i+1)*blocks_per_seq)`` (``caching/paged/cache.py:779-791``).  ``num_blocks``
        overrides the pool size for callers that manage page ids themselves."""
        if num_seqs <= 0:
            raise ValueError("num_seqs must be positive")
        if max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        device = torch.device(device if device is not None else "cuda")
        bits = _resolve_bits(cache_dtype, cache_bits)
        mode = str(cache_dtype or "auto").lower()
        pool_dtype = _TORCH_DTYPES.get(mode, _resolve_dtype(dtype))
        blocks_per_seq = math.ceil(max_seq_len / block_size)
        nb = int(num_blocks) if num_blocks is not None else blocks_per_seq * num_seqs
        tables = torch.arange(blocks_per_seq * num_seqs, dtype=torch.int32, device=device).reshape(num_seqs, blocks_per_seq)
        kv_lens = torch.zeros(num_seqs, dtype=torch.int32, device=device)
        extra: dict = {}
        if bits:
            kc = torch.zeros((nb, block_size, num_kv_heads, head_dim * bits // 8), dtype=torch.uint8, device=device)
            vc = torch.zeros((nb, num_kv_heads, head_dim, block_size * bits // 8), dtype=torch.uint8, device=device)
            sb = (nb, num_kv_heads, block_size, head_dim // QUANT_GROUP)
            extra = dict(k_scales=torch.zeros(sb, dtype=torch.float16, device=device),
                         k_biases=torch.zeros(sb, dtype=torch.float16, device=device),
                         v_scales=torch.zeros(sb, dtype=torch.float16, device=device),
                         v_biases=torch.zeros(sb, dtype=torch.float16, device=device), cache_bits=bits)
        else:
            kc = torch.zeros((nb, block_size, num_kv_heads, head_dim), dtype=pool_dtype, device=device)
            vc = torch.zeros_like(kc)
        return cls(key_cache=kc, value_cache=vc, block_tables=tables, kv_lens=kv_lens, block_size=block_size,
                   num_kv_heads=num_kv_heads, head_dim=head_dim, **extra)

    allocate = init

    def can_append(self, seq_idx: int, num_new_tokens: int) -> bool:
        if num_new_tokens < 0:
            raise ValueError("num_new_tokens must be non-negative.")
        if seq_idx < 0 or seq_idx >= self.num_seqs:
            raise IndexError(f"Invalid seq_idx {seq_idx}")
        return int(self.kv_lens[seq_idx].item()) + int(num_new_tokens) <= self.max_seq_len

    # ------------------------------------------------------------------ native descriptors
    def native_pool(self) -> nv.Pool:
        p = nv.Pool()
        p.key_cache, p.value_cache = self.key_cache.data_ptr(), self.value_cache.data_ptr()
        if self.is_affine:
            p.k_scale, p.k_bias = self.k_scales.data_ptr(), self.k_biases.data_ptr()
            p.v_scale, p.v_bias = self.v_scales.data_ptr(), self.v_biases.data_ptr()
            p.kv_format, p.kv_dtype = self.cache_bits, nv.F16
        else:
            p.kv_format, p.kv_dtype = nv.KV_FLOAT, nv.dtype_code(self.key_cache.dtype)
        p.num_blocks, p.block_size = self.num_blocks, self.block_size
        p.num_kv_heads, p.head_dim = self.num_kv_heads, self.head_dim
        return p

    # ------------------------------------------------------------------ writes
    def _write_batch(self, keys: torch.Tensor, values: torch.Tensor, query_lens_dev: torch.Tensor,
                     slots_dev: torch.Tensor, total_tokens: int, plan_for: tuple | None = None,
                     advance: bool = True, rope=None, queries: torch.Tensor | None = None,
                     single_token: bool = False):
        """Batch metadata, attention work list and KV write for one packed batch: one launch for up to 2048 sequences
        (``single_token``: every sequence brings exactly one token, no prefix sum needed), else the metadata kernel
        followed by the write kernel.  Returns ``(qsl, block_tables, kv_lens)`` of the scheduled rows;
        ``self.kv_lens`` is advanced in place."""
        nv.require_cuda(keys, values, self.key_cache)
        dev = self.key_cache.device
        lib, stream = nv.lib(), nv.stream_ptr(dev)
        s = int(slots_dev.shape[0])
        qsl = torch.empty(s + 1, dtype=torch.int32, device=dev)
        bt = torch.empty((s, self.blocks_per_seq), dtype=torch.int32, device=dev)
        lens = torch.empty(s, dtype=torch.int32, device=dev)
        slot_mapping = torch.empty(max(total_tokens, 1), dtype=torch.int64, device=dev)
        positions = torch.empty(max(total_tokens, 1), dtype=torch.int32, device=dev) if rope is not None else None
        rotated_q = None
        if self.block_tables.dtype != torch.int32 or self.kv_lens.dtype != torch.int32:
            raise ValueError("block_tables and kv_lens must be int32")
        if not (self.block_tables.is_contiguous() and self.kv_lens.is_contiguous()):
            raise ValueError("block_tables and kv_lens must be contiguous")
        plan = None
        hq = window = max_q = plan_bytes = flags = 0
        if plan_for is not None and total_tokens > 0 and (
                self.block_size == 128 or (not self.is_affine and self.block_size in (16, 32, 64))):
            hq, window, max_q = plan_for[:3]
            flags = int(lib.emlx_attn_plan_flags(self.cache_bits if self.is_affine else nv.KV_FLOAT, hq,
                                                 self.num_kv_heads, self.head_dim))
            if self.is_affine and len(plan_for) > 3 and plan_for[3] > 0 and wide_units_geometry(hq, self.num_kv_heads, self.head_dim):
                flags |= 1  # long rows in 128-row units: the attention call expands their pages for the tcgen05 kernel
            plan_bytes = int(lib.emlx_attn_plan_bytes(s, total_tokens, hq, self.num_kv_heads))
            plan = torch.empty(plan_bytes, dtype=torch.uint8, device=dev)
        if total_tokens > 0:
            if keys.shape != values.shape:
                raise ValueError("key and value must have the same shape")
            if keys.ndim != 3 or keys.shape[1] != self.num_kv_heads or keys.shape[2] != self.head_dim:
                raise ValueError("key/value must be [num_tokens, num_kv_heads, head_dim] matching the cache")
            if keys.dtype != values.dtype:
                raise ValueError("key and value must have the same dtype")
            keys, values = keys.contiguous(), values.contiguous()
            if rope is not None:
                if not hasattr(rope, "native"):
                    raise TypeError("rope must be an easymlx_b200.layers.rotary.RotaryEmbedding (see get_rope)")
                if queries.dtype != keys.dtype:
                    raise ValueError("queries and keys must have the same dtype when RoPE is fused into the write")
                queries = queries.contiguous()
                rotated_q = torch.empty_like(queries)
        if 0 < total_tokens and 0 < s <= _FUSED_STEP_MAX_SEQS:
            # metadata, work list and write in one launch (the reference's concatenate_to_cache, cache.py:1123-1306);
            # a batch of single tokens (its decode fast path, :1155-1206) skips the prefix sum of the query lengths
            decode = single_token and total_tokens == s
            nv.check(lib.emlx_kv_write_step(
                nv.ptr(queries) if rope is not None else None, nv.ptr(rotated_q), nv.ptr(keys), nv.ptr(values),
                nv.dtype_code(keys.dtype), None if decode else nv.ptr(query_lens_dev), nv.ptr(slots_dev), s, total_tokens,
                nv.ptr(self.block_tables), self.num_seqs, self.blocks_per_seq, nv.ptr(self.kv_lens), 1 if advance else 0,
                self.native_pool(), rope.native(dev) if rope is not None else None, nv.ptr(qsl), nv.ptr(bt), nv.ptr(lens),
                hq if plan is not None else (int(queries.shape[1]) if rope is not None else 0), window, max_q, flags,
                nv.ptr(plan), plan_bytes, nv.ptr(self.ticket), nv.ptr(self.status), stream))
            if _CHECK and not torch.cuda.is_current_stream_capturing():
                self.check()
            return qsl, bt, lens, (None if plan is None else (plan, hq, window, flags)), rotated_q
        nv.check(lib.emlx_build_metadata(
            nv.ptr(query_lens_dev), nv.ptr(slots_dev), s, total_tokens, nv.ptr(self.block_tables), self.num_seqs,
            self.blocks_per_seq, nv.ptr(self.kv_lens), self.block_size, 1 if advance else 0, nv.ptr(qsl), nv.ptr(bt),
            nv.ptr(lens), nv.ptr(slot_mapping), nv.ptr(positions), self.num_blocks, nv.ptr(self.status), hq, self.num_kv_heads, window, max_q,
            flags, nv.ptr(plan), plan_bytes, stream))
        if total_tokens > 0:
            pool = self.native_pool()
            if rope is None:
                nv.check(lib.emlx_kv_write(nv.ptr(keys), nv.ptr(values), nv.dtype_code(keys.dtype), total_tokens,
                                           nv.ptr(slot_mapping), pool, nv.ptr(self.status), stream))
            else:
                nv.check(lib.emlx_kv_write_rope(
                    nv.ptr(queries), nv.ptr(rotated_q), int(queries.shape[1]), nv.ptr(keys), nv.ptr(values),
                    nv.dtype_code(keys.dtype), total_tokens, nv.ptr(slot_mapping), nv.ptr(positions),
                    rope.native(dev), pool, nv.ptr(self.status), stream))
        if _CHECK and not torch.cuda.is_current_stream_capturing():
            self.check()
        return qsl, bt, lens, (None if plan is None else (plan, hq, window, flags)), rotated_q

    def append(self, seq_idx: int, key: torch.Tensor, value: torch.Tensor) -> None:
        """Append ``[num_tokens, num_kv_heads, head_dim]`` rows to one slot (``cache.py:834-872``)."""
        if key.shape != value.shape:
            raise ValueError("key and value must have the same shape")
        if key.ndim != 3:
            raise ValueError("key/value must be rank-3: [num_tokens, num_kv_heads, head_dim]")
        if key.shape[1] != self.num_kv_heads or key.shape[2] != self.head_dim:
            raise ValueError("key/value head dims do not match cache")
        if seq_idx < 0 or seq_idx >= self.num_seqs:
            raise IndexError(f"Invalid seq_idx {seq_idx}")
        n = int(key.shape[0])
        dev = self.key_cache.device
        self._write_batch(key, value, _uploaded.get((n,), dev), _uploaded.get((int(seq_idx),), dev), n)  # noqa

    def reset(self, seq_idx: int) -> None:
        """Zero a slot's length.  (The reference also zero-fills the slot's pages; stale rows beyond
        ``kv_lens`` are never read by the kernels, so only the length is reset here.)"""
        if seq_idx < 0 or seq_idx >= self.num_seqs:
            raise IndexError(f"Invalid seq_idx {seq_idx}")
        self.kv_lens[seq_idx] = 0

    def reset_batch(self, seq_indices: tp.Sequence[int]) -> None:
        for i in seq_indices:
            self.reset(int(i))

    def clear(self, seq_idx: int | None = None) -> None:
        if seq_idx is None:
            self.kv_lens.zero_()
            return
        self.reset(int(seq_idx))

    def clear_many(self, seq_indices: tp.Iterable[int]) -> None:
        for i in seq_indices:
            self.reset(int(i))

    # ------------------------------------------------------------------ page maintenance
    def _int32_on_device(self, values, cols: int | None = None) -> tuple[torch.Tensor, torch.Tensor | None]:
        """(device int32 tensor, host copy or None when the caller passed a device tensor)."""
        dev = self.key_cache.device
        if isinstance(values, torch.Tensor) and values.is_cuda:
            t = values.to(dtype=torch.int32).contiguous()
            host = None
        else:
            host = torch.as_tensor(values, dtype=torch.int32).reshape(-1, cols) if cols else \
                torch.as_tensor(values, dtype=torch.int32).reshape(-1)
            t = host.to(dev)
        return t, host

    def copy_blocks(self, block_mapping, *, assume_independent: bool = False) -> None:
        """Copy-on-write page copies (``caching/paged/cache.py:944-972``): ``block_mapping [num_pairs, 2]`` holds
        ``(src_block, dst_block)`` rows; every destination receives its source as it was before the call.

        A mapping given on the host is inspected: when no page is both read and written and no destination
        repeats, one in-place launch does it.  Otherwise (or for a device-resident mapping, unless
        ``assume_independent``) the pages go through a staging buffer in two launches."""
        if isinstance(block_mapping, torch.Tensor):
            if block_mapping.ndim != 2 or block_mapping.shape[1] != 2:
                raise ValueError("block_mapping must be rank-2 with shape [num_pairs, 2]")
        mapping, host = self._int32_on_device(block_mapping, cols=2)
        if mapping.ndim != 2 or mapping.shape[1] != 2:
            raise ValueError("block_mapping must be rank-2 with shape [num_pairs, 2]")
        pairs = int(mapping.shape[0])
        if pairs == 0:
            return
        independent = assume_independent
        if host is not None:
            src, dst = set(host[:, 0].tolist()), host[:, 1].tolist()
            independent = len(set(dst)) == len(dst) and not (src & set(dst))
        pool = self.native_pool()
        lib = nv.lib()
        dev = self.key_cache.device
        staging, staging_bytes = None, 0
        if not independent:
            staging_bytes = pairs * int(lib.emlx_page_staging_bytes(pool))
            staging = torch.empty(staging_bytes, dtype=torch.uint8, device=dev)
        nv.check(lib.emlx_copy_blocks(pool, nv.ptr(mapping), pairs, nv.ptr(staging), staging_bytes, nv.ptr(self.status),
                                      nv.stream_ptr(dev)))
        if _CHECK and not torch.cuda.is_current_stream_capturing():
            self.check()

    def zero_pages(self, page_ids) -> None:
        """Zero the listed pages in every array of the pool; ids below zero or past the pool are skipped
        (``inference/esurge/runners/model_runner.py:1058-1094``)."""
        ids, _ = self._int32_on_device(page_ids)
        if ids.numel() == 0:
            return
        dev = self.key_cache.device
        nv.check(nv.lib().emlx_zero_pages(self.native_pool(), nv.ptr(ids), int(ids.numel()), nv.stream_ptr(dev)))

    def gather_kv_cache(self, block_table, cu_seq_lens, *, out_dtype=None) -> tuple[torch.Tensor, torch.Tensor]:
        """Contiguous ``[total_tokens, num_kv_heads, head_dim]`` K and V of the sequences whose pages ``block_table
        [num_seqs, max_blocks]`` lists and whose lengths ``cu_seq_lens [num_seqs + 1]`` accumulates
        (``caching/paged/cache.py:974-1027``).  Affine pools come back dequantised."""
        dev = self.key_cache.device
        bt = torch.as_tensor(block_table).to(device=dev, dtype=torch.int32).contiguous()
        if bt.ndim != 2:
            raise ValueError("block_table must be rank-2: [num_seqs, max_blocks_per_seq]")
        cu_host = cu_seq_lens.tolist() if isinstance(cu_seq_lens, torch.Tensor) else list(cu_seq_lens)
        if len(cu_host) != bt.shape[0] + 1:
            raise ValueError("cu_seq_lens must have num_seqs + 1 entries")
        total = int(cu_host[-1])
        cu = torch.as_tensor(cu_host, dtype=torch.int32).to(dev)
        if out_dtype is None:
            out_dtype = torch.float16 if self.is_affine else self.key_cache.dtype
        out_dtype = _resolve_dtype(out_dtype)
        k_out = torch.empty((total, self.num_kv_heads, self.head_dim), dtype=out_dtype, device=dev)
        v_out = torch.empty_like(k_out)
        nv.check(nv.lib().emlx_gather_kv_cache(self.native_pool(), nv.ptr(bt), int(bt.shape[0]), int(bt.shape[1]), nv.ptr(cu),
                                               total, nv.dtype_code(out_dtype), nv.ptr(k_out), nv.ptr(v_out),
                                               nv.ptr(self.status), nv.stream_ptr(dev)))
        if _CHECK and not torch.cuda.is_current_stream_capturing():
            self.check()
        return k_out, v_out

    def dequantize_kv_cache(self, key_cache: torch.Tensor, value_cache: torch.Tensor, *, block_tables=None,
                            out_dtype=torch.float16) -> tuple[torch.Tensor, torch.Tensor]:
        """Float pools are returned as they are (``cache.py:1050-1086`` does the same when the pool is not quantised); an
        affine pool comes back as ``[num_blocks, block_size, num_kv_heads, head_dim]`` tensors of ``out_dtype``."""
        del block_tables
        if not self.is_affine:
            return key_cache, value_cache
        nb, bs = self.num_blocks, self.block_size
        table = torch.arange(nb, dtype=torch.int32, device=self.key_cache.device).reshape(nb, 1)
        cu = [i * bs for i in range(nb + 1)]
        k, v = self.gather_kv_cache(table, cu, out_dtype=out_dtype)
        shape = (nb, bs, self.num_kv_heads, self.head_dim)
        return k.reshape(shape), v.reshape(shape)

    def concatenate_to_cache(self, queries: torch.Tensor, keys: torch.Tensor, values: torch.Tensor, *,
                             cache_metadata: tp.Any, rope: tp.Any = None,
                             slot_ids: tp.Sequence[int] | None = None,
                             query_lens: tp.Sequence[int] | None = None, advance: bool = True):
        """Append the batch's K/V to the pool and resolve the metadata (``cache.py:1088-1306``).

        Returns ``(prepared_queries, key_cache, value_cache, resolved_metadata)``; the metadata carries the
        scheduled slots' page-table rows and their lengths after the write.  ``rope`` (a ``RotaryEmbedding``) is
        applied to queries and keys at each token's position in its sequence, inside the write kernel.  ``slot_ids`` and
        ``query_lens`` are host sequences, as in the reference; when ``query_lens`` is omitted the lengths
        are derived on the device from ``cache_metadata.query_start_loc``.  ``advance=False`` (an extension)
        writes the rows and resolves the metadata but leaves ``self.kv_lens`` untouched, so that the same batch
        can be replayed (benchmarks, speculative what-if steps).
        """
        if slot_ids is None:
            slot_ids = getattr(cache_metadata, "slot_ids", None) or ()
        slots = tuple(int(s) for s in slot_ids)
        dev = self.key_cache.device
        total = int(queries.shape[0])
        max_q = 0
        qlens = None
        if query_lens is not None:
            qlens = tuple(max(0, int(q)) for q in query_lens)
            qlens_dev = _uploaded.get(qlens, dev)
            max_q = max(qlens, default=0)
            single = bool(qlens) and total == len(qlens) and max_q == 1 and min(qlens) == 1
        else:
            qsl_in = cache_metadata.query_start_loc
            if not isinstance(qsl_in, torch.Tensor):
                qsl_in = torch.as_tensor(list(qsl_in), dtype=torch.int32)
                qlens = tuple(int(x) for x in (qsl_in[1:] - qsl_in[:-1]).tolist())[: len(slots)]
                qlens_dev = _uploaded.get(tuple(max(0, q) for q in qlens), dev)
                max_q = max(qlens, default=0)
                single = bool(qlens) and total == len(qlens) and all(q == 1 for q in qlens)
            else:
                qlens_dev = (qsl_in[1:len(slots) + 1] - qsl_in[:len(slots)]).to(device=dev, dtype=torch.int32).contiguous()
                single = bool(getattr(cache_metadata, "is_single_token_decode", False)) and total == len(slots)
                max_q = 1 if single else 0
        window = int(getattr(cache_metadata, "sliding_window", None) or 0)
        if rope is not None and hasattr(rope, "select"):
            # longrope: one table per batch, chosen from the longest scheduled sequence after the step
            longest = int(getattr(cache_metadata, "max_kv_len", 0) or 0)
            if longest <= 0 and slots:
                longest = int((self.kv_lens[_uploaded.get(slots, dev).long()] + qlens_dev[: len(slots)]).max().item())
            rope = rope.select(longest)
        group = max(1, int(queries.shape[1]) // self.num_kv_heads)
        long_seqs = expanded_page_hint(qlens, group)
        qsl, bt, lens, plan, rotated_q = self._write_batch(
            keys, values, qlens_dev, _uploaded.get(slots, dev), total,
            plan_for=(int(queries.shape[1]), window, max_q, long_seqs), advance=advance, rope=rope, queries=queries,
            single_token=single and len(slots) == total)
        if rotated_q is not None:
            queries = rotated_q
        meta = PageMetadata(
            query_start_loc=qsl, sliding_window=getattr(cache_metadata, "sliding_window", None),
            is_single_token_decode=bool(getattr(cache_metadata, "is_single_token_decode", False)) or single,
            slot_ids=getattr(cache_metadata, "slot_ids", None) or slots, max_query_len=max_q, plan=plan,
            query_len_set=None if qlens is None else tuple(sorted(set(q for q in qlens if q > 0))),
            long_seqs=long_seqs,
        ).with_cache_state(block_tables=bt, kv_lens=lens, block_size=self.block_size)
        return queries, self.key_cache, self.value_cache, meta


class PageCacheConfig:
    """Static configuration of a multi-layer paged cache (``cache.py:1309-1375``)."""

    def __init__(self, *, num_hidden_layers: int, num_kv_heads: int, head_dim: int, page_size: int = 16,
                 max_num_reqs: int = 4, max_model_length: int = 4096, memory_utilization: float = 0.85,
                 dtype=torch.float16, cache_dtype: str | None = None, cache_bits: int | None = None,
                 device=None) -> None:
        self.num_hidden_layers, self.num_kv_heads, self.head_dim = int(num_hidden_layers), int(num_kv_heads), int(head_dim)
        self.page_size, self.max_num_reqs, self.max_model_length = int(page_size), int(max_num_reqs), int(max_model_length)
        self.memory_utilization = float(memory_utilization)
        self.dtype, self.cache_dtype = dtype, cache_dtype
        self.cache_bits = int(cache_bits) if cache_bits is not None else None
        self.device = device

    @property
    def num_pages(self) -> int:
        return math.ceil(self.max_model_length / self.page_size) * self.max_num_reqs

    @classmethod
    def create(cls, **kwargs) -> "PageCacheConfig":
        return cls(**kwargs)


class PageCache:
    """One ``PageCacheView`` per layer (``cache.py:1378-1445``)."""

    def __init__(self, views: list[PageCacheView], config: PageCacheConfig | None = None) -> None:
        self.views, self.config = views, config

    def __getitem__(self, index: int) -> PageCacheView:
        return self.views[index]

    def __setitem__(self, index: int, view: PageCacheView) -> None:
        self.views[index] = view

    def __len__(self) -> int:
        return len(self.views)

    def __iter__(self):
        return iter(self.views)

    @classmethod
    def init_cache(cls, config: PageCacheConfig) -> "PageCache":
        views = [
            PageCacheView.init(num_seqs=config.max_num_reqs, max_seq_len=config.max_model_length,
                               num_kv_heads=config.num_kv_heads, head_dim=config.head_dim,
                               block_size=config.page_size, dtype=config.dtype, cache_dtype=config.cache_dtype,
                               cache_bits=config.cache_bits, device=config.device)
            for _ in range(config.num_hidden_layers)
        ]
        return cls(views=views, config=config)

    def clear(self) -> None:
        for view in self.views:
            view.clear()

    def copy_blocks(self, block_mapping) -> None:
        """Copy pages in every layer's pool (``caching/paged/cache.py:1437-1445``)."""
        for view in self.views:
            view.copy_blocks(block_mapping)


__all__ = ("PageCache", "PageCacheConfig", "PageCacheView", "PageMetadata", "build_query_start_loc")
