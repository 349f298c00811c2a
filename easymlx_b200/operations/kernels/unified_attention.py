"""Unified ragged paged attention on B200.

Host-side mirror of easymlx ``operations/kernels/unified_attention.py``:
``paged_attention`` (``:1377-1512``), ``UnifiedAttnMetadata`` (``:44-66``),
``UnifiedAttnConfig`` (``:69-82``) and the registered ``UnifiedAttention`` operation
(``:1515-1684``) keep their names, arguments, defaults and error behaviour.  The work is
done by the CUDA library behind ``include/easymlx_b200.h``; there is no CPU path, so
where the reference would fall back to NumPy this module raises.
"""

from __future__ import annotations

import math
import os
import typing as tp
from dataclasses import dataclass

import torch

from ... import _native as nv
from .._attention_outputs import AttentionOutput
from .._base_operation import BaseOperation, OperationRegistry
from ..requirements import ExecutionMode, MetadataField, RequirementsBuilder

_CHECK = os.environ.get("EASYMLX_B200_CHECK", "0") not in ("", "0")
_TILED_HEAD_DIMS = (64, 128)
_TILED_BLOCK_SIZES_FLOAT = (16, 32, 64, 128)  # a 128-token tile is one page or 2 / 4 / 8 pages
_TILED_BLOCK_SIZE_AFFINE = 128              # affine pools keep values transposed inside a 128-token page


@dataclass
class UnifiedAttnMetadata:
    block_tables: tp.Any
    kv_lens: tp.Any
    query_start_loc: tp.Any
    block_size: int
    sliding_window: int | None = None
    is_single_token_decode: bool = False


@dataclass
class UnifiedAttnConfig:
    """Kept for signature compatibility; the Metal-specific knobs have no effect here."""

    use_metal_kernel: bool = True
    allow_fallback: bool = True
    threadgroup_size: int = 256


def _validate_inputs(queries, key_cache, value_cache, block_tables, kv_lens, query_start_loc, affine: bool) -> None:
    if queries.ndim != 3:
        raise ValueError("queries must be rank-3: [total_tokens, num_q_heads, head_dim]")
    if key_cache.ndim != 4 or value_cache.ndim != 4:
        raise ValueError("key_cache/value_cache must be rank-4: [num_blocks, block_size, num_kv_heads, head_dim]")
    if not affine:
        if key_cache.shape != value_cache.shape:
            raise ValueError("key_cache and value_cache must have the same shape")
        if queries.shape[2] != key_cache.shape[3]:
            raise ValueError("queries head_dim must match key/value cache head_dim")
    if queries.shape[1] % key_cache.shape[2] != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads (GQA)")
    if block_tables.ndim != 2:
        raise ValueError("block_tables must be rank-2: [num_seqs, max_blocks_per_seq]")
    if kv_lens.ndim != 1 or query_start_loc.ndim != 1:
        raise ValueError("kv_lens/query_start_loc must be rank-1")
    if query_start_loc.shape[0] != block_tables.shape[0] + 1:
        raise ValueError("query_start_loc must have length num_seqs + 1")


def _as_int32(value, device) -> torch.Tensor:
    if isinstance(value, torch.Tensor):
        if value.dtype != torch.int32 or value.device != device or not value.is_contiguous():
            value = value.to(device=device, dtype=torch.int32).contiguous()
        return value
    return torch.as_tensor(value, dtype=torch.int32).to(device)


class _Scratch:
    """Plan / workspace / status buffers per (device, stream), grown on demand and reused across calls.

    The workspace must start zeroed (its counters reset themselves after every merge), so it is
    zero-filled whenever it is (re)allocated.  Calls issued on one stream run one after the other and may
    share these buffers; calls on different streams may overlap on the GPU, so each stream gets its own
    set.  Two ``AttentionCall`` objects built on the same stream share the work list: build, plan and launch
    one call before constructing the next (``paged_attention`` does).
    """

    def __init__(self):
        self.buffers: dict = {}
        self.marks: dict = {}

    def get(self, device, kind: str, nbytes: int, zero: bool) -> torch.Tensor:
        key = (str(device), int(torch.cuda.current_stream(device).cuda_stream), kind)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < nbytes:
            size = max(256, int(nbytes))
            buf = torch.zeros(size, dtype=torch.uint8, device=device) if zero else \
                torch.empty(size, dtype=torch.uint8, device=device)
            self.buffers[key] = buf
        return buf


_scratch = _Scratch()


def _make_pool(key_cache, value_cache, head_dim, k_scale, v_scale, k_bias, v_bias) -> tuple[nv.Pool, bool]:
    p = nv.Pool()
    affine = key_cache.dtype == torch.uint8
    p.key_cache, p.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
    p.num_blocks, p.block_size, p.num_kv_heads = int(key_cache.shape[0]), int(key_cache.shape[1]), int(key_cache.shape[2])
    p.head_dim = int(head_dim)
    if affine:
        if k_scale is None or v_scale is None or k_bias is None or v_bias is None:
            raise ValueError("a uint8 (affine) KV pool needs k_scale, v_scale, k_bias and v_bias")
        width = int(key_cache.shape[3])
        if width == head_dim:
            bits = 8
        elif width * 2 == head_dim:
            bits = 4
        else:
            raise ValueError("affine key_cache last dimension must be head_dim (8-bit) or head_dim/2 (4-bit)")
        expect_v = (p.num_blocks, p.num_kv_heads, head_dim, p.block_size * bits // 8)
        if tuple(value_cache.shape) != expect_v:
            raise ValueError(f"affine value_cache must be [num_blocks, num_kv_heads, head_dim, block_size*bits/8] = {expect_v}")
        sb_shape = (p.num_blocks, p.num_kv_heads, p.block_size, head_dim // 64)
        for t in (k_scale, k_bias, v_scale, v_bias):
            if tuple(t.shape) != sb_shape or t.dtype != torch.float16 or not t.is_contiguous():
                raise ValueError(f"affine scale/bias must be contiguous float16 {sb_shape}")
        p.k_scale, p.k_bias, p.v_scale, p.v_bias = k_scale.data_ptr(), k_bias.data_ptr(), v_scale.data_ptr(), v_bias.data_ptr()
        p.kv_format, p.kv_dtype = bits, nv.F16
    else:
        p.kv_format, p.kv_dtype = nv.KV_FLOAT, nv.dtype_code(key_cache.dtype)
    return p, affine


class AttentionCall:
    """One validated attention call, split into ``plan()`` (work list built on the GPU) and ``launch()``
    (the attention kernels) so that a caller can build the plan once per engine step and launch once per
    layer, or time the kernels alone.  ``paged_attention`` is ``AttentionCall(...).plan().launch()``."""

    def __init__(self, queries, key_cache, value_cache, block_tables, kv_lens, query_start_loc, *,
                 softmax_scale: float | None = None, sliding_window: int | None = None,
                 k_scale=None, v_scale=None, k_bias=None, v_bias=None, kernel: str | None = None,
                 max_query_len: int = 0, plan=None, query_len_set: tp.Sequence[int] | None = None, gather=None,
                 long_seqs: int = 0):
        nv.require_cuda(queries, key_cache, value_cache)
        dev = queries.device
        affine = key_cache.dtype == torch.uint8
        self.block_tables = _as_int32(block_tables, dev)
        self.kv_lens = _as_int32(kv_lens, dev)
        self.query_start_loc = _as_int32(query_start_loc, dev)
        _validate_inputs(queries, key_cache, value_cache, self.block_tables, self.kv_lens, self.query_start_loc, affine)
        self.total, self.hq, self.d = int(queries.shape[0]), int(queries.shape[1]), int(queries.shape[2])
        self.scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(self.d)
        self.window = int(sliding_window or 0)
        self.device = dev
        self.queries = queries.contiguous()
        self.out = None
        self.kernel = kernel
        # KV heads sharded over GPUs (``easymlx_b200.distributed.GatherTarget``): the short-row kernels store this
        # rank's heads into every rank's full output instead of a local [T, Hq, D] tensor
        self.gather = gather
        if gather is not None:
            if kernel not in (None, "decode"):
                raise ValueError("a gathering call runs the short-row kernels (kernel='decode')")
            if self.total > gather.out.shape[0] or self.d != gather.out.shape[2] or queries.dtype != gather.out.dtype:
                raise ValueError("the gather target does not fit this call's tokens / head_dim / dtype")
            self.kernel = "decode"
        if self.total == 0:
            return
        if not (key_cache.is_contiguous() and value_cache.is_contiguous()):
            raise ValueError("key_cache and value_cache must be contiguous")
        self.key_cache, self.value_cache = key_cache, value_cache
        self.scales = (k_scale, v_scale, k_bias, v_bias)
        self.pool, _ = _make_pool(key_cache, value_cache, self.d, k_scale, v_scale, k_bias, v_bias)
        tiled_ok = (
            (self.pool.block_size == _TILED_BLOCK_SIZE_AFFINE if affine else self.pool.block_size in _TILED_BLOCK_SIZES_FLOAT)
            and self.d in _TILED_HEAD_DIMS
            and queries.dtype in (torch.float16, torch.bfloat16)
            and (affine or key_cache.dtype == queries.dtype)
        )
        if self.kernel is None:
            self.kernel = "tiled" if tiled_ok else "generic"
        if self.kernel != "generic" and not tiled_ok:
            raise NotImplementedError(
                "the tiled kernels need page size 128 (or 16/32/64 with a 16-bit pool), head_dim 64 or 128, fp16/bf16 queries and a pool of the "
                "same dtype (or an affine pool)")
        self.num_seqs = int(self.block_tables.shape[0])
        self.status = _scratch.get(dev, "status", 4, zero=True)
        a = nv.AttnArgs()
        a.queries = self.queries.data_ptr()
        a.block_tables, a.kv_lens = self.block_tables.data_ptr(), self.kv_lens.data_ptr()
        a.query_start_loc = self.query_start_loc.data_ptr()
        a.total_tokens, a.num_seqs, a.num_q_heads = self.total, self.num_seqs, self.hq
        a.max_blocks_per_seq, a.q_dtype = int(self.block_tables.shape[1]), nv.dtype_code(queries.dtype)
        a.sliding_window, a.softmax_scale = self.window, self.scale
        a.max_query_len = max(0, int(max_query_len))
        a.row_class_mask = 0
        a.status = self.status.data_ptr()
        self.args = a
        if self.kernel != "generic":
            lib = nv.lib()
            hkv = self.pool.num_kv_heads
            self.plan_bytes = int(lib.emlx_attn_plan_bytes(self.num_seqs, self.total, self.hq, hkv))
            ws_bytes = int(lib.emlx_attn_workspace_bytes(self.num_seqs, self.total, self.hq, hkv, self.d))
            self.planned = False
            # the flags decide which row classes the work list holds; the launch has to use the ones it was built with
            # (the decode entry point serves the short-row classes only: its work list is built without 128-row units)
            recommended = int(lib.emlx_attn_plan_flags(self.pool.kv_format, self.hq, hkv, self.d))
            # An affine pool serves rows of more than 16 (prefill chunks) on the tcgen05 kernel when the caller says how
            # many sequences have such rows: their pages are expanded to 16-bit rows in scratch memory behind the
            # workspace, sized from that count (``long_seqs``, a host-side hint like ``query_len_set``).
            from ...caching.paged.cache import wide_units_geometry
            expandable = affine and self.kernel == "tiled" and int(long_seqs) > 0 and wide_units_geometry(self.hq, hkv, self.d)
            if expandable:
                recommended |= 1
            self.plan_flags = recommended & ~1 if self.kernel == "decode" else recommended
            usable = plan is not None and plan[1] == self.hq and plan[2] == self.window and plan[0].numel() >= self.plan_bytes
            if usable and self.kernel == "decode" and (int(plan[3]) & 1):
                usable = False   # that work list holds 128-row units, which the short-row entry points do not serve
            if usable and affine and (int(plan[3]) & 1) and not expandable:
                usable = False   # 128-row units over an affine pool need the scratch, and the scratch needs the count
            if usable:
                self.plan_buf, self.planned = plan[0], True   # built together with the batch metadata
                self.plan_flags = int(plan[3])
            else:
                self.plan_buf = _scratch.get(dev, "plan", self.plan_bytes, zero=False)
            a.plan_flags = self.plan_flags
            wide = bool(self.plan_flags & 1)
            if query_len_set:
                # the host knows which query lengths occur: launch only the kernels of those row classes
                group = self.hq // hkv
                for q_len in set(int(x) for x in query_len_set):
                    rows = q_len * group
                    if rows > 0:
                        a.row_class_mask |= 1 << (0 if rows <= 8 else 1 if rows <= 16 else (3 if wide else 2))
            if affine and wide:
                # The expanded pages sit behind the workspace proper.  Where that ends depends on the batch, so this
                # buffer is kept apart from the one ordinary calls share (whose counters must stay zero), and its own
                # workspace part is zeroed again whenever a call of another geometry takes it over.
                base_bytes = ws_bytes
                ws_bytes += int(lib.emlx_attn_dequant_bytes(self.pool, self.num_seqs, int(self.block_tables.shape[1]),
                                                            int(long_seqs), self.total, self.hq, nv.dtype_code(queries.dtype)))
                self.workspace = _scratch.get(dev, "workspace+pages", ws_bytes, zero=True)
                key = (str(dev), int(torch.cuda.current_stream(dev).cuda_stream), "workspace+pages")
                if _scratch.marks.get(key) not in (None, base_bytes):
                    self.workspace[: max(base_bytes, _scratch.marks[key])].zero_()
                _scratch.marks[key] = base_bytes
            else:
                self.workspace = _scratch.get(dev, "workspace", ws_bytes, zero=True)
            a.plan, a.plan_bytes = self.plan_buf.data_ptr(), self.plan_bytes
            # (the size this call asked for, not the shared buffer's: the library sizes the expansion's grid from it)
            a.workspace, a.workspace_bytes = self.workspace.data_ptr(), ws_bytes

    def plan(self) -> "AttentionCall":
        if self.total and self.kernel != "generic" and not self.planned:
            nv.check(nv.lib().emlx_attn_plan(
                nv.ptr(self.query_start_loc), nv.ptr(self.kv_lens), self.num_seqs, self.total, self.hq,
                self.pool.num_kv_heads, self.pool.block_size, self.window, int(self.args.max_query_len),
                self.plan_flags, nv.ptr(self.plan_buf), self.plan_bytes, nv.stream_ptr(self.device)))
            self.planned = True
        return self

    def launch(self) -> torch.Tensor:
        if self.total == 0:
            return torch.zeros_like(self.queries) if self.gather is None else self.gather.out[:0]
        lib = nv.lib()
        if self.gather is not None:
            g = self.gather
            self.out = g.out[: self.total]
            self.args.out = g.out.data_ptr()
            nv.check(lib.emlx_attn_decode_gather(self.args, self.pool, g.flag_block, g.total_q_heads, g.head_offset,
                                                 nv.stream_ptr(self.device)))
            self._report_status(lib)
            return self.out
        self.out = torch.empty_like(self.queries)
        if _CHECK:
            self.out.fill_(float("nan"))  # a row no kernel writes shows up in the caller's checks
        self.args.out = self.out.data_ptr()
        entry = {"generic": lib.emlx_attn_generic, "tiled": lib.emlx_attn_unified, "decode": lib.emlx_attn_decode,
                 "prefill": lib.emlx_attn_prefill}[self.kernel]
        nv.check(entry(self.args, self.pool, nv.stream_ptr(self.device)))
        self._report_status(lib)
        return self.out

    def _report_status(self, lib) -> None:
        # (reading the status synchronises the stream, which a stream capture does not allow)
        if not _CHECK or torch.cuda.is_current_stream_capturing():
            return
        rc = lib.emlx_read_status(nv.ptr(self.status), nv.stream_ptr(self.device))
        if rc != nv.EMLX_OK:
            self.status.zero_()  # report once
            ws = getattr(self, "workspace", None)
            if ws is not None:
                ws.zero_()  # a wait that gave up may have left split-KV arrival counters set
        nv.check(rc)


def paged_attention(
    queries: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables,
    kv_lens,
    query_start_loc,
    *,
    softmax_scale: float | None = None,
    sliding_window: int | None = None,
    use_metal: bool | None = None,
    single_token_decode: bool | None = None,
    threadgroup_size: int = 256,
    allow_fallback: bool = True,
    k_scale: torch.Tensor | None = None,
    v_scale: torch.Tensor | None = None,
    k_bias: torch.Tensor | None = None,
    v_bias: torch.Tensor | None = None,
    kernel: str | None = None,
    max_query_len: int = 0,
    plan=None,
    query_len_set: tp.Sequence[int] | None = None,
    gather=None,
    long_seqs: int = 0,
) -> torch.Tensor:
    """Ragged causal attention of packed queries over a paged KV pool.

    Same arguments as the reference.  ``kv_lens`` are the lengths after this step's write;
    ``block_tables`` / ``kv_lens`` hold one row per scheduled sequence.  ``use_metal``,
    ``threadgroup_size`` and ``allow_fallback`` are accepted and ignored.  For affine pools
    ``k_scale``/``v_scale`` are per-group fp16 arrays and ``k_bias``/``v_bias`` join them.
    ``single_token_decode`` / ``max_query_len`` are host-side hints (an upper bound on the query tokens of
    any sequence) and ``query_len_set`` (the distinct query lengths of the batch); without them the kernels for every
    row class are launched and the empty ones return at once.  ``kernel`` (``None`` = automatic, ``"generic"``, ``"tiled"``, ``"decode"``, ``"prefill"``) selects
    an entry point explicitly; tests and benchmarks use it.  ``long_seqs`` (the number of sequences with more than 16
    query rows, another host hint) lets an affine pool serve those rows on the tcgen05 kernel.  ``gather`` (a ``distributed.GatherTarget``) makes the call
    store its heads into every rank's full output (KV heads sharded over GPUs) and return this rank's copy of it.
    """
    del use_metal, threadgroup_size, allow_fallback
    if single_token_decode and not max_query_len:
        max_query_len = 1
    return AttentionCall(queries, key_cache, value_cache, block_tables, kv_lens, query_start_loc,
                         softmax_scale=softmax_scale, sliding_window=sliding_window, k_scale=k_scale, v_scale=v_scale,
                         k_bias=k_bias, v_bias=v_bias, kernel=kernel, max_query_len=max_query_len,
                         plan=plan, query_len_set=query_len_set, gather=gather, long_seqs=long_seqs).plan().launch()


@OperationRegistry.register
class UnifiedAttention(BaseOperation):
    """Paged (unified) attention operation for block-tabled KV caches.

    Registered under the reference's names.  Every batch - decode rows, prefill chunks, one
    multi-token sequence - goes to the same CUDA entry point; the reference's separate dense route
    for a single multi-token sequence (``unified_attention.py:1658-1673``) differs from it only by
    rounding the probabilities to the value dtype, which lies inside the op's tolerance.
    """

    def __init__(self, metadata: tp.Any | None = None, *, use_metal: bool = True):
        super().__init__(metadata=metadata)
        self.use_metal = bool(use_metal)

    @classmethod
    def get_impl_name(cls) -> str | tuple[str, ...]:
        return ("unified_attention", "unified", "paged", "full_attention", "linear_attention")

    @classmethod
    def get_requirements(cls, mode: ExecutionMode = ExecutionMode.MIXED):
        from ...caching.paged.cache import PageCacheView

        return (
            RequirementsBuilder("unified_attention")
            .require_metadata(MetadataField.QUERY_START_LOC, MetadataField.BLOCK_TABLES, MetadataField.KV_LENS,
                              MetadataField.BLOCK_SIZE)
            .optional_metadata(MetadataField.SLIDING_WINDOW)
            .require_cache(PageCacheView)
            .build()
        )

    def forward_native(self, *, query, key, value, cache_metadata=None, cache_view=None, scale: float | None = None,
                       use_metal: bool | None = None, threadgroup_size: int = 256, **_: tp.Any) -> AttentionOutput:
        from ...caching.paged.cache import PageMetadata

        if cache_metadata is None:
            raise ValueError("UnifiedAttention requires cache_metadata.")
        if isinstance(cache_metadata, PageMetadata):
            if cache_metadata.block_tables is None or cache_metadata.kv_lens is None or cache_metadata.block_size is None:
                raise ValueError("PageMetadata must be resolved before unified attention execution.")
        extra: dict[str, tp.Any] = {}
        if cache_view is not None and getattr(cache_view, "is_affine", False) and key.dtype == torch.uint8:
            extra = dict(k_scale=cache_view.k_scales, v_scale=cache_view.v_scales,
                         k_bias=cache_view.k_biases, v_bias=cache_view.v_biases)
        outputs = paged_attention(
            query, key, value, cache_metadata.block_tables, cache_metadata.kv_lens, cache_metadata.query_start_loc,
            softmax_scale=scale, sliding_window=cache_metadata.sliding_window,
            single_token_decode=cache_metadata.is_single_token_decode,
            max_query_len=int(getattr(cache_metadata, "max_query_len", 0) or 0),
            plan=getattr(cache_metadata, "plan", None), query_len_set=getattr(cache_metadata, "query_len_set", None),
            long_seqs=int(getattr(cache_metadata, "long_seqs", 0) or 0), **extra,
        )
        return AttentionOutput(attention_outputs=outputs, cache_view=cache_view)


__all__ = ("AttentionCall", "UnifiedAttention", "UnifiedAttnConfig", "UnifiedAttnMetadata", "paged_attention")
