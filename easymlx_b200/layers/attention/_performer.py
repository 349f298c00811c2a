"""Caller of the paged path: reshape, cache write, operation dispatch.

Mirrors the paged branch of easymlx ``layers/attention/_performer.py``
(``prepare_paged_attention_inputs`` ``:63-128``, ``AttentionPerformer._forward_paged`` ``:219-274``):
``[B, L, H, D]`` inputs are flattened to ``[T, H, D]``, new K/V go through
``PageCacheView.concatenate_to_cache``, the registered ``"unified_attention"`` operation attends, and an
empty batch returns the queries unchanged.
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass

import torch

from ...caching.paged.cache import PageCacheView, PageMetadata
from ...operations import ExecutionMode, OperationExecutor, OperationRegistry


@dataclass
class PagedAttentionInputs:
    queries: torch.Tensor
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    metadata: PageMetadata


def prepare_paged_attention_inputs(queries, keys, values, *, kv_cache: PageCacheView,
                                   query_start_loc: tp.Sequence[int] | PageMetadata,
                                   slot_ids: tp.Sequence[int] | None = None, rope: tp.Any = None,
                                   sliding_window: int | None = None) -> PagedAttentionInputs:
    meta = query_start_loc if isinstance(query_start_loc, PageMetadata) else PageMetadata(
        query_start_loc=query_start_loc, sliding_window=int(sliding_window) if sliding_window is not None else 0)
    slots = slot_ids or getattr(meta, "slot_ids", None) or ()
    query_lens = (1,) * len(slots) if getattr(meta, "is_single_token_decode", False) and slots else None
    q, kc, vc, resolved = kv_cache.concatenate_to_cache(queries, keys, values, cache_metadata=meta, slot_ids=slots,
                                                        query_lens=query_lens, rope=rope)
    return PagedAttentionInputs(queries=q, key_cache=kc, value_cache=vc, metadata=resolved)


class AttentionPerformer:
    """Single entry for a model's attention layers on the paged path."""

    def __init__(self, scale: float | None = None, attn_mechanism: str = "unified_attention"):
        self.scale = scale
        self.executor = OperationExecutor.from_operations(mixin=OperationRegistry.create(attn_mechanism))

    def __call__(self, queries, keys, values, *, cache_view: PageCacheView, cache_metadata: PageMetadata | None,
                 rope: tp.Any = None) -> torch.Tensor:
        return self._forward_paged(queries, keys, values, cache_view=cache_view, cache_metadata=cache_metadata, rope=rope)

    def _forward_paged(self, queries, keys, values, *, cache_view, cache_metadata, rope) -> torch.Tensor:
        batched = queries.ndim == 4
        if batched:
            b, l = queries.shape[0], queries.shape[1]
            queries = queries.reshape(-1, queries.shape[-2], queries.shape[-1])
            keys = keys.reshape(-1, keys.shape[-2], keys.shape[-1])
            values = values.reshape(-1, values.shape[-2], values.shape[-1])
        prepared = prepare_paged_attention_inputs(queries, keys, values, kv_cache=cache_view,
                                                  query_start_loc=cache_metadata, rope=rope)
        if prepared.queries.shape[0] == 0:
            out = queries
        else:
            op = self.executor.get_operation(ExecutionMode.MIXED)
            out = op(query=prepared.queries, key=prepared.key_cache, value=prepared.value_cache,
                     cache_metadata=prepared.metadata, cache_view=cache_view, scale=self.scale).attention_outputs
        return out.reshape(b, l, out.shape[-2], out.shape[-1]) if batched else out


__all__ = ("AttentionPerformer", "PagedAttentionInputs", "prepare_paged_attention_inputs")
