"""The page-table and batch-format part of the reference's ``ModelRunner``, kept on the device.

``ModelRunner`` (``inference/esurge/runners/model_runner.py``) edits ``block_tables`` / ``kv_lens`` row by row from
Python and pads token ids with a compiled helper; here the same operations are kernels behind the C ABI, so the
tables the attention kernels read never leave the GPU.  Method names and meaning follow the reference:

  _clear_row_mapping     model_runner.py:1010-1025
  _zero_pages            model_runner.py:1058-1094
  _assign_row_mapping    model_runner.py:1096-1131
  _move_cache_row        model_runner.py:1192-1213   (exchanges two rows)
  compact_rows           model_runner.py:1215-1241   (the sequence buffer's moves are passed in)
  _flatten_sequence_tokens / _pad_batch_token_ids    model_runner.py:1243-1290
  extract_last_tokens    modules/_base/causal_lm_module.py:176-207
"""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass

import torch

from ...._native import EMLX_OK  # noqa: F401  (re-exported for callers that test return codes)
from .... import _native as nv
from ....caching.paged.cache import PageCacheView, PageMetadata, _uploaded, build_query_start_loc
from .execution_types import ScheduledSequence, build_positions


def _status_ptr(cache: PageCacheView):
    return nv.ptr(cache.status)


def extract_last_tokens(hidden_states: torch.Tensor, cache_metadata: tp.Any) -> torch.Tensor:
    """Last token's hidden state of every sequence of a packed ``[T, hidden]`` batch.

    Rank-3 inputs, a missing ``cache_metadata`` and single-token decode batches are returned unchanged, as in the
    reference."""
    if hidden_states.ndim != 2 or cache_metadata is None or bool(getattr(cache_metadata, "is_single_token_decode", False)):
        return hidden_states
    nv.require_cuda(hidden_states)
    qsl = cache_metadata.query_start_loc
    if not isinstance(qsl, torch.Tensor):
        qsl = torch.as_tensor(list(qsl), dtype=torch.int32)
    qsl = qsl.to(device=hidden_states.device, dtype=torch.int32).contiguous()
    hidden_states = hidden_states.contiguous()
    num_seqs = int(qsl.shape[0]) - 1
    out = torch.empty((num_seqs, hidden_states.shape[1]), dtype=hidden_states.dtype, device=hidden_states.device)
    status = torch.zeros(1, dtype=torch.int32, device=hidden_states.device)
    row_bytes = int(hidden_states.shape[1]) * hidden_states.element_size()
    nv.check(nv.lib().emlx_gather_last_tokens(nv.ptr(hidden_states), int(hidden_states.shape[0]), row_bytes, nv.ptr(qsl),
                                              num_seqs, nv.ptr(out), nv.ptr(status), nv.stream_ptr(hidden_states.device)))
    return out


class PageTableRunner:
    """Holds the per-layer caches (``kv_caches``) and edits their page tables on the device."""

    def __init__(self, kv_caches: tp.Sequence[PageCacheView]):
        self.kv_caches = list(kv_caches)

    # ------------------------------------------------------------------ rows
    def _rows_update(self, ops: list[int], count: int, mode: int) -> None:
        for cache in self.kv_caches:
            dev = cache.block_tables.device
            t = _uploaded.get(tuple(ops), dev)
            nv.check(nv.lib().emlx_rows_update(nv.ptr(cache.block_tables), nv.ptr(cache.kv_lens), cache.num_seqs,
                                               cache.blocks_per_seq, nv.ptr(t), count, mode, _status_ptr(cache),
                                               nv.stream_ptr(dev)))

    def _clear_row_mapping(self, row_index: int) -> None:
        if not self.kv_caches:
            return
        rows = [int(row_index)]
        # the reference silently ignores a row past the table here
        if any(row_index >= c.num_seqs or row_index < 0 for c in self.kv_caches):
            return
        self._rows_update(rows, 1, 2)

    def _assign_row_mapping(self, row_index: int, page_ids: list[int], *, cached_tokens: int = 0) -> None:
        for cache in self.kv_caches:
            if row_index >= cache.num_seqs:
                raise RuntimeError(f"Row index {row_index} exceeds cache capacity {cache.num_seqs}")
            dev = cache.block_tables.device
            count = min(len(page_ids), cache.blocks_per_seq)
            ids = _uploaded.get(tuple(int(p) for p in page_ids[:count]), dev) if count else None
            nv.check(nv.lib().emlx_rows_assign(nv.ptr(cache.block_tables), nv.ptr(cache.kv_lens), cache.num_seqs,
                                               cache.blocks_per_seq, int(row_index), nv.ptr(ids), count,
                                               int(cached_tokens), nv.stream_ptr(dev)))

    def _move_cache_row(self, from_index: int, to_index: int) -> None:
        if from_index == to_index or not self.kv_caches:
            return
        self._rows_update([int(from_index), int(to_index)], 1, 1)

    def compact_rows(self, moves: tp.Sequence[tuple[int, int]]) -> list[tuple[int, int]]:
        """Apply the sequence buffer's ``(from_index, to_index)`` moves, in order, to every cache."""
        moves = [(int(a), int(b)) for a, b in moves]
        if not moves or not self.kv_caches:
            return moves
        flat = [x for m in moves for x in m]
        self._rows_update(flat, len(moves), 0)
        return moves

    def _zero_pages(self, page_ids: list[int]) -> None:
        if not page_ids or not self.kv_caches:
            return
        valid = [int(p) for p in page_ids if int(p) >= 0]
        if not valid:
            return
        for cache in self.kv_caches:
            cache.zero_pages(valid)

    # ------------------------------------------------------------------ batch format
    @staticmethod
    def _flatten_sequence_tokens(sequences: tp.Sequence[tp.Any], device=None) -> tuple[torch.Tensor, list[int]]:
        """One int32 vector of all scheduled token ids (staged in pinned memory) and the per-sequence lengths."""
        query_lens = [len(sequence.token_ids) for sequence in sequences]
        flat = torch.tensor([int(t) for sequence in sequences for t in sequence.token_ids], dtype=torch.int32)
        if device is not None and torch.device(device).type == "cuda":
            flat = flat.pin_memory().to(device, non_blocking=True)
        return flat, query_lens

    def _pad_batch_token_ids(self, sequences: tp.Sequence[tp.Any], device=None) -> tuple[torch.Tensor, list[int]]:
        """``[num_seqs, max_query_len]`` int32 ids, zero past each sequence's length."""
        if device is None:
            device = self.kv_caches[0].block_tables.device if self.kv_caches else "cuda"
        flat, query_lens = self._flatten_sequence_tokens(sequences, device=device)
        max_query_len = max(query_lens, default=0)
        out = torch.zeros((len(sequences), max_query_len), dtype=torch.int32, device=device)
        if not sequences or max_query_len == 0:
            return out, query_lens
        qsl = build_query_start_loc(query_lens, device=device)
        nv.check(nv.lib().emlx_pad_token_ids(nv.ptr(flat), int(flat.numel()), nv.ptr(qsl), len(sequences), max_query_len,
                                             nv.ptr(out), nv.stream_ptr(torch.device(device))))
        return out, query_lens




@dataclass
class StepBatch:
    """The packed batch of one step, resident on the device, in the form the attention path takes it."""

    token_ids: torch.Tensor          # int32 [T]
    positions: torch.Tensor          # int32 [T]
    query_lens: list[int]
    slot_ids: tuple[int, ...]
    cache_metadata: PageMetadata


def prepare_step(runner: PageTableRunner, sequences: tp.Sequence[ScheduledSequence], *, bind_pages: bool = True,
                 device=None) -> StepBatch:
    """Turn the scheduler's selection into the kernels' inputs: bind each row's pages (when the sequence carries
    them), flatten token ids and positions, and build the metadata for ``concatenate_to_cache`` /
    ``paged_attention`` (``model_runner.py:1308-1500`` does the same on the host, per forward step)."""
    if device is None:
        device = runner.kv_caches[0].block_tables.device if runner.kv_caches else "cuda"
    if bind_pages:
        for seq in sequences:
            if seq.page_ids:
                runner._assign_row_mapping(int(seq.row_index), list(seq.page_ids), cached_tokens=int(seq.num_computed_tokens))
    flat, query_lens = runner._flatten_sequence_tokens(sequences, device=device)
    pos = [p for row in build_positions(sequences) for p in row]
    positions = torch.tensor(pos, dtype=torch.int32)
    if torch.device(device).type == "cuda":
        positions = positions.pin_memory().to(device, non_blocking=True)
    slot_ids = tuple(int(s.row_index) for s in sequences)
    single = bool(sequences) and all(n == 1 for n in query_lens)
    meta = PageMetadata(query_start_loc=build_query_start_loc(query_lens, device=device), slot_ids=slot_ids,
                        is_single_token_decode=single, max_query_len=max(query_lens, default=0))
    return StepBatch(token_ids=flat, positions=positions, query_lens=query_lens, slot_ids=slot_ids, cache_metadata=meta)


__all__ = ("PageTableRunner", "ScheduledSequence", "StepBatch", "extract_last_tokens", "prepare_step")
