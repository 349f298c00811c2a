"""CPU restatement (NumPy) of the reference's batch and page-table maintenance around the attention path.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the benchmark's CPU baseline; the product never
routes through it.

Pinned against the reference's own functions, executed through the NumPy stand-in for ``mlx.core``
(tests/golden/table_ops.npz, made by tests/golden/make_golden_table_ops.py), except ``copy_blocks``: the reference
has only a Metal kernel for it (caching/paged/cache.py:95-132), so that one is a restatement of the kernel text
-- parity unpinned.
"""

from __future__ import annotations

import numpy as np


def extract_last_tokens(hidden_states: np.ndarray, query_start_loc) -> np.ndarray:
    """modules/_base/causal_lm_module.py:176-207: ``take(hidden, qsl[1:] - 1, axis=0)`` (an index of -1 wraps)."""
    qsl = np.asarray(query_start_loc, dtype=np.int32)
    return np.take(hidden_states, qsl[1:] - 1, axis=0)


def flatten_sequence_tokens(token_lists) -> tuple[np.ndarray, list[int]]:
    """inference/esurge/runners/model_runner.py:1243-1248."""
    lens = [len(t) for t in token_lists]
    flat = np.asarray([int(x) for t in token_lists for x in t], dtype=np.int32)
    return flat, lens


def pad_batch_token_ids(flat_ids: np.ndarray, query_lens, max_query_len: int | None = None) -> np.ndarray:
    """model_runner.py:1250-1290: rows of ``max_query_len`` ids, zero past each sequence's length."""
    lens = np.asarray(query_lens, dtype=np.int32)
    max_q = int(lens.max()) if max_query_len is None and lens.size else int(max_query_len or 0)
    out = np.zeros((lens.size, max_q), dtype=np.int32)
    if lens.size == 0 or max_q == 0:
        return out
    offsets = np.cumsum(lens) - lens
    pos = np.arange(max_q, dtype=np.int32)[None, :]
    safe = np.minimum(offsets[:, None] + pos, max(int(flat_ids.shape[0]), 1) - 1)
    gathered = np.take(flat_ids, safe.reshape(-1)).reshape(lens.size, max_q) if flat_ids.size else out
    return np.where(pos < lens[:, None], gathered, 0).astype(np.int32)


def clear_row(block_tables: np.ndarray, kv_lens: np.ndarray, row: int) -> None:
    """model_runner.py:1010-1025."""
    if row < block_tables.shape[0]:
        block_tables[row, :] = -1
    if row < kv_lens.shape[0]:
        kv_lens[row] = 0


def assign_row(block_tables: np.ndarray, kv_lens: np.ndarray, row: int, page_ids, cached_tokens: int = 0) -> None:
    """model_runner.py:1096-1131."""
    if row >= block_tables.shape[0]:
        raise RuntimeError(f"Row index {row} exceeds cache capacity {block_tables.shape[0]}")
    block_tables[row, :] = -1
    count = min(len(page_ids), block_tables.shape[1])
    if count:
        block_tables[row, :count] = np.asarray(page_ids[:count], dtype=np.int32)
    kv_lens[row] = max(int(cached_tokens), 0)


def swap_rows(block_tables: np.ndarray, kv_lens: np.ndarray, from_index: int, to_index: int) -> None:
    """model_runner.py:1192-1213 (named a move there; it exchanges the two rows)."""
    if from_index == to_index:
        return
    a, b = block_tables[from_index].copy(), block_tables[to_index].copy()
    la, lb = int(kv_lens[from_index]), int(kv_lens[to_index])
    block_tables[to_index], kv_lens[to_index] = a, la
    block_tables[from_index], kv_lens[from_index] = b, lb


def compact_rows(block_tables: np.ndarray, kv_lens: np.ndarray, moves) -> None:
    """model_runner.py:1215-1241: for every (from, to) in order, move the row and clear its old place."""
    for from_index, to_index in moves:
        if from_index == to_index:
            continue
        block_tables[to_index] = block_tables[from_index].copy()
        kv_lens[to_index] = int(kv_lens[from_index])
        block_tables[from_index, :] = -1
        kv_lens[from_index] = 0


def zero_pages(arrays, page_ids) -> None:
    """model_runner.py:1058-1094: zero the listed pages (ids < 0 or past the pool are dropped) in every array."""
    for a in arrays:
        ids = [int(p) for p in page_ids if 0 <= int(p) < a.shape[0]]
        if ids:
            a[ids] = 0


def copy_blocks(arrays, block_mapping) -> None:
    """caching/paged/cache.py:95-132,944-972: every destination page receives its source page as it was BEFORE the
    call (the kernel reads the input arrays and writes fresh output arrays)."""
    mapping = np.asarray(block_mapping, dtype=np.int64).reshape(-1, 2)
    for a in arrays:
        before = a.copy()
        for src, dst in mapping:
            a[dst] = before[src]
