"""Chunked-prefill and decode slicing (``inference/esurge/scheduler/scheduler.py:327-372``): which tokens of a
request run in this step.  These decide the ragged batches the attention kernels see (prefill chunk sizes, single
decode rows)."""

from __future__ import annotations

import typing as tp


def make_prefill_slice(all_token_ids: tp.Sequence[int], num_computed_tokens: int, remaining_prefill_tokens: int,
                       budget_available: int, *, chunked_prefill_enabled: bool = False,
                       long_prefill_token_threshold: int | None = None) -> tuple[list[int], int]:
    """``(token_ids, token_count)`` of the next prefill chunk: the rest of the prompt, cut to the step's token
    budget and, with chunked prefill, to the long-prefill threshold."""
    remaining = int(remaining_prefill_tokens)
    if remaining <= 0 or budget_available <= 0:
        return [], 0
    planned = min(remaining, int(budget_available))
    threshold = long_prefill_token_threshold
    if bool(chunked_prefill_enabled) and threshold is not None and threshold > 0:
        planned = min(planned, int(threshold))
    start = int(num_computed_tokens)
    return list(all_token_ids[start:start + planned]), planned


def make_decode_slice(generated_token_ids: tp.Sequence[int], prompt_token_ids: tp.Sequence[int],
                      remaining_generation_budget: int, budget_available: int) -> tuple[list[int], int]:
    """``([last_token], 1)``: the last generated token, else the last prompt token, else 0."""
    if budget_available <= 0 or remaining_generation_budget <= 0:
        return [], 0
    last = generated_token_ids[-1] if generated_token_ids else (prompt_token_ids[-1] if prompt_token_ids else 0)
    return [int(last)], 1
