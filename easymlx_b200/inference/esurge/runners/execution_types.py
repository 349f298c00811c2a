"""What the runner receives per step (``inference/esurge/runners/execution_types.py:30-60`` of the reference)."""

from __future__ import annotations

import typing as tp
from dataclasses import dataclass, field


@dataclass(slots=True)
class ScheduledSequence:
    """One request row selected for this step."""

    request_id: str
    row_index: int
    token_ids: list[int]
    num_computed_tokens: int = 0
    page_ids: tuple[int, ...] = ()
    meta: dict[str, tp.Any] = field(default_factory=dict)

    @property
    def query_len(self) -> int:
        return len(self.token_ids)


def build_positions(sequences: tp.Sequence[ScheduledSequence]) -> list[list[int]]:
    """Per-sequence position ids starting at ``num_computed_tokens`` (``model_runner.py:1292-1306``)."""
    return [list(range(int(s.num_computed_tokens), int(s.num_computed_tokens) + len(s.token_ids))) for s in sequences]
