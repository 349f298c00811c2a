"""The scheduler -> runner batch format (``inference/esurge/scheduler/output.py:26-89`` of the reference).

Only the data carried to the runner is mirrored; queueing, preemption and budgeting policy stay with the
embedding engine."""

from __future__ import annotations

import time
from dataclasses import dataclass, field


@dataclass(slots=True)
class ScheduledRequest:
    """One request's slice of a step: the tokens to run, its row in the page table and its pages."""

    request_id: str
    row_index: int
    token_ids: list[int]
    is_prefill: bool
    num_tokens: int
    page_ids: list[int] = field(default_factory=list)
    cache_group: str = "default"
    prefix_cache_hit: bool = False


@dataclass(slots=True)
class SchedulerStepOutput:
    """Everything scheduled for one engine step."""

    scheduled: list[ScheduledRequest] = field(default_factory=list)
    preempted_request_ids: list[str] = field(default_factory=list)
    newly_running_request_ids: list[str] = field(default_factory=list)
    finished_request_ids: list[str] = field(default_factory=list)
    num_scheduled: int = 0
    num_waiting: int = 0
    num_running: int = 0
    token_budget_remaining: int = 0
    decode_only: bool = False
    pending_structured_output_tokens: bool = False
    timestamp: float = field(default_factory=time.time)

    @classmethod
    def from_scheduled(cls, scheduled: list[ScheduledRequest], **kwargs) -> "SchedulerStepOutput":
        """Fill the derived fields the way ``Scheduler.schedule`` does (``scheduler/scheduler.py:440-452``)."""
        return cls(scheduled=scheduled, num_scheduled=len(scheduled),
                   decode_only=bool(scheduled) and all(not entry.is_prefill for entry in scheduled), **kwargs)
