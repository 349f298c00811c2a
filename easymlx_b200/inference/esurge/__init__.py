"""eSurge-side batch format and page-table helpers (device resident)."""

from .runners import PageTableRunner, ScheduledSequence, StepBatch, build_positions, extract_last_tokens, prepare_step
from .scheduler import ScheduledRequest, SchedulerStepOutput, make_decode_slice, make_prefill_slice

__all__ = ("PageTableRunner", "ScheduledRequest", "ScheduledSequence", "SchedulerStepOutput", "StepBatch", "build_positions",
           "extract_last_tokens", "make_decode_slice", "make_prefill_slice", "prepare_step")
