from .execution_types import ScheduledSequence, build_positions
from .model_runner import PageTableRunner, StepBatch, extract_last_tokens, prepare_step

__all__ = ("PageTableRunner", "ScheduledSequence", "StepBatch", "build_positions", "extract_last_tokens", "prepare_step")
