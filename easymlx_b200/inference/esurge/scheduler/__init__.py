from .output import ScheduledRequest, SchedulerStepOutput
from .slicing import make_decode_slice, make_prefill_slice

__all__ = ("ScheduledRequest", "SchedulerStepOutput", "make_decode_slice", "make_prefill_slice")
