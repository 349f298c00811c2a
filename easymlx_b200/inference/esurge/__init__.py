"""eSurge-side batch and page-table helpers (device resident)."""

from .runners.model_runner import PageTableRunner, extract_last_tokens

__all__ = ("PageTableRunner", "extract_last_tokens")
