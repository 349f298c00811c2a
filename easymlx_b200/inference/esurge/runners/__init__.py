from .model_runner import PageTableRunner, extract_last_tokens

__all__ = ("PageTableRunner", "extract_last_tokens")
