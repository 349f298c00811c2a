"""Result container of attention operations (``operations/_attention_outputs.py:33-50`` of easymlx)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch


@dataclass
class AttentionOutput:
    attention_outputs: torch.Tensor | None = None
    attention_weights: torch.Tensor | None = None
    cache_view: Any | None = None


__all__ = ("AttentionOutput",)
