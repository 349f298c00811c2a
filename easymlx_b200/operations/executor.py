"""Per-mode operation selection, mirroring ``operations/executor.py:31-121`` of easymlx."""

from __future__ import annotations

from dataclasses import dataclass

from ._base_operation import BaseOperation
from .requirements import ExecutionMode, OperationRequirements


@dataclass
class OperationExecutor:
    """Holds up to three implementations; decode falls back to prefill, both fall back to mixin."""

    prefill_impl: BaseOperation | None = None
    decode_impl: BaseOperation | None = None
    mixin_impl: BaseOperation | None = None

    @property
    def prefill_operation(self) -> BaseOperation | None:
        return self.prefill_impl or self.mixin_impl

    @property
    def decode_operation(self) -> BaseOperation | None:
        return self.decode_impl or self.prefill_impl or self.mixin_impl

    def get_operation(self, mode: ExecutionMode) -> BaseOperation | None:
        return self.decode_operation if mode == ExecutionMode.DECODE else self.prefill_operation

    def get_requirements(self, mode: ExecutionMode = ExecutionMode.MIXED) -> OperationRequirements:
        op = self.get_operation(mode)
        return OperationRequirements.default() if op is None else op.get_instance_requirements(mode)

    def get_combined_requirements(self) -> OperationRequirements:
        pre, dec = self.prefill_operation, self.decode_operation
        parts = []
        if pre is not None:
            parts.append(pre.get_instance_requirements(ExecutionMode.PREFILL))
        if dec is not None:
            parts.append(dec.get_instance_requirements(ExecutionMode.DECODE))
        if not parts:
            return OperationRequirements.default()
        return parts[0] if len(parts) == 1 else parts[0] | parts[1]

    @classmethod
    def from_operations(cls, *, prefill=None, decode=None, mixin=None) -> "OperationExecutor":
        return cls(prefill_impl=prefill, decode_impl=decode, mixin_impl=mixin)


__all__ = ("OperationExecutor",)
