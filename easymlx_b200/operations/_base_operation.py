"""Operation plugin API: abstract operation and name registry.

Mirrors ``operations/_base_operation.py:34-198`` of easymlx (``BaseOperation``,
``OperationRegistry.register/get/create/available_impls``).
"""

from __future__ import annotations

import abc
import typing as tp

from .requirements import ExecutionMode, OperationRequirements


class BaseOperation(abc.ABC):
    """An attention implementation; calling it runs ``forward_native``."""

    metadata: tp.Any | None = None

    def __init__(self, metadata: tp.Any | None = None):
        self.metadata = metadata

    @classmethod
    @abc.abstractmethod
    def get_impl_name(cls) -> str | tuple[str, ...]:
        """Name, or tuple of alias names, the registry files this class under."""

    @classmethod
    def get_requirements(cls, mode: ExecutionMode = ExecutionMode.MIXED) -> OperationRequirements:
        names = cls.get_impl_name()
        return OperationRequirements.default(str(names[0] if isinstance(names, tuple) else names))

    def get_instance_requirements(self, mode: ExecutionMode = ExecutionMode.MIXED) -> OperationRequirements:
        return self.get_requirements(mode)

    def get_impl_metadata(self) -> tp.Any | None:
        return self.metadata

    @abc.abstractmethod
    def forward_native(self, *args, **kwargs) -> tp.Any:
        """Run the operation."""

    def __call__(self, *args, **kwargs) -> tp.Any:
        return self.forward_native(*args, **kwargs)


class OperationRegistry:
    """Process-wide map from implementation name to operation class."""

    _registry: tp.ClassVar[dict[str, type[BaseOperation]]] = {}

    @classmethod
    def register(cls, operation_cls: type[BaseOperation]) -> type[BaseOperation]:
        names = operation_cls.get_impl_name()
        for name in (names,) if isinstance(names, str) else names:
            cls._registry[str(name)] = operation_cls
        return operation_cls

    @classmethod
    def get(cls, name: str) -> type[BaseOperation]:
        if name not in cls._registry:
            raise KeyError(f"Unknown operation '{name}'. Available: {', '.join(sorted(cls._registry))}")
        return cls._registry[name]

    @classmethod
    def create(cls, name: str, *, metadata: tp.Any | None = None) -> BaseOperation:
        return cls.get(name)(metadata=metadata)

    @classmethod
    def available_impls(cls) -> list[str]:
        return sorted(cls._registry)


Operation = BaseOperation

__all__ = ("BaseOperation", "Operation", "OperationRegistry")
