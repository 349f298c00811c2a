"""Requirement declarations of the operation plugin API.

Mirrors ``operations/requirements/{types,requirements,builder}.py`` of easymlx: the
same enum members and the same builder calls, so that an operation written against
the reference registers here unchanged.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field, replace


class ExecutionMode(enum.Enum):
    PREFILL = "prefill"
    DECODE = "decode"
    MIXED = "mixed"


class MetadataField(enum.Flag):
    NONE = 0
    MASK = enum.auto()
    SINKS = enum.auto()
    QUERY_START_LOC = enum.auto()
    BLOCK_TABLES = enum.auto()
    KV_LENS = enum.auto()
    BLOCK_SIZE = enum.auto()
    SLIDING_WINDOW = enum.auto()

    @classmethod
    def basic(cls) -> "MetadataField":
        return cls.MASK | cls.SINKS

    @classmethod
    def paged(cls) -> "MetadataField":
        return cls.QUERY_START_LOC | cls.BLOCK_TABLES | cls.KV_LENS | cls.BLOCK_SIZE | cls.SLIDING_WINDOW


class CacheType(enum.Flag):
    NONE = 0
    TRANSFORMER = enum.auto()
    PAGED = enum.auto()
    RECURRENT = enum.auto()
    HYBRID = enum.auto()

    @classmethod
    def any(cls) -> "CacheType":
        return cls.TRANSFORMER | cls.PAGED | cls.RECURRENT | cls.HYBRID

    @classmethod
    def attention(cls) -> "CacheType":
        return cls.TRANSFORMER | cls.PAGED

    def is_compatible_with(self, other: "CacheType") -> bool:
        return bool(self & other)


@dataclass(frozen=True)
class OperationRequirements:
    """What an operation needs from its caller; ``a | b`` is the union of two declarations."""

    name: str = ""
    required_metadata: MetadataField = MetadataField.NONE
    optional_metadata: MetadataField = MetadataField.NONE
    requires_cache: bool = False
    cache_view_cls: type | None = None

    def __or__(self, other: "OperationRequirements") -> "OperationRequirements":
        if self.cache_view_cls is None:
            view = other.cache_view_cls
        elif other.cache_view_cls is None or other.cache_view_cls is self.cache_view_cls:
            view = self.cache_view_cls
        else:
            view = object  # two different view classes: anything goes
        return OperationRequirements(
            name="+".join(n for n in (self.name, other.name) if n),
            required_metadata=self.required_metadata | other.required_metadata,
            optional_metadata=self.optional_metadata | other.optional_metadata,
            requires_cache=self.requires_cache or other.requires_cache,
            cache_view_cls=view,
        )

    @classmethod
    def create(cls, **fields) -> "OperationRequirements":
        return cls(**fields)

    @classmethod
    def default(cls, name: str = "") -> "OperationRequirements":
        return cls(name=name, optional_metadata=MetadataField.basic())


@dataclass
class RequirementsBuilder:
    name: str
    _req: OperationRequirements = field(default_factory=OperationRequirements, repr=False)

    def require_metadata(self, *fields: MetadataField) -> "RequirementsBuilder":
        for f in fields:
            self._req = replace(self._req, required_metadata=self._req.required_metadata | f)
        return self

    def optional_metadata(self, *fields: MetadataField) -> "RequirementsBuilder":
        for f in fields:
            self._req = replace(self._req, optional_metadata=self._req.optional_metadata | f)
        return self

    def require_cache(self, cache_view_cls: type | None = None) -> "RequirementsBuilder":
        self._req = replace(self._req, requires_cache=True, cache_view_cls=cache_view_cls)
        return self

    def build(self) -> OperationRequirements:
        return replace(self._req, name=self.name)


__all__ = ("CacheType", "ExecutionMode", "MetadataField", "OperationRequirements", "RequirementsBuilder")
