"""Operation plugin API and the paged-attention operation registered in it."""

from ._attention_outputs import AttentionOutput
from ._base_operation import BaseOperation, Operation, OperationRegistry
from .executor import OperationExecutor
from .kernels import UnifiedAttention, UnifiedAttnConfig, UnifiedAttnMetadata, paged_attention
from .requirements import CacheType, ExecutionMode, MetadataField, OperationRequirements, RequirementsBuilder

__all__ = (
    "AttentionOutput", "BaseOperation", "CacheType", "ExecutionMode", "MetadataField", "Operation",
    "OperationExecutor", "OperationRegistry", "OperationRequirements", "RequirementsBuilder",
    "UnifiedAttention", "UnifiedAttnConfig", "UnifiedAttnMetadata", "paged_attention",
)
