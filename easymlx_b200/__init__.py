"""B200-native ragged paged attention behind easymlx's attention-operation interface."""

from .caching import PageCache, PageCacheConfig, PageCacheView, PageMetadata, build_query_start_loc
from .layers.attention import AttentionPerformer
from .operations import (AttentionOutput, BaseOperation, ExecutionMode, MetadataField, OperationExecutor,
                         OperationRegistry, UnifiedAttention, UnifiedAttnMetadata, paged_attention)

__version__ = "0.1.0"

__all__ = (
    "AttentionOutput", "AttentionPerformer", "BaseOperation", "ExecutionMode", "MetadataField", "OperationExecutor",
    "OperationRegistry", "PageCache", "PageCacheConfig", "PageCacheView", "PageMetadata", "UnifiedAttention",
    "UnifiedAttnMetadata", "build_query_start_loc", "paged_attention",
)
