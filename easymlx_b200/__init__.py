"""B200-native ragged paged attention behind easymlx's attention-operation interface."""

from .caching import PageCache, PageCacheConfig, PageCacheView, PageMetadata, build_query_start_loc
from .inference.esurge import PageTableRunner, extract_last_tokens
from .layers.attention import AttentionPerformer
from .operations import (AttentionOutput, BaseOperation, ExecutionMode, MetadataField, OperationExecutor,
                         OperationRegistry, UnifiedAttention, UnifiedAttnMetadata, paged_attention)

__version__ = "0.1.0"

__all__ = (
    "AttentionOutput", "AttentionPerformer", "BaseOperation", "ExecutionMode", "MetadataField", "OperationExecutor",
    "OperationRegistry", "PageCache", "PageCacheConfig", "PageCacheView", "PageMetadata", "PageTableRunner",
    "UnifiedAttention", "UnifiedAttnMetadata", "build_query_start_loc", "extract_last_tokens", "paged_attention",
)
