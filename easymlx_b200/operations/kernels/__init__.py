from .unified_attention import UnifiedAttention, UnifiedAttnConfig, UnifiedAttnMetadata, paged_attention

__all__ = ("UnifiedAttention", "UnifiedAttnConfig", "UnifiedAttnMetadata", "paged_attention")
