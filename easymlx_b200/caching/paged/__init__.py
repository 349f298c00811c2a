from .cache import PageCache, PageCacheConfig, PageCacheView, PageMetadata, build_query_start_loc

__all__ = ("PageCache", "PageCacheConfig", "PageCacheView", "PageMetadata", "build_query_start_loc")
