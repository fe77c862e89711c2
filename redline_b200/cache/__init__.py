from .manager import CacheError, CacheManager, GroupInfo, PageAllocator, RequestCache
