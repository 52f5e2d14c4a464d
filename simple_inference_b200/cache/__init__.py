from .allocator import OutOfPages, PageAllocator
from .manager import CacheManager, PageGroup, pages_for

__all__ = ["OutOfPages", "PageAllocator", "CacheManager", "PageGroup", "pages_for"]
