"""Cache manager: paged keys and values with block tables, and per-request state slots."""
from .manager import CacheManager, PagedBinding, StateBinding
from .pages import OutOfPages, PagePool

__all__ = ["CacheManager", "PagedBinding", "StateBinding", "OutOfPages", "PagePool"]
