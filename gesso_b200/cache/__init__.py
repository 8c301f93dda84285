"""Cache manager: paged keys/values with block tables, and per-request state slots."""
from .manager import FREED, CacheManager, IndexPool, PagedGroupSpec

__all__ = ["FREED", "CacheManager", "IndexPool", "PagedGroupSpec"]
