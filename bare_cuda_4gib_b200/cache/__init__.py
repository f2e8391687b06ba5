"""Cache manager: page pools, cache groups, block tables and per-request state slots."""

from .manager import CacheDemand, CacheGroup, CacheManager  # noqa: F401
from .page_pool import PagePool  # noqa: F401
