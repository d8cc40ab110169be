from .manager import CacheManager, PagedGroup
from .pages import OutOfPages, PageAccountingError, PagePool
