from .allocators import CacheError, IndexPool  # noqa: F401
from .cache import PAGE, Cache, pages_for  # noqa: F401
