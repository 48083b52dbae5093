from .cache import CacheManager  # noqa: F401
from .table import TableManager  # noqa: F401
