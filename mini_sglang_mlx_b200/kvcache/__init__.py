from .base import BaseCacheHandle, SizeInfo  # noqa: F401
from .mha_pool import MHAKVCache  # noqa: F401
from .naive_manager import NaiveCacheManager  # noqa: F401
from .radix_manager import RadixCacheHandle, RadixCacheManager  # noqa: F401


def create_cache_manager(device=None, type: str = "radix", page_size: int = 1):
    """``radix`` or ``naive`` (reference: mini_sglang_mlx/kvcache/__init__.py).  ``page_size`` > 1
    keeps the radix tree page-aligned (the reference has one token per page)."""
    if type == "radix":
        return RadixCacheManager(device=device, page_size=page_size)
    if type == "naive":
        return NaiveCacheManager(device=device)
    raise ValueError(f"unknown cache manager type {type!r}")
