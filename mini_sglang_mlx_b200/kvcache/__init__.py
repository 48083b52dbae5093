from .mha_pool import MHAKVCache  # noqa: F401
