"""B200-native paged attention behind the ``mini_sglang_mlx_kernel`` op surface.

``mini_sglang_mlx_b200.kernel`` exposes the operators with the reference's
names and keyword arguments over CUDA ``torch.Tensor`` inputs;
``mini_sglang_mlx_b200.attention`` and ``mini_sglang_mlx_b200.kvcache`` mirror
the reference's ``AttnBackend`` and ``MHAKVCache`` that call them.
"""
from .kernel import (  # noqa: F401
    fast_compare_key,
    qk_norm_rope_store,
    gather_kv_indices,
    paged_decode_attention,
    paged_decode_attention_p16,
    paged_prefill_attention,
    paged_prefill_attention_p16,
    store_kv_cache,
)

__all__ = [
    "paged_decode_attention",
    "paged_prefill_attention",
    "paged_decode_attention_p16",
    "paged_prefill_attention_p16",
    "store_kv_cache",
    "gather_kv_indices",
    "fast_compare_key",
    "qk_norm_rope_store",
]
