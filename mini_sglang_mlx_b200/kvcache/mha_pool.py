"""KV page pool in HBM: per layer one K and one V tensor
``(num_pages, num_kv_heads, head_dim)``, written through ``store_kv_cache``.

Mirror of the reference's ``MHAKVCache``
(mini_sglang_mlx/kvcache/mha_pool.py:10-56).  A "page" of the reference holds
one token; the row index is the slot id that page tables and ``kv_indices``
carry.  Both tensors of all layers are carved from one allocation so that a
pool sized for most of the 180 GB of a B200 is a single request to the
allocator.  Unlike the reference, ``store_kv`` does not synchronise the
device: the scatter is ordered before the attention call by the stream.
"""
from __future__ import annotations

import torch

from ..kernel import store_kv_cache


class MHAKVCache:
    def __init__(self, num_kv_heads: int, num_layers: int, head_dim: int, num_pages: int,
                 dtype: torch.dtype, device="cuda") -> None:
        self._num_layers = num_layers
        self._dtype = dtype
        self._storage_shape = (num_pages, num_kv_heads, head_dim)
        # (2, layers, pages, heads, dim): K planes then V planes
        self._buffer = torch.zeros((2, num_layers, num_pages, num_kv_heads, head_dim),
                                   dtype=dtype, device=device)
        self._k_buffer = [self._buffer[0, i] for i in range(num_layers)]
        self._v_buffer = [self._buffer[1, i] for i in range(num_layers)]

    def k_cache(self, index: int) -> torch.Tensor:
        return self._k_buffer[index]

    def v_cache(self, index: int) -> torch.Tensor:
        return self._v_buffer[index]

    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None:
        assert out_loc.dtype == torch.int32, "out_loc must be int32"
        if len(out_loc) != k.shape[0] or len(out_loc) != v.shape[0]:
            raise ValueError(
                f"store_kv shape mismatch: len(out_loc)={len(out_loc)}, "
                f"k.shape={tuple(k.shape)}, v.shape={tuple(v.shape)}")
        store_kv_cache(k_cache=self._k_buffer[layer_id], v_cache=self._v_buffer[layer_id],
                       indices=out_loc, k=k, v=v)

    @property
    def dtype(self) -> torch.dtype:
        return self._dtype

    @property
    def num_layers(self) -> int:
        return self._num_layers

    @property
    def num_pages(self) -> int:
        return self._storage_shape[0]
