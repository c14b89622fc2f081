"""Per-layer INT8 cache registry behind the interface of the reference's vllm_int8/cache_manager.py:8-70
(`LayerInt8Cache`, `INT8_CACHE_POOL`, `has_layer_cache`, `get_layer_cache`, `allocate_layer_cache`,
`clear_cache_pool`).  Every layer owns zero-initialised int8 caches [num_blocks, block_size, Hkv, D] — the
layout both kernels read and write — and its static scales."""

from __future__ import annotations

from typing import Dict, NamedTuple

import torch


class LayerInt8Cache(NamedTuple):
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor


class _Pool(dict):
    """layer name -> LayerInt8Cache"""

    def allocate(self, layer_name: str, shape, k_scale, v_scale, device) -> LayerInt8Cache:
        keys = torch.zeros(shape, dtype=torch.int8, device=device)
        self[layer_name] = LayerInt8Cache(keys, torch.zeros_like(keys), k_scale, v_scale)
        return self[layer_name]


INT8_CACHE_POOL: Dict[str, LayerInt8Cache] = _Pool()

has_layer_cache = INT8_CACHE_POOL.__contains__
get_layer_cache = INT8_CACHE_POOL.__getitem__
clear_cache_pool = INT8_CACHE_POOL.clear


def allocate_layer_cache(*, layer_name, num_blocks, block_size, num_kv_heads, head_dim, k_scale, v_scale, device):
    return INT8_CACHE_POOL.allocate(layer_name, (num_blocks, block_size, num_kv_heads, head_dim), k_scale, v_scale, device)
