"""Per-layer INT8 cache registry with the interface of the reference's vllm_int8/cache_manager.py:8-70:
each layer owns zero-initialised int8 caches [num_blocks, block_size, Hkv, D] and its static scales."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict

import torch


@dataclass
class LayerInt8Cache:
    key_cache: torch.Tensor
    value_cache: torch.Tensor
    k_scale: torch.Tensor
    v_scale: torch.Tensor


INT8_CACHE_POOL: Dict[str, LayerInt8Cache] = {}


def has_layer_cache(layer_name: str) -> bool:
    return layer_name in INT8_CACHE_POOL


def get_layer_cache(layer_name: str) -> LayerInt8Cache:
    return INT8_CACHE_POOL[layer_name]


def allocate_layer_cache(*, layer_name, num_blocks, block_size, num_kv_heads, head_dim, k_scale, v_scale, device):
    shape = (num_blocks, block_size, num_kv_heads, head_dim)
    entry = LayerInt8Cache(
        key_cache=torch.zeros(shape, dtype=torch.int8, device=device),
        value_cache=torch.zeros(shape, dtype=torch.int8, device=device),
        k_scale=k_scale,
        v_scale=v_scale,
    )
    INT8_CACHE_POOL[layer_name] = entry
    return entry


def clear_cache_pool() -> None:
    INT8_CACHE_POOL.clear()
