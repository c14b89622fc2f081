"""Drop-in for the reference module vllm_int8/vllm_int8_cache_ops.py: `runtime_int8_cache_write` (:281-306, the
static-scale write used by the attention path) and the dynamic per-(token, head) scheme with its helpers
(`reshape_and_cache_int8` :134-210, `allocate_int8_kv_cache` :213-247, `dequantize_int8_cache` :250-256,
`print_int8_cache_memory` :263-277).  `int8_paged_attention_dynamic` is an addition: the decode attention that reads
the caches and scale caches of the dynamic scheme, for which the reference has a writer and a debug dequantiser only."""

from __future__ import annotations

import torch

from ..ops import int8_kv_cache_write, int8_paged_attention_dynamic, reshape_and_cache_int8  # noqa: F401


def runtime_int8_cache_write(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
) -> None:
    assert key.ndim == 3
    assert value.shape == key.shape
    assert key_cache.dtype == torch.int8
    assert value_cache.dtype == torch.int8
    assert slot_mapping.ndim == 1
    assert slot_mapping.numel() == key.shape[0]
    assert k_scale.shape == (key.shape[1],)
    assert v_scale.shape == (key.shape[1],)
    int8_kv_cache_write(key, value, key_cache, value_cache, slot_mapping, k_scale, v_scale)


def allocate_int8_kv_cache(num_blocks: int, block_size: int, num_kv_heads: int, head_dim: int, device="cuda"):
    """(key_cache, value_cache int8 [num_blocks, BS, Hkv, D], k_scale_cache, v_scale_cache fp32 [num_blocks, BS, Hkv])."""
    key_cache = torch.empty((num_blocks, block_size, num_kv_heads, head_dim), device=device, dtype=torch.int8)
    k_scale_cache = torch.empty((num_blocks, block_size, num_kv_heads), device=device, dtype=torch.float32)
    return key_cache, torch.empty_like(key_cache), k_scale_cache, torch.empty_like(k_scale_cache)


def dequantize_int8_cache(cache: torch.Tensor, scale_cache: torch.Tensor) -> torch.Tensor:
    """Debug helper: INT8 cache times its per-(slot, head) scale -> fp32."""
    assert cache.dtype == torch.int8
    return cache.float() * scale_cache[..., None]


def int8_cache_memory_bytes(key_cache, value_cache, k_scale_cache, v_scale_cache):
    """(INT8 payload bytes, scale bytes)."""
    nbytes = lambda x: x.numel() * x.element_size()
    return nbytes(key_cache) + nbytes(value_cache), nbytes(k_scale_cache) + nbytes(v_scale_cache)


def print_int8_cache_memory(key_cache, value_cache, k_scale_cache, v_scale_cache) -> None:
    kv_bytes, scale_bytes = int8_cache_memory_bytes(key_cache, value_cache, k_scale_cache, v_scale_cache)
    print(f"K/V INT8 : {kv_bytes / 1024**2:.3f} MB")
    print(f"Scales    : {scale_bytes / 1024**2:.3f} MB")
    print(f"Total     : {(kv_bytes + scale_bytes) / 1024**2:.3f} MB")
