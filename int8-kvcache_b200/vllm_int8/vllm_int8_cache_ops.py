"""Drop-in for `runtime_int8_cache_write` of the reference module vllm_int8/vllm_int8_cache_ops.py:281-306:
the shape checks vLLM's runtime tensors must pass, then the INT8 cache write."""

from __future__ import annotations

import torch

from ..ops import int8_kv_cache_write


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
