"""Drop-in for the reference module src/triton_ops/int8_cache_write.py.

`int8_kv_cache_write` is the sm_100a CUDA operator.  The two helpers below exist because the
reference's tests import them from this module (tests/test_int8_paged_attention.py:6-9); they are
plain device-agnostic PyTorch for debugging and are never called by the operator.
"""

from __future__ import annotations

import torch

from ..ops import int8_kv_cache_write  # noqa: F401


def torch_int8_kv_cache_write_reference(key, value, key_cache, value_cache, slot_mapping, k_scale, v_scale):
    """Debug helper with the reference's name (src/triton_ops/int8_cache_write.py:152-183): round-half-even
    quantisation in PyTorch and an indexed scatter; later tokens win when a slot repeats."""
    assert key.ndim == 3
    block_size = key_cache.shape[1]
    slots = slot_mapping.reshape(-1).long()
    live = (slots >= 0).nonzero().reshape(-1).tolist()
    ks = k_scale.float().reshape(1, -1, 1)
    vs = v_scale.float().reshape(1, -1, 1)
    kq = torch.clamp(torch.round(key.float() / ks), -127, 127).to(torch.int8)
    vq = torch.clamp(torch.round(value.float() / vs), -127, 127).to(torch.int8)
    for t in live:
        s = int(slots[t])
        key_cache[s // block_size, s % block_size] = kq[t]
        value_cache[s // block_size, s % block_size] = vq[t]


def dequantize_paged_cache_for_debug(cache: torch.Tensor, scale: torch.Tensor):
    """int8 cache [num_blocks, BS, Hkv, D] * scale[Hkv] -> float32 (src/triton_ops/int8_cache_write.py:186-189)."""
    assert cache.dtype == torch.int8
    return cache.float() * scale.float().reshape(1, 1, -1, 1)
