"""The KV-cache-update call site of the reference's shadow-cache patch (vllm_int8/vllm_shadow_cache_patch.py:26-191):
after the engine's own cache update, mirror the step's new K/V rows into the layer's INT8 cache, which is
allocated on first use from the page geometry of the engine's cache and the layer's static scales.

`shadow_cache_update` is the mirror step on its own; `apply_shadow_cache_patch` wraps the
`do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping)` method of an attention-implementation class
(vLLM's TritonAttentionImpl when none is given) so that it runs after the original.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..ops import int8_kv_cache_write
from .cache_manager import allocate_layer_cache, get_layer_cache, has_layer_cache
from .static_scales import get_layer_scales

WRITE_CALL_COUNT: Dict[str, int] = {}
NATIVE_CACHE_BYTES_BY_LAYER: Dict[str, int] = {}
_PATCHED_CLASSES = set()


def _infer_native_page_dims(kv_cache: torch.Tensor, num_kv_heads: int) -> Tuple[int, int]:
    """(num_blocks, block_size) of the engine's own cache; three layouts are recognised:
    fused [num_blocks, Hkv, block_size, 2*D], split [num_blocks, 2, block_size, Hkv, D],
    older split [2, num_blocks, block_size, Hkv, D]."""
    shape = tuple(kv_cache.shape)
    if len(shape) == 4 and shape[1] == num_kv_heads:
        return int(shape[0]), int(shape[2])
    if len(shape) == 5 and shape[1] == 2:
        return int(shape[0]), int(shape[2])
    if len(shape) == 5 and shape[0] == 2:
        return int(shape[1]), int(shape[2])
    raise ValueError(f"Unsupported vLLM kv_cache shape {shape} for Hkv={num_kv_heads}")


def shadow_cache_update(layer, key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                        slot_mapping: torch.Tensor, *, writer=int8_kv_cache_write) -> None:
    """Mirror key/value [T, Hkv, D] into the INT8 cache of `layer.layer_name` at slot_mapping."""
    name = layer.layer_name
    NATIVE_CACHE_BYTES_BY_LAYER.setdefault(name, kv_cache.numel() * kv_cache.element_size())
    assert key.ndim == 3 and value.ndim == 3
    num_tokens, num_kv_heads, head_dim = key.shape
    if not has_layer_cache(name):
        num_blocks, block_size = _infer_native_page_dims(kv_cache, num_kv_heads)
        k_scale, v_scale = get_layer_scales(name, key.device)
        allocate_layer_cache(layer_name=name, num_blocks=num_blocks, block_size=block_size, num_kv_heads=num_kv_heads,
                             head_dim=head_dim, k_scale=k_scale, v_scale=v_scale, device=key.device)
    shadow = get_layer_cache(name)
    slots = slot_mapping.reshape(-1).contiguous()
    assert slots.numel() == num_tokens, f"slot_mapping={tuple(slots.shape)}, key={tuple(key.shape)}"
    writer(key, value, shadow.key_cache, shadow.value_cache, slots, shadow.k_scale, shadow.v_scale)
    WRITE_CALL_COUNT[name] = WRITE_CALL_COUNT.get(name, 0) + 1


def apply_shadow_cache_patch(impl_cls=None, verbose_layer: int = 0):
    """Wrap impl_cls.do_kv_cache_update: original first, then the INT8 mirror.  Idempotent per class."""
    del verbose_layer  # accepted for call compatibility; this module does not print
    if impl_cls is None:
        from vllm.v1.attention.backends.triton_attn import TritonAttentionImpl as impl_cls
    if impl_cls in _PATCHED_CLASSES:
        return impl_cls
    original = impl_cls.do_kv_cache_update

    def patched_do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        original(self, layer, key, value, kv_cache, slot_mapping)
        shadow_cache_update(layer, key, value, kv_cache, slot_mapping)

    impl_cls.do_kv_cache_update = patched_do_kv_cache_update
    _PATCHED_CLASSES.add(impl_cls)
    return impl_cls
