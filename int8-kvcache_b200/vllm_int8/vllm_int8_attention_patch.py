"""The attention call site of the reference's patch (vllm_int8/vllm_int8_attention_patch.py:60-334): the gate that
recognises a pure decode step, the call that serves it from the layer's INT8 cache, and the wrapper of an
attention implementation's `forward` in the reference's three modes:

  shadow     run the original, run INT8 beside it, record cosine / relative L2 / MAE, return the original
  takeover   same comparison, but the INT8 result overwrites the output
  int8_only  INT8 alone (no comparison, no host synchronisation: the reference's operator reads seq_lens back on
             the host twice per call, src/triton_ops/int8_paged_attention.py:720-721, this call site passes an upper
             bound instead, so a decode step can be captured in a CUDA graph), counted in ATTN_INT8_HITS

Anything that is not a decode step, or a layer without an INT8 cache, goes to the original forward.
"""

from __future__ import annotations

from typing import Dict, List

import torch

from ..ops import int8_paged_attention
from .cache_manager import get_layer_cache, has_layer_cache

ATTN_COMPARE_COUNT: Dict[str, int] = {}
ATTN_METRICS: Dict[str, List[dict]] = {}
ATTN_INT8_HITS: Dict[str, int] = {}
ATTN_INT8_STATS: Dict[str, int] = {"last_batch": 0, "max_batch": 0}
_PATCHED_CLASSES = set()


def _get_block_table(attn_metadata):
    table = getattr(attn_metadata, "block_table", None)
    return table if table is not None else getattr(attn_metadata, "block_tables", None)


def _is_supported_decode(query, attn_metadata) -> bool:
    """True for a step with exactly one new query token per sequence (any batch size)."""
    if attn_metadata is None or query.ndim != 3:
        return False
    seq_lens = getattr(attn_metadata, "seq_lens", None)
    table = _get_block_table(attn_metadata)
    if seq_lens is None or table is None or table.ndim != 2:
        return False
    batch = int(seq_lens.numel())
    if batch <= 0 or table.shape[0] != batch:
        return False
    tokens = getattr(attn_metadata, "num_actual_tokens", None)
    if int(query.shape[0] if tokens is None else tokens) != batch:
        return False
    max_query_len = getattr(attn_metadata, "max_query_len", None)
    return max_query_len is None or int(max_query_len) == 1


def _max_seq_len_bound(attn_metadata, block_table, block_size: int) -> int:
    """An upper bound of seq_lens that costs no device read: the engine's own max_seq_len when its metadata carries
    one (a host integer), else what the block table can address."""
    bound = getattr(attn_metadata, "max_seq_len", None)
    limit = int(block_table.shape[1]) * int(block_size)
    if bound is None or isinstance(bound, torch.Tensor):  # a device tensor would have to be read back
        return limit
    return max(1, min(int(bound), limit))


def _run_int8_attention(layer, query, attn_metadata):
    """query may be padded beyond num_actual_tokens; the slice is a view and is passed on as such.  No device value
    is read on the host: the sequence-length bound comes from the metadata or from the table's width."""
    shadow = get_layer_cache(layer.layer_name)
    tokens = int(getattr(attn_metadata, "num_actual_tokens", query.shape[0]))
    block_table = _get_block_table(attn_metadata)
    return int8_paged_attention(
        query[:tokens],
        shadow.key_cache,
        shadow.value_cache,
        block_table,
        attn_metadata.seq_lens,
        shadow.k_scale,
        shadow.v_scale,
        quantize_q=False,
        max_seq_len=_max_seq_len_bound(attn_metadata, block_table, shadow.key_cache.shape[1]),
    )


def _compare(int8_out: torch.Tensor, ref_out: torch.Tensor) -> dict:
    a, b = int8_out.float().reshape(-1), ref_out.float().reshape(-1)
    return {
        "cosine": float(torch.nn.functional.cosine_similarity(a, b, dim=0)),
        "relative_l2": float((a - b).norm() / b.norm().clamp_min(1e-12)),
        "mae": float((a - b).abs().mean()),
    }


def apply_int8_attention_patch(impl_cls=None, *, mode: str = "shadow", verbose_layer: int = 0, max_compare_calls: int = 8):
    """Wrap impl_cls.forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
    output_block_scale=None) in the given mode; vLLM's TritonAttentionImpl is patched when no class is given."""
    del verbose_layer, max_compare_calls  # accepted for call compatibility; this module does not print
    if mode not in ("shadow", "takeover", "int8_only"):
        raise ValueError(f"Unknown mode: {mode}")
    if impl_cls is None:
        from vllm.v1.attention.backends.triton_attn import TritonAttentionImpl as impl_cls
    if impl_cls in _PATCHED_CLASSES:
        raise RuntimeError("Attention has already been patched in this Python process.")
    original_forward = impl_cls.forward

    def patched_forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                        output_block_scale=None):
        name = getattr(layer, "layer_name", None)
        if name is None or not has_layer_cache(name) or not _is_supported_decode(query, attn_metadata):
            return original_forward(self, layer, query, key, value, kv_cache, attn_metadata, output,
                                    output_scale=output_scale, output_block_scale=output_block_scale)
        if mode == "int8_only":
            int8_out = _run_int8_attention(layer, query, attn_metadata)
            ATTN_INT8_HITS[name] = ATTN_INT8_HITS.get(name, 0) + 1
            batch = int(attn_metadata.seq_lens.numel())
            ATTN_INT8_STATS["last_batch"] = batch
            ATTN_INT8_STATS["max_batch"] = max(ATTN_INT8_STATS.get("max_batch", 0), batch)
            n = int8_out.shape[0]
            output[:n].copy_(int8_out.reshape_as(output[:n]))
            return output
        result = original_forward(self, layer, query, key, value, kv_cache, attn_metadata, output,
                                  output_scale=output_scale, output_block_scale=output_block_scale)
        int8_out = _run_int8_attention(layer, query, attn_metadata)
        n = int8_out.shape[0]
        ref_out = output[:n].detach().reshape(int8_out.shape)
        ATTN_COMPARE_COUNT[name] = ATTN_COMPARE_COUNT.get(name, 0) + 1
        ATTN_METRICS.setdefault(name, []).append(_compare(int8_out, ref_out))
        if mode == "shadow":
            return result
        assert not torch.isnan(int8_out).any() and not torch.isinf(int8_out).any()
        output[:n].copy_(int8_out.reshape_as(output[:n]))
        ATTN_INT8_HITS[name] = ATTN_INT8_HITS.get(name, 0) + 1
        return output

    impl_cls.forward = patched_forward
    _PATCHED_CLASSES.add(impl_cls)
    return impl_cls
