"""The decode call site of the reference's attention patch (vllm_int8/vllm_int8_attention_patch.py:60-137):
the gate that recognises a pure decode step and the call that serves it from the layer's INT8 cache.
The monkey-patching of vLLM itself is outside this package."""

from __future__ import annotations

from ..ops import int8_paged_attention
from .cache_manager import get_layer_cache


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


def _run_int8_attention(layer, query, attn_metadata):
    """query may be padded beyond num_actual_tokens; the slice is a view and is passed on as such."""
    shadow = get_layer_cache(layer.layer_name)
    tokens = int(getattr(attn_metadata, "num_actual_tokens", query.shape[0]))
    return int8_paged_attention(
        query[:tokens],
        shadow.key_cache,
        shadow.value_cache,
        _get_block_table(attn_metadata).contiguous(),
        attn_metadata.seq_lens.contiguous(),
        shadow.k_scale,
        shadow.v_scale,
        quantize_q=False,
    )
