"""Oracle: fp32 decode attention over a paged cache (test infrastructure).

Restates src/attention_ref.py:11-28 (fp32 scores / sqrt(D), softmax over the
tokens, GQA by contiguous groups: query head h reads KV head h // (Hq/Hkv)),
the dequantise-then-attend chain used by the reference's loop reference
(src/triton_ops/int8_paged_attention.py:776-814), and the split-KV merge
(src/triton_ops/int8_paged_attention.py:330-388) expressed on (out, lse) pairs.
"""

from __future__ import annotations

import math
from typing import Sequence, Tuple

import torch

from .paged_cache import gather_paged_cache
from .quant import dequant_per_head


def decode_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """q [Hq, D], k/v [Hkv, T, D] (one sequence) -> [Hq, D] fp32."""
    Hq, D = q.shape
    Hkv = k.shape[0]
    assert Hq % Hkv == 0
    group = Hq // Hkv
    qg = q.to(torch.float32).reshape(Hkv, group, D)
    kf = k.to(torch.float32)
    vf = v.to(torch.float32)
    scores = torch.matmul(qg, kf.transpose(1, 2)) / math.sqrt(D)  # [Hkv, group, T]
    probs = torch.softmax(scores, dim=-1)
    return torch.matmul(probs, vf).reshape(Hq, D)


def partial_attention_with_lse(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention over a token subset plus its natural-log sum-exp per query head.

    An empty subset returns zeros and lse = -inf, which the merge ignores.
    """
    Hq, D = q.shape
    Hkv, T, _ = k.shape
    if T == 0:
        return torch.zeros(Hq, D), torch.full((Hq,), -math.inf)
    group = Hq // Hkv
    qg = q.to(torch.float32).reshape(Hkv, group, D)
    scores = torch.matmul(qg, k.to(torch.float32).transpose(1, 2)) / math.sqrt(D)
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.matmul(torch.softmax(scores, dim=-1), v.to(torch.float32))
    return out.reshape(Hq, D), lse.reshape(Hq)


def merge_partials(outs: torch.Tensor, lses: torch.Tensor) -> torch.Tensor:
    """outs [R, ..., D], lses [R, ...] -> [..., D]; weights exp(lse_r - max lse)."""
    top = torch.amax(lses, dim=0, keepdim=True)
    top = torch.where(torch.isinf(top), torch.zeros_like(top), top)
    w = torch.exp(lses - top)  # exp(-inf) = 0 for empty parts
    denom = torch.clamp_min(w.sum(dim=0), 1e-20)
    return (outs * w.unsqueeze(-1)).sum(dim=0) / denom.unsqueeze(-1)


def quantize_query_per_head(q: torch.Tensor) -> torch.Tensor:
    """The reference's optional INT8 query (src/triton_ops/int8_paged_attention.py:798-802, kernel side :137-146):
    per query head, scale = max(absmax / 127, 1e-6), q8 = clamp(round_half_away_from_zero(q / scale), -127, 127),
    and the dot product uses q8 * scale.  q [..., D] -> fp32 of the same shape."""
    qf = q.to(torch.float32)
    scale = torch.clamp(qf.abs().amax(dim=-1, keepdim=True) / 127.0, min=1e-6)
    x = qf / scale
    q8 = torch.where(x >= 0, torch.floor(x + 0.5), -torch.floor(-x + 0.5))
    return torch.clamp(q8, -127, 127) * scale


def int8_paged_attention_oracle(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: Sequence[int],
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    quantize_q: bool = False,
) -> torch.Tensor:
    """[B, Hq, D] fp32: gather pages -> int8 * scale[head] -> fp32 attention.  quantize_q: the query is first
    replaced by its per-head INT8 quantisation (quantize_query_per_head)."""
    ks, vs = gather_paged_cache(key_cache, value_cache, block_tables, seq_lens)
    rows = []
    for b in range(query.shape[0]):
        k = dequant_per_head(ks[b], k_scale, head_axis=0)
        v = dequant_per_head(vs[b], v_scale, head_axis=0)
        q = quantize_query_per_head(query[b]) if quantize_q else query[b]
        rows.append(decode_attention(q, k, v))
    return torch.stack(rows)


def float_paged_attention_oracle(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: Sequence[int],
) -> torch.Tensor:
    """Same attention on an un-quantised (bf16/fp16/fp32) paged cache; fp32 result."""
    ks, vs = gather_paged_cache(key_cache, value_cache, block_tables, seq_lens)
    return torch.stack([decode_attention(query[b], ks[b], vs[b]) for b in range(query.shape[0])])


def dynamic_int8_paged_attention_oracle(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    k_scale_cache: torch.Tensor,
    v_scale_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: Sequence[int],
) -> torch.Tensor:
    """[B, Hq, D] fp32 attention over an INT8 cache with one scale per (block, slot, head): the cache is first
    dequantised as the reference's `dequantize_int8_cache` does (vllm_int8/vllm_int8_cache_ops.py:250-256,
    `cache.float() * scale_cache[..., None]`), then attended with the fp32 reference attention."""
    kf = key_cache.float() * k_scale_cache.float()[..., None]
    vf = value_cache.float() * v_scale_cache.float()[..., None]
    return float_paged_attention_oracle(query, kf, vf, block_tables, seq_lens)
