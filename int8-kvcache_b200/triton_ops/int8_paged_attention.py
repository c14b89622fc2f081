"""Drop-in for the reference module src/triton_ops/int8_paged_attention.py.

`int8_paged_attention` is the sm_100a CUDA operator.  `torch_int8_paged_attention_reference` exists
because the reference's tests import it from this module (tests/test_int8_paged_attention.py:10-13);
it is plain PyTorch for debugging and is never called by the operator.
"""

from __future__ import annotations

import math

import torch

from ..ops import int8_paged_attention  # noqa: F401


def torch_int8_paged_attention_reference(
    query, key_cache, value_cache, block_tables, seq_lens, k_scale, v_scale, *, quantize_q: bool = False
):
    """Debug helper with the reference's name (src/triton_ops/int8_paged_attention.py:776-814):
    gather the pages of each sequence, dequantise per head, fp32 softmax attention, result in query.dtype."""
    B, Hq, D = query.shape
    block_size, Hkv = key_cache.shape[1], key_cache.shape[2]
    assert Hq % Hkv == 0
    group = Hq // Hkv
    rows = []
    for b in range(B):
        T = int(seq_lens[b])
        ids = block_tables[b, : (T + block_size - 1) // block_size].long()
        k = key_cache[ids].reshape(-1, Hkv, D)[:T].float() * k_scale.float().reshape(1, -1, 1)
        v = value_cache[ids].reshape(-1, Hkv, D)[:T].float() * v_scale.float().reshape(1, -1, 1)
        q = query[b].float()
        if quantize_q:
            qs = torch.clamp(q.abs().amax(dim=-1, keepdim=True) / 127.0, min=1e-6)
            x = q / qs
            q = torch.clamp(torch.where(x >= 0, torch.floor(x + 0.5), -torch.floor(-x + 0.5)), -127, 127) * qs
        qg = q.reshape(Hkv, group, D)
        score = torch.einsum("hgd,thd->hgt", qg, k) / math.sqrt(D)
        rows.append(torch.einsum("hgt,thd->hgd", torch.softmax(score, dim=-1), v).reshape(Hq, D))
    return torch.stack(rows).to(query.dtype)
