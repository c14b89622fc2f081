"""Oracle: static symmetric per-KV-head INT8 quantisation (test infrastructure).

Follows src/quant.py:37-40 (`quant_kv_static_per_head`) and src/quant.py:33-34
(`dequant_kv_per_head`) of the reference: the quotient is formed in fp32
(bf16/fp16 inputs are promoted first, exactly what torch's type promotion does
for `x_bf16 / scale_fp32`), rounded half-to-even, clamped to [-127, 127] and
narrowed to int8.  The reference's Triton write kernel additionally floors the
scale at 1e-6 (src/triton_ops/int8_cache_write.py:50-51); `floor_scale=True`
reproduces that, and is a no-op for every scale >= 1e-6.
"""

from __future__ import annotations

import torch

SCALE_FLOOR = 1e-6


def _as_head_broadcast(scale: torch.Tensor, ndim: int, head_axis: int) -> torch.Tensor:
    shape = [1] * ndim
    shape[head_axis] = scale.numel()
    return scale.reshape(shape)


def static_quant_per_head(
    x: torch.Tensor,
    scale: torch.Tensor,
    head_axis: int = 1,
    floor_scale: bool = False,
) -> torch.Tensor:
    """x: any float tensor with a KV-head axis; scale: [Hkv] -> int8, same shape as x."""
    s = scale.detach().to(torch.float32).reshape(-1)
    if floor_scale:
        s = torch.clamp_min(s, SCALE_FLOOR)
    quotient = x.to(torch.float32) / _as_head_broadcast(s, x.ndim, head_axis)
    rounded = torch.round(quotient)  # IEEE round-half-to-even, as torch.round in the reference
    return torch.clamp(rounded, -127.0, 127.0).to(torch.int8)


def dequant_per_head(
    q: torch.Tensor, scale: torch.Tensor, head_axis: int = 1, dtype=torch.float32
) -> torch.Tensor:
    """int8 -> float: q * scale[head] (src/quant.py:33-34)."""
    s = scale.detach().to(dtype).reshape(-1)
    return q.to(dtype) * _as_head_broadcast(s, q.ndim, head_axis)


def dynamic_quant_per_token_head(x: torch.Tensor):
    """x [T, Hkv, D] -> (int8 [T, Hkv, D], fp32 scale [T, Hkv]): one scale per (token, head),
    scale = max(absmax / 127, 1e-6), q = clamp(x / scale, +-127) rounded half away from zero in fp32.

    Follows the arithmetic of the reference's dynamic write kernel
    (vllm_int8/vllm_int8_cache_ops.py:70-93), which is its only definition of this scheme; the reference pins it
    only through a dequantisation-error bound (tests/test_vllm_int8_cache_ops.py: mean abs error < 0.02)."""
    xf = x.to(torch.float32)
    scale = torch.clamp_min(xf.abs().amax(dim=-1) / 127.0, SCALE_FLOOR)
    q = torch.clamp(xf / scale.unsqueeze(-1), -127.0, 127.0)
    q = torch.where(q >= 0, torch.floor(q + 0.5), torch.ceil(q - 0.5))
    return q.to(torch.int8), scale
