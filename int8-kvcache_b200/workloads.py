"""Seeded synthetic inputs shaped like the decode-attention layers the kernels serve.

The distributions stand in for real Qwen2.5 K/V activations (no model weights are
available offline): queries are N(0,1); keys are N(0,1) with four outlier channels per
KV head scaled x8 (real keys show a few dominant channels per head); values are
N(0, 0.5).  Static per-KV-head scales are absmax/127 over a separate seeded calibration
draw, floored at 1e-6 — the formula of the reference's calibration script
(scripts/04_calibrate_static_scale.py:50-56), so values outside the calibrated range
saturate at +-127 exactly as they would in production.

Everything here is host-side input construction; nothing in this file computes attention.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class LayerShape:
    """One attention layer: query heads, KV heads, head dim, tokens per cache block."""

    num_q_heads: int = 28
    num_kv_heads: int = 4
    head_dim: int = 128
    block_size: int = 16

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads


QWEN25_7B = LayerShape(28, 4, 128, 16)
QWEN25_72B = LayerShape(64, 8, 128, 16)

OUTLIERS_PER_HEAD = 4
OUTLIER_GAIN = 8.0
V_STD = 0.5
CALIBRATION_TOKENS = 2048


def _gen(seed: int, device="cpu") -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def outlier_channels(shape: LayerShape, seed: int) -> torch.Tensor:
    """[Hkv, 4] channel indices that carry the x8 gain, from a seeded permutation per head."""
    g = _gen(seed * 7919 + 17)
    rows = [torch.randperm(shape.head_dim, generator=g)[:OUTLIERS_PER_HEAD] for _ in range(shape.num_kv_heads)]
    return torch.stack(rows)


def channel_gain(shape: LayerShape, seed: int, device="cpu") -> torch.Tensor:
    """[Hkv, D] multiplicative gain for keys: 8 on the outlier channels, 1 elsewhere."""
    gain = torch.ones(shape.num_kv_heads, shape.head_dim)
    gain.scatter_(1, outlier_channels(shape, seed), OUTLIER_GAIN)
    return gain.to(device)


def draw_kv(
    num_tokens: int,
    shape: LayerShape,
    gen: torch.Generator,
    gain: torch.Tensor,
    dtype=torch.bfloat16,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """(key, value) of shape [T, Hkv, D] on the generator's device."""
    dev = gen.device
    k = torch.randn(num_tokens, shape.num_kv_heads, shape.head_dim, generator=gen, device=dev)
    k = k * gain.to(dev)
    v = torch.randn(num_tokens, shape.num_kv_heads, shape.head_dim, generator=gen, device=dev) * V_STD
    return k.to(dtype), v.to(dtype)


def draw_query(batch: int, shape: LayerShape, gen: torch.Generator, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.randn(batch, shape.num_q_heads, shape.head_dim, generator=gen, device=gen.device).to(dtype)


def calibrate_scales(shape: LayerShape, seed: int, layer: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Static (k_scale, v_scale), fp32 [Hkv], from a 2048-token CPU calibration draw.

    `layer` perturbs the draw so that each layer of a multi-layer workload has its own scales.
    """
    g = _gen(seed * 104729 + 31 * layer + 5)
    k, v = draw_kv(CALIBRATION_TOKENS, shape, g, channel_gain(shape, seed))
    k_scale = (k.float().abs().amax(dim=(0, 2)) / 127.0).clamp_min(1e-6)
    v_scale = (v.float().abs().amax(dim=(0, 2)) / 127.0).clamp_min(1e-6)
    return k_scale, v_scale


def blocks_needed(seq_lens: Sequence[int], block_size: int) -> torch.Tensor:
    s = torch.as_tensor(list(seq_lens), dtype=torch.long)
    return (s + block_size - 1) // block_size


def permuted_block_tables(
    seq_lens: Sequence[int],
    block_size: int,
    num_blocks: int,
    seed: int,
    table_width: Optional[int] = None,
    dtype=torch.int32,
) -> torch.Tensor:
    """[B, width] logical->physical block ids drawn from a seeded permutation of the pool.

    Entries past a sequence's last block are 0 (the convention of the reference's test
    helper, tests/test_int8_paged_attention.py:16-43); kernels must never read through them.
    """
    need = blocks_needed(seq_lens, block_size)
    total = int(need.sum())
    assert total <= num_blocks, "block pool too small"
    width = int(need.max()) if table_width is None else int(table_width)
    perm = torch.randperm(num_blocks, generator=_gen(seed * 31337 + 3))[:total]
    tables = torch.zeros(len(need), width, dtype=dtype)
    ends = torch.cumsum(need, 0)
    starts = ends - need
    for b in range(len(need)):
        tables[b, : int(need[b])] = perm[int(starts[b]) : int(ends[b])].to(dtype)
    return tables


def slot_mapping_for(block_tables: torch.Tensor, seq_lens: Sequence[int], block_size: int) -> torch.Tensor:
    """int64 slot (= block*block_size + offset) of every token, sequences concatenated in order."""
    parts = []
    bt = block_tables.to(torch.long)
    for b, T in enumerate(seq_lens):
        tok = torch.arange(int(T), dtype=torch.long, device=bt.device)
        parts.append(bt[b, tok // block_size] * block_size + tok % block_size)
    return torch.cat(parts) if parts else torch.zeros(0, dtype=torch.long)


@dataclass
class DecodeCase:
    """Inputs of one decode-attention call plus the bf16 K/V the caches were built from."""

    shape: LayerShape
    query: torch.Tensor  # [B, Hq, D]
    key: torch.Tensor  # [sum(seq), Hkv, D] bf16, sequences concatenated
    value: torch.Tensor
    block_tables: torch.Tensor  # [B, width] int32
    seq_lens: torch.Tensor  # [B] int32
    slot_mapping: torch.Tensor  # [sum(seq)] int64
    k_scale: torch.Tensor  # [Hkv] fp32
    v_scale: torch.Tensor
    num_blocks: int

    def to(self, device) -> "DecodeCase":
        moved = {
            f: (getattr(self, f).to(device) if isinstance(getattr(self, f), torch.Tensor) else getattr(self, f))
            for f in self.__dataclass_fields__
        }
        return DecodeCase(**moved)


def make_decode_case(
    seq_lens: Sequence[int],
    shape: LayerShape = QWEN25_7B,
    seed: int = 0,
    num_blocks: Optional[int] = None,
    pool_factor: float = 2.0,
    layer: int = 0,
    dtype=torch.bfloat16,
) -> DecodeCase:
    """CPU-generated case: seeded K/V/query, static scales, permuted block pool."""
    seq_lens = [int(s) for s in seq_lens]
    need = int(blocks_needed(seq_lens, shape.block_size).sum())
    if num_blocks is None:
        num_blocks = max(1, int(round(need * pool_factor)))
    g = _gen(seed * 2654435761 % (2**31) + 101 * layer + 1)
    gain = channel_gain(shape, seed)
    total = sum(seq_lens)
    key, value = draw_kv(total, shape, g, gain, dtype=dtype)
    query = draw_query(len(seq_lens), shape, g, dtype=dtype)
    k_scale, v_scale = calibrate_scales(shape, seed, layer)
    tables = permuted_block_tables(seq_lens, shape.block_size, num_blocks, seed + 13 * layer)
    return DecodeCase(
        shape=shape,
        query=query,
        key=key,
        value=value,
        block_tables=tables,
        seq_lens=torch.tensor(seq_lens, dtype=torch.int32),
        slot_mapping=slot_mapping_for(tables, seq_lens, shape.block_size),
        k_scale=k_scale,
        v_scale=v_scale,
        num_blocks=num_blocks,
    )


def config1_case(seed: int = 0) -> DecodeCase:
    """B=1, 512 context tokens (+1 to be written), 64-block permuted pool, Qwen2.5-7B layer shape.

    The case holds 513 tokens; the first 512 are the context, token 512 is the new one whose
    slot is `slot_mapping[512]` (first offset of the 33rd block).
    """
    return make_decode_case([513], QWEN25_7B, seed=seed, num_blocks=64)


def prefill_write_case(
    num_seqs: int = 8,
    tokens_per_seq: int = 2048,
    shape: LayerShape = QWEN25_7B,
    seed: int = 0,
    pad_fraction: float = 0.03,
    device="cpu",
):
    """Prefill-style cache write: key/value [num_seqs*tokens, Hkv, D] bf16, a permuted block pool
    that exactly covers the tokens, and about `pad_fraction` of the slots set to -1 (padding that the
    write must skip).  Returns (key, value, slot_mapping int64, k_scale, v_scale, num_blocks)."""
    total = num_seqs * tokens_per_seq
    num_blocks = -(-total // shape.block_size)
    g = _gen(seed * 48271 + 11, device)
    key, value = draw_kv(total, shape, g, channel_gain(shape, seed, device))
    cpu = _gen(seed * 16807 + 7)
    perm = torch.randperm(num_blocks, generator=cpu)
    tok = torch.arange(total)
    slots = perm[tok // shape.block_size] * shape.block_size + tok % shape.block_size
    drop = torch.rand(total, generator=cpu) < pad_fraction
    slots = torch.where(drop, torch.full_like(slots, -1), slots)
    k_scale, v_scale = calibrate_scales(shape, seed)
    return key, value, slots.to(device), k_scale.to(device), v_scale.to(device), num_blocks
