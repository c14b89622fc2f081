"""Oracle: paged KV cache layout and the slot_mapping scatter write (test infrastructure).

Layout facts restated from the reference:
  * a cache is [num_blocks, block_size, Hkv, D]; logical block `lb` of sequence
    `b` lives in physical block `block_tables[b, lb]`; tokens past `seq_len` in
    the last block are padding                       (src/paged_cache.py:4-59)
  * the write maps token t to slot = block*block_size + offset, skips slot < 0
    and leaves every other cache byte untouched
                                    (src/triton_ops/int8_cache_write.py:152-183)
"""

from __future__ import annotations

import random
from typing import List, Sequence, Tuple

import torch

from .quant import static_quant_per_head


def build_paged_cache(k: torch.Tensor, v: torch.Tensor, block_size: int = 16):
    """k, v: [B, Hkv, T, D] -> (kc, vc, block_tables int32 [B, nblk], seq_lens int32 [B]).

    Blocks are handed out in order, sequence after sequence (src/paged_cache.py:24-27).
    """
    B, Hkv, T, D = k.shape
    per_seq = -(-T // block_size)
    kc = k.new_zeros((B * per_seq, block_size, Hkv, D))
    vc = v.new_zeros((B * per_seq, block_size, Hkv, D))
    tables = torch.arange(B * per_seq, dtype=torch.int32).reshape(B, per_seq)
    k_tm = k.permute(0, 2, 1, 3)  # [B, T, Hkv, D]
    v_tm = v.permute(0, 2, 1, 3)
    for b in range(B):
        flat_k = kc[b * per_seq : (b + 1) * per_seq].reshape(per_seq * block_size, Hkv, D)
        flat_v = vc[b * per_seq : (b + 1) * per_seq].reshape(per_seq * block_size, Hkv, D)
        flat_k[:T] = k_tm[b]
        flat_v[:T] = v_tm[b]
    seq_lens = torch.full((B,), T, dtype=torch.int32)
    return kc, vc, tables, seq_lens


def gather_paged_cache(
    kc: torch.Tensor, vc: torch.Tensor, block_tables: torch.Tensor, seq_lens
) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """Inverse of the paging: per sequence, [Hkv, T_b, D] tensors (ragged lengths allowed).

    Follows src/paged_cache.py:39-59, but returns lists so that sequences of
    different lengths can be gathered in one call.
    """
    block_size = kc.shape[1]
    ks, vs = [], []
    for b in range(block_tables.shape[0]):
        T = int(seq_lens[b])
        nblk = -(-T // block_size)
        ids = block_tables[b, :nblk].to(torch.long)
        k = kc[ids].reshape(nblk * block_size, *kc.shape[2:])[:T]
        v = vc[ids].reshape(nblk * block_size, *vc.shape[2:])[:T]
        ks.append(k.permute(1, 0, 2))
        vs.append(v.permute(1, 0, 2))
    return ks, vs


def cache_write(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    floor_scale: bool = True,
) -> None:
    """Quantise key/value [T, Hkv, D] and scatter them into the int8 caches in place.

    When a slot appears more than once the last token in order wins, as in the
    reference's sequential loop (src/triton_ops/int8_cache_write.py:164-183).
    """
    block_size = key_cache.shape[1]
    slots = slot_mapping.reshape(-1).to(torch.long)
    keep = torch.nonzero(slots >= 0).reshape(-1)
    if keep.numel() == 0:
        return
    kq = static_quant_per_head(key, k_scale, head_axis=1, floor_scale=floor_scale)
    vq = static_quant_per_head(value, v_scale, head_axis=1, floor_scale=floor_scale)
    # python loop only where duplicates exist; otherwise one vectorised scatter
    s = slots[keep]
    blk = torch.div(s, block_size, rounding_mode="floor")
    off = s - blk * block_size
    if torch.unique(s).numel() == s.numel():
        key_cache[blk, off] = kq[keep]
        value_cache[blk, off] = vq[keep]
    else:
        for i, t in enumerate(keep.tolist()):
            key_cache[blk[i], off[i]] = kq[t]
            value_cache[blk[i], off[i]] = vq[t]


def slots_for_sequences(block_tables: torch.Tensor, seq_lens: Sequence[int], block_size: int):
    """slot of every token of every sequence, concatenated in order (int64)."""
    out = []
    for b, T in enumerate(seq_lens):
        tok = torch.arange(int(T), dtype=torch.long)
        phys = block_tables[b, torch.div(tok, block_size, rounding_mode="floor")].to(torch.long)
        out.append(phys * block_size + tok % block_size)
    return torch.cat(out) if out else torch.zeros(0, dtype=torch.long)


def random_block_tables(seq_lens: Sequence[int], block_size: int, num_blocks: int, rng: random.Random):
    """Shuffle the pool, hand consecutive slices to the sequences, zero-pad the rest.

    Same procedure as the helper in the reference's tests
    (tests/test_int8_paged_attention.py:16-43).
    """
    need = [-(-int(T) // block_size) for T in seq_lens]
    pool = list(range(num_blocks))
    rng.shuffle(pool)
    tables = torch.zeros((len(seq_lens), max(need) if need else 0), dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        tables[b, :n] = torch.tensor(pool[at : at + n], dtype=torch.int32)
        at += n
    return tables
