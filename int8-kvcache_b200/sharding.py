"""Multi-GPU partitioning of the decode path: one process per GPU.

Two partitions need no collective at all, because every (sequence, KV head) pair is independent:
tensor-parallel by KV head and data-parallel by batch.  Each rank calls the unchanged operators on
its slice (local Hq, Hkv, B); outputs stay head/batch-sharded, as they are under a tensor-parallel
model before the output projection.

The third partition splits the SEQUENCE across ranks for very long contexts: rank r holds a
contiguous range of every sequence's logical blocks in its own cache, computes unmerged partial
attention rows (normalised out | log-sum-exp), the rows of all ranks are brought into LOCAL memory,
and a local merge kernel combines them.  The merge reads local memory only.  Two exchanges exist:
an NCCL all-gather, and PeerExchange, where every rank stores its rows straight into the other
ranks' buffers over NVLink (plain stores to peer-mapped memory, every value paired with the step's
number) and the merge kernel itself waits, with a bound, until the values it reads carry that number.

The reference prototype is single-GPU (its README states TP=1); the split-KV partial/merge math that
this generalises is its src/triton_ops/int8_paged_attention.py:293-388.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch


# ---------------------------------------------------------------------------------------------------
# KV-head x batch partition (no collective)
# ---------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class HeadBatchShard:
    rank: int
    world: int
    kv_heads: Tuple[int, int]  # [start, stop) of KV heads
    batch: Tuple[int, int]  # [start, stop) of sequences
    group: int  # query heads per KV head

    @property
    def q_heads(self) -> Tuple[int, int]:
        return self.kv_heads[0] * self.group, self.kv_heads[1] * self.group


def head_batch_partition(world: int, num_q_heads: int, num_kv_heads: int, batch: int) -> List[HeadBatchShard]:
    """Shards for `world` ranks: KV heads are divided first (up to one head per rank), the batch next.

    world=2 on 4 KV heads -> heads {0,1},{2,3}; world=4 -> one head each; world=8 -> one head x half the
    batch.  Raises if the division is not exact.
    """
    assert world >= 1 and num_q_heads % num_kv_heads == 0
    tp = min(world, num_kv_heads)
    while tp > 1 and (num_kv_heads % tp or world % tp):
        tp -= 1
    dp = world // tp
    if tp * dp != world or batch % dp:
        raise ValueError(f"cannot shard Hkv={num_kv_heads}, B={batch} over {world} ranks")
    hp, bp = num_kv_heads // tp, batch // dp
    group = num_q_heads // num_kv_heads
    return [
        HeadBatchShard(r, world, ((r % tp) * hp, (r % tp + 1) * hp), ((r // tp) * bp, (r // tp + 1) * bp), group)
        for r in range(world)
    ]


def shard_decode_inputs(shard: HeadBatchShard, query, key_cache, value_cache, block_tables, seq_lens, k_scale, v_scale):
    """Views (no copies) of one rank's slice of a full decode call's tensors."""
    h0, h1 = shard.kv_heads
    q0, q1 = shard.q_heads
    b0, b1 = shard.batch
    return (
        query[b0:b1, q0:q1],
        key_cache[:, :, h0:h1],
        value_cache[:, :, h0:h1],
        block_tables[b0:b1],
        seq_lens[b0:b1],
        k_scale[h0:h1],
        v_scale[h0:h1],
    )


# ---------------------------------------------------------------------------------------------------
# sequence partition (one all-gather + local merge)
# ---------------------------------------------------------------------------------------------------
def sequence_split(seq_lens: Sequence[int], rank: int, world: int, block_size: int,
                   blocks_per_rank: Optional[int] = None) -> Tuple[int, int, List[int]]:
    """Logical block range [lo, hi) owned by `rank` and the number of tokens of each sequence inside it.

    Every rank owns the same block range of every sequence (rank r: blocks [r*per, (r+1)*per)); a sequence
    shorter than a rank's range start contributes 0 tokens there, which the partial kernel reports as
    lse = -inf and the merge ignores.
    """
    longest = max(seq_lens) if len(seq_lens) else 0
    total_blocks = -(-longest // block_size)
    per = blocks_per_rank if blocks_per_rank is not None else max(1, -(-total_blocks // world))
    lo, hi = rank * per, (rank + 1) * per
    local = [max(0, min(int(s) - lo * block_size, per * block_size)) for s in seq_lens]
    return lo, hi, local


def gather_partials(local_rows: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather [B, Hq, row] partial rows into a local [world, B, Hq, row] buffer."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    shape = tuple(local_rows.shape)
    flat = torch.empty((world * shape[0],) + shape[1:], dtype=local_rows.dtype, device=local_rows.device)
    dist.all_gather_into_tensor(flat, local_rows.contiguous(), group=group)  # rank r fills rows [r*B, (r+1)*B)
    return flat.view((world,) + shape)


class PeerExchange:
    """Peer-mapped exchange buffers for sequence_parallel_int8_attention(..., exchange=...): one buffer per rank in
    symmetric memory (torch.distributed._symmetric_memory: every rank allocates the same size and the allocator maps
    all of them into every process), laid out as include/int8kv_b200.h describes for int8kv_exchange.  Collective:
    every rank of `group` must construct it, with the same shape.  Only plain peer stores are used on these buffers,
    so the allocator's NVLink multicast binding is switched off for them."""

    def __init__(self, batch: int, num_q_heads: int, head_dim: int, device, group=None):
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shape = (int(batch), int(num_q_heads), int(head_dim))
        nbytes = _lib.load().int8kv_exchange_bytes(self.world, *self.shape)
        if nbytes <= 0:
            raise ValueError(f"no exchange layout for {self.world} ranks and shape {self.shape}")
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.handle = symm_mem.rendezvous(self.buffer, group)
        self.buffer.zero_()  # control words and slabs start at zero on every rank ...
        torch.cuda.synchronize(device)
        dist.barrier(group)  # ... before anyone's first push can arrive
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(ptrs) == self.world and ptrs[self.rank] == self.buffer.data_ptr()
        self.exchange = _lib.Exchange(self.world, self.rank, (_lib._VP * 16)(*ptrs), nbytes)
        self._group = group

    def close(self) -> None:
        """Collective: every rank stops using the buffers before any of them lets go of its own."""
        import torch.distributed as dist

        if self.buffer is not None:
            torch.cuda.synchronize(self.buffer.device)
            dist.barrier(self._group)
            self.exchange = self.handle = self.buffer = None


def sequence_parallel_int8_attention(query, local_key_cache, local_value_cache, local_block_tables, local_seq_lens,
                                     k_scale, v_scale, *, group=None, out_dtype=None, max_seq_len=None, exchange=None):
    """INT8 paged decode attention with the sequence split across the ranks of `group`.

    Every rank passes the full query [B, Hq, D], its own caches/block tables (local physical block ids) and
    the number of tokens of each sequence that it holds.  Returns the merged [B, Hq, D] on every rank.
    exchange: a PeerExchange built for this batch and head layout; the partial rows then travel by peer stores
    instead of an NCCL all-gather (same result).
    """
    from . import ops

    if exchange is not None:
        B, Hq, D = query.shape
        assert exchange.shape == (B, Hq, D)
        ops.int8_paged_attention_partial_push(query, local_key_cache, local_value_cache, local_block_tables,
                                              local_seq_lens, k_scale, v_scale, exchange.exchange,
                                              max_seq_len=max_seq_len)
        return ops.merge_exchanged(exchange.exchange, B, Hq, D, dtype=out_dtype or query.dtype, device=query.device)
    rows = ops.int8_paged_attention_partial(query, local_key_cache, local_value_cache, local_block_tables,
                                            local_seq_lens, k_scale, v_scale, max_seq_len=max_seq_len)
    gathered = gather_partials(rows, group)
    return ops.merge_partials(gathered, query.shape[-1], dtype=out_dtype or query.dtype)
