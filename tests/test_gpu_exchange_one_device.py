"""The sequence-parallel exchange on ONE device: the kernels that store partial rows as {value, step number} pairs,
and the merge that polls them, with every "rank's" buffer in this GPU's memory.  What needs two GPUs (NVLink stores,
symmetric memory, two processes) is in test_gpu_sequence_parallel.py; this file covers the same kernels where only one
GPU is visible: a world of one against the ordinary operator (bit-identical), two and nine ranks emulated one after
the other against the all-gather path's merge (bit-identical), CUDA-graph replay, and a rank that never pushes (the
bounded wait runs out, the status word says so, the context stays usable)."""

import pytest
import torch

import oracle
from conftest import cosine, max_abs, package

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _exchange(lib_mod, world, rank, buffers):
    ptrs = (lib_mod._VP * 16)(*[b.data_ptr() for b in buffers])
    return lib_mod.Exchange(world, rank, ptrs, buffers[0].numel())


def _buffers(lib_mod, world, B, Hq, D):
    n = lib_mod.load().int8kv_exchange_bytes(world, B, Hq, D)
    assert n > 0
    return [torch.zeros(n, dtype=torch.uint8, device=DEV) for _ in range(world)]


def _case(wl, lens, seed, shape=None):
    shape = shape or wl.QWEN25_7B
    case = wl.make_decode_case(lens, shape, seed=seed)
    kc = torch.zeros(case.num_blocks, shape.block_size, shape.num_kv_heads, shape.head_dim, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
    return case, kc, vc


@pytest.mark.parametrize("num_splits", [None, 1, 4, "planned"])
def test_world_of_one_equals_the_ordinary_call(kv, workloads, num_splits):
    """One rank: its rows go through the slab and come back through the polling merge.  With one part per row that
    merge multiplies by 1 and divides by 1, so the output has the bits of int8_paged_attention with the same split
    (automatic, 4, planned on the device: the split-KV merge stores its rows into the slab, rows of sequences with a
    single part are forwarded from the staging area; 1: the attention kernel stages and a copy kernel pushes)."""
    lib_mod = package("_lib")
    lens = [1500, 333, 64, 1, 0, 4096]
    case, kc, vc = _case(workloads, lens, seed=5)
    args = [t.to(DEV) for t in (case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)]
    want = kv.int8_paged_attention(*args, num_splits=num_splits, max_seq_len=max(lens))
    bufs = _buffers(lib_mod, 1, len(lens), 28, 128)
    ex = _exchange(lib_mod, 1, 0, bufs)
    for step in range(3):  # the slabs alternate
        kv.int8_paged_attention_partial_push(*args, ex, num_splits=num_splits, max_seq_len=max(lens))
        got = kv.merge_exchanged(ex, len(lens), 28, 128, device=DEV)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"step {step}"
    assert kv.device_status() == 0
    assert int(bufs[0][:8].view(torch.int32)[1]) == 3  # the step count lives in the buffer


@pytest.mark.parametrize("hq,hkv,d,num_splits", [(8, 2, 64, None), (8, 2, 64, 1), (6, 2, 66, 3), (16, 1, 256, None)])
def test_head_dims_outside_the_tiled_kernels_go_through_the_exchange(kv, workloads, hq, hkv, d, num_splits):
    """Head dims 64, 66 (not a multiple of 4: the row's last 16-byte piece holds the lse and padding) and 256 (two
    pieces per lane in the merge): world of one, the bits of the ordinary call."""
    lib_mod = package("_lib")
    shape = workloads.LayerShape(hq, hkv, d, 16)
    lens = [700, 33, 1, 0, 257]
    case, kc, vc = _case(workloads, lens, seed=3, shape=shape)
    args = [t.to(DEV) for t in (case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)]
    want = kv.int8_paged_attention(*args, num_splits=num_splits, max_seq_len=max(lens))
    ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    assert max_abs(want.float().cpu(), ref.to(torch.bfloat16).float()) <= 2e-2
    bufs = _buffers(lib_mod, 1, len(lens), hq, d)
    ex = _exchange(lib_mod, 1, 0, bufs)
    for step in range(2):
        kv.int8_paged_attention_partial_push(*args, ex, num_splits=num_splits, max_seq_len=max(lens))
        got = kv.merge_exchanged(ex, len(lens), hq, d, device=DEV)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"step {step}"
    assert kv.device_status() == 0


@pytest.mark.parametrize("num_splits", ["planned", 8, None])
def test_many_ragged_sequences_through_the_exchange(kv, workloads, num_splits):
    """64 ragged sequences x 4 kv heads, device-planned parts included, with sequences of a single part, an empty one
    and a one-token one among them.  World of one: the bits of the ordinary call with the same split."""
    lib_mod = package("_lib")
    g = torch.Generator().manual_seed(11)
    lens = [int(x) for x in torch.randint(1, 3000, (64,), generator=g)]
    lens[3], lens[17], lens[40] = 0, 1, 2999
    case, kc, vc = _case(workloads, lens, seed=21)
    args = [t.to(DEV) for t in (case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)]
    want = kv.int8_paged_attention(*args, num_splits=num_splits, max_seq_len=max(lens))
    ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    assert max_abs(want.float().cpu(), ref.to(torch.bfloat16).float()) <= 2e-2
    bufs = _buffers(lib_mod, 1, len(lens), 28, 128)
    ex = _exchange(lib_mod, 1, 0, bufs)
    for step in range(3):
        kv.int8_paged_attention_partial_push(*args, ex, num_splits=num_splits, max_seq_len=max(lens))
        got = kv.merge_exchanged(ex, len(lens), 28, 128, device=DEV)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"step {step}"
    assert kv.device_status() == 0


@pytest.mark.parametrize("world,num_splits", [(2, None), (9, None), (2, "planned"), (3, 1), (2, 6), (8, None), (8, 1),
                                              (16, None), (4, "planned"), (7, 4)])
def test_emulated_ranks_equal_the_gathered_merge_and_replay_as_a_graph(kv, workloads, world, num_splits):
    """Several "ranks" on one device, run one after the other on one stream: all of them push into all buffers (the
    last rank first), then each merges (its wait finds everything there).  All must return what merge_partials gives
    for the ranks' rows stacked, bit for bit, eagerly and replayed as a CUDA graph.  Nine ranks make the merge take
    the other ranks' rows in two batches; four, seven, eight and sixteen ranks (the 112 rows divide by them) use the
    scatter form:
    a row goes to its owner only, the owner's merged row to every rank's output slab, and a last kernel writes out."""
    lib_mod, sh = package("_lib"), package("sharding")
    lens = [2000, 333, 64, 1]
    case, kc, vc = _case(workloads, lens, seed=77)
    rank_args = []
    for rank in range(world):
        lo, hi, local_lens = sh.sequence_split(lens, rank, world, 16)
        hi = min(hi, case.block_tables.shape[1])
        tables = torch.zeros(len(lens), max(hi - lo, 1), dtype=torch.int32)
        lkc = torch.zeros(len(lens) * max(hi - lo, 1) + 1, 16, 4, 128, dtype=torch.int8)
        lvc = torch.zeros_like(lkc)
        nxt = 1
        for b, n in enumerate(local_lens):
            for j in range((n + 15) // 16):
                src = int(case.block_tables[b, lo + j])
                lkc[nxt], lvc[nxt] = kc[src], vc[src]
                tables[b, j] = nxt
                nxt += 1
        rank_args.append(([t.to(DEV) for t in (case.query, lkc, lvc, tables, torch.tensor(local_lens, dtype=torch.int32),
                                               case.k_scale, case.v_scale)], max(max(local_lens), 1)))
    rows = torch.stack([kv.int8_paged_attention_partial(*a, max_seq_len=m, num_splits=num_splits) for a, m in rank_args])
    want = kv.merge_partials(rows, 128)
    ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    assert max_abs(want.float().cpu(), ref.to(torch.bfloat16).float()) <= 2e-2 and cosine(want.float().cpu(), ref) >= 0.9999

    bufs = _buffers(lib_mod, world, len(lens), 28, 128)
    exs = [_exchange(lib_mod, world, r, bufs) for r in range(world)]
    outs = [torch.empty_like(want) for _ in range(world)]

    def step():
        for r in reversed(range(world)):
            kv.int8_paged_attention_partial_push(*rank_args[r][0], exs[r], max_seq_len=rank_args[r][1],
                                                 num_splits=num_splits)
        # one phase for all ranks, then the other: in the scatter form a rank's second phase needs every owner's first
        for phase in (lib_mod.EXCHANGE_MERGE_PHASE, lib_mod.EXCHANGE_GATHER_PHASE):
            for r in range(world):
                kv.merge_exchanged(exs[r], len(lens), 28, 128, out=outs[r], phase=phase)

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(2):
            step()
        stream.synchronize()
        assert all(torch.equal(o, want) for o in outs)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
        for _ in range(3):
            for o in outs:
                o.zero_()
            g.replay()
        stream.synchronize()
        assert all(torch.equal(o, want) for o in outs)
        assert kv.device_status() == 0
    del g


def test_a_rank_that_never_pushes_runs_the_wait_out(kv, workloads):
    """Two ranks, only rank 0 ever pushes: its merge waits about a second for rank 1's rows, gives up, sets
    INT8KV_DEV_WAIT_TIMEOUT and leaves the output unwritten.  The kernel returns normally: the next call works."""
    lib_mod = package("_lib")
    lens = [300, 17]
    case, kc, vc = _case(workloads, lens, seed=9)
    args = [t.to(DEV) for t in (case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)]
    bufs = _buffers(lib_mod, 2, len(lens), 28, 128)
    ex = _exchange(lib_mod, 2, 0, bufs)
    assert kv.device_status() == 0
    out = torch.full((len(lens), 28, 128), 7.0, dtype=torch.bfloat16, device=DEV)
    kv.int8_paged_attention_partial_push(*args, ex, max_seq_len=max(lens))
    kv.merge_exchanged(ex, len(lens), 28, 128, out=out)
    torch.cuda.synchronize()
    assert kv.device_status() == lib_mod.DEV_WAIT_TIMEOUT
    assert bool((out == 7.0).all())
    want = kv.int8_paged_attention(*args, max_seq_len=max(lens))
    ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    assert max_abs(want.float().cpu(), ref.to(torch.bfloat16).float()) <= 2e-2
    assert kv.device_status() == 0
