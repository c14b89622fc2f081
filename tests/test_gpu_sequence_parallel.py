"""Sequence-parallel INT8 attention on two GPUs: every rank holds a contiguous block range of every sequence
in its own cache, computes partial rows, brings the rows of all ranks into local memory (an NCCL all-gather, or
peer stores of {value, step number} pairs) and merges locally.  The result must equal single-GPU attention over the whole
sequence.  Skipped when fewer than two GPUs are visible.
Also checks the collective-free KV-head x batch sharding on each rank against the oracle."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from conftest import cosine, max_abs, package

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        kv, sh, wl = package(), package("sharding"), package("workloads")
        lens = [2000, 333, 64, 1]
        case = wl.make_decode_case(lens, wl.QWEN25_7B, seed=77)
        kc = torch.zeros(case.num_blocks, 16, 4, 128, dtype=torch.int8)
        vc = torch.zeros_like(kc)
        oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
        want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)

        # --- sequence split: this rank's local cache holds only its block range, with local block ids
        lo, hi, local_lens = sh.sequence_split(lens, rank, world, 16)
        width = case.block_tables.shape[1]
        hi = min(hi, width)
        local_tables = torch.zeros(len(lens), max(hi - lo, 1), dtype=torch.int32)
        local_kc = torch.zeros(len(lens) * max(hi - lo, 1) + 1, 16, 4, 128, dtype=torch.int8)
        local_vc = torch.zeros_like(local_kc)
        nxt = 1
        for b, n in enumerate(local_lens):
            for j in range((n + 15) // 16):
                src = int(case.block_tables[b, lo + j])
                local_kc[nxt], local_vc[nxt] = kc[src], vc[src]
                local_tables[b, j] = nxt
                nxt += 1
        out = sh.sequence_parallel_int8_attention(
            case.query.to(dev), local_kc.to(dev), local_vc.to(dev), local_tables.to(dev),
            torch.tensor(local_lens, dtype=torch.int32, device=dev), case.k_scale.to(dev), case.v_scale.to(dev))
        torch.cuda.synchronize()
        got = out.float().cpu()
        seq_err, seq_cos = max_abs(got, want.to(torch.bfloat16).float()), cosine(got, want)
        # the same split with the rows exchanged by peer stores instead of the all-gather (the split-KV merge stores
        # its rows into the peers' buffers itself): several
        # steps in a row (the buffers alternate between two slabs), then the same steps replayed as a CUDA graph
        peer = sh.PeerExchange(len(lens), 28, 128, dev)
        args = (case.query.to(dev), local_kc.to(dev), local_vc.to(dev), local_tables.to(dev),
                torch.tensor(local_lens, dtype=torch.int32, device=dev), case.k_scale.to(dev), case.v_scale.to(dev))
        for _ in range(3):
            out_p = sh.sequence_parallel_int8_attention(*args, exchange=peer, max_seq_len=max(max(local_lens), 1))
        torch.cuda.synchronize()
        peer_equal = bool(torch.equal(out_p, out))
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            sh.sequence_parallel_int8_attention(*args, exchange=peer, max_seq_len=max(max(local_lens), 1))
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                out_g = sh.sequence_parallel_int8_attention(*args, exchange=peer, max_seq_len=max(max(local_lens), 1))
            for _ in range(3):
                out_g.zero_()
                g.replay()
            stream.synchronize()
        peer_equal = peer_equal and bool(torch.equal(out_g, out))
        del g
        # an unsplit call leaves its rows in the staging area and a copy kernel pushes them: same exchange, other sender
        kv.int8_paged_attention_partial_push(*args, peer.exchange, num_splits=1, max_seq_len=max(max(local_lens), 1))
        out_1 = kv.merge_exchanged(peer.exchange, len(lens), 28, 128, device=dev)
        torch.cuda.synchronize()
        got_1 = out_1.float().cpu()
        unsplit_ok = max_abs(got_1, want.to(torch.bfloat16).float()) <= 2e-2 and cosine(got_1, want) >= 0.9999
        peer_equal = peer_equal and unsplit_ok
        # a forced split count: same bits as gathering the same rows through NCCL
        for _ in range(2):
            kv.int8_paged_attention_partial_push(*args, peer.exchange, num_splits=6, max_seq_len=max(max(local_lens), 1))
            out_6 = kv.merge_exchanged(peer.exchange, len(lens), 28, 128, device=dev)
        rows_6 = kv.int8_paged_attention_partial(*args, num_splits=6, max_seq_len=max(max(local_lens), 1))
        want_6 = kv.merge_partials(sh.gather_partials(rows_6), 128)
        torch.cuda.synchronize()
        peer_equal = peer_equal and bool(torch.equal(out_6, want_6))
        peer.close()

        # --- head x batch shard of this rank, no collective
        shard = sh.head_batch_partition(world, 28, 4, len(lens))[rank]
        args = sh.shard_decode_inputs(shard, case.query.to(dev), kc.to(dev), vc.to(dev), case.block_tables.to(dev),
                                      case.seq_lens.to(dev), case.k_scale.to(dev), case.v_scale.to(dev))
        part = kv.int8_paged_attention(*args).float().cpu()
        q0, q1 = shard.q_heads
        b0, b1 = shard.batch
        ref = want[b0:b1, q0:q1]
        ret[rank] = (seq_err, seq_cos, max_abs(part, ref.to(torch.bfloat16).float()), cosine(part, ref),
                     int(kv.device_status(dev)), peer_equal)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sequence_split_and_head_shards_match_the_oracle():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(240)
            assert p.exitcode == 0
        assert len(ret) == world
        for seq_err, seq_cos, shard_err, shard_cos, status, peer_equal in ret.values():
            assert seq_err <= 2e-2 and seq_cos >= 0.9999
            assert shard_err <= 2e-2 and shard_cos >= 0.9999
            assert status == 0
            assert peer_equal  # the two exchanges deliver the same rows to the same merge: bit-identical outputs
