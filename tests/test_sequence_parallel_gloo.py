"""world_size-2 run of the sequence-parallel plumbing on CPU (gloo): partition, all-gather of partial rows,
merge.  The arithmetic of each rank is done by the CPU oracle here; on GPUs the same host code calls the
partial-attention and merge kernels."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from conftest import package


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        sh = package("sharding")
        wl = package("workloads")
        lens = [300, 47, 16]
        case = wl.make_decode_case(lens, wl.QWEN25_7B, seed=21)
        kc = torch.zeros(case.num_blocks, 16, 4, 128, dtype=torch.int8)
        vc = torch.zeros_like(kc)
        oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
        lo, hi, local_lens = sh.sequence_split(lens, rank, world, 16)
        # this rank's rows: out (128) | lse | pad, as the GPU partial kernel lays them out
        rows = torch.zeros(len(lens), 28, 132)
        ks, vs = oracle.gather_paged_cache(kc, vc, case.block_tables, lens)
        for b, n in enumerate(local_lens):
            k = oracle.dequant_per_head(ks[b][:, lo * 16 : lo * 16 + n], case.k_scale, head_axis=0)
            v = oracle.dequant_per_head(vs[b][:, lo * 16 : lo * 16 + n], case.v_scale, head_axis=0)
            o, lse = oracle.partial_attention_with_lse(case.query[b], k, v)
            rows[b, :, :128] = o
            rows[b, :, 128] = lse
        gathered = sh.gather_partials(rows)
        assert gathered.shape == (world, len(lens), 28, 132)
        merged = oracle.merge_partials(gathered[..., :128], gathered[..., 128])
        want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
        ret[rank] = float((merged - want).abs().max())
    finally:
        dist.destroy_process_group()


def test_two_rank_sequence_split_equals_single_rank():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, ret)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert len(ret) == world and max(ret.values()) < 2e-6
