#!/usr/bin/env python
"""Benchmark of the INT8 paged decode-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c4|c2|c3|c5]

Default workload (`c4`): large-batch decode over 28 layers, each layer with its own INT8 cache and its own
static scales — B=256 sequences with seq_lens uniform in [1024, 8192], Hq=28, Hkv=4, D=128, block_size=16
(1.2 GB of K+V per layer call, 34 GB per step: every call reads its pages from HBM).  One step = one decode pass
over the 28 layers = 28 int8_paged_attention calls.  On N GPUs (one process per GPU, torchrun) the workload is
sharded by KV head first and by batch next — heads {0,1},{2,3} at N=2, one head each at N=4, one head x half the
batch at N=8 — with no collective on the data path; the total work is fixed, so the scaling is "strong".

Printed JSON (one line, rank 0):
  value         achieved GB/s of algorithmic bytes of the whole job, device-resident inputs, step replayed as a
                CUDA graph, max over ranks
  e2e           same metric through the Python operators with pinned-host inputs copied in and the results
                copied out inside the timed region
  roofline      the attention call against the measured HBM copy peak
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch CPU path) on a bounded sample of the workload
  bf16_baseline the same calls on un-quantised bf16 caches with identical block tables
  shard_check   the timed calls' outputs for a few sequences against the CPU oracle (outside the timed region)
  c2_cell, cells  (N=1) the single-GPU kernel sweep B in {1,2,4,8} x seq in {512..4096}, largest cell separately
  c3_write      (N=1) the prefill-style INT8 cache write of 16384 tokens
  c5            long context B=32 x 65536, Hq=64/Hkv=8: whole on one GPU; on N GPUs head-parallel (no collective)
                and sequence-parallel (partial rows exchanged over NVLink, then merged), the latter checked
                against single-device attention over the same tokens
`--impl reference` times the CPU path alone with all host threads.  `--shape Hq,Hkv,D,BLOCK[,BATCH,SEQ]` times one
layer of any other shape (head_dim 64, 96, 256 ..., larger groups, odd block sizes) instead.
"""

from __future__ import annotations

import argparse
import gc
import importlib
import json
import os
import statistics
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

# dram__bytes_read.sum + dram__bytes_write.sum of one paged_attn_int8_kernel launch per algorithmic byte of the
# launch, from one-pass ncu captures of this script's own workloads (profiles/bench_default__launch_list.md for c4
# and c2); the c5 figure comes from a capture of a smaller batch of the same shape
# (profiles/paged_attn_int8_kernel__c4_first64.md names the method) and is scaled by the bytes a full launch
# processes: traffic grows in proportion, every page is read once.
C3_NCU_DRAM_BYTES_IN_KERNEL = 32_677_000 + 18_700  # profiles/cache_write_vec_kernel__c3_prefill.md: read + written, one launch
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {"c2": 35601446 / 33677376, "c4": 1243505426 / 1206481112, "c5": 1.002}
HBM_NOMINAL_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0
METRIC = "int8_paged_decode_attn_achieved_hbm_gbps"


# ---------------------------------------------------------------------------------------------------
# workload description
# ---------------------------------------------------------------------------------------------------
def workload_spec(name: str):
    """(hq, hkv, seq_lens of the whole job, layers, description)"""
    gen = torch.Generator().manual_seed(1234)
    if name == "c2":
        return 28, 4, [4096] * 8, 28, "sweep cell B=8 seq=4096, 28 distinct layer caches"
    if name == "c3":  # cache-write workload; handled by leg_cache_write
        return 28, 4, [2048] * 8, 1, "prefill cache write, 8 x 2048 tokens"
    if name == "c4":
        lens = torch.randint(1024, 8193, (256,), generator=gen).tolist()
        return 28, 4, lens, 28, "B=256 seq~U[1024,8192], 28 layers, each with its own INT8 cache and static scales"
    if name == "c5":
        return 64, 8, [65536] * 32, 1, "B=32 ctx 65536 Hq=64 Hkv=8, one layer"
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(seq_lens, hq, hkv, d=128, bs=16, elem=1) -> int:
    """K+V bytes + block ids + query in / out + scales + seq_lens, per call."""
    tok = sum(seq_lens)
    blocks = sum((s + bs - 1) // bs for s in seq_lens)
    return tok * hkv * d * 2 * elem + blocks * 4 + len(seq_lens) * hq * d * 2 * 2 + 8 * hkv + 4 * len(seq_lens)


class Layer:
    pass


def build_layers(kv, wl, device, hq, hkv, seq_lens, layers, seed, with_bf16=False, common_seed=None):
    """Per layer: INT8 caches filled through the product write kernel from seeded bf16 K/V draws (and, with
    `with_bf16`, bf16 caches holding the same un-quantised rows at the same slots).  `seed` drives the K/V draws
    and the block placement; `common_seed` (default: seed) drives what ranks of one job must agree on: the static
    scales, the outlier channels and the queries.  All layers share one block table and one seq_lens tensor, as
    the layers of a model do in a serving engine (a sequence's block ids are the same in every layer's cache); the
    caches themselves are distinct allocations with distinct contents."""
    common_seed = seed if common_seed is None else common_seed
    shape = wl.LayerShape(hq, hkv, 128, 16)
    B = len(seq_lens)
    need = int(wl.blocks_needed(seq_lens, 16).sum())
    # small pools get the 2x slack of the reference's microbenchmark; large ones an eighth, to bound memory
    num_blocks = need * 2 if need * 16 * hkv * 128 < (256 << 20) else need + max(64, need // 8)
    lens_t = torch.tensor(seq_lens, dtype=torch.long, device=device)
    seq_of_tok = torch.repeat_interleave(torch.arange(B, device=device), lens_t)
    pos = torch.arange(int(lens_t.sum()), device=device) - (torch.cumsum(lens_t, 0) - lens_t)[seq_of_tok]
    chunk = 1 << 17  # tokens per draw: bounds the fp32/bf16 staging memory to about a gigabyte
    out = []
    gen = torch.Generator(device=device)
    qgen = torch.Generator(device=device)
    gain = wl.channel_gain(shape, common_seed, device)
    block_tables = wl.permuted_block_tables(seq_lens, 16, num_blocks, seed).to(device)
    seq_lens_dev = torch.tensor(seq_lens, dtype=torch.int32, device=device)
    slots = block_tables[seq_of_tok, pos // 16].long() * 16 + pos % 16
    for li in range(layers):
        L = Layer()
        L.k_scale, L.v_scale = [t.to(device) for t in wl.calibrate_scales(shape, common_seed, li)]
        L.block_tables, L.seq_lens = block_tables, seq_lens_dev
        L.kc = torch.zeros(num_blocks, 16, hkv, 128, dtype=torch.int8, device=device)
        L.vc = torch.zeros_like(L.kc)
        if with_bf16:
            L.kb = torch.zeros(num_blocks, 16, hkv, 128, dtype=torch.bfloat16, device=device)
            L.vb = torch.zeros_like(L.kb)
        gen.manual_seed(seed * 1000003 + li)
        for t0 in range(0, slots.numel(), chunk):
            s = slots[t0:t0 + chunk]
            k, v = wl.draw_kv(s.numel(), shape, gen, gain)
            kv.int8_kv_cache_write(k, v, L.kc, L.vc, s, L.k_scale, L.v_scale)
            if with_bf16:
                L.kb.view(-1, hkv, 128)[s] = k
                L.vb.view(-1, hkv, 128)[s] = v
        qgen.manual_seed(common_seed * 7919 + li)
        L.query = wl.draw_query(B, shape, qgen)
        L.out = torch.empty_like(L.query)
        out.append(L)
    torch.cuda.synchronize(device)
    return out


# ---------------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU every few milliseconds while a region runs
    (NVML reads only; nothing is set)."""

    REASONS = {
        "hw_slowdown": 0x8,
        "sw_thermal_slowdown": 0x20,
        "hw_thermal_slowdown": 0x40,
        "sw_power_cap": 0x4,
    }

    def __init__(self, gpu_index: int, period_s: float = 0.004):
        self.idx = gpu_index
        self.period = period_s
        self.samples, self.reason_bits = [], 0
        self.max_mhz = None
        self._stop = None
        self._thread = None
        self._err = None

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip()]
            if self.idx < len(ids) and ids[self.idx].isdigit():
                return int(ids[self.idx])
        return self.idx

    def start(self):
        import threading

        try:
            import pynvml

            pynvml.nvmlInit()
            try:  # the CUDA device's own UUID is unambiguous under any CUDA_VISIBLE_DEVICES remapping
                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.idx).uuid)
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report that instead of clocks
            self._err = f"nvml unavailable: {type(e).__name__}"
            return
        self._stop = threading.Event()

        def loop():
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop.is_set():
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    self.reason_bits |= int(get_reasons(h))
                except Exception:
                    pass
                self._stop.wait(self.period)

        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self._err or "not sampled"]}
        self._stop.set()
        self._thread.join(2)
        reasons = sorted(n for n, bit in self.REASONS.items() if self.reason_bits & bit)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.samples), "reasons": reasons}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle (port of the reference's PyTorch CPU path)
# ---------------------------------------------------------------------------------------------------
def cpu_layer_inputs(wl, hq, hkv, seq_lens, seed=0):
    import oracle

    case = wl.make_decode_case(seq_lens, wl.LayerShape(hq, hkv, 128, 16), seed=seed)
    kc = torch.zeros(case.num_blocks, 16, hkv, 128, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
    return case, kc, vc


def cpu_one_call(case, kc, vc):
    import oracle

    B = case.query.shape[0]
    # decode step of one layer: write one new token per sequence over its last slot, then attend
    last = torch.tensor([int(case.seq_lens[:b + 1].sum()) - 1 for b in range(B)])
    oracle.cache_write(case.key[last], case.value[last], kc, vc, case.slot_mapping[last], case.k_scale, case.v_scale)
    return oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, case.seq_lens.tolist(),
                                              case.k_scale, case.v_scale)


def time_cpu(wl, hq, hkv, seq_lens, budget_s, min_reps=3, warm=1):
    # bound the sample: at most ~64k tokens of context per call
    sample = list(seq_lens)
    while sum(sample) > 65536 and len(sample) > 1:
        sample = sample[: len(sample) // 2]
    if sum(sample) > 65536:
        sample = [65536]
    torch.set_num_threads(os.cpu_count() or 1)
    case, kc, vc = cpu_layer_inputs(wl, hq, hkv, sample)
    for _ in range(warm):
        cpu_one_call(case, kc, vc)
    times = []
    t_end = time.perf_counter() + budget_s
    while len(times) < min_reps or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        cpu_one_call(case, kc, vc)
        times.append(time.perf_counter() - t0)
        if len(times) >= 200:
            break
    med = statistics.median(times)
    nbytes = algorithmic_bytes(sample, hq, hkv)
    desc = (f"one layer call (write {len(sample)} tokens + attention) on the first {len(sample)} sequences of the "
            f"workload, {sum(sample)} context tokens, {len(times)} reps, median")
    return nbytes / med / 1e9, med, torch.get_num_threads(), desc, sample


# ---------------------------------------------------------------------------------------------------
# run context: device, ranks, timing
# ---------------------------------------------------------------------------------------------------
class Ctx:
    def __init__(self, args, rank, local_rank, world):
        self.args, self.rank, self.local_rank, self.world = args, rank, local_rank, world
        self.kv = importlib.import_module("int8-kvcache_b200")
        self.wl = importlib.import_module("int8-kvcache_b200.workloads")
        self.sh = importlib.import_module("int8-kvcache_b200.sharding")
        torch.cuda.set_device(local_rank)
        self.device = torch.device("cuda", local_rank)
        self.dist = None
        if world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        self.stream = torch.cuda.Stream(self.device)
        peaks_path = REPO / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            self.peak = float(json.loads(peaks_path.read_text())["hbm_gbs"])
            self.peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            self.peak, self.peak_src = FALLBACK_PEAK_GBS, "fallback 6.65 TB/s"
        self.sm = torch.cuda.get_device_properties(self.device).multi_processor_count

    def barrier(self):
        torch.cuda.synchronize(self.device)
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize(self.device)

    def reduce(self, values, op="max"):
        """max / sum / min of a list of floats over the ranks."""
        if self.dist is None:
            return [float(v) for v in values]
        t = torch.tensor([float(v) for v in values], device=self.device, dtype=torch.float64)
        ops = {"max": self.dist.ReduceOp.MAX, "sum": self.dist.ReduceOp.SUM, "min": self.dist.ReduceOp.MIN}
        self.dist.all_reduce(t, op=ops[op])
        return [float(x) for x in t.tolist()]

    def time_device(self, fn, steps=None, graph=True, sampler=None):
        """Milliseconds per call of `fn` on this rank: warm-up, then `steps` calls between two CUDA events on the
        launching stream, bracketed by barrier + synchronise; captured once as a CUDA graph and replayed unless
        graph=False.  Callers take the max over ranks."""
        steps = steps or self.args.steps
        with torch.cuda.stream(self.stream):
            for _ in range(2):
                fn()
            self.stream.synchronize()
            run, g = fn, None
            if graph and not self.args.no_graph:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.stream):
                    fn()
                run = g.replay
            for _ in range(self.args.warmup):
                run()
            self.barrier()
            if sampler is not None:
                sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(steps):
                run()
            e1.record(self.stream)
            self.barrier()
            ms = e0.elapsed_time(e1) / steps
        # a live CUDA graph that holds captured NCCL work blocks the communicator's teardown: release it here
        run = g = None
        return ms

    def time_host(self, step, steps=None):
        """Wall-clock seconds per call of `step` (which synchronises its stream itself), barrier on both sides."""
        steps = steps or self.args.steps
        with torch.cuda.stream(self.stream):
            for _ in range(self.args.warmup):
                step()
            self.barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                step()
            self.barrier()
            return (time.perf_counter() - t0) / steps


def _without_nan(x):
    """Legs that were skipped hold NaN; JSON has no NaN, so they become null."""
    if isinstance(x, dict):
        return {k: _without_nan(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_without_nan(v) for v in x]
    if isinstance(x, float) and (x != x or x in (float("inf"), float("-inf"))):
        return None
    return x


def _release(*objs):
    del objs
    gc.collect()
    torch.cuda.empty_cache()


# ---------------------------------------------------------------------------------------------------
# checks against the CPU oracle (outside every timed region)
# ---------------------------------------------------------------------------------------------------
def oracle_check(L, out, hkv, picks):
    """The kernel's output rows of sequences `picks` of one layer against the CPU oracle on the same INT8 pages
    (gathered through the block table into a compact cache).  Returns (max-abs vs the bf16-rounded oracle,
    cosine vs the fp32 oracle)."""
    import oracle

    lens = [int(L.seq_lens[b]) for b in picks]
    ids, tables = [], torch.zeros(len(picks), max((n + 15) // 16 for n in lens), dtype=torch.int32)
    nxt = 0
    for i, (b, n) in enumerate(zip(picks, lens)):
        nb = (n + 15) // 16
        ids.append(L.block_tables[b, :nb].long())
        tables[i, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
        nxt += nb
    ids = torch.cat(ids)
    kc, vc = L.kc[ids].cpu(), L.vc[ids].cpu()
    want = oracle.int8_paged_attention_oracle(L.query[picks].cpu(), kc, vc, tables, lens, L.k_scale.cpu(), L.v_scale.cpu())
    got = out[picks].float().cpu()
    err = float((got - want.to(torch.bfloat16).float()).abs().max())
    cos = float(torch.nn.functional.cosine_similarity(got.reshape(-1).double(), want.reshape(-1).double(), dim=0))
    return err, cos


def sequence_parallel_check(ctx, L, local_lens, merged, picks):
    """Merged sequence-parallel output of sequences `picks` against single-device attention (the CPU oracle) over
    the same tokens: every rank contributes the INT8 rows it holds of those sequences (NCCL all-gather, outside the
    timed region), rank 0 strings them together in rank order and attends.  Returns a dict on rank 0."""
    import oracle

    dist, hkv = ctx.dist, L.kc.shape[2]
    ks, vs = [], []
    for b in picks:
        n = local_lens[b]
        ids = L.block_tables[b, :(n + 15) // 16].long()
        ks.append(L.kc[ids].reshape(-1, hkv, 128)[:n])
        vs.append(L.vc[ids].reshape(-1, hkv, 128)[:n])
    mine = torch.stack([torch.stack(ks), torch.stack(vs)]).contiguous()  # [2, picks, n_local, Hkv, D] (equal n_local)
    everyone = torch.empty((ctx.world,) + tuple(mine.shape), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(everyone.view(-1, *mine.shape[1:]), mine)
    if ctx.rank != 0:
        return None
    everyone = everyone.cpu()
    err, cos = 0.0, 1.0
    for i, b in enumerate(picks):
        k = torch.cat([everyone[r, 0, i] for r in range(ctx.world)]).permute(1, 0, 2)  # [Hkv, T, D]
        v = torch.cat([everyone[r, 1, i] for r in range(ctx.world)]).permute(1, 0, 2)
        want = oracle.decode_attention(L.query[b].cpu(), oracle.dequant_per_head(k, L.k_scale.cpu(), head_axis=0),
                                       oracle.dequant_per_head(v, L.v_scale.cpu(), head_axis=0))
        got = merged[b].float().cpu()
        err = max(err, float((got - want.to(torch.bfloat16).float()).abs().max()))
        cos = min(cos, float(torch.nn.functional.cosine_similarity(got.reshape(-1).double(), want.reshape(-1).double(), dim=0)))
    return {"sequences": list(picks), "tokens_each": int(k.shape[1]), "max_abs": err, "cosine": cos,
            "ok": bool(err <= 2e-2 and cos >= 0.9999),
            "against": "CPU oracle attention over the concatenated tokens of all ranks"}


# ---------------------------------------------------------------------------------------------------
# legs
# ---------------------------------------------------------------------------------------------------
def leg_cache_write(ctx):
    """Prefill-style INT8 cache write: 8 sequences x 2048 new tokens ([16384, 4, 128] bf16), a permuted pool of 1024
    blocks, ~3% padding slots, rotated over 8 distinct input/cache sets (400 MB, larger than L2); one step = 8
    writes replayed as a CUDA graph."""
    kv, wl, device, args = ctx.kv, ctx.wl, ctx.device, ctx.args
    sets = []
    for i in range(8):
        key, value, slots, ks, vs, nb = wl.prefill_write_case(8, 2048, seed=i, device=device)
        kc = torch.zeros(nb, 16, 4, 128, dtype=torch.int8, device=device)
        sets.append((key, value, slots, ks, vs, kc, torch.zeros_like(kc)))
    valid = sum(int((s[2] >= 0).sum()) for s in sets) / len(sets)
    nbytes = 16384 * 4 * 128 * 4 + valid * 4 * 128 * 2 + 8 * 16384 + 32
    dynamic = args.scales == "dynamic"
    if dynamic:  # the per-(token, head) scheme: no input scales, one fp32 scale written per row of K and of V
        nbytes += valid * 4 * 2 * 4 - 32
        scale_caches = [(torch.zeros(s[5].shape[:3], device=device), torch.zeros(s[5].shape[:3], device=device)) for s in sets]

    def step():
        for i, (key, value, slots, ks, vs, kc, vc) in enumerate(sets):
            if dynamic:
                kv.reshape_and_cache_int8(key, value, kc, vc, scale_caches[i][0], scale_caches[i][1], slots)
            else:
                kv.int8_kv_cache_write(key, value, kc, vc, slots, ks, vs)

    us = ctx.time_device(step) * 1e3 / len(sets)
    gbs = nbytes / us / 1e3
    # yardstick: what a plain device copy reaches at this launch size (same total bytes read + written per launch, same
    # 8-set rotation, same graph replay) - the roofline's peak is a long copy, whose ramp and tail weigh nothing
    half = int(nbytes // 2) // 16 * 16
    srcs = [torch.rand(half // 4, dtype=torch.float32, device=device) for _ in sets]
    dsts = [torch.empty_like(x) for x in srcs]

    def copies():
        for a, b in zip(srcs, dsts):
            torch.neg(a, out=b)

    copy_us = ctx.time_device(copies) * 1e3 / len(sets)
    del srcs, dsts
    return {
        "same_bytes_copy": {"us_per_call": copy_us, "frac": 2 * half / copy_us / 1e3 / ctx.peak,
                            "what": "torch.neg on fp32, bytes/2 read and bytes/2 written per launch, timed the same way (an "
                                    "elementwise kernel of PyTorch, not of this library)"},
        "metric": "int8_dynamic_scale_kv_cache_write_achieved_hbm_gbps" if dynamic else "int8_kv_cache_write_achieved_hbm_gbps",
        "value": gbs, "unit": "GB/s", "us_per_call": us, "frac": gbs / ctx.peak, "frac_of_8TBps": gbs / HBM_NOMINAL_GBS,
        "gpu_launches": len(sets) * args.steps, "ms_per_step": us * len(sets) / 1e3,
        "workload": "c3: prefill cache write, 16384 tokens x 4 heads x 128, permuted 1024-block pool, ~3% slots = -1, "
                    "8 rotated sets (larger than L2)",
        "kernel": "cache_write_dynamic_vec_kernel<bf16>" if dynamic else "cache_write_vec_kernel<bf16>",
        "algorithmic_bytes_per_call": nbytes,
        # ncu, one launch: rows in from DRAM; the INT8 output is still in L2 at kernel end (written back later)
        "traffic": None if dynamic else C3_NCU_DRAM_BYTES_IN_KERNEL,
    }


def layered_steps(ctx, layers_data, max_seq, num_splits=None, bf16=False, mode=None):
    """The step function of a device-timed leg: all layers of `layers_data` (INT8 caches, or their bf16 twins).
    --launch chained (default): one DecodeStepLayers call with the inputs-ready promise, i.e. one launch per layer,
    each carrying the previous layer's split-KV merge; per-call: one operator call per layer, each with the promise;
    ordered: one operator call per layer, fully ordered behind the previous one."""
    kv, mode = ctx.kv, mode or ctx.args.launch
    L0 = layers_data[0]
    outs = torch.empty((len(layers_data),) + tuple(L0.query.shape), dtype=L0.query.dtype, device=L0.query.device)
    for i, L in enumerate(layers_data):
        L.out = outs[i]
    if mode == "chained":
        with torch.cuda.stream(ctx.stream):
            if bf16:
                plan = kv.DecodeStepLayers([L.query for L in layers_data], None, None, [L.kb for L in layers_data],
                                           [L.vb for L in layers_data], None, L0.block_tables, L0.seq_lens, None, None,
                                           max_seq_len=max_seq, num_splits=num_splits, out=outs, inputs_ready=True)
            else:
                plan = kv.DecodeStepLayers([L.query for L in layers_data], None, None, [L.kc for L in layers_data],
                                           [L.vc for L in layers_data], None, L0.block_tables, L0.seq_lens,
                                           [L.k_scale for L in layers_data], [L.v_scale for L in layers_data],
                                           max_seq_len=max_seq, num_splits=num_splits, out=outs, inputs_ready=True)
        return plan
    ready = mode == "per-call"

    def step():  # writes this call's own `outs`, whatever L.out names by the time it runs
        for L, out in zip(layers_data, outs):
            if bf16:
                kv.bf16_paged_attention(L.query, L.kb, L.vb, L.block_tables, L.seq_lens, num_splits=num_splits,
                                        max_seq_len=max_seq, out=out, inputs_ready=ready)
            else:
                kv.int8_paged_attention(L.query, L.kc, L.vc, L.block_tables, L.seq_lens, L.k_scale, L.v_scale,
                                        num_splits=num_splits, max_seq_len=max_seq, out=out, inputs_ready=ready)

    return step


LAUNCH_MODES = {
    "chained": "all layers of a step behind one int8kv_decode_step_layers call with the inputs-ready promise: one launch "
               "per layer, each carrying the previous layer's split-KV merge (INT8 and BF16 alike)",
    "per-call": "one operator call per layer, each with the inputs-ready promise (INT8KV_FLAG_INPUTS_READY)",
    "ordered": "one operator call per layer, every call fully ordered behind the previous one",
}


def leg_shape(ctx, spec: str):
    """int8_paged_attention on one layer of an arbitrary shape, "--shape Hq,Hkv,D,block[,batch,seq]": the layers outside
    the headline workloads (all of them head_dim 128), which the library serves with its non-tiled kernels.  The
    cache holds random INT8 bytes (the kernels' time does not depend on the values), the block table is the
    identity, and two distinct caches are visited in turn so that every call reads its pages from DRAM; launched
    eagerly.  GB/s counts the K and V bytes of the tokens attended, once."""
    kv, dev, args = ctx.kv, ctx.device, ctx.args
    vals = [int(x) for x in spec.split(",")]
    hq, hkv, d, bs = vals[:4]
    batch = vals[4] if len(vals) > 4 else 64
    seq = vals[5] if len(vals) > 5 else 2048
    per_seq = (seq + bs - 1) // bs
    nblk = per_seq * batch
    gen = torch.Generator(device=dev).manual_seed(1)
    caches = [tuple(torch.randint(-127, 128, (nblk, bs, hkv, d), device=dev, dtype=torch.int8, generator=gen)
                    for _ in range(2)) for _ in range(2)]
    bt = torch.arange(nblk, device=dev, dtype=torch.int32).view(batch, per_seq)
    sl = torch.full((batch,), seq, device=dev, dtype=torch.int32)
    q = torch.randn(batch, hq, d, device=dev, generator=gen).to(torch.bfloat16)
    ks = torch.full((hkv,), 0.02, device=dev)
    out = torch.empty_like(q)

    def calls():
        for kc, vc in caches:
            kv.int8_paged_attention(q, kc, vc, bt, sl, ks, ks, max_seq_len=seq, out=out, num_splits=args.num_splits)

    us = ctx.time_device(calls, graph=False) * 1e3 / len(caches)
    nbytes = batch * seq * hkv * d * 2
    return {"shape": {"q_heads": hq, "kv_heads": hkv, "head_dim": d, "block_size": bs, "batch": batch, "seq": seq},
            "caches": len(caches), "num_splits": args.num_splits, "us_per_call": round(us, 2), "bytes_per_call": nbytes,
            "gb_per_s": round(nbytes / us / 1e3, 1), "device_status": kv.device_status(dev)}


def leg_sweep(ctx, variants=True):
    """The single-GPU sweep B in {1,2,4,8} x seq in {512,1024,2048,4096} at Hq=28/Hkv=4 (the grid of the reference's
    bench/bench_paged_attention.py): microseconds per call for INT8 (automatic split), the same-run BF16 baseline
    and, as in the reference's table, INT8 with quantize_q and INT8 with a forced split of 8; each cell rotates
    over enough distinct layer caches to exceed the L2."""
    kv, wl, device = ctx.kv, ctx.wl, ctx.device
    hq, hkv = wl.QWEN25_7B.num_q_heads, wl.QWEN25_7B.num_kv_heads
    ready = ctx.args.launch != "ordered"  # every input of a step is resident before the step starts
    cells = []
    for B in (1, 2, 4, 8):
        for seq in (512, 1024, 2048, 4096):
            cell_bytes = B * seq * hkv * 128 * 2 * 3  # INT8 and BF16 caches of one layer
            layers = 28 if (B, seq) == (8, 4096) else max(4, min(64, int(600e6 / cell_bytes)))
            L = build_layers(kv, wl, device, hq, hkv, [seq] * B, layers, seed=5, with_bf16=True)

            def int8_variant(**kw):  # the reference's other table columns, one operator call per layer
                for x in L:
                    kv.int8_paged_attention(x.query, x.kc, x.vc, x.block_tables, x.seq_lens, x.k_scale, x.v_scale,
                                            max_seq_len=seq, out=x.out, inputs_ready=ready, **kw)

            i8 = ctx.time_device(layered_steps(ctx, L, seq)) / layers * 1e3
            bf = ctx.time_device(layered_steps(ctx, L, seq, bf16=True)) / layers * 1e3
            nb = algorithmic_bytes([seq] * B, hq, hkv)
            cell = {"batch": B, "seq_len": seq, "layer_caches": layers, "int8_us": i8, "bf16_us": bf,
                    "int8_speedup": bf / i8, "int8_gbs": nb / i8 / 1e3}
            if variants:
                cell["int8_quantize_q_us"] = ctx.time_device(lambda: int8_variant(quantize_q=True)) / layers * 1e3
                cell["int8_split8_us"] = ctx.time_device(lambda: int8_variant(num_splits=8)) / layers * 1e3
            cells.append(cell)
            del L
            _release()
    return cells


def leg_decode(ctx, name, hq, hkv, seq_lens, layers, config, sub=False):
    """One decode workload on this job's ranks (KV-head x batch sharded when there is more than one): device-timed
    INT8 attention, the BF16 baseline, the host-to-host leg and the oracle check.  Returns the JSON line's body
    (on every rank; only rank 0's is printed)."""
    kv, wl, args, device, world, rank = ctx.kv, ctx.wl, ctx.args, ctx.device, ctx.world, ctx.rank
    parts = world if world > 1 else (args.one_shard_of or 1)
    if parts > 1:
        shard = ctx.sh.head_batch_partition(parts, hq, hkv, len(seq_lens))[rank]
        group = hq // hkv
        hkv = shard.kv_heads[1] - shard.kv_heads[0]
        hq = hkv * group
        seq_lens = seq_lens[shard.batch[0]:shard.batch[1]]
        config["parallelism"] = (f"KV-head x batch sharded over {parts} ranks, no collective: {hkv} KV head(s) x "
                                 f"{len(seq_lens)} sequences per rank" + ("" if world > 1 else " (one rank's shard alone, on one GPU)"))
        config["batch_per_gpu"], config["kv_heads_per_gpu"] = len(seq_lens), hkv
    dynamic = args.scales == "dynamic"
    want_bf16 = args.bf16_baseline and not dynamic
    layers_data = build_layers(kv, wl, device, hq, hkv, seq_lens, layers, seed=100 + rank, with_bf16=want_bf16)
    max_seq, B = max(seq_lens), len(seq_lens)
    nbytes_call = algorithmic_bytes(seq_lens, hq, hkv)
    metric = METRIC
    if dynamic:
        # one fp32 K scale and one fp32 V scale per (token, head) are read on top of the INT8 bytes
        nbytes_call += sum(seq_lens) * hkv * 8
        metric = "int8_dynamic_scale_paged_decode_attn_achieved_hbm_gbps"
        config["scales"] = "per (token, head) fp32 scale caches [num_blocks, 16, Hkv], seeded uniform [0.005, 0.025]"
        gen_s = torch.Generator(device=device)
        for li, L in enumerate(layers_data):
            gen_s.manual_seed(7000 + li)
            L.ksc = torch.rand(L.kc.shape[:3], device=device, generator=gen_s) * 0.02 + 0.005
            L.vsc = torch.rand(L.kc.shape[:3], device=device, generator=gen_s) * 0.02 + 0.005
    nbytes_step = nbytes_call * layers
    # Every input of a step (queries, caches, tables, lengths, scales) is resident before the step starts and no
    # layer reads what another writes, which is what the inputs-ready promise asks for; see LAUNCH_MODES.
    ready = args.launch != "ordered"
    config["launch"] = f"{args.launch}: {LAUNCH_MODES[args.launch]}"
    if dynamic:
        def device_step():
            for L in layers_data:
                kv.int8_paged_attention_dynamic(L.query, L.kc, L.vc, L.ksc, L.vsc, L.block_tables, L.seq_lens,
                                                num_splits=args.num_splits, max_seq_len=max_seq, out=L.out,
                                                inputs_ready=ready)
    else:
        device_step = layered_steps(ctx, layers_data, max_seq, args.num_splits)
    main_out0 = layers_data[0].out  # layer 0's output buffer of the timed mode (other legs bring their own)

    lib = kv._lib.load()
    splits = args.num_splits or lib.int8kv_choose_splits(B, hkv, max_seq, 16, ctx.sm)
    launches_per_call = 1 + (1 if splits > 1 else 0)
    chained = args.launch == "chained" and not dynamic and layers > 1
    split_plan = None
    with torch.cuda.stream(ctx.stream):
        device_step()
        ctx.stream.synchronize()
        if args.num_splits is None:
            plan = kv.last_split_plan(device)
            if plan is not None:
                split_plan = {"items": plan[0], "part_tiles": plan[1], "waves": plan[2]}
                splits, launches_per_call = "planned on the device", 2

    sampler = ClockSampler(ctx.local_rank) if rank == 0 and not sub else None
    dev_ms = ctx.time_device(device_step, sampler=sampler)
    clocks = sampler.stop() if sampler is not None else None

    # ---- the same step in the other launch modes, for the record (see LAUNCH_MODES) ---------------------------
    other_modes = {}
    if not dynamic and not sub and not args.no_graph:
        for m in LAUNCH_MODES:
            if m != args.launch:
                other_modes[m] = ctx.time_device(layered_steps(ctx, layers_data, max_seq, args.num_splits, mode=m))
        with torch.cuda.stream(ctx.stream):
            main_out0.fill_(float("nan"))
            device_step()  # the timed mode once more: its result is what the check below reads
            ctx.stream.synchronize()

    # ---- oracle check of the timed calls' result (layer 0, a few sequences of this rank's shard) -------------
    check = None
    if not dynamic:
        picks = sorted(set([0, B // 2, B - 1]))[: (3 if max_seq <= 16384 else 1)]
        err, cos = oracle_check(layers_data[0], main_out0, hkv, picks)
        err, = ctx.reduce([err], "max")
        cos, = ctx.reduce([cos], "min")
        check = {"layer": 0, "sequences_per_rank": picks, "max_abs": err, "cosine": cos,
                 "ok": bool(err <= 2e-2 and cos >= 0.9999), "against": "CPU oracle on the same INT8 pages, every rank's shard"}

    # ---- the same calls on ONE layer's cache, labelled L2-warm (only where a layer's pages fit the L2) -------
    warm_ms = float("nan")
    if not dynamic and not args.no_graph and not sub and nbytes_call < 100e6:
        L0 = layers_data[0]

        def warm_step():
            for _ in range(layers):
                kv.int8_paged_attention(L0.query, L0.kc, L0.vc, L0.block_tables, L0.seq_lens, L0.k_scale, L0.v_scale,
                                        num_splits=args.num_splits, max_seq_len=max_seq, out=L0.out, inputs_ready=ready)

        warm_ms = ctx.time_device(warm_step)

    # ---- same-run BF16 baseline on identical block tables and the same K/V rows (one step = the same calls) ----
    bf16_ms = float("nan")
    if want_bf16:
        bf16_step = layered_steps(ctx, layers_data, max_seq, args.num_splits, bf16=True)
        bf16_ms = ctx.time_device(bf16_step)
        for L in layers_data:
            del L.kb, L.vb
        _release()

    # ---- e2e: the decode step a serving engine runs, from host buffers to host buffers ---------------
    # Inputs of one step (every layer's new query / key / value rows, the block tables, sequence lengths and
    # write slots) sit in ONE pinned host buffer; a step copies it to the device, runs cache write +
    # attention for every layer through the Python operators, and copies every layer's output back to a
    # pinned host buffer.  Measured three ways: launched eagerly from Python, through one
    # int8kv_decode_step_layers call per step, and with the calls captured once into a CUDA graph and replayed.
    e2e_s = e2e_eager_s = e2e_layers_s = e2e_per_layer_s = float("nan")
    e2e_agree = None
    e2e_from = "CUDA graph replay"
    h2d = d2h = 0
    if not args.no_e2e and not dynamic and not sub:
        shape = wl.LayerShape(hq, hkv, 128, 16)
        g = torch.Generator().manual_seed(7)
        n_q, n_kv = B * hq * 128, B * hkv * 128
        width = layers_data[0].block_tables.shape[1]
        per_layer = (n_q + 2 * n_kv) * 2
        meta_bytes = (B * width * 4 + B * 4 + B * 8 + 8 + 15) // 16 * 16
        h_in = torch.empty(layers * per_layer + meta_bytes, dtype=torch.uint8).pin_memory()
        d_in = torch.empty_like(h_in, device=device)
        h_out = torch.empty(layers, B, hq, 128, dtype=torch.bfloat16).pin_memory()
        d_out = torch.empty(layers, B, hq, 128, dtype=torch.bfloat16, device=device)

        def views(buf):
            per = []
            for i in range(layers):
                base = buf[i * per_layer:(i + 1) * per_layer].view(torch.bfloat16)
                per.append((base[:n_q].view(B, hq, 128), base[n_q:n_q + n_kv].view(B, hkv, 128),
                            base[n_q + n_kv:].view(B, hkv, 128)))
            m = buf[layers * per_layer:]
            bt = m[:B * width * 4].view(torch.int32).view(B, width)
            sl = m[B * width * 4:B * width * 4 + B * 4].view(torch.int32)
            so = (B * width * 4 + B * 4 + 7) // 8 * 8
            slots = m[so:so + B * 8].view(torch.int64)
            return per, bt, sl, slots

        hv, h_bt, h_sl, h_slots = views(h_in)
        gain0 = wl.channel_gain(shape, 0)
        for i in range(layers):
            hv[i][0].copy_(wl.draw_query(B, shape, g))
            k, v = wl.draw_kv(B, shape, g, gain0)
            hv[i][1].copy_(k)
            hv[i][2].copy_(v)
        # all layers share the step's metadata, as in a serving engine (layer 0's tables are used for every layer)
        L0 = layers_data[0]
        h_bt.copy_(L0.block_tables.cpu())
        h_sl.copy_(L0.seq_lens.cpu())
        last = torch.tensor([s - 1 for s in seq_lens])
        h_slots.copy_(L0.block_tables.cpu()[torch.arange(B), last // 16].long() * 16 + last % 16)
        dv, d_bt, d_sl, d_slots = views(d_in)
        h2d, d2h = h_in.numel(), h_out.numel() * 2
        stream = ctx.stream

        # Copies and compute overlap layer by layer, as a serving engine's copy engines would run them: the inputs
        # of layer l+1 travel to the device and the output of layer l-1 travels back while layer l computes.
        # Every byte of the step still moves inside the timed region.
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        meta_h, meta_d = h_in[layers * per_layer:], d_in[layers * per_layer:]

        overlap_copies = per_layer >= (1 << 20)  # a megabyte of input per layer and more

        def e2e_enqueue():
            main = torch.cuda.current_stream(device)
            if not overlap_copies:
                # small steps: per-layer copies and events would cost more host time than the copies take
                d_in.copy_(h_in, non_blocking=True)
                for i, L in enumerate(layers_data):
                    q, k, v = dv[i]
                    kv.int8_decode_step(q, k, v, L.kc, L.vc, d_slots, d_bt, d_sl, L.k_scale, L.v_scale,
                                        num_splits=args.num_splits, max_seq_len=max_seq, out=d_out[i],
                                        inputs_ready=ready and i > 0)
                h_out.copy_(d_out, non_blocking=True)
                return
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            ready_in = []
            with torch.cuda.stream(s_in):
                meta_d.copy_(meta_h, non_blocking=True)
                for i in range(layers):
                    d_in[i * per_layer:(i + 1) * per_layer].copy_(h_in[i * per_layer:(i + 1) * per_layer], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                    ready_in.append(ev)
            for i, L in enumerate(layers_data):
                q, k, v = dv[i]
                main.wait_event(ready_in[i])
                # the first layer's kernel follows the host-to-device copy and orders itself behind it
                kv.int8_decode_step(q, k, v, L.kc, L.vc, d_slots, d_bt, d_sl, L.k_scale, L.v_scale,
                                    num_splits=args.num_splits, max_seq_len=max_seq, out=d_out[i],
                                    inputs_ready=ready and i > 0)
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    h_out[i].copy_(d_out[i], non_blocking=True)
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        def eager_step():
            e2e_enqueue()
            stream.synchronize()

        # The same step with the layers chained in groups (--launch chained): one int8kv_decode_step_layers call per
        # group of layers, the group's inputs copied in beside the previous group's compute and its outputs copied
        # out beside the next group's.  Steps too small for that (see overlap_copies) are one group.
        group_len = 4 if overlap_copies else layers
        groups = [(a, min(a + group_len, layers)) for a in range(0, layers, group_len)]
        chained_e2e = args.launch == "chained"
        if chained_e2e:
            with torch.cuda.stream(stream):
                group_plans = [kv.DecodeStepLayers(
                    [dv[i][0] for i in range(a, b)], [dv[i][1] for i in range(a, b)], [dv[i][2] for i in range(a, b)],
                    [L.kc for L in layers_data[a:b]], [L.vc for L in layers_data[a:b]], d_slots, d_bt, d_sl,
                    [L.k_scale for L in layers_data[a:b]], [L.v_scale for L in layers_data[a:b]],
                    num_splits=args.num_splits, max_seq_len=max_seq, out=d_out[a:b], inputs_ready=True) for a, b in groups]

        def e2e_enqueue_grouped():
            main = torch.cuda.current_stream(device)
            if len(groups) == 1:
                d_in.copy_(h_in, non_blocking=True)
                group_plans[0]()
                h_out.copy_(d_out, non_blocking=True)
                return
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            ready_in = []
            with torch.cuda.stream(s_in):
                meta_d.copy_(meta_h, non_blocking=True)
                for a, b in groups:
                    d_in[a * per_layer:b * per_layer].copy_(h_in[a * per_layer:b * per_layer], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                    ready_in.append(ev)
            for gi, (a, b) in enumerate(groups):
                main.wait_event(ready_in[gi])
                group_plans[gi]()
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(done)
                    h_out[a:b].copy_(d_out[a:b], non_blocking=True)
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        def eager_grouped_step():
            e2e_enqueue_grouped()
            stream.synchronize()

        e2e_eager_s = ctx.time_host(eager_grouped_step if chained_e2e else eager_step)
        with torch.cuda.stream(stream):
            # the same step through the L-layer entry point: one library call per step, arguments marshalled once
            plan = kv.DecodeStepLayers([dv[i][0] for i in range(layers)], [dv[i][1] for i in range(layers)],
                                       [dv[i][2] for i in range(layers)], [L.kc for L in layers_data],
                                       [L.vc for L in layers_data], d_slots, d_bt, d_sl,
                                       [L.k_scale for L in layers_data], [L.v_scale for L in layers_data],
                                       num_splits=args.num_splits, max_seq_len=max_seq, out=d_out, inputs_ready=ready)

        def layers_step():
            d_in.copy_(h_in, non_blocking=True)
            plan()
            h_out.copy_(d_out, non_blocking=True)
            stream.synchronize()

        e2e_layers_s = ctx.time_host(layers_step)
        def graphed(enqueue):
            with torch.cuda.stream(stream):
                enqueue()  # once eagerly on this stream: workspaces reach their size before the capture
                stream.synchronize()
                g3 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g3, stream=stream):
                    enqueue()

            def graph_step():
                g3.replay()
                stream.synchronize()

            return ctx.time_host(graph_step)

        e2e_per_layer_s = graphed(e2e_enqueue)
        per_layer_out = h_out.clone()
        h_out.zero_()
        e2e_s = graphed(e2e_enqueue_grouped) if chained_e2e else e2e_per_layer_s
        # same inputs, same caches: the two variants differ at most in their split counts (bf16 rounding of the output)
        e2e_agree = {"bit_identical": bool(torch.equal(h_out, per_layer_out)),
                     "max_abs": float((h_out.float() - per_layer_out.float()).abs().max()),
                     "largest_output": float(per_layer_out.float().abs().max())}
        e2e_agree["ok"] = e2e_agree["max_abs"] <= 2e-2 * max(1.0, e2e_agree["largest_output"])
        del plan
        if chained_e2e:
            del group_plans

    dev_ms, e2e_ms, e2e_eager_ms, bf16_ms, e2e_layers_ms, warm_ms, e2e_per_layer_ms = ctx.reduce(
        [dev_ms, e2e_s * 1e3, e2e_eager_s * 1e3, bf16_ms, e2e_layers_s * 1e3, warm_ms, e2e_per_layer_s * 1e3], "max")
    e2e_graph_ms = e2e_ms
    if args.launch == "chained" and e2e_eager_ms < e2e_ms:  # launched from Python it can be the faster of the two
        e2e_ms, e2e_from = e2e_eager_ms, "launched from Python every step"
    mode_names = sorted(other_modes)
    mode_ms = dict(zip(mode_names, ctx.reduce([other_modes[m] for m in mode_names], "max"))) if mode_names else {}
    mode_ms[args.launch] = dev_ms
    total_step_bytes, total_token_layers, h2d_all, d2h_all = ctx.reduce(
        [nbytes_step, B * layers, h2d, d2h], "sum")
    status = kv.device_status(device)
    status, = ctx.reduce([status], "max")
    del layers_data
    _release()

    value = total_step_bytes / (dev_ms * 1e-3) / 1e9
    per_call_s = dev_ms * 1e-3 / layers
    achieved = nbytes_call / per_call_s / 1e9  # rank 0's shard per call; the ranks' shards are alike
    traffic = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get(name)
    line = {
        "metric": metric, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms, "higher_is_better": True,
        "scaling": "strong" if name in ("c4", "c5") else args.scaling,
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config,
        "us_per_call": per_call_s * 1e6,
        "tokens_layers_per_s": total_token_layers / (dev_ms * 1e-3),
        "frac_of_8TBps": value / world / HBM_NOMINAL_GBS,
        "num_splits": splits, "split_plan": split_plan,
        "launch_modes_us_per_call": {m: v * 1e3 / layers for m, v in sorted(mode_ms.items())},
        "gpu_launches": ((layers + (1 if launches_per_call > 1 else 0)) if chained else launches_per_call * layers) * args.steps,
        "clocks": clocks, "device_status": int(status), "shard_check": check,
        "e2e": {"value": total_step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": int(h2d_all), "d2h_bytes_per_step": int(d2h_all),
                "ms_per_step": e2e_ms, "graph_ms_per_step": e2e_graph_ms, "eager_ms_per_step": e2e_eager_ms,
                "eager_value": total_step_bytes / (e2e_eager_ms * 1e-3) / 1e9,
                "one_call_ms_per_step": e2e_layers_ms,
                "one_call_value": total_step_bytes / (e2e_layers_ms * 1e-3) / 1e9,
                "value_from": e2e_from,
                "outputs_agree_with_per_layer_calls": e2e_agree,
                "per_layer_calls_ms_per_step": e2e_per_layer_ms,
                "per_layer_calls_value": total_step_bytes / (e2e_per_layer_ms * 1e-3) / 1e9,
                "what": "per step and rank: pinned-host inputs (every layer's new q/k/v rows; block tables, seq_lens, "
                        "slots) -> device, the decode step (cache write + attention) of every layer through the Python "
                        "operators, every layer's output -> pinned host, all streams synchronised.  With --launch chained "
                        "the layers run as int8kv_decode_step_layers calls over groups of 4 layers, a group's inputs "
                        "travelling in beside the previous group's compute and its outputs out beside the next group's, "
                        "on streams of their own (steps with less than a megabyte of input per layer are one group with "
                        "one copy before and one after); the step is timed as one CUDA graph replay and launched from "
                        "Python every step (`eager_value`), `value` is the faster of the two (`value_from`); `per_layer_calls_value` is a graph of one int8_decode_step "
                        "call per layer with per-layer copies beside them (what `value` is under --launch per-call or "
                        "ordered); `one_call_value` copies everything in, runs one int8kv_decode_step_layers call over "
                        "all layers and copies everything out (no graph, no overlap); bytes are summed over ranks"},
        "l2_warm": {"us_per_call": warm_ms * 1e3 / layers,
                    "what": "the same calls repeated on one layer's cache (re-read from L2 when it fits): not the "
                            "headline, which reads a different cache per call"},
        "bf16_baseline": {"us_per_call": bf16_ms * 1e3 / layers, "int8_speedup": bf16_ms / dev_ms,
                          "what": "bf16_paged_attention on caches holding the same rows un-quantised, same block "
                                  "tables, same graph replay timing, same sharding"} if want_bf16 else None,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": ctx.peak, "unit": "GB/s", "frac": achieved / ctx.peak,
                     "traffic": int(traffic * nbytes_call) if traffic and not (args.batch or dynamic) else None,
                     "traffic_source": "ncu dram bytes of a smaller launch of the same shape, scaled by algorithmic bytes"
                     if name == "c5" or parts > 1 else "ncu dram bytes of this launch (serialised: the carried merge "
                     "re-reads the previous layer's partial rows from DRAM there, from L2 in the timed run)",
                     "peak_source": ctx.peak_src,
                     "kernel": "paged_attn_int8_kernel (+ merge_partials_kernel when split), per call inside the graph",
                     "algorithmic_bytes_per_call": nbytes_call},
    }
    return line


def leg_sequence_parallel(ctx, hq, hkv, seq_lens):
    """Long-context sequence split: rank r holds blocks [r*per, (r+1)*per) of every sequence in its own cache (all KV
    heads, local block ids); one step = partial attention over the local tokens, exchange of the [B, Hq, D+4] fp32
    partial rows, local merge.  Returns a dict with the microseconds per step (max over ranks) of each exchange
    variant and the check of the merged result against single-device attention."""
    kv, wl, sh, device, args, rank, world = ctx.kv, ctx.wl, ctx.sh, ctx.device, ctx.args, ctx.rank, ctx.world
    _, _, local_lens = sh.sequence_split(seq_lens, rank, world, 16)
    assert len(set(local_lens)) == 1, "the check gathers equal token counts from every rank"
    layer = build_layers(kv, wl, device, hq, hkv, local_lens, 1, seed=300 + rank, common_seed=300)[0]
    max_local = max(local_lens)
    result = {}
    merged = {}

    def nccl_step():
        merged["nccl"] = sh.sequence_parallel_int8_attention(
            layer.query, layer.kc, layer.vc, layer.block_tables, layer.seq_lens, layer.k_scale, layer.v_scale,
            max_seq_len=max_local)

    variants = [("nccl_all_gather", nccl_step, "nccl")]
    peer = None
    if not args.no_peer_exchange:
        try:
            peer = sh.PeerExchange(len(seq_lens), hq, 128, device)
        except Exception as e:  # no symmetric-memory mapping on this box: the NCCL variant stands alone
            result["peer_stores"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if peer is not None:

        def peer_step():
            merged["peer"] = sh.sequence_parallel_int8_attention(
                layer.query, layer.kc, layer.vc, layer.block_tables, layer.seq_lens, layer.k_scale, layer.v_scale,
                max_seq_len=max_local, exchange=peer)

        variants.append(("peer_stores", peer_step, "peer"))

    nbytes = algorithmic_bytes(seq_lens, hq, hkv)
    picks = [0, len(seq_lens) - 1]
    for label, step, key in variants:
        ms, = ctx.reduce([ctx.time_device(step)], "max")
        eager_ms, = ctx.reduce([ctx.time_device(step, graph=False)], "max")
        with torch.cuda.stream(ctx.stream):
            step()
            ctx.stream.synchronize()
        chk = sequence_parallel_check(ctx, layer, local_lens, merged[key], picks)
        result[label] = {"us_per_step": ms * 1e3, "eager_us_per_step": eager_ms * 1e3,
                         "value": nbytes / (ms * 1e-3) / 1e9, "seq_parallel_check": chk}
    if peer is not None:
        # where a peer-store step spends its time: the rank's own attention (parts + their merge into rows), the same
        # followed by the push (nobody waits for the flags), and the whole step
        B, D = len(seq_lens), 128
        rows = torch.empty((B, hq, 132), device=device, dtype=torch.float32)  # out (128) | lse | pad

        def partial_only():
            kv.int8_paged_attention_partial(layer.query, layer.kc, layer.vc, layer.block_tables, layer.seq_lens,
                                            layer.k_scale, layer.v_scale, max_seq_len=max_local, out=rows)

        def partial_push():
            kv.int8_paged_attention_partial_push(layer.query, layer.kc, layer.vc, layer.block_tables,
                                                     layer.seq_lens, layer.k_scale, layer.v_scale, peer.exchange,
                                                     max_seq_len=max_local)

        a_ms, = ctx.reduce([ctx.time_device(partial_only)], "max")
        b_ms, = ctx.reduce([ctx.time_device(partial_push)], "max")
        result["peer_stores"]["breakdown_us"] = {
            "partial_rows": a_ms * 1e3, "partial_rows_and_push": b_ms * 1e3,
            "whole_step": result["peer_stores"]["us_per_step"],
            "what": "max over ranks of: the rank's attention and the merge of its parts into rows; the same followed by "
                    "the push (to every rank, or from four ranks on to the rows' owner ranks; nobody waits); the whole step with "
                    "the kernels that poll for the other ranks' rows, merge them and write the output"}
    status, = ctx.reduce([kv.device_status(device)], "max")
    result["device_status"] = int(status)
    result["collective"] = {"bytes_per_rank": len(seq_lens) * hq * 132 * 4,
                            "rows": "fp32 [B, Hq, 132] = normalised out (128) | lse | pad, one slab per rank"}
    result["tokens_per_rank_per_sequence"] = max_local
    if peer is not None:
        peer.close()
    del layer
    _release()
    return result


def leg_c5(ctx):
    """Long context (Hq=64, Hkv=8, B=32, 65536 tokens each, 4.29 GB of INT8 K+V, 2 GiB per cache tensor).  One GPU:
    the whole call and its BF16 twin.  N GPUs: head-parallel shards (no collective) and the sequence-parallel form."""
    hq, hkv, seq_lens, layers, desc = workload_spec("c5")
    config = {"workload": f"c5: {desc}", "Hq": hq, "Hkv": hkv, "head_dim": 128, "block_size": 16}
    body = leg_decode(ctx, "c5", hq, hkv, seq_lens, layers, config, sub=True)
    rec = {"workload": config["workload"], "parallelism": config.get("parallelism", "single GPU"),
           "us_per_call": body["us_per_call"], "value": body["value"], "frac": body["roofline"]["frac"],
           "frac_of_8TBps": body["frac_of_8TBps"], "num_splits": body["num_splits"], "split_plan": body["split_plan"],
           "bf16_baseline": body["bf16_baseline"], "shard_check": body["shard_check"],
           "algorithmic_bytes_per_call_per_rank": body["roofline"]["algorithmic_bytes_per_call"]}
    if ctx.world > 1:
        rec["sequence_parallel"] = leg_sequence_parallel(ctx, hq, hkv, seq_lens)
    return rec


# ---------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c4", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--num-splits", type=int, default=None)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="c2 only (c4 and c5 are always sharded by KV head and batch): weak = every rank runs the cell")
    ap.add_argument("--seq-parallel", action="store_true",
                    help="c5 only: print the sequence-parallel record alone (partial rows exchanged and merged)")
    ap.add_argument("--no-peer-exchange", action="store_true", help="sequence-parallel: NCCL all-gather variant only")
    ap.add_argument("--no-sub", action="store_true", help="skip the c2 / c3 / c5 sub-records of the default line")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host leg (profiling runs)")
    ap.add_argument("--no-bf16", dest="bf16_baseline", action="store_false", help="skip the same-run BF16 baseline")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--launch", default="chained", choices=sorted(LAUNCH_MODES),
                    help="how the layers of a device-timed step are launched: " + "; ".join(f"{k} = {v}" for k, v in LAUNCH_MODES.items()))
    ap.add_argument("--scales", default="static", choices=["static", "dynamic"],
                    help="dynamic: time the attention over per-(token, head) scale caches (device leg only)")
    ap.add_argument("--sweep", action="store_true",
                    help="c2 only, one GPU: time all 16 cells of the sweep and list them under `cells`")
    ap.add_argument("--shape", default=None, metavar="Hq,Hkv,D,BLOCK[,BATCH,SEQ]",
                    help="time int8_paged_attention on one layer of any shape (one GPU) and print that record alone")
    ap.add_argument("--one-shard-of", type=int, default=None, metavar="N",
                    help="one GPU: run rank 0's shard of an N-way KV-head x batch partition alone (what one rank of an "
                         "N-GPU job computes); the printed value covers that shard only")
    ap.add_argument("--batch", type=int, default=None, help="use only the first BATCH sequences of the workload")
    ap.add_argument("--layers", type=int, default=None, help="override the number of distinct layer caches")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if "WORLD_SIZE" not in os.environ and args.gpus > 1:
        # started bare with --gpus N: run the same command as one process per GPU
        port = os.environ.get("MASTER_PORT", "29541")
        os.execvp(sys.executable, [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
                                   f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1", "--master-port", port,
                                   str(Path(__file__).resolve())] + sys.argv[1:])
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world:
        raise SystemExit(f"bench.py: --gpus {args.gpus} but the launcher started {world} rank(s) (WORLD_SIZE); "
                         "launch with python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    hq, hkv, seq_lens, layers, desc = workload_spec(args.workload)
    if args.batch:
        seq_lens = seq_lens[: args.batch]
        desc += f" (first {len(seq_lens)} sequences)"
    if args.layers:
        layers = args.layers
        desc += f" ({layers} layer caches)"
    config = {"workload": f"{args.workload}: {desc}", "Hq": hq, "Hkv": hkv, "head_dim": 128, "block_size": 16,
              "batch": len(seq_lens), "batch_per_gpu": len(seq_lens), "layers": layers,
              "arithmetic": "int8 cache; QK^T on int8 tensor cores, PV in fp16 MMA, fp32 softmax and accumulation",
              "l2": "inputs larger than L2: each call reads a different layer's cache",
              "parallelism": "single GPU"}

    # ---------------- reference arm: the CPU path on the host cores -------------------------------
    if args.impl == "reference":
        if rank != 0:
            return
        wl = importlib.import_module("int8-kvcache_b200.workloads")
        gbs, med, cores, sample_desc, sample = time_cpu(wl, hq, hkv, seq_lens, budget_s=0.0,
                                                        min_reps=max(1, args.steps), warm=max(0, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": med * 1e3, "higher_is_better": True,
                "scaling": "strong" if args.workload in ("c4", "c5") else args.scaling, "vs_baseline": None,
                "dtype": "int8", "data": "synthetic", "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample_desc},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "us_per_call": med * 1e6, "gpu_launches": 0}
        print(json.dumps(line))
        return

    # ---------------- our arm ------------------------------------------------------------------------
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the kernels)")
    ctx = Ctx(args, rank, local_rank, world)
    try:
        if args.shape:
            print(json.dumps(leg_shape(ctx, args.shape)))
            return
        if args.workload == "c3":
            rec = leg_cache_write(ctx)
            line = {"metric": rec.pop("metric"), "value": rec["value"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
                    "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                    "us_per_call": rec["us_per_call"], "gpu_launches": rec["gpu_launches"],
                    "same_bytes_copy": rec["same_bytes_copy"], "config": {"workload": rec["workload"]},
                    "roofline": {"bound": "hbm", "achieved": rec["value"], "peak": ctx.peak, "unit": "GB/s",
                                 "frac": rec["frac"], "traffic": C3_NCU_DRAM_BYTES_IN_KERNEL, "kernel": rec["kernel"],
                                 "traffic_note": "ncu, dram__bytes_read.sum + dram__bytes_write.sum of one launch: the rows "
                                                 "of the tokens that are written come in, the INT8 output is still in L2 when "
                                                 "the kernel ends and is written back under later kernels",
                                 "algorithmic_bytes_per_call": rec["algorithmic_bytes_per_call"]}}
            if rank == 0:
                print(json.dumps(_without_nan(line)))
            return
        if args.sweep:
            if args.workload != "c2" or world > 1:
                raise SystemExit("--sweep runs the c2 grid on one GPU")
            cells = leg_sweep(ctx)
            top = cells[-1]
            print(json.dumps(_without_nan({
                "metric": METRIC, "value": top["int8_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": top["int8_us"] * top["layer_caches"] / 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": "c2 sweep: B in {1,2,4,8} x seq in {512,1024,2048,4096}, value = the largest cell",
                           "Hq": 28, "Hkv": 4, "head_dim": 128, "block_size": 16,
                           "l2": "inputs larger than L2: each call reads a different layer's cache"},
                "us_per_call": top["int8_us"], "cells": cells, "device_status": ctx.kv.device_status(ctx.device)})))
            return
        if args.seq_parallel:
            if args.workload != "c5" or world < 2:
                raise SystemExit("--seq-parallel runs c5 on two or more GPUs")
            rec = leg_sequence_parallel(ctx, hq, hkv, seq_lens)
            if rank == 0:
                best = min(v["us_per_step"] for v in rec.values() if isinstance(v, dict) and "us_per_step" in v)
                config["parallelism"] = f"sequence split over {world} ranks, partial rows exchanged and merged"
                print(json.dumps(_without_nan({
                    "metric": METRIC, "value": algorithmic_bytes(seq_lens, hq, hkv) / (best * 1e-6) / 1e9, "unit": "GB/s",
                    "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": best / 1e3,
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8",
                    "data": "synthetic", "config": config, "us_per_call": best, "sequence_parallel": rec})))
            return

        line = leg_decode(ctx, args.workload, hq, hkv, seq_lens, layers, config)
        main_shape = (hq, hkv, seq_lens)
        if args.workload == "c4" and not args.no_sub and not (args.batch or args.layers or args.scales == "dynamic"):
            if world == 1:
                cells = leg_sweep(ctx)
                top = cells[-1]
                nb = algorithmic_bytes([4096] * 8, 28, 4)
                line["c2_cell"] = {"workload": "c2: sweep cell B=8 seq=4096, 28 distinct layer caches",
                                   "us_per_call": top["int8_us"], "value": top["int8_gbs"],
                                   "frac": top["int8_gbs"] / ctx.peak, "bf16_us_per_call": top["bf16_us"],
                                   "int8_speedup": top["int8_speedup"], "algorithmic_bytes_per_call": nb}
                line["cells"] = cells
                line["c3_write"] = leg_cache_write(ctx)
            line["c5"] = leg_c5(ctx)
        if rank == 0:
            if not args.no_cpu:
                gbs, med, cores, sample_desc, _ = time_cpu(ctx.wl, main_shape[0], main_shape[1], main_shape[2],
                                                           budget_s=args.cpu_seconds)
                line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                        "sample": sample_desc, "ms_per_call": med * 1e3}
            print(json.dumps(_without_nan(line)))
    finally:
        if ctx.dist is not None:
            gc.collect()
            torch.cuda.synchronize(ctx.device)
            ctx.dist.barrier()
            ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
