#!/usr/bin/env python
"""Benchmark of the INT8 paged decode-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c4|c5]

Default workload (`c2`): the largest cell of the single-GPU kernel sweep — B=8 sequences of 4096
tokens, Hq=28, Hkv=4, D=128, block_size=16 — for 28 layers, each with its own INT8 cache (28 x 67 MB,
larger than L2, so every call reads its pages from HBM).  One step = one decode pass over the 28
layers = 28 int8_paged_attention calls.  Under torchrun every rank runs the same shard (its own batch
of sequences on its own GPU, no collective): weak scaling.

Printed JSON (one line, rank 0):
  value      achieved GB/s of algorithmic bytes, device-resident inputs, step replayed as a CUDA graph
  e2e        same metric through the Python operators with pinned-host inputs copied in and the result
             copied out inside the timed region
  roofline   the attention call against the measured HBM copy peak
  cpu_baseline  the CPU oracle (a port of the reference's PyTorch CPU path) on one layer of the workload
`--impl reference` times that CPU path alone with all host threads.
"""

from __future__ import annotations

import argparse
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

# dram__bytes_read.sum + dram__bytes_write.sum of one paged_attn_int8_kernel launch, from a one-pass ncu capture of
# this script's default workload (the launch-list summary under profiles/)
NCU_DRAM_TRAFFIC_PER_LAUNCH = {"c2": 33690154}
HBM_NOMINAL_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0


# ---------------------------------------------------------------------------------------------------
# workload description
# ---------------------------------------------------------------------------------------------------
def workload_spec(name: str):
    """(shape kwargs, seq_lens per rank, layers, description)"""
    gen = torch.Generator().manual_seed(1234)
    if name == "c2":
        return dict(hq=28, hkv=4), [4096] * 8, 28, "sweep cell B=8 seq=4096, 28 distinct layer caches"
    if name == "c3":  # cache-write workload; handled by bench_cache_write
        return dict(hq=28, hkv=4), [2048] * 8, 1, "prefill cache write, 8 x 2048 tokens"
    if name == "c4":
        lens = torch.randint(1024, 8193, (256,), generator=gen).tolist()
        return dict(hq=28, hkv=4), lens, 4, "B=256 seq~U[1024,8192], 4 distinct layer caches"
    if name == "c5":
        return dict(hq=64, hkv=8), [65536] * 32, 1, "B=32 ctx 65536 Hq=64 Hkv=8, one layer"
    raise SystemExit(f"unknown workload {name}")


def algorithmic_bytes(seq_lens, hq, hkv, d=128, bs=16, elem=1) -> int:
    """K+V bytes + block ids + query in / out + scales + seq_lens, per call."""
    tok = sum(seq_lens)
    blocks = sum((s + bs - 1) // bs for s in seq_lens)
    return tok * hkv * d * 2 * elem + blocks * 4 + len(seq_lens) * hq * d * 2 * 2 + 8 * hkv + 4 * len(seq_lens)


class Layer:
    pass


def build_layers(kv, wl, device, hq, hkv, seq_lens, layers, seed, with_bf16=False):
    """Per layer: INT8 caches filled through the product write kernel from seeded bf16 K/V."""
    shape = wl.LayerShape(hq, hkv, 128, 16)
    B = len(seq_lens)
    need = int(wl.blocks_needed(seq_lens, 16).sum())
    num_blocks = need * 2 if need * 2 * 16 * hkv * 128 < (8 << 30) else need + 64
    out = []
    gen = torch.Generator(device=device)
    for li in range(layers):
        L = Layer()
        L.k_scale, L.v_scale = [t.to(device) for t in wl.calibrate_scales(shape, seed, li)]
        tables = wl.permuted_block_tables(seq_lens, 16, num_blocks, seed + 13 * li)
        L.block_tables = tables.to(device)
        L.seq_lens = torch.tensor(seq_lens, dtype=torch.int32, device=device)
        L.kc = torch.zeros(num_blocks, 16, hkv, 128, dtype=torch.int8, device=device)
        L.vc = torch.zeros_like(L.kc)
        if with_bf16:
            L.kb = torch.zeros(num_blocks, 16, hkv, 128, dtype=torch.bfloat16, device=device)
            L.vb = torch.zeros_like(L.kb)
        gain = wl.channel_gain(shape, seed, device)
        gen.manual_seed(seed * 1000003 + li)
        for b in range(B):  # one sequence at a time bounds the bf16 staging memory
            T = seq_lens[b]
            k, v = wl.draw_kv(T, shape, gen, gain)
            tok = torch.arange(T, device=device)
            slots = L.block_tables[b, tok // 16].long() * 16 + tok % 16
            kv.int8_kv_cache_write(k, v, L.kc, L.vc, slots, L.k_scale, L.v_scale)
            if with_bf16:
                L.kb.view(-1, hkv, 128)[slots] = k
                L.vb.view(-1, hkv, 128)[slots] = v
        L.query = wl.draw_query(B, shape, gen)
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
    desc = f"one layer call (write {len(sample)} tokens + attention), B={len(sample)}, {sum(sample)} context tokens, {len(times)} reps, median"
    return nbytes / med / 1e9, med, torch.get_num_threads(), desc, sample


# ---------------------------------------------------------------------------------------------------
def bench_cache_write(kv, wl, device, args):
    """Prefill-style INT8 cache write (BASELINE config 3): 8 x 2048 tokens, ~3% padding slots, rotated over
    8 distinct input/cache sets (400 MB, larger than L2); one step = 8 writes replayed as a CUDA graph."""
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

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        if args.no_graph:
            replay = step
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            replay = graph.replay
        for _ in range(max(args.warmup, 3)):
            replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            replay()
        e1.record(stream)
        stream.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps / len(sets)
    peaks_path = REPO / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else FALLBACK_PEAK_GBS
    gbs = nbytes / us / 1e3
    print(json.dumps({
        "metric": "int8_dynamic_scale_kv_cache_write_achieved_hbm_gbps" if dynamic else "int8_kv_cache_write_achieved_hbm_gbps",
        "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": us * len(sets) / 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "us_per_call": us, "gpu_launches": len(sets) * args.steps,
        "config": {"workload": "c3: prefill cache write, 16384 tokens x 4 heads x 128, permuted 1024-block pool, "
                               "~3% slots = -1, 8 rotated sets (larger than L2)"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "traffic": None,
                     "kernel": "cache_write_dynamic_vec_kernel<bf16>" if dynamic else "cache_write_vec_kernel<bf16>",
                     "algorithmic_bytes_per_call": nbytes},
    }))


def _time_graph(fn, stream, steps, warmup):
    """ms per replay of `fn` captured as a CUDA graph on `stream` (CUDA events on that stream)."""
    with torch.cuda.stream(stream):
        fn()
        fn()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            fn()
        for _ in range(max(warmup, 3)):
            graph.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        stream.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_sweep(kv, wl, device, args):
    """The whole single-GPU sweep of BASELINE config 2 (B in {1,2,4,8} x seq in {512,1024,2048,4096}, the grid of
    the reference's bench/bench_paged_attention.py): microseconds per call for the INT8 kernels and the same-run
    BF16 baseline, each cell rotated over enough distinct layer caches to exceed the L2."""
    hq, hkv = wl.QWEN25_7B.num_q_heads, wl.QWEN25_7B.num_kv_heads
    stream = torch.cuda.Stream(device)
    cells = []
    for B in (1, 2, 4, 8):
        for seq in (512, 1024, 2048, 4096):
            cell_bytes = B * seq * hkv * 128 * 2 * 3  # INT8 and BF16 caches of one layer
            layers = max(4, min(64, int(600e6 / cell_bytes)))
            L = build_layers(kv, wl, device, hq, hkv, [seq] * B, layers, seed=5, with_bf16=True)

            def int8_step():
                for x in L:
                    kv.int8_paged_attention(x.query, x.kc, x.vc, x.block_tables, x.seq_lens, x.k_scale, x.v_scale,
                                            max_seq_len=seq, out=x.out)

            def bf16_step():
                for x in L:
                    kv.bf16_paged_attention(x.query, x.kb, x.vb, x.block_tables, x.seq_lens, max_seq_len=seq, out=x.out)

            i8 = _time_graph(int8_step, stream, args.steps, args.warmup) / layers * 1e3
            bf = _time_graph(bf16_step, stream, args.steps, args.warmup) / layers * 1e3
            nb = algorithmic_bytes([seq] * B, hq, hkv)
            cells.append({"batch": B, "seq_len": seq, "layer_caches": layers, "int8_us": i8, "bf16_us": bf,
                          "int8_speedup": bf / i8, "int8_gbs": nb / i8 / 1e3})
            del L
            torch.cuda.empty_cache()
    top = cells[-1]
    print(json.dumps({
        "metric": "int8_paged_decode_attn_achieved_hbm_gbps", "value": top["int8_gbs"], "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": top["int8_us"] * top["layer_caches"] / 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "c2 sweep: B in {1,2,4,8} x seq in {512,1024,2048,4096}, value = the largest cell",
                   "Hq": hq, "Hkv": hkv, "head_dim": 128, "block_size": 16,
                   "l2": "inputs larger than L2: each call reads a different layer's cache"},
        "us_per_call": top["int8_us"], "cells": cells, "device_status": kv.device_status(device),
    }))


def bench_sequence_parallel(kv, wl, device, args, rank, world, hq, hkv, seq_lens, config, metric):
    """Long-context sequence split: rank r holds blocks [r*per, (r+1)*per) of every sequence in its own cache (all KV
    heads); one step = partial attention over the local tokens, NCCL all-gather of the [B, Hq, D+4] fp32 partial
    rows into local memory, local merge.  value = bytes of the whole context / max-over-ranks time."""
    import torch.distributed as dist

    sh = importlib.import_module("int8-kvcache_b200.sharding")
    _, _, local_lens = sh.sequence_split(seq_lens, rank, world, 16)
    layer = build_layers(kv, wl, device, hq, hkv, local_lens, 1, seed=300 + rank)[0]
    max_local = max(local_lens)

    def step():
        return sh.sequence_parallel_int8_attention(layer.query, layer.kc, layer.vc, layer.block_tables, layer.seq_lens,
                                                   layer.k_scale, layer.v_scale, max_seq_len=max_local)

    # The step (partial kernel, NCCL all-gather, merge) is captured once into a CUDA graph and replayed, as a decode
    # loop would run it; --no-graph launches it from Python every step.
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        run, launched = step, "eager"
        if not args.no_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            run, launched = graph.replay, "cuda graph"
            for _ in range(3):
                run()
        torch.cuda.synchronize(device)
        dist.barrier()
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        torch.cuda.synchronize(device)
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        ms = float(t.item())
        nbytes = algorithmic_bytes(seq_lens, hq, hkv)
        config["parallelism"] = (f"sequence split over {world} ranks ({max_local} tokens of every sequence per rank), "
                                 "NCCL all-gather of partial rows + local merge")
        config["batch_per_gpu"] = len(seq_lens)
        print(json.dumps({
            "metric": metric, "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": config, "us_per_call": ms * 1e3,
            "gpu_launches": 2 * args.steps,
            "collective": {"op": "all_gather_into_tensor", "bytes_per_rank": len(seq_lens) * hq * 132 * 4},
            "launched": launched,
        }))
    # a live CUDA graph that holds captured NCCL work blocks the communicator's teardown: release it first
    run = graph = None
    import gc

    gc.collect()
    torch.cuda.synchronize(device)
    dist.barrier()
    dist.destroy_process_group()


def _without_nan(x):
    """Legs that were skipped hold NaN; JSON has no NaN, so they become null."""
    if isinstance(x, dict):
        return {k: _without_nan(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_without_nan(v) for v in x]
    if isinstance(x, float) and x != x:
        return None
    return x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c4", "c5"])
    ap.add_argument("--num-splits", type=int, default=None)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank runs the whole workload shape; strong: the workload is sharded by KV head "
                         "and batch over the ranks (no collective)")
    ap.add_argument("--seq-parallel", action="store_true",
                    help="c5 only: split every sequence over the ranks; partial rows are all-gathered with NCCL and merged")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-to-host leg (profiling runs)")
    ap.add_argument("--no-bf16", dest="bf16_baseline", action="store_false", help="skip the same-run BF16 baseline")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--scales", default="static", choices=["static", "dynamic"],
                    help="dynamic: time the attention over per-(token, head) scale caches (device leg only)")
    ap.add_argument("--sweep", action="store_true",
                    help="c2 only, one GPU: time all 16 cells of the sweep, INT8 and BF16, and list them under `cells`")
    ap.add_argument("--batch", type=int, default=None, help="use only the first BATCH sequences of the workload")
    ap.add_argument("--layers", type=int, default=None, help="override the number of distinct layer caches")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    shape_kw, seq_lens, layers, desc = workload_spec(args.workload)
    if args.batch:
        seq_lens = seq_lens[: args.batch]
        desc += f" (first {len(seq_lens)} sequences)"
    if args.layers:
        layers = args.layers
        desc += f" ({layers} layer caches)"
    hq, hkv = shape_kw["hq"], shape_kw["hkv"]
    wl = importlib.import_module("int8-kvcache_b200.workloads")
    metric = "int8_paged_decode_attn_achieved_hbm_gbps"
    config = {"workload": f"{args.workload}: {desc}", "Hq": hq, "Hkv": hkv, "head_dim": 128, "block_size": 16,
              "batch_per_gpu": len(seq_lens), "layers": layers,
              "arithmetic": "int8 cache; QK^T on int8 tensor cores, PV in fp16 MMA, fp32 softmax and accumulation",
              "l2": "inputs larger than L2: each call reads a different layer's cache",
              "parallelism": f"batch-sharded x{world}, no collective" if world > 1 else "single GPU"}

    # ---------------- reference arm: the CPU path on the host cores -------------------------------
    if args.impl == "reference":
        if rank != 0:
            return
        gbs, med, cores, sample_desc, sample = time_cpu(wl, hq, hkv, seq_lens, budget_s=0.0,
                                                        min_reps=max(1, args.steps), warm=max(0, args.warmup))
        line = {"impl": "reference", "metric": metric, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": med * 1e3, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": config,
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample_desc},
                "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "us_per_call": med * 1e6, "gpu_launches": 0}
        print(json.dumps(line))
        return

    # ---------------- our arm ------------------------------------------------------------------------
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback exists for the kernels)")
    kv = importlib.import_module("int8-kvcache_b200")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if args.workload == "c3":
        return bench_cache_write(kv, wl, device, args)
    if args.sweep:
        if args.workload != "c2" or world > 1:
            raise SystemExit("--sweep runs the c2 grid on one GPU")
        return bench_sweep(kv, wl, device, args)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    if args.seq_parallel:
        return bench_sequence_parallel(kv, wl, device, args, rank, world, hq, hkv, seq_lens, config, metric)
    if args.scaling == "strong" and world > 1:
        sh = importlib.import_module("int8-kvcache_b200.sharding")
        shard = sh.head_batch_partition(world, hq, hkv, len(seq_lens))[rank]
        group = hq // hkv
        hkv = shard.kv_heads[1] - shard.kv_heads[0]
        hq = hkv * group
        seq_lens = seq_lens[shard.batch[0]:shard.batch[1]]
        config["parallelism"] = (f"KV-head x batch sharded over {world} ranks, no collective: {hkv} KV head(s) x "
                                 f"{len(seq_lens)} sequences per rank")
        config["batch_per_gpu"] = len(seq_lens)
    layers_data = build_layers(kv, wl, device, hq, hkv, seq_lens, layers, seed=100 + rank)
    max_seq = max(seq_lens)
    B = len(seq_lens)
    nbytes_call = algorithmic_bytes(seq_lens, hq, hkv)
    dynamic = args.scales == "dynamic"
    if dynamic:
        # one fp32 K scale and one fp32 V scale per (token, head) are read on top of the INT8 bytes
        nbytes_call += sum(seq_lens) * hkv * 8
        metric = "int8_dynamic_scale_paged_decode_attn_achieved_hbm_gbps"
        config["scales"] = "per (token, head) fp32 scale caches [num_blocks, 16, Hkv], seeded uniform [0.005, 0.025]"
        args.no_e2e, args.bf16_baseline, args.no_cpu = True, False, True
        gen_s = torch.Generator(device=device)
        for li, L in enumerate(layers_data):
            gen_s.manual_seed(7000 + li)
            L.ksc = torch.rand(L.kc.shape[:3], device=device, generator=gen_s) * 0.02 + 0.005
            L.vsc = torch.rand(L.kc.shape[:3], device=device, generator=gen_s) * 0.02 + 0.005
    nbytes_step = nbytes_call * layers

    def device_step():
        for L in layers_data:
            if dynamic:
                kv.int8_paged_attention_dynamic(L.query, L.kc, L.vc, L.ksc, L.vsc, L.block_tables, L.seq_lens,
                                                num_splits=args.num_splits, max_seq_len=max_seq, out=L.out)
            else:
                kv.int8_paged_attention(L.query, L.kc, L.vc, L.block_tables, L.seq_lens, L.k_scale, L.v_scale,
                                        num_splits=args.num_splits, max_seq_len=max_seq, out=L.out)

    lib = kv._lib.load()
    sm = torch.cuda.get_device_properties(device).multi_processor_count
    splits = args.num_splits or lib.int8kv_choose_splits(B, hkv, max_seq, 16, sm)
    launches_per_call = 1 + (1 if splits > 1 else 0)
    split_plan = None  # filled in after the warm-up when the library planned the parts on the device

    # warm up eagerly (kernel attribute set-up, workspace allocation), then capture one step as a CUDA graph
    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(2):
            device_step()
        stream.synchronize()
        if args.num_splits is None:
            plan = kv.last_split_plan(device)
            if plan is not None:
                split_plan = {"items": plan[0], "part_tiles": plan[1], "waves": plan[2]}
                splits, launches_per_call = "planned on the device", 2
        if args.no_graph:
            class _Eager:
                replay = staticmethod(device_step)
            graph = _Eager()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                device_step()
        for _ in range(args.warmup):
            graph.replay()
        stream.synchronize()

        def barrier():
            torch.cuda.synchronize(device)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(device)

        sampler = ClockSampler(local_rank)
        barrier()
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        dev_ms = e0.elapsed_time(e1)

        # ---- the same calls on ONE layer's cache, labelled L2-warm: whatever fits the 126 MB L2 is re-read from it
        # (reported beside the headline, never as it) ----------------------------------------------------
        warm_ms = float("nan")
        if not dynamic and not args.no_graph:
            L0 = layers_data[0]

            def warm_step():
                for _ in range(layers):
                    kv.int8_paged_attention(L0.query, L0.kc, L0.vc, L0.block_tables, L0.seq_lens, L0.k_scale, L0.v_scale,
                                            num_splits=args.num_splits, max_seq_len=max_seq, out=L0.out)

            warm_step()
            gw = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gw, stream=stream):
                warm_step()
            for _ in range(args.warmup):
                gw.replay()
            barrier()
            w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            w0.record(stream)
            for _ in range(args.steps):
                gw.replay()
            w1.record(stream)
            barrier()
            warm_ms = w0.elapsed_time(w1) / args.steps
            del gw

        # ---- same-run BF16 baseline on identical block tables (one step = the same 28 calls) --------------
        bf16_ms = float("nan")
        if args.bf16_baseline:
            shape = wl.LayerShape(hq, hkv, 128, 16)
            gen = torch.Generator(device=device)
            for li, L in enumerate(layers_data):
                L.kb = torch.zeros(L.kc.shape, dtype=torch.bfloat16, device=device)
                L.vb = torch.zeros_like(L.kb)
                gen.manual_seed(9000 + li)
                gain = wl.channel_gain(shape, 100 + rank, device)
                for b in range(B):
                    T = seq_lens[b]
                    k, v = wl.draw_kv(T, shape, gen, gain)
                    tok = torch.arange(T, device=device)
                    slots = L.block_tables[b, tok // 16].long() * 16 + tok % 16
                    L.kb.view(-1, hkv, 128)[slots] = k
                    L.vb.view(-1, hkv, 128)[slots] = v

            def bf16_step():
                for L in layers_data:
                    kv.bf16_paged_attention(L.query, L.kb, L.vb, L.block_tables, L.seq_lens,
                                            max_seq_len=max_seq, out=L.out)

            for _ in range(2):
                bf16_step()
            stream.synchronize()
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=stream):
                bf16_step()
            for _ in range(args.warmup):
                g2.replay()
            barrier()
            b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record(stream)
            for _ in range(args.steps):
                g2.replay()
            b1.record(stream)
            barrier()
            bf16_ms = b0.elapsed_time(b1) / args.steps
            for L in layers_data:
                del L.kb, L.vb

        # ---- e2e: the decode step a serving engine runs, from host buffers to host buffers ---------------
        # Inputs of one step (every layer's new query / key / value rows, the block tables, sequence lengths and
        # write slots) sit in ONE pinned host buffer; a step copies it to the device, runs cache write +
        # attention for every layer through the Python operators, and copies every layer's output back to a
        # pinned host buffer.  Measured twice: launched eagerly from Python, and with the same calls captured
        # once into a CUDA graph (how decode loops are run in production) and replayed per step.
        shape = wl.LayerShape(hq, hkv, 128, 16)
        g = torch.Generator().manual_seed(7)
        n_q, n_kv = B * hq * 128, B * hkv * 128
        width = layers_data[0].block_tables.shape[1]
        per_layer = (n_q + 2 * n_kv) * 2
        meta_bytes = B * width * 4 + B * 4 + B * 8
        meta_bytes = (meta_bytes + 15) // 16 * 16
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
            so = B * width * 4 + B * 4
            so = (so + 7) // 8 * 8
            slots = m[so:so + B * 8].view(torch.int64)
            return per, bt, sl, slots

        hv, h_bt, h_sl, h_slots = views(h_in)
        for i in range(layers):
            hv[i][0].copy_(wl.draw_query(B, shape, g))
            k, v = wl.draw_kv(B, shape, g, wl.channel_gain(shape, 0))
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

        def e2e_enqueue():
            d_in.copy_(h_in, non_blocking=True)
            for i, L in enumerate(layers_data):
                q, k, v = dv[i]
                kv.int8_decode_step(q, k, v, L.kc, L.vc, d_slots, d_bt, d_sl, L.k_scale, L.v_scale,
                                    num_splits=args.num_splits, max_seq_len=max_seq, out=d_out[i])
            h_out.copy_(d_out, non_blocking=True)

        def time_steps(step):
            for _ in range(args.warmup):
                step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                step()
            barrier()
            return time.perf_counter() - t0

        e2e_s = e2e_eager_s = e2e_layers_s = float("nan")
        if not args.no_e2e:
            def eager_step():
                e2e_enqueue()
                stream.synchronize()

            e2e_eager_s = time_steps(eager_step)
            # the same step through the L-layer entry point: one library call per step, arguments marshalled once
            plan = kv.DecodeStepLayers([dv[i][0] for i in range(layers)], [dv[i][1] for i in range(layers)],
                                       [dv[i][2] for i in range(layers)], [L.kc for L in layers_data],
                                       [L.vc for L in layers_data], d_slots, d_bt, d_sl,
                                       [L.k_scale for L in layers_data], [L.v_scale for L in layers_data],
                                       num_splits=args.num_splits, max_seq_len=max_seq, out=d_out)

            def layers_step():
                d_in.copy_(h_in, non_blocking=True)
                plan()
                h_out.copy_(d_out, non_blocking=True)
                stream.synchronize()

            e2e_layers_s = time_steps(layers_step)
            g3 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g3, stream=stream):
                e2e_enqueue()

            def graph_step():
                g3.replay()
                stream.synchronize()

            e2e_s = time_steps(graph_step)
        clocks = sampler.stop() if rank == 0 else None

    times = torch.tensor([dev_ms, e2e_s * 1e3, e2e_eager_s * 1e3, bf16_ms, e2e_layers_s * 1e3], device=device,
                         dtype=torch.float64)
    total = torch.tensor([float(nbytes_step), float(B * layers)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
        dist.all_reduce(total, op=dist.ReduceOp.SUM)
    total_step_bytes, total_token_layers = [float(x) for x in total.tolist()]
    dev_ms, e2e_ms, e2e_eager_ms, bf16_ms, e2e_layers_ms = [float(x) for x in times.tolist()]
    status = kv.device_status(device)

    if rank == 0:
        ms_per_step = dev_ms / args.steps
        value = total_step_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = total_step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9
        peaks_path = REPO / "MEASURED_PEAKS.json"
        if peaks_path.exists():
            peak, peak_src = float(json.loads(peaks_path.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = FALLBACK_PEAK_GBS, "fallback 6.65 TB/s"
        per_call_s = ms_per_step * 1e-3 / layers
        achieved = nbytes_call / per_call_s / 1e9
        line = {
            "metric": metric, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "int8",
            "data": "synthetic", "config": config,
            "us_per_call": per_call_s * 1e6,
            "tokens_layers_per_s": total_token_layers / (ms_per_step * 1e-3),
            "frac_of_8TBps": value / world / HBM_NOMINAL_GBS,
            "num_splits": splits,
            "split_plan": split_plan,
            "gpu_launches": launches_per_call * layers * args.steps,
            "clocks": clocks,
            "device_status": status,
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "eager_ms_per_step": e2e_eager_ms / args.steps,
                    "eager_value": total_step_bytes / (e2e_eager_ms / args.steps * 1e-3) / 1e9,
                    "one_call_ms_per_step": e2e_layers_ms / args.steps,
                    "one_call_value": total_step_bytes / (e2e_layers_ms / args.steps * 1e-3) / 1e9,
                    "what": "per step: one pinned-host buffer (all layers' new q/k/v rows, block tables, seq_lens, "
                            "slots) -> device, int8_decode_step (cache write + attention) per layer through the Python operators, all "
                            "outputs -> pinned host, stream synchronised; `value` replays those calls as one CUDA "
                            "graph, `eager_value` launches them from Python every step, `one_call_value` launches them "
                            "every step through one int8kv_decode_step_layers call (no graph)"},
            "l2_warm": {"us_per_call": warm_ms * 1e3 / layers,
                        "what": "the same calls repeated on one layer's cache (re-read from L2 when it fits): not the "
                                "headline, which reads a different cache per call"},
            "bf16_baseline": {"us_per_call": bf16_ms * 1e3 / layers, "int8_speedup": bf16_ms / ms_per_step,
                              "what": "bf16_paged_attention on un-quantised caches, same block tables, same graph "
                                      "replay timing"} if args.bf16_baseline else None,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_DRAM_TRAFFIC_PER_LAUNCH.get(args.workload)
                         if not (args.batch or args.layers or dynamic) else None,
                         "peak_source": peak_src,
                         "kernel": "paged_attn_int8_kernel (+ merge_partials_kernel when split), per call inside the graph",
                         "algorithmic_bytes_per_call": nbytes_call},
        }
        if not args.no_cpu:
            gbs, med, cores, sample_desc, _ = time_cpu(wl, hq, hkv, seq_lens, budget_s=args.cpu_seconds)
            line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                    "sample": sample_desc, "ms_per_call": med * 1e3}
        print(json.dumps(_without_nan(line)))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
