"""Time int8_paged_attention on one layer of an arbitrary shape (any head_dim, group and block size).

    python int8-kvcache_b200/shape_bench.py --q-heads 32 --kv-heads 8 --head-dim 64 --batch 64 --seq 2048

bench.py at the repository root measures the headline workloads, all of them head_dim 128; this script is for the
shapes outside them, which the library serves with its non-tiled kernels.  The cache holds random INT8 bytes (the
kernels' time does not depend on the values), the block table is the identity, and `--caches` distinct caches are
visited in turn so that every call reads its pages from DRAM.  Prints one JSON line; GB/s counts the K and V bytes
of the tokens attended, once.
"""

import argparse
import importlib
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--caches", type=int, default=2, help="distinct caches visited in turn (keeps the reads out of L2)")
    ap.add_argument("--num-splits", type=int, default=None)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("shape_bench needs a CUDA device")
    kv = importlib.import_module("int8-kvcache_b200")
    dev = torch.device("cuda:0")
    bs, hkv, d = a.block_size, a.kv_heads, a.head_dim
    per_seq = (a.seq + bs - 1) // bs
    nblk = per_seq * a.batch
    gen = torch.Generator(device=dev).manual_seed(1)
    caches = []
    for _ in range(a.caches):
        kc = torch.randint(-127, 128, (nblk, bs, hkv, d), device=dev, dtype=torch.int8, generator=gen)
        vc = torch.randint(-127, 128, (nblk, bs, hkv, d), device=dev, dtype=torch.int8, generator=gen)
        caches.append((kc, vc))
    bt = torch.arange(nblk, device=dev, dtype=torch.int32).view(a.batch, per_seq)
    sl = torch.full((a.batch,), a.seq, device=dev, dtype=torch.int32)
    q = torch.randn(a.batch, a.q_heads, d, device=dev, generator=gen).to(torch.bfloat16)
    ks = torch.full((hkv,), 0.02, device=dev)
    vs = torch.full((hkv,), 0.02, device=dev)
    out = torch.empty_like(q)

    def calls():
        for kc, vc in caches:
            kv.int8_paged_attention(q, kc, vc, bt, sl, ks, vs, max_seq_len=a.seq, out=out, num_splits=a.num_splits)

    stream = torch.cuda.Stream(dev)
    with torch.cuda.stream(stream):
        for _ in range(a.warmup):
            calls()
        stream.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(a.reps):
            calls()
        t1.record(stream)
        stream.synchronize()
    us = t0.elapsed_time(t1) * 1e3 / (a.reps * a.caches)
    nbytes = a.batch * a.seq * hkv * d * 2
    print(json.dumps({"shape": {"q_heads": a.q_heads, "kv_heads": hkv, "head_dim": d, "block_size": bs,
                                "batch": a.batch, "seq": a.seq}, "caches": a.caches, "num_splits": a.num_splits,
                      "us_per_call": round(us, 2), "bytes_per_call": nbytes, "gb_per_s": round(nbytes / us / 1e3, 1),
                      "device_status": kv.device_status()}))


if __name__ == "__main__":
    main()
