"""Seeded random shapes through the whole device chain: the cache is written by the CUDA write kernel, attention
reads it, and both are held to the oracle — bit-exact cache bytes, attention within the path's tolerances.  Every
case draws its own batch, lengths, head layout, block size, dtypes, index widths, split mode and views."""

import random

import pytest
import torch

import oracle
from conftest import cosine, max_abs

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MIN_COS = 0.9999
HEADS = [(28, 4), (32, 8), (8, 1), (16, 2), (12, 4), (40, 8), (6, 6)]  # (Hq, Hkv): groups 7, 4, 8, 8, 3, 5, 1


def _draw(seed):
    r = random.Random(seed)
    hq, hkv = r.choice(HEADS)
    return dict(
        seed=seed, hq=hq, hkv=hkv,
        block_size=r.choice([16, 16, 32, 64]),
        lens=[r.choice([1, 2, 15, 16, 17, r.randint(1, 900), r.randint(1, 200)]) for _ in range(r.randint(1, 7))],
        q_dtype=r.choice([torch.bfloat16, torch.bfloat16, torch.float16, torch.float32]),
        kv_dtype=r.choice([torch.bfloat16, torch.float16, torch.float32]),
        wide_index=r.random() < 0.5,
        splits=r.choice([None, None, 1, 2, 3, 5, 16, "planned"]),
        strided_query=r.random() < 0.3,
        table_slack=r.randint(0, 3),
    )


@pytest.mark.parametrize("seed", range(24))
def test_write_then_attend_on_a_random_shape(kv, workloads, seed):
    c = _draw(1000 + seed)
    shape = workloads.LayerShape(c["hq"], c["hkv"], 128, c["block_size"])
    case = workloads.make_decode_case(c["lens"], shape, seed=c["seed"], dtype=c["kv_dtype"])
    bs, hkv = shape.block_size, shape.num_kv_heads
    dev = "cuda"
    # device write into a cache full of a canary, slots as the case maps them
    canary = 0x55
    kc = torch.full((case.num_blocks, bs, hkv, 128), canary, dtype=torch.int8, device=dev)
    vc = torch.full_like(kc, canary)
    slots = case.slot_mapping.to(torch.int64 if c["wide_index"] else torch.int32)
    kv.int8_kv_cache_write(case.key.to(dev), case.value.to(dev), kc, vc, slots.to(dev), case.k_scale.to(dev),
                           case.v_scale.to(dev))
    kc_o = torch.full((case.num_blocks, bs, hkv, 128), canary, dtype=torch.int8)
    vc_o = torch.full_like(kc_o, canary)
    oracle.cache_write(case.key, case.value, kc_o, vc_o, case.slot_mapping, case.k_scale, case.v_scale)
    assert torch.equal(kc.cpu(), kc_o) and torch.equal(vc.cpu(), vc_o)

    want = oracle.int8_paged_attention_oracle(case.query.float(), kc_o, vc_o, case.block_tables, c["lens"],
                                              case.k_scale, case.v_scale)
    # block table with unused columns of garbage to the right, optionally 64-bit; query optionally a strided view
    bt = case.block_tables
    if c["table_slack"]:
        junk = torch.full((bt.shape[0], c["table_slack"]), 2**30, dtype=bt.dtype)
        bt = torch.cat([bt, junk], dim=1)
    bt = bt.to(torch.int64 if c["wide_index"] else torch.int32).to(dev)
    sl = case.seq_lens.to(torch.int64 if c["wide_index"] else torch.int32).to(dev)
    q = case.query.to(c["q_dtype"]).to(dev)
    if c["strided_query"]:
        wide = torch.zeros(q.shape[0], q.shape[1], 256, dtype=q.dtype, device=dev)
        wide[:, :, 64:192] = q
        q = wide[:, :, 64:192]
    tiled = shape.group <= 8 and bs % 16 == 0
    splits = c["splits"] if (tiled or c["splits"] != "planned") else None
    out = kv.int8_paged_attention(q, kc, vc, bt, sl, case.k_scale.to(dev), case.v_scale.to(dev), num_splits=splits)
    assert out.dtype == c["q_dtype"] and out.shape == q.shape
    got = out.float().cpu()
    # the oracle saw the query in its original precision; a narrower query dtype is part of the operator's input
    want_q = oracle.int8_paged_attention_oracle(case.query.to(c["q_dtype"]).float(), kc_o, vc_o, case.block_tables,
                                                c["lens"], case.k_scale, case.v_scale)
    assert torch.isfinite(got).all()
    assert cosine(got, want_q) >= MIN_COS, c
    bound = MAX_ABS * max(1.0, float(want_q.abs().max()))
    assert max_abs(got, want_q.to(c["q_dtype"]).float()) <= bound, c
    assert cosine(got, want) >= 0.999
    assert kv.device_status() == 0
