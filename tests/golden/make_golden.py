"""Generate the golden fixtures in this directory by running the REFERENCE's own Python code.

Run it where the reference checkout is importable (it is pure PyTorch on CPU; the Triton kernels
are not launched):

    python tests/golden/make_golden.py --reference /path/to/Int8-kvcache

Every fixture stores the seeded inputs and what the reference's functions returned for them:
`src.quant.quant_kv_static_per_head`, `src.quant.dequant_kv_per_head`,
`src.paged_cache.make_paged_cache` / `gather_from_paged_cache`,
`src.attention_ref.decode_attention_ref`,
`src.triton_ops.int8_cache_write.torch_int8_kv_cache_write_reference`,
`src.triton_ops.int8_paged_attention.torch_int8_paged_attention_reference`, and the block-table /
slot-mapping helpers of the reference's tests.  bf16 tensors are stored as their uint16 bit patterns.
The fixtures are consumed by tests/test_oracle_golden.py (oracle vs reference) and by the GPU parity
tests (CUDA kernels vs the same vectors); nothing reads the reference at test time.
"""

from __future__ import annotations

import argparse
import importlib
import os
import random
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16/fp16 tensor -> uint16 bit pattern array."""
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def save(name: str, **arrays) -> None:
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = bits(v) if v.dtype in (torch.bfloat16, torch.float16) else v.contiguous().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(HERE / f"{name}.npz", **out)
    size = (HERE / f"{name}.npz").stat().st_size
    print(f"{name}.npz  {size / 1024:.1f} KB")


def chain_attention(ref, query, kc, vc, block_tables, seq_lens, k_scale, v_scale):
    """gather -> dequant -> decode_attention_ref with the reference's functions, one sequence at a time
    (its gather stacks sequences and therefore needs equal lengths)."""
    rows = []
    for b in range(query.shape[0]):
        k8, v8 = ref["gather"](kc, vc, block_tables[b : b + 1], seq_lens[b : b + 1])
        k = ref["dequant"](k8, k_scale.reshape(1, -1, 1, 1))
        v = ref["dequant"](v8, v_scale.reshape(1, -1, 1, 1))
        rows.append(ref["attn"](query[b : b + 1], k, v)[0])
    return torch.stack(rows)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("INT8KV_REFERENCE"),
                    help="checkout of cjsmt/Int8-kvcache to import (or set INT8KV_REFERENCE)")
    args = ap.parse_args()
    if not args.reference:
        ap.error("--reference (or INT8KV_REFERENCE) must name a checkout of the reference")
    sys.path.insert(0, args.reference)
    sys.path.insert(0, str(REPO))
    quant = importlib.import_module("src.quant")
    paged = importlib.import_module("src.paged_cache")
    attn = importlib.import_module("src.attention_ref")
    wr = importlib.import_module("src.triton_ops.int8_cache_write")
    pa = importlib.import_module("src.triton_ops.int8_paged_attention")
    rtests = importlib.import_module("tests.test_int8_paged_attention")
    ref = {"gather": paged.gather_from_paged_cache, "dequant": quant.dequant_kv_per_head,
           "attn": attn.decode_attention_ref}
    workloads = importlib.import_module("int8-kvcache_b200.workloads")

    # 1. cache write, T=37, fixed scales, gapped slots (tests/test_cache_write.py)
    torch.manual_seed(41)
    key = torch.randn(37, 4, 128, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    k_scale = torch.tensor([0.03, 0.025, 0.04, 0.035])
    v_scale = torch.tensor([0.035, 0.03, 0.025, 0.04])
    slots = torch.tensor(list(range(16, 32)) + list(range(64, 80)) + list(range(96, 101)), dtype=torch.int64)[:37]
    kc = torch.zeros(8, 16, 4, 128, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    wr.torch_int8_kv_cache_write_reference(key, value, kc, vc, slots, k_scale, v_scale)
    kq = quant.quant_kv_static_per_head(key.permute(1, 0, 2)[None], k_scale.reshape(1, 4, 1, 1))
    save("write_t37", key=key, value=value, k_scale=k_scale, v_scale=v_scale, slot_mapping=slots,
         key_cache=kc, value_cache=vc, key_q_static=kq)

    # 2. runtime cache write, N=23, slots 7..29 crossing a block boundary (tests/test_runtime_cache_write.py)
    torch.manual_seed(0)
    key = torch.randn(23, 4, 128, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    k_scale = (key.float().abs().amax(dim=(0, 2)) / 127).clamp_min(1e-6)
    v_scale = (value.float().abs().amax(dim=(0, 2)) / 127).clamp_min(1e-6)
    slots = torch.arange(7, 30, dtype=torch.long)
    kc = torch.zeros(16, 16, 4, 128, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    wr.torch_int8_kv_cache_write_reference(key, value, kc, vc, slots, k_scale, v_scale)
    save("write_n23", key=key, value=value, k_scale=k_scale, v_scale=v_scale, slot_mapping=slots,
         key_cache=kc, value_cache=vc)

    # 3./4. write + attention on ragged sequences (tests/test_int8_paged_attention.py:107-323)
    for name, seed, seq_lens_list, pool in (("attn_127_301", 0, [127, 301], None), ("attn_97_256", 1, [97, 256], 512)):
        torch.manual_seed(seed)
        random.seed(seed)
        B, Hq, Hkv, D, bs = 2, 28, 4, 128, 16
        query = torch.randn(B, Hq, D, dtype=torch.bfloat16)
        keys, values = [], []
        for T in seq_lens_list:
            keys.append(torch.randn(T, Hkv, D, dtype=torch.bfloat16))
            values.append(torch.randn_like(keys[-1]))
        all_k, all_v = torch.cat(keys).float(), torch.cat(values).float()
        k_scale = (all_k.abs().amax(dim=(0, 2)) / 127.0).clamp_min(1e-6)
        v_scale = (all_v.abs().amax(dim=(0, 2)) / 127.0).clamp_min(1e-6)
        need = sum((x + bs - 1) // bs for x in seq_lens_list)
        num_blocks = pool if pool else need + 20
        tables = rtests.create_random_block_tables(B, seq_lens_list, bs, num_blocks, "cpu")
        seq_lens = torch.tensor(seq_lens_list, dtype=torch.int32)
        slots = rtests.build_slot_mapping(tables, seq_lens_list, bs)
        kc = torch.zeros(num_blocks, bs, Hkv, D, dtype=torch.int8)
        vc = torch.zeros_like(kc)
        wr.torch_int8_kv_cache_write_reference(torch.cat(keys), torch.cat(values), kc, vc, slots, k_scale, v_scale)
        out_loop = pa.torch_int8_paged_attention_reference(query, kc, vc, tables, seq_lens, k_scale, v_scale)
        out_loop_qq = pa.torch_int8_paged_attention_reference(query, kc, vc, tables, seq_lens, k_scale, v_scale,
                                                              quantize_q=True)
        out_chain = chain_attention(ref, query, kc, vc, tables, seq_lens, k_scale, v_scale)
        out_bf16 = rtests.torch_bf16_attention_reference(query, keys, values)
        save(name, query=query, key=torch.cat(keys), value=torch.cat(values), k_scale=k_scale, v_scale=v_scale,
             block_tables=tables, seq_lens=seq_lens, slot_mapping=slots, key_cache=kc, value_cache=vc,
             out_loop_bf16=out_loop, out_loop_quantize_q_bf16=out_loop_qq, out_chain_f32=out_chain,
             out_unquantised_bf16=out_bf16)

    # 5. config 1: B=1, 512 context tokens + 1 written token, outlier keys, calibrated scales, 64-block pool
    case = workloads.config1_case(seed=0)
    sh = case.shape
    k_ctx = case.key[:512].permute(1, 0, 2)[None]  # [1, Hkv, 512, D]
    v_ctx = case.value[:512].permute(1, 0, 2)[None]
    k8 = quant.quant_kv_static_per_head(k_ctx, case.k_scale.reshape(1, -1, 1, 1))
    v8 = quant.quant_kv_static_per_head(v_ctx, case.v_scale.reshape(1, -1, 1, 1))
    kc_seq, vc_seq, bt_seq, _ = paged.make_paged_cache(k8, v8, sh.block_size)  # 32 blocks in order
    kc = torch.zeros(case.num_blocks, sh.block_size, sh.num_kv_heads, sh.head_dim, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    ids = case.block_tables[0, :32].long()
    kc[ids] = kc_seq
    vc[ids] = vc_seq
    out_512 = chain_attention(ref, case.query, kc, vc, case.block_tables, torch.tensor([512]), case.k_scale, case.v_scale)
    wr.torch_int8_kv_cache_write_reference(case.key[512:], case.value[512:], kc, vc, case.slot_mapping[512:],
                                           case.k_scale, case.v_scale)
    out_513 = chain_attention(ref, case.query, kc, vc, case.block_tables, torch.tensor([513]), case.k_scale, case.v_scale)
    save("config1", query=case.query, key=case.key, value=case.value, k_scale=case.k_scale, v_scale=case.v_scale,
         block_tables=case.block_tables, slot_mapping=case.slot_mapping, key_cache=kc, value_cache=vc,
         out_ctx512_f32=out_512, out_ctx513_f32=out_513)

    # 6. paged layout identity (tests/test_paged_cache.py), on int8 payloads to keep the file small
    g = torch.Generator().manual_seed(5)
    k = torch.randint(-127, 128, (2, 4, 127, 128), generator=g, dtype=torch.int8)
    v = torch.randint(-127, 128, (2, 4, 127, 128), generator=g, dtype=torch.int8)
    kc, vc, bt, sl = paged.make_paged_cache(k, v, 16)
    k2, v2 = paged.gather_from_paged_cache(kc, vc, bt, sl)
    assert torch.equal(k, k2) and torch.equal(v, v2)
    save("paged_layout", k=k, v=v, key_cache=kc, value_cache=vc, block_tables=bt, seq_lens=sl)

    # 7. real activations: layer 27 of the reference's K/V sample with its calibrated static scales
    scales = torch.load(os.path.join(args.reference, "outputs/static_per_head_scales.pt"))
    sample = torch.load(os.path.join(args.reference, "outputs/kv_sample.pt"))
    k = sample[27]["k"]  # [4 prompts, Hkv, 10, D] fp16
    v = sample[27]["v"]
    ks, vs = scales["k_scale"][27], scales["v_scale"][27]
    kq = quant.quant_kv_static_per_head(k, ks.reshape(1, -1, 1, 1))
    vq = quant.quant_kv_static_per_head(v, vs.reshape(1, -1, 1, 1))
    save("real_layer27", k=k, v=v, k_scale=ks, v_scale=vs, k_q=kq, v_q=vq,
         all_k_scale=scales["k_scale"], all_v_scale=scales["v_scale"])


if __name__ == "__main__":
    main()
