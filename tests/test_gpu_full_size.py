"""Full-size configurations through size-independent properties (the CPU oracle cannot attend over gigabytes in
seconds, so it checks a few sequences; the rest is invariance):

  * large ragged batch (B=256, seq ~ U[1024, 8192], one layer): sampled sequences against the oracle, and the
    result must not depend on the number of KV splits beyond rounding;
  * long context (B=32 x 65536 tokens, Hq=64, Hkv=8): cache tensors larger than 2 GiB, so block offsets need
    64 bits; the sequence whose blocks sit highest in the pool is checked against the oracle, and physical block
    placement must not matter: the same logical content in a differently permuted pool gives identical bits.
"""

import pytest
import torch

import oracle
from conftest import cosine, max_abs

pytestmark = pytest.mark.gpu


def _fill(kv, wl, shape, seq_lens, tables, num_blocks, seed, dev):
    kc = torch.zeros(num_blocks, 16, shape.num_kv_heads, 128, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    ks, vs = [t.to(dev) for t in wl.calibrate_scales(shape, seed)]
    gain = wl.channel_gain(shape, seed, dev)
    gen = torch.Generator(device=dev)
    bt = tables.to(dev)
    for b, T in enumerate(seq_lens):
        gen.manual_seed(seed * 100003 + b)  # content depends on the sequence only, not on its placement
        k, v = wl.draw_kv(T, shape, gen, gain)
        tok = torch.arange(T, device=dev)
        slots = bt[b, tok // 16].long() * 16 + tok % 16
        kv.int8_kv_cache_write(k, v, kc, vc, slots, ks, vs)
    return kc, vc, ks, vs


def _oracle_rows(q, kc, vc, tables, seq_lens, ks, vs, rows):
    out = {}
    for b in rows:
        T = seq_lens[b]
        ids = tables[b, : (T + 15) // 16].long().to(kc.device)
        k1, v1 = kc[ids].cpu(), vc[ids].cpu()  # this sequence's blocks only, renumbered 0..n-1
        bt1 = torch.arange(ids.numel(), dtype=torch.int32)[None]
        out[b] = oracle.int8_paged_attention_oracle(q[b : b + 1].cpu(), k1, v1, bt1, [T], ks.cpu(), vs.cpu())[0]
    return out


def test_large_ragged_batch(kv, workloads):
    dev = "cuda"
    shape = workloads.QWEN25_7B
    g = torch.Generator().manual_seed(1234)
    seq_lens = torch.randint(1024, 8193, (256,), generator=g).tolist()
    need = int(workloads.blocks_needed(seq_lens, 16).sum())
    num_blocks = need + 4096
    tables = workloads.permuted_block_tables(seq_lens, 16, num_blocks, seed=5)
    kc, vc, ks, vs = _fill(kv, workloads, shape, seq_lens, tables, num_blocks, 5, dev)
    q = workloads.draw_query(256, shape, torch.Generator().manual_seed(6)).to(dev)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=dev)
    bt = tables.to(dev)
    auto = kv.int8_paged_attention(q, kc, vc, bt, sl, ks, vs, max_seq_len=max(seq_lens))
    one = kv.int8_paged_attention(q, kc, vc, bt, sl, ks, vs, max_seq_len=max(seq_lens), num_splits=1)
    many = kv.int8_paged_attention(q, kc, vc, bt, sl, ks, vs, max_seq_len=max(seq_lens), num_splits=16)
    assert kv.device_status() == 0
    # peaked rows reach magnitudes of 2-4, where one bf16 ulp is already 0.016: the bound scales with the output
    bound = 2e-2 * max(1.0, float(auto.float().abs().max()))
    worst = 0.0
    for other in (one, many):
        worst = max(worst, max_abs(auto.float(), other.float()))
        assert max_abs(auto.float(), other.float()) <= bound and cosine(auto.float(), other.float()) >= 0.9999
    print(f"split invariance on the 256-sequence ragged batch: worst max-abs between split counts {worst:.4g} "
          f"(bound {bound:.4g}, largest |out| {float(auto.float().abs().max()):.4g})")
    rows = [0, 255, int(torch.tensor(seq_lens).argmax()), int(torch.tensor(seq_lens).argmin())]
    for b, want in _oracle_rows(q, kc, vc, tables, seq_lens, ks, vs, rows).items():
        got = auto[b].float().cpu()
        assert cosine(got, want) >= 0.9999 and max_abs(got, want.to(torch.bfloat16).float()) <= 2e-2


def test_long_context_beyond_2gib_and_placement_invariance(kv, workloads):
    dev = "cuda"
    shape = workloads.QWEN25_72B
    B, T = 32, 65536
    seq_lens = [T] * B
    num_blocks = B * T // 16 + 1024  # 132 096 blocks x 16 KB = 2.06 GiB per cache tensor
    assert num_blocks * 16 * shape.num_kv_heads * 128 > 2 ** 31
    q = workloads.draw_query(B, shape, torch.Generator().manual_seed(8)).to(dev)
    sl = torch.tensor(seq_lens, dtype=torch.int32, device=dev)
    outs = []
    for placement in (1, 2):
        tables = workloads.permuted_block_tables(seq_lens, 16, num_blocks, seed=placement)
        kc, vc, ks, vs = _fill(kv, workloads, shape, seq_lens, tables, num_blocks, 9, dev)
        out = kv.int8_paged_attention(q, kc, vc, tables.to(dev), sl, ks, vs, max_seq_len=T)
        assert kv.device_status() == 0
        outs.append(out)
        if placement == 1:
            high = int(tables.float().mean(dim=1).argmax())  # the sequence living highest in the pool
            assert int(tables[high].max()) * 16 * shape.num_kv_heads * 128 > 2 ** 31
            want = _oracle_rows(q, kc, vc, tables, seq_lens, ks, vs, [high])[high]
            got = out[high].float().cpu()
            assert cosine(got, want) >= 0.9999 and max_abs(got, want.to(torch.bfloat16).float()) <= 2e-2
        del kc, vc
        torch.cuda.empty_cache()
    assert torch.equal(outs[0], outs[1])
