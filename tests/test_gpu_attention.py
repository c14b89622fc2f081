"""GPU parity of INT8 paged decode attention and of the BF16 baseline, through the C ABI.

Bars: max-abs <= 2e-2 against the reference's result in bf16, cosine >= 0.9999 against the fp32
dequantise-then-attend oracle."""

import math

import pytest
import torch

import oracle
from conftest import cosine, load_golden, max_abs

pytestmark = pytest.mark.gpu
MAX_ABS = 2e-2
MIN_COS = 0.9999


def _dev(*ts):
    return [t.cuda() for t in ts]


def _check(out, want_f32, want_bf16=None):
    out = out.float().cpu()
    assert torch.isfinite(out).all()
    assert cosine(out, want_f32) >= MIN_COS
    ref = want_f32.to(torch.bfloat16).float() if want_bf16 is None else want_bf16.float()
    assert max_abs(out, ref) <= MAX_ABS


def _run_int8(kv, g, seq_lens=None, **kw):
    q, kc, vc, bt, ks, vs = _dev(g["query"], g["key_cache"], g["value_cache"], g["block_tables"], g["k_scale"], g["v_scale"])
    sl = (g["seq_lens"] if seq_lens is None else torch.tensor(seq_lens, dtype=torch.int32)).cuda()
    out = kv.int8_paged_attention(q, kc, vc, bt, sl, ks, vs, **kw)
    torch.cuda.synchronize()
    assert kv.device_status() == 0
    return out


@pytest.mark.parametrize("name", ["attn_127_301", "attn_97_256"])
@pytest.mark.parametrize("splits", [None, 1, 2, 4, 7, 64])
def test_golden_cases(kv, name, splits):
    g = load_golden(name)
    out = _run_int8(kv, g, num_splits=splits)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (2, 28, 128)
    _check(out, g["out_chain_f32"], g["out_loop_bf16"])


@pytest.mark.parametrize("impl", ["auto", "v3", "v4"])
def test_impl_names_are_accepted(kv, impl):
    g = load_golden("attn_97_256")
    _check(_run_int8(kv, g, impl=impl), g["out_chain_f32"], g["out_loop_bf16"])


def test_unknown_impl_raises(kv):
    g = load_golden("attn_97_256")
    with pytest.raises(ValueError):
        _run_int8(kv, g, impl="v5")


def test_config1_before_and_after_the_written_token(kv):
    g = load_golden("config1")
    dev = "cuda"
    kc = torch.zeros(g["key_cache"].shape, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    ks, vs, slots = g["k_scale"].cuda(), g["v_scale"].cuda(), g["slot_mapping"].cuda()
    key, value = g["key"].cuda(), g["value"].cuda()
    kv.int8_kv_cache_write(key[:512], value[:512], kc, vc, slots[:512], ks, vs)
    q, bt = g["query"].cuda(), g["block_tables"].cuda()
    out512 = kv.int8_paged_attention(q, kc, vc, bt, torch.tensor([512], dtype=torch.int32, device=dev), ks, vs)
    _check(out512, g["out_ctx512_f32"])
    kv.int8_kv_cache_write(key[512:], value[512:], kc, vc, slots[512:], ks, vs)
    assert torch.equal(kc.cpu(), g["key_cache"]) and torch.equal(vc.cpu(), g["value_cache"])
    out513 = kv.int8_paged_attention(q, kc, vc, bt, torch.tensor([513], dtype=torch.int32, device=dev), ks, vs)
    _check(out513, g["out_ctx513_f32"])


def _case_on_gpu(kv, workloads, seq_lens, shape=None, seed=0, **kw):
    case = workloads.make_decode_case(seq_lens, shape or workloads.QWEN25_7B, seed=seed, **kw)
    sh = case.shape
    kc = torch.zeros(case.num_blocks, sh.block_size, sh.num_kv_heads, sh.head_dim, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
    return case, kc, vc


def test_every_length_1_to_48_and_every_split(kv, workloads):
    """Ragged tails, single-token sequences, splits that end up empty."""
    lens = list(range(1, 49))
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=2)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    q, kcd, vcd, bt, sl, ks, vs = _dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    for splits in (None, 1, 2, 3, 5):
        out = kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs, num_splits=splits)
        _check(out, want)
    assert kv.device_status() == 0


@pytest.mark.parametrize("B,seq", [(1, 512), (2, 1024), (4, 2048), (8, 4096)])
def test_sweep_cells_int8_and_bf16_baseline(kv, workloads, B, seq):
    case, kc, vc = _case_on_gpu(kv, workloads, [seq] * B, seed=B)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, [seq] * B, case.k_scale, case.v_scale)
    q, kcd, vcd, bt, sl, ks, vs = _dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    out = kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs)
    _check(out, want)
    # determinism: same launch twice gives the same bits
    out2 = kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs)
    assert torch.equal(out, out2)
    # BF16 baseline on the un-quantised cache with identical block tables
    sh = case.shape
    kb = torch.zeros(case.num_blocks, sh.block_size, sh.num_kv_heads, sh.head_dim, dtype=torch.bfloat16)
    vb = torch.zeros_like(kb)
    s = case.slot_mapping
    kb[s // 16, s % 16] = case.key
    vb[s // 16, s % 16] = case.value
    want_b = oracle.float_paged_attention_oracle(case.query, kb, vb, case.block_tables, [seq] * B)
    bf = package_bf16(kv)(q, kb.cuda(), vb.cuda(), bt, sl)
    _check(bf, want_b)
    assert kv.device_status() == 0


def package_bf16(kv):
    return kv.bf16_paged_attention


def test_bf16_baseline_ragged_with_nan_padding(kv, workloads):
    """Rows past seq_len in the last block may hold anything, NaN included; they must not leak."""
    lens = [1, 15, 16, 17, 100, 333]
    case = workloads.make_decode_case(lens, seed=4)
    sh = case.shape
    for dtype in (torch.bfloat16, torch.float16):
        kb = torch.full((case.num_blocks, 16, sh.num_kv_heads, sh.head_dim), float("nan"), dtype=dtype)
        vb = torch.full_like(kb, float("nan"))
        s = case.slot_mapping
        kb[s // 16, s % 16] = case.key.to(dtype)
        vb[s // 16, s % 16] = case.value.to(dtype)
        want = oracle.float_paged_attention_oracle(case.query, kb, vb, case.block_tables, lens)
        for splits in (None, 1, 3):
            out = kv.bf16_paged_attention(case.query.cuda(), kb.cuda(), vb.cuda(), case.block_tables.cuda(),
                                          case.seq_lens.cuda(), num_splits=splits)
            _check(out, want)


@pytest.mark.parametrize("qdtype", [torch.float16, torch.float32])
def test_query_dtypes_int64_tables_and_views(kv, workloads, qdtype):
    lens = [77, 513, 260]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=6)
    q = case.query.to(qdtype)
    want = oracle.int8_paged_attention_oracle(q, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    # query as a non-owning slice of a padded buffer, int64 tables wider than needed with garbage beyond the end
    padded = torch.zeros(8, 28, 128, dtype=qdtype, device="cuda")
    padded[:3] = q.cuda()
    wide = torch.full((3, case.block_tables.shape[1] + 9), 10 ** 6, dtype=torch.int64)
    for b, T in enumerate(lens):
        n = (T + 15) // 16
        wide[b, :n] = case.block_tables[b, :n]
    out = kv.int8_paged_attention(padded[:3], kc.cuda(), vc.cuda(), wide.cuda(), case.seq_lens.to(torch.int64).cuda(),
                                  case.k_scale.double().cuda(), case.v_scale.double().cuda())
    assert out.dtype == qdtype
    out_f = out.float().cpu()
    assert cosine(out_f, want) >= MIN_COS and max_abs(out_f, want) <= MAX_ABS
    assert kv.device_status() == 0


def test_generic_path_shapes(kv, workloads):
    """Shapes outside the tiled kernels: head_dim 64, block size 8, GQA group 16, MHA."""
    for (hq, hkv, d, bs) in [(8, 2, 64, 8), (32, 2, 128, 16), (4, 4, 96, 16)]:
        shape = workloads.LayerShape(hq, hkv, d, bs)
        lens = [5, 64, 131]
        case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=hq)
        want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
        for splits in (None, 1, 3):
            out = kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, case.seq_lens,
                                                case.k_scale, case.v_scale), num_splits=splits)
            _check(out, want)
    # the per-query-head kernel: a group of 17, a head_dim that is not a multiple of 4
    for (hq, hkv, d, bs) in [(34, 2, 128, 16), (4, 2, 66, 16)]:
        shape = workloads.LayerShape(hq, hkv, d, bs)
        lens = [5, 64, 131]
        case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=hq)
        want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
        for splits in (None, 2):
            _check(kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, case.seq_lens,
                                                 case.k_scale, case.v_scale), num_splits=splits), want)
    # the grouped kernel on rows that are not 4-byte aligned (a view into a wider cache), with the INT8 query
    # option, and the 16-bit baseline on a head_dim of 64
    shape = workloads.LayerShape(8, 2, 64, 16)
    lens = [70, 9, 200]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=77)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    wide_k = torch.zeros(kc.shape[0], 16, 2, 66, dtype=torch.int8, device="cuda")
    wide_v = torch.zeros_like(wide_k)
    wide_k[..., 1:65], wide_v[..., 1:65] = kc.cuda(), vc.cuda()
    q, bt, sl, ks, vs = _dev(case.query, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    _check(kv.int8_paged_attention(q, wide_k[..., 1:65], wide_v[..., 1:65], bt, sl, ks, vs), want)
    wantq = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale,
                                               quantize_q=True)
    _check(kv.int8_paged_attention(q, kc.cuda(), vc.cuda(), bt, sl, ks, vs, quantize_q=True), wantq)
    kb = torch.zeros(case.num_blocks, 16, 2, 64, dtype=torch.bfloat16)
    vb = torch.zeros_like(kb)
    s_ = case.slot_mapping
    kb[s_ // 16, s_ % 16], vb[s_ // 16, s_ % 16] = case.key, case.value
    _check(kv.bf16_paged_attention(q, kb.cuda(), vb.cuda(), bt, sl),
           oracle.float_paged_attention_oracle(case.query, kb, vb, case.block_tables, lens))
    assert kv.device_status() == 0


@pytest.mark.parametrize("hq,hkv,d,bs", [
    (14, 2, 128, 8),    # group 7 on a block size the tiled kernels do not take
    (14, 2, 64, 16),    # group 7, two tokens per V load
    (32, 2, 64, 16),    # group 16, two tokens per V load
    (8, 2, 256, 16),    # eight dims per lane
    (16, 2, 256, 16),   # group 8 with eight dims per lane
    (4, 2, 132, 16),    # head_dim % 8 == 4 and % 16 != 0: word K loads, byte V loads
    (4, 2, 32, 16),     # half of the lanes idle in P.V
    (2, 1, 16, 16),     # one K load per row
    (8, 2, 64, 24),     # block sizes that do not divide a 32-token step
    (8, 2, 64, 5),
    (8, 2, 96, 48),
])
def test_grouped_kernel_variants(kv, workloads, hq, hkv, d, bs):
    """Every instantiation and lane layout of the kernel that serves INT8 caches outside the tiled shapes, over
    ragged lengths (a part that ends inside a step, a one-token sequence) and several split counts."""
    shape = workloads.LayerShape(hq, hkv, d, bs)
    lens = [1, 5, 64, 131, 300]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=hq + d + bs)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    args = _dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    for splits in (None, 1, 3, 16):
        _check(kv.int8_paged_attention(*args, num_splits=splits), want)
    assert kv.device_status() == 0


def test_larger_block_size_and_group_of_8(kv, workloads):
    shape = workloads.LayerShape(64, 8, 128, 32)  # 72B-style GQA 8:1, 32-token blocks
    lens = [31, 32, 33, 700]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=8)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    for splits in (None, 1, 4):
        out = kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, case.seq_lens,
                                            case.k_scale, case.v_scale), num_splits=splits)
        _check(out, want)
    assert kv.device_status() == 0


@pytest.mark.parametrize("name", ["attn_127_301", "attn_97_256"])
def test_quantize_q_matches_the_reference_vectors(kv, name):
    """quantize_q=True against what the reference's own loop returned for it on the golden cases (generated by
    tests/golden/make_golden.py from src/triton_ops/int8_paged_attention.py:776-814), for the automatic split and
    forced ones, and against the oracle's restatement on a seeded case."""
    g = load_golden(name)
    want = oracle.int8_paged_attention_oracle(g["query"], g["key_cache"], g["value_cache"], g["block_tables"],
                                              g["seq_lens"].tolist(), g["k_scale"], g["v_scale"], quantize_q=True)
    for splits in (None, 1, 4):
        out = _run_int8(kv, g, quantize_q=True, num_splits=splits)
        _check(out, want, g["out_loop_quantize_q_bf16"])


def test_quantize_q_on_a_seeded_case(kv, workloads):
    lens = [200, 45]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=10)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale,
                                              quantize_q=True)
    out = kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, case.seq_lens,
                                        case.k_scale, case.v_scale), quantize_q=True)
    _check(out, want)


def test_max_seq_len_hint_skips_validation_and_zero_length_is_safe(kv, workloads):
    lens = [40, 0, 17]
    case = workloads.make_decode_case([40, 1, 17], seed=12)
    sh = case.shape
    kc = torch.zeros(case.num_blocks, 16, sh.num_kv_heads, sh.head_dim, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
    sl = torch.tensor(lens, dtype=torch.int32)
    out = kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, sl, case.k_scale, case.v_scale),
                                  max_seq_len=48)
    out = out.float().cpu()
    assert torch.isfinite(out).all() and float(out[1].abs().max()) == 0.0
    want = oracle.int8_paged_attention_oracle(case.query[[0, 2]], kc, vc, case.block_tables[[0, 2]], [40, 17],
                                              case.k_scale, case.v_scale)
    assert cosine(out[[0, 2]], want) >= MIN_COS
    with pytest.raises(AssertionError):  # the reference's host check: every seq_len > 0
        kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, sl, case.k_scale, case.v_scale))


def test_partial_rows_and_merge_reproduce_a_sequence_split(kv, workloads):
    """Each 'rank' holds a contiguous range of every sequence's blocks in its own local cache; partial rows
    merged on one device must equal attention over the whole sequence."""
    lens = [1000, 333, 64]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=14)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    R = 4
    per_rank_blocks = 16  # rank r owns logical blocks [16r, 16r+16)
    parts = []
    for r in range(R):
        lo = r * per_rank_blocks
        local_bt = case.block_tables[:, lo : lo + per_rank_blocks].contiguous()
        local_len = torch.tensor([max(0, min(T - lo * 16, per_rank_blocks * 16)) for T in lens], dtype=torch.int32)
        if local_bt.shape[1] == 0:
            local_bt = torch.zeros(len(lens), 1, dtype=torch.int32)
        parts.append(kv.int8_paged_attention_partial(*_dev(case.query, kc, vc, local_bt, local_len,
                                                           case.k_scale, case.v_scale)))
    merged = kv.merge_partials(torch.stack(parts).contiguous(), 128, dtype=torch.bfloat16)
    _check(merged, want)
    assert kv.device_status() == 0


def test_decode_step_equals_write_then_attend(kv, workloads):
    lens = [513, 97, 1030, 16]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=16)
    dev = "cuda"
    last = torch.tensor([sum(lens[: b + 1]) - 1 for b in range(len(lens))])
    # caches hold everything but each sequence's last token
    kc0, vc0 = torch.zeros_like(kc), torch.zeros_like(vc)
    keep = torch.ones(sum(lens), dtype=torch.bool)
    keep[last] = False
    oracle.cache_write(case.key[keep], case.value[keep], kc0, vc0, case.slot_mapping[keep], case.k_scale, case.v_scale)
    kcd, vcd = kc0.to(dev), vc0.to(dev)
    out = kv.int8_decode_step(case.query.to(dev), case.key[last].to(dev), case.value[last].to(dev), kcd, vcd,
                              case.slot_mapping[last].to(dev), case.block_tables.to(dev), case.seq_lens.to(dev),
                              case.k_scale.to(dev), case.v_scale.to(dev), max_seq_len=max(lens))
    assert torch.equal(kcd.cpu(), kc) and torch.equal(vcd.cpu(), vc)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    _check(out, want)
    two = kv.int8_paged_attention(*_dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale))
    assert torch.equal(out, two)
    assert kv.device_status() == 0
    # every split count, fp16 new rows, int32 slots, a padding row (slot -1: nothing written, attention unchanged)
    for splits in (1, 2, 8):
        kcd, vcd = kc0.to(dev), vc0.to(dev)
        slots = case.slot_mapping[last].to(torch.int32)
        slots[3] = -1
        out = kv.int8_decode_step(case.query.to(dev), case.key[last].half().to(dev), case.value[last].half().to(dev),
                                  kcd, vcd, slots.to(dev), case.block_tables.to(dev), case.seq_lens.to(dev),
                                  case.k_scale.to(dev), case.v_scale.to(dev), max_seq_len=max(lens), num_splits=splits)
        kc_e, vc_e = kc.clone(), vc.clone()
        s3 = int(case.slot_mapping[last][3])
        kc_e[s3 // 16, s3 % 16], vc_e[s3 // 16, s3 % 16] = kc0[s3 // 16, s3 % 16], vc0[s3 // 16, s3 % 16]
        assert torch.equal(kcd.cpu(), kc_e) and torch.equal(vcd.cpu(), vc_e)
        _check(out[:3], want[:3])
    assert kv.device_status() == 0
    # a slot that is not the last token's is written all the same, and reported
    kcd, vcd = kc0.to(dev), vc0.to(dev)
    wrong = case.slot_mapping[last].clone()
    wrong[0] = int(case.slot_mapping[5])
    kv.int8_decode_step(case.query.to(dev), case.key[last].to(dev), case.value[last].to(dev), kcd, vcd, wrong.to(dev),
                        case.block_tables.to(dev), case.seq_lens.to(dev), case.k_scale.to(dev), case.v_scale.to(dev),
                        max_seq_len=max(lens))
    torch.cuda.synchronize()
    s5 = int(case.slot_mapping[5])
    q_last = oracle.static_quant_per_head(case.key[last][0:1], case.k_scale, head_axis=1)[0]
    assert torch.equal(kcd.cpu()[s5 // 16, s5 % 16], q_last)
    assert kv.device_status() == 2
    # shapes outside the tiled kernel take the two-call form behind the same entry point
    shape = workloads.LayerShape(8, 2, 64, 8)
    lens2 = [33, 9]
    c2 = workloads.make_decode_case(lens2, shape, seed=3)
    k2 = torch.zeros(c2.num_blocks, 8, 2, 64, dtype=torch.int8)
    v2 = torch.zeros_like(k2)
    last2 = torch.tensor([32, 41])
    keep2 = torch.ones(42, dtype=torch.bool)
    keep2[last2] = False
    oracle.cache_write(c2.key[keep2], c2.value[keep2], k2, v2, c2.slot_mapping[keep2], c2.k_scale, c2.v_scale)
    k2d, v2d = k2.to(dev), v2.to(dev)
    o2 = kv.int8_decode_step(c2.query.to(dev), c2.key[last2].to(dev), c2.value[last2].to(dev), k2d, v2d,
                             c2.slot_mapping[last2].to(dev), c2.block_tables.to(dev), c2.seq_lens.to(dev),
                             c2.k_scale.to(dev), c2.v_scale.to(dev), max_seq_len=33)
    oracle.cache_write(c2.key[last2], c2.value[last2], k2, v2, c2.slot_mapping[last2], c2.k_scale, c2.v_scale)
    assert torch.equal(k2d.cpu(), k2) and torch.equal(v2d.cpu(), v2)
    _check(o2, oracle.int8_paged_attention_oracle(c2.query, k2, v2, c2.block_tables, lens2, c2.k_scale, c2.v_scale))


def test_decode_step_layers_equals_per_layer_calls(kv, workloads):
    """The L-layer entry point computes, layer by layer, exactly what L single-layer calls compute."""
    lens = [513, 97, 1030, 16]
    dev = "cuda"
    L = 3
    last = torch.tensor([sum(lens[: b + 1]) - 1 for b in range(len(lens))])
    keep = torch.ones(sum(lens), dtype=torch.bool)
    keep[last] = False
    cases, full, start = [], [], []
    c0 = workloads.make_decode_case(lens, workloads.QWEN25_7B, seed=40)
    for l in range(L):  # every layer shares one block table and slot mapping, as in a model
        case = workloads.make_decode_case(lens, workloads.QWEN25_7B, seed=40 + l)
        kc = torch.zeros(c0.num_blocks, 16, 4, 128, dtype=torch.int8)
        vc, kc0, vc0 = torch.zeros_like(kc), torch.zeros_like(kc), torch.zeros_like(kc)
        oracle.cache_write(case.key, case.value, kc, vc, c0.slot_mapping, case.k_scale, case.v_scale)
        oracle.cache_write(case.key[keep], case.value[keep], kc0, vc0, c0.slot_mapping[keep], case.k_scale, case.v_scale)
        cases.append(case), full.append((kc, vc)), start.append((kc0, vc0))
    bt, sl, slots = c0.block_tables.to(dev), c0.seq_lens.to(dev), c0.slot_mapping[last].to(dev)
    queries = torch.stack([c.query for c in cases]).to(dev)
    keys = torch.stack([c.key[last] for c in cases]).to(dev)
    values = torch.stack([c.value[last] for c in cases]).to(dev)
    kcs = [s[0].to(dev) for s in start]
    vcs = [s[1].to(dev) for s in start]
    kscales = torch.stack([c.k_scale for c in cases]).to(dev)
    vscales = torch.stack([c.v_scale for c in cases]).to(dev)
    out = kv.int8_decode_step_layers(queries, keys, values, kcs, vcs, slots, bt, sl, kscales, vscales, max_seq_len=max(lens))
    assert out.shape == (L, len(lens), 28, 128)
    for l in range(L):
        assert torch.equal(kcs[l].cpu(), full[l][0]) and torch.equal(vcs[l].cpu(), full[l][1])
        kcd, vcd = start[l][0].to(dev), start[l][1].to(dev)
        one = kv.int8_decode_step(queries[l], keys[l], values[l], kcd, vcd, slots, bt, sl, kscales[l], vscales[l],
                                  max_seq_len=max(lens))
        assert torch.equal(out[l], one)
        _check(out[l], oracle.int8_paged_attention_oracle(cases[l].query, full[l][0], full[l][1], c0.block_tables, lens,
                                                          cases[l].k_scale, cases[l].v_scale))
    # attention only (no new rows): lists of tensors, preallocated output, explicit split count
    pre = torch.empty(L, len(lens), 28, 128, dtype=torch.bfloat16, device=dev)
    got = kv.int8_decode_step_layers([q for q in queries], None, None, kcs, vcs, None, bt, sl, [k for k in kscales],
                                     [v for v in vscales], max_seq_len=max(lens), num_splits=4, out=pre)
    assert got is pre
    for l in range(L):
        one = kv.int8_paged_attention(queries[l], kcs[l], vcs[l], bt, sl, kscales[l], vscales[l], num_splits=4,
                                      max_seq_len=max(lens))
        assert torch.equal(pre[l], one)
    assert kv.device_status() == 0
    # a layer that fails is named
    bad = [k for k in kcs]
    bad[1] = kcs[1][:, :, :, :64]  # not the shape of layer 0
    with pytest.raises(AssertionError):
        kv.int8_decode_step_layers(queries, None, None, bad, vcs, None, bt, sl, kscales, vscales, max_seq_len=max(lens))


def test_inputs_ready_promise_changes_timing_not_results(kv, workloads):
    """A chain of calls that carry the inputs-ready promise (each starts reading while the previous call's merge is
    still running, and orders itself behind it only before its first write) returns bit for bit what the fully ordered
    chain returns: INT8 with fixed, automatic and device-planned splits, the BF16 baseline, the fused decode step and
    the L-layer entry point, launched eagerly and replayed as a CUDA graph.  All inputs are resident before the
    chain starts and every call has its own cache and output, which is what the promise asks for."""
    dev = "cuda"
    lens = [700, 45, 260, 1, 2048, 130]
    layers = []
    for li in range(6):
        case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=50 + li)
        kb = torch.zeros(case.num_blocks, 16, 4, 128, dtype=torch.bfloat16)
        vb = torch.zeros_like(kb)
        s_ = case.slot_mapping
        kb[s_ // 16, s_ % 16], vb[s_ // 16, s_ % 16] = case.key, case.value
        layers.append(dict(case=case, q=case.query.to(dev), kc=kc.to(dev), vc=vc.to(dev), kb=kb.to(dev), vb=vb.to(dev),
                           bt=case.block_tables.to(dev), sl=case.seq_lens.to(dev), ks=case.k_scale.to(dev),
                           vs=case.v_scale.to(dev)))
    mx = max(lens)
    split_modes = [None, 1, 4, "planned", 16, None]

    def chain(ready, outs):
        for i, (L, sp) in enumerate(zip(layers, split_modes)):
            kv.int8_paged_attention(L["q"], L["kc"], L["vc"], L["bt"], L["sl"], L["ks"], L["vs"], num_splits=sp,
                                    max_seq_len=mx, out=outs[0][i], inputs_ready=ready)
        for i, (L, sp) in enumerate(zip(layers, split_modes)):
            kv.bf16_paged_attention(L["q"], L["kb"], L["vb"], L["bt"], L["sl"], num_splits=sp, max_seq_len=mx,
                                    out=outs[1][i], inputs_ready=ready)

    def fresh():
        return [torch.full((6, len(lens), 28, 128), float("nan"), dtype=torch.bfloat16, device=dev) for _ in range(2)]

    want = fresh()
    chain(False, want)
    torch.cuda.synchronize()
    for L, o in zip(layers, want[0]):
        c = L["case"]
        _check(o, oracle.int8_paged_attention_oracle(c.query, L["kc"].cpu(), L["vc"].cpu(), c.block_tables, lens,
                                                     c.k_scale, c.v_scale))
    got = fresh()
    for _ in range(3):  # back to back, so that calls really overlap their predecessors
        chain(True, got)
    torch.cuda.synchronize()
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    # the same chain replayed as a CUDA graph
    got2 = fresh()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        chain(True, got2)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            chain(True, got2)
        for o in got2:
            o.fill_(float("nan"))
        for _ in range(3):
            g.replay()
        stream.synchronize()
    assert torch.equal(got2[0], want[0]) and torch.equal(got2[1], want[1])
    del g
    # fused decode step per layer and the L-layer entry point: the new rows rewrite each sequence's last token
    last = torch.tensor([sum(lens[: b + 1]) - 1 for b in range(len(lens))])
    c0 = layers[0]["case"]
    slots = c0.slot_mapping[last].to(dev)

    def step_chain(ready, outs, caches):
        for i, L in enumerate(layers):
            c = L["case"]
            kv.int8_decode_step(L["q"], c.key[last].to(dev), c.value[last].to(dev), caches[i][0], caches[i][1],
                                c.slot_mapping[last].to(dev), L["bt"], L["sl"], L["ks"], L["vs"], max_seq_len=mx,
                                out=outs[i], inputs_ready=ready and i > 0)

    caches_a = [(L["kc"].clone(), L["vc"].clone()) for L in layers]
    caches_b = [(L["kc"].clone(), L["vc"].clone()) for L in layers]
    wa, wb = fresh()[0], fresh()[0]
    step_chain(False, wa, caches_a)
    for _ in range(2):
        step_chain(True, wb, caches_b)
    torch.cuda.synchronize()
    assert torch.equal(wa, wb)
    for (ka, va), (kb_, vb_) in zip(caches_a, caches_b):
        assert torch.equal(ka, kb_) and torch.equal(va, vb_)
    # L layers behind one call, attention only, planned splits
    del slots
    outs = fresh()[0]
    plan = kv.DecodeStepLayers([L["q"] for L in layers], None, None, [L["kc"] for L in layers],
                               [L["vc"] for L in layers], None, layers[0]["bt"], layers[0]["sl"],
                               [L["ks"] for L in layers], [L["vs"] for L in layers], max_seq_len=mx,
                               num_splits="planned", out=outs, inputs_ready=True)
    ordered = fresh()[0]
    plain = kv.DecodeStepLayers([L["q"] for L in layers], None, None, [L["kc"] for L in layers],
                                [L["vc"] for L in layers], None, layers[0]["bt"], layers[0]["sl"],
                                [L["ks"] for L in layers], [L["vs"] for L in layers], max_seq_len=mx,
                                num_splits="planned", out=ordered)
    plain()
    for _ in range(3):
        plan()
    torch.cuda.synchronize()
    assert torch.equal(outs, ordered)
    assert kv.device_status() == 0


@pytest.mark.parametrize("lens,splits", [
    ([700, 45, 260, 1, 2048, 130], 4),          # every sequence split four ways
    ([700, 45, 260, 1, 2048, 130], None),       # automatic count
    ([700, 45, 260, 1, 2048, 130], "planned"),  # parts planned on the device, some sequences unsplit
    ([40, 17], 1),                              # no split at all: nothing to chain, outputs written directly
    ([3000] * 12, 32),                          # enough items for four-warp thread blocks
])
def test_chained_layers_match_single_calls(kv, workloads, lens, splits):
    """The L-layer entry point with the inputs-ready promise chains its layers: every layer works in its own half of
    the workspace and its split-KV merge is carried, as extra thread blocks, by the next layer's launch (the last one
    by a closing merge).  Outputs must be bit for bit those of one ordinary call per layer: INT8 attention, the
    fused decode step (cache bytes included) and the BF16 baseline, for odd and even layer counts, launched
    eagerly several times in a row and replayed as a CUDA graph."""
    dev = "cuda"
    B, mx = len(lens), max(lens)
    base, kc0, vc0 = _case_on_gpu(kv, workloads, lens, seed=70)
    bt, sl = base.block_tables.to(dev), base.seq_lens.to(dev)
    last = torch.tensor([sum(lens[: b + 1]) - 1 for b in range(B)])
    slots = base.slot_mapping[last].to(dev)
    g = torch.Generator().manual_seed(71)
    for L in (5, 2):
        layers = []
        for li in range(L):
            # same block table for all layers, own cache contents, scales, queries and new rows per layer
            k = (torch.randn(base.key.shape, generator=g) * (1 + 0.1 * li)).to(torch.bfloat16)
            v = (torch.randn(base.value.shape, generator=g) * 0.5).to(torch.bfloat16)
            ks = (k.float().abs().amax(dim=(0, 2)) / 127).clamp_min(1e-6)
            vs = (v.float().abs().amax(dim=(0, 2)) / 127).clamp_min(1e-6)
            kc, vc = torch.zeros_like(kc0), torch.zeros_like(vc0)
            oracle.cache_write(k, v, kc, vc, base.slot_mapping, ks, vs)
            kb = torch.zeros(base.num_blocks, 16, 4, 128, dtype=torch.bfloat16)
            vb = torch.zeros_like(kb)
            s_ = base.slot_mapping
            kb[s_ // 16, s_ % 16], vb[s_ // 16, s_ % 16] = k, v
            q = torch.randn(B, 28, 128, generator=g).to(torch.bfloat16)
            layers.append(dict(q=q.to(dev), kc=kc.to(dev), vc=vc.to(dev), kb=kb.to(dev), vb=vb.to(dev), ks=ks.to(dev),
                               vs=vs.to(dev), nk=torch.randn(B, 4, 128, generator=g).to(torch.bfloat16).to(dev),
                               nv=(torch.randn(B, 4, 128, generator=g) * 0.5).to(torch.bfloat16).to(dev),
                               q_cpu=q, kc_cpu=kc, vc_cpu=vc, ks_cpu=ks, vs_cpu=vs))
        # --- what single calls return
        want_i8 = torch.stack([kv.int8_paged_attention(x["q"], x["kc"], x["vc"], bt, sl, x["ks"], x["vs"],
                                                       num_splits=splits, max_seq_len=mx) for x in layers])
        want_bf = torch.stack([kv.bf16_paged_attention(x["q"], x["kb"], x["vb"], bt, sl, num_splits=splits,
                                                       max_seq_len=mx) for x in layers])
        torch.cuda.synchronize()
        _check(want_i8[0], oracle.int8_paged_attention_oracle(layers[0]["q_cpu"], layers[0]["kc_cpu"], layers[0]["vc_cpu"],
                                                              base.block_tables, lens, layers[0]["ks_cpu"], layers[0]["vs_cpu"]))
        # --- attention only, chained
        out = torch.full_like(want_i8, float("nan"))
        plan = kv.DecodeStepLayers([x["q"] for x in layers], None, None, [x["kc"] for x in layers],
                                   [x["vc"] for x in layers], None, bt, sl, [x["ks"] for x in layers],
                                   [x["vs"] for x in layers], max_seq_len=mx, num_splits=splits, out=out,
                                   inputs_ready=True)
        for _ in range(3):
            plan()
        torch.cuda.synchronize()
        assert torch.equal(out, want_i8)
        # --- the BF16 baseline through the same chaining
        out_b = torch.full_like(want_bf, float("nan"))
        plan_b = kv.DecodeStepLayers([x["q"] for x in layers], None, None, [x["kb"] for x in layers],
                                     [x["vb"] for x in layers], None, bt, sl, None, None, max_seq_len=mx,
                                     num_splits=splits, out=out_b, inputs_ready=True)
        for _ in range(3):
            plan_b()
        torch.cuda.synchronize()
        assert torch.equal(out_b, want_bf)
        # --- both replayed as one CUDA graph, INT8 and BF16 chains back to back
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            p1 = kv.DecodeStepLayers([x["q"] for x in layers], None, None, [x["kc"] for x in layers],
                                     [x["vc"] for x in layers], None, bt, sl, [x["ks"] for x in layers],
                                     [x["vs"] for x in layers], max_seq_len=mx, num_splits=splits, out=out,
                                     inputs_ready=True)
            p2 = kv.DecodeStepLayers([x["q"] for x in layers], None, None, [x["kb"] for x in layers],
                                     [x["vb"] for x in layers], None, bt, sl, None, None, max_seq_len=mx,
                                     num_splits=splits, out=out_b, inputs_ready=True)
            p1(), p2()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                p1(), p2()
            out.fill_(float("nan"))
            out_b.fill_(float("nan"))
            for _ in range(3):
                graph.replay()
            stream.synchronize()
        assert torch.equal(out, want_i8) and torch.equal(out_b, want_bf)
        del graph
        # --- the fused decode step, chained, against one int8_decode_step per layer: outputs and cache bytes
        ca = [(x["kc"].clone(), x["vc"].clone()) for x in layers]
        cb = [(x["kc"].clone(), x["vc"].clone()) for x in layers]
        want_s = torch.stack([kv.int8_decode_step(x["q"], x["nk"], x["nv"], ca[i][0], ca[i][1], slots, bt, sl, x["ks"],
                                                  x["vs"], max_seq_len=mx, num_splits=splits)
                              for i, x in enumerate(layers)])
        out_s = torch.full_like(want_s, float("nan"))
        plan_s = kv.DecodeStepLayers([x["q"] for x in layers], [x["nk"] for x in layers], [x["nv"] for x in layers],
                                     [c[0] for c in cb], [c[1] for c in cb], slots, bt, sl, [x["ks"] for x in layers],
                                     [x["vs"] for x in layers], max_seq_len=mx, num_splits=splits, out=out_s,
                                     inputs_ready=True)
        for _ in range(2):
            plan_s()
        torch.cuda.synchronize()
        assert torch.equal(out_s, want_s)
        for (ka, va), (kb_, vb_) in zip(ca, cb):
            assert torch.equal(ka, kb_) and torch.equal(va, vb_)
    assert kv.device_status() == 0


def test_device_planned_splits(kv, workloads):
    """num_splits="planned": the kernel reads seq_lens and cuts the sequences into parts of one common length that
    fill whole waves of warps; every operator that takes the tiled path accepts it."""
    lens = [513, 97, 1030, 16, 1, 31, 2048, 300]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=31)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    q, kcd, vcd, bt, sl, ks, vs = _dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    kv.release_workspaces()
    assert kv.last_split_plan() is None
    out = kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs, num_splits="planned")
    _check(out, want)
    items, part, waves = kv.last_split_plan()
    tiles = [(n + 15) // 16 for n in lens]
    assert waves >= 1 and part >= 8
    assert items == 4 * sum(max(1, -(-t // part)) for t in tiles)
    assert items <= waves * 148 * 12
    # lengths below the hint, zero-length sequences, int64 metadata: no host synchronisation, zeros for empty rows
    sl2 = torch.tensor([513, 0, 700, 16, 0, 31, 1000, 300])
    want2 = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, sl2.tolist(), case.k_scale, case.v_scale)
    out2 = kv.int8_paged_attention(q, kcd, vcd, bt.long(), sl2.cuda(), ks, vs, num_splits="planned", max_seq_len=2048)
    live = sl2 > 0
    _check(out2[live.cuda()], want2[live])
    assert float(out2[(~live).cuda()].abs().max()) == 0.0
    # partial rows for a cross-device merge, planned: sequences with one part write their row themselves
    rows = kv.int8_paged_attention_partial(q, kcd, vcd, bt, sl2.cuda(), ks, vs, num_splits="planned", max_seq_len=2048)
    merged = kv.merge_partials(rows[None].contiguous(), 128, dtype=torch.float32)
    _check(merged[live.cuda()], want2[live])
    assert float(merged[(~live).cuda()].abs().max()) == 0.0
    lse = rows[:, :, 128].cpu()
    assert torch.isinf(lse[~live]).all() and torch.isfinite(lse[live]).all()
    # the other operators of the tiled path
    kb = torch.full((case.num_blocks, 16, 4, 128), float("nan"), dtype=torch.bfloat16)
    vb = torch.full_like(kb, float("nan"))
    s_ = case.slot_mapping
    kb[s_ // 16, s_ % 16], vb[s_ // 16, s_ % 16] = case.key, case.value
    wantb = oracle.float_paged_attention_oracle(case.query, kb, vb, case.block_tables, lens)
    _check(kv.bf16_paged_attention(q, kb.cuda(), vb.cuda(), bt, sl, num_splits="planned"), wantb)
    wantq = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale,
                                               quantize_q=True)
    _check(kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs, num_splits="planned", quantize_q=True), wantq)
    assert kv.device_status() == 0


def test_device_planned_splits_many_sequences(kv, workloads):
    """More sequences than lanes (each lane of the planning warp owns a run of them), ragged lengths, and enough
    tiles that the parts are longer than one tile; every sequence is checked against the oracle."""
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(1, 1500, (150,), generator=g).tolist()
    lens[7], lens[100] = 4000, 3999
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=33)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    q, kcd, vcd, bt, sl, ks, vs = _dev(case.query, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    kv.release_workspaces()
    out = kv.int8_paged_attention(q, kcd, vcd, bt, sl, ks, vs, num_splits="planned")
    _check(out, want)
    items, part, waves = kv.last_split_plan()
    tiles = [(n + 15) // 16 for n in lens]
    assert part > 1 and items == 4 * sum(max(1, -(-t // part)) for t in tiles) and items <= waves * 148 * 12
    # the most sequences a plan covers (16 per lane of the planning warp), two KV heads, some of them empty
    shape = workloads.LayerShape(14, 2, 128, 16)
    lens = torch.randint(1, 400, (512,), generator=g).tolist()
    case, kc, vc = _case_on_gpu(kv, workloads, lens, shape=shape, seed=34)
    sl = case.seq_lens.clone()
    sl[::37] = 0
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, sl.tolist(), case.k_scale, case.v_scale)
    q, kcd, vcd, bt, ks, vs = _dev(case.query, kc, vc, case.block_tables, case.k_scale, case.v_scale)
    out = kv.int8_paged_attention(q, kcd, vcd, bt, sl.cuda(), ks, vs, num_splits="planned", max_seq_len=400)
    live = sl > 0
    _check(out[live.cuda()], want[live])
    assert float(out[(~live).cuda()].abs().max()) == 0.0
    # one sequence more is refused, not mis-planned
    from conftest import package

    with pytest.raises(package("_lib").Int8KVError):
        kv.int8_paged_attention(q[:1].expand(513, -1, -1).contiguous(), kcd, vcd, bt[:1].expand(513, -1).contiguous(),
                                sl[:1].expand(513).contiguous().cuda() + 1, ks, vs, num_splits="planned", max_seq_len=400)
    assert kv.device_status() == 0


def _plan_restated(lens, hkv, cap_tokens, k_max, min_part, grid_items, slots=148 * 12):
    """The planning arithmetic of the kernels restated on the host: (items, part length in tiles, waves)."""
    tiles = [(min(max(n, 0), cap_tokens) + 15) // 16 for n in lens]
    total, longest, B = sum(tiles), max(tiles), len(lens)
    parts = lambda P: sum(max(1, -(-t // P)) for t in tiles)
    floor_p = max(1, -(-longest // 128))
    k, P = max(k_max, 1), 1
    while k >= 1:
        room = k * slots - hkv * B // 2
        if room > 0:
            P = -(-(total * hkv) // room)
            if P >= min_part or k == 1:
                break
        k -= 1
    k = max(k, 1)
    P = max(P, floor_p, 8)
    target = min(k * slots, grid_items)
    for rnd in range(64):
        if parts(P) * hkv <= target or P >= longest:
            break
        P += max(1, P >> 4) if rnd < 16 else P
    return parts(P) * hkv, P, k


def test_device_plan_matches_its_restatement_on_random_batches(kv, workloads):
    """Random batch sizes, head counts and length distributions: the plan the kernels leave in the workspace equals
    the host restatement of the same arithmetic, fills at most the waves it aimed for, and the planned result
    equals the result with a fixed split count."""
    g = torch.Generator().manual_seed(2024)
    dev = "cuda"
    for trial, (B, hkv, lo, hi) in enumerate([(300, 4, 800, 2400), (37, 1, 4000, 30000), (512, 2, 16, 900),
                                              (96, 8, 1, 6000), (200, 4, 3000, 3001), (5, 4, 20000, 60000)]):
        lens = torch.randint(lo, hi + 1, (B,), generator=g).tolist()
        hq = hkv * (7 if hkv <= 4 else 8)
        width = -(-max(lens) // 16)
        nblocks = sum(-(-n // 16) for n in lens)
        gd = torch.Generator(device=dev).manual_seed(trial)
        kc = torch.randint(-127, 128, (nblocks, 16, hkv, 128), generator=gd, device=dev, dtype=torch.int8)
        vc = torch.randint(-127, 128, (nblocks, 16, hkv, 128), generator=gd, device=dev, dtype=torch.int8)
        bt = torch.zeros(B, width, dtype=torch.int32)
        perm = torch.randperm(nblocks, generator=g).to(torch.int32)
        at = 0
        for b, n in enumerate(lens):
            nb = -(-n // 16)
            bt[b, :nb] = perm[at : at + nb]
            at += nb
        q = torch.randn(B, hq, 128, generator=gd, device=dev, dtype=torch.float32).to(torch.bfloat16)
        ks = torch.rand(hkv, generator=gd, device=dev) * 0.02 + 0.01
        vs = torch.rand(hkv, generator=gd, device=dev) * 0.02 + 0.01
        sl = torch.tensor(lens, dtype=torch.int32, device=dev)
        kv.release_workspaces()
        out = kv.int8_paged_attention(q, kc, vc, bt.to(dev), sl, ks, vs, num_splits="planned", max_seq_len=max(lens))
        plan = kv.last_split_plan()
        assert plan is not None
        # what the host passes to the kernel for this shape: waves from the nominal lengths, 48-tile parts above one wave
        nominal = (max(lens) + 15) // 16
        k_max = 1
        for k in (4, 3, 2, 1):
            room = k * 1776 - B * hkv // 2
            if room > 0 and (-(-(B * hkv * nominal) // room) >= 48 or k == 1):
                k_max = k
                break
        want = _plan_restated(lens, hkv, width * 16, k_max, 48, max(k_max * 1776, B * hkv))
        assert plan == want, (trial, plan, want)
        assert plan[0] <= plan[2] * 1776 or plan[1] >= max(-(-n // 16) for n in lens)
        fixed = kv.int8_paged_attention(q, kc, vc, bt.to(dev), sl, ks, vs, num_splits=3, max_seq_len=max(lens))
        assert cosine(out.float().cpu(), fixed.float().cpu()) > 0.99999
        assert max_abs(out.float().cpu(), fixed.float().cpu()) <= 2e-2 * max(1.0, float(fixed.float().abs().max()))
    assert kv.device_status() == 0


def test_device_planned_splits_in_decode_step_and_dynamic_scales(kv, workloads):
    lens = [513, 97, 1030, 16]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=16)
    dev = "cuda"
    last = torch.tensor([sum(lens[: b + 1]) - 1 for b in range(len(lens))])
    kc0, vc0 = torch.zeros_like(kc), torch.zeros_like(vc)
    keep = torch.ones(sum(lens), dtype=torch.bool)
    keep[last] = False
    oracle.cache_write(case.key[keep], case.value[keep], kc0, vc0, case.slot_mapping[keep], case.k_scale, case.v_scale)
    kcd, vcd = kc0.to(dev), vc0.to(dev)
    out = kv.int8_decode_step(case.query.to(dev), case.key[last].to(dev), case.value[last].to(dev), kcd, vcd,
                              case.slot_mapping[last].to(dev), case.block_tables.to(dev), case.seq_lens.to(dev),
                              case.k_scale.to(dev), case.v_scale.to(dev), max_seq_len=max(lens), num_splits="planned")
    assert torch.equal(kcd.cpu(), kc) and torch.equal(vcd.cpu(), vc)
    _check(out, oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale))
    lens = [513, 97, 1030, 16, 1, 31, 2048]
    case, kc, vc, ksc, vsc = _dynamic_case(workloads, lens, workloads.QWEN25_7B, seed=21)
    want = oracle.dynamic_int8_paged_attention_oracle(case.query, kc, vc, ksc, vsc, case.block_tables, lens)
    q, kcd, vcd, kscd, vscd, bt, sl = _dev(case.query, kc, vc, ksc, vsc, case.block_tables, case.seq_lens)
    _check(kv.int8_paged_attention_dynamic(q, kcd, vcd, kscd, vscd, bt, sl, num_splits="planned"), want)
    # shapes outside the tiled kernels cannot be planned: the library says so
    shape = workloads.LayerShape(8, 2, 64, 8)
    c2, k2, v2 = _case_on_gpu(kv, workloads, [33, 9], shape=shape, seed=3)
    from conftest import package

    with pytest.raises(package("_lib").Int8KVError):
        kv.int8_paged_attention(*_dev(c2.query, k2, v2, c2.block_tables, c2.seq_lens, c2.k_scale, c2.v_scale),
                                num_splits="planned")
    assert kv.device_status() == 0


def _dynamic_case(workloads, lens, shape, seed, v_gain=None):
    """A paged cache filled by the dynamic per-(token, head) scheme on the CPU (oracle arithmetic); unused slots
    hold garbage bytes and NaN scales, which attention must never read into its result."""
    case = workloads.make_decode_case(lens, shape, seed=seed)
    value = case.value.float()
    if v_gain is not None:
        value = value * v_gain[:, None, None]
    kq, ks = oracle.dynamic_quant_per_token_head(case.key)
    vq, vs = oracle.dynamic_quant_per_token_head(value)
    nb, bs, h, d = case.num_blocks, shape.block_size, shape.num_kv_heads, shape.head_dim
    g = torch.Generator().manual_seed(seed + 99)
    kc = torch.randint(-128, 128, (nb * bs, h, d), generator=g, dtype=torch.int8)
    vc = torch.randint(-128, 128, (nb * bs, h, d), generator=g, dtype=torch.int8)
    ksc = torch.full((nb * bs, h), float("nan"))
    vsc = torch.full((nb * bs, h), float("nan"))
    kc[case.slot_mapping], vc[case.slot_mapping] = kq, vq
    ksc[case.slot_mapping], vsc[case.slot_mapping] = ks, vs
    return case, kc.view(nb, bs, h, d), vc.view(nb, bs, h, d), ksc.view(nb, bs, h), vsc.view(nb, bs, h)


def test_dynamic_scale_attention_tiled_path(kv, workloads):
    """Attention over the per-(token, head) scale scheme equals the fp32 attention of the dequantised cache.
    Parity unpinned (no CPU definition in the reference): it has a writer and a dequantiser for this scheme but no
    attention over it; the expectation is fp32 attention over what its dequantize_int8_cache formula reconstructs."""
    lens = [513, 97, 1030, 16, 1, 31, 2048]
    case, kc, vc, ksc, vsc = _dynamic_case(workloads, lens, workloads.QWEN25_7B, seed=21)
    want = oracle.dynamic_int8_paged_attention_oracle(case.query, kc, vc, ksc, vsc, case.block_tables, lens)
    assert torch.isfinite(want).all()
    q, kcd, vcd, kscd, vscd, bt, sl = _dev(case.query, kc, vc, ksc, vsc, case.block_tables, case.seq_lens)
    for splits in (None, 1, 2, 3, 8, 32):
        out = kv.int8_paged_attention_dynamic(q, kcd, vcd, kscd, vscd, bt, sl, num_splits=splits)
        _check(out, want)
    # no host synchronisation with max_seq_len; fp32 query and output; int64 tables
    out = kv.int8_paged_attention_dynamic(q.float(), kcd, vcd, kscd, vscd, bt.long(), sl.long(), max_seq_len=2048)
    assert out.dtype == torch.float32
    out = out.cpu()
    assert max_abs(out, want) < 5e-3 and cosine(out, want) > 0.99999
    assert kv.device_status() == 0


def test_dynamic_scale_attention_wide_value_range(kv, workloads):
    """Token scales that differ by orders of magnitude inside one sequence (tiny first tokens, huge later ones and
    the reverse) keep their precision through the fp16 P.V product.  Parity unpinned (no CPU definition in the
    reference), as for the test above."""
    lens = [700, 700, 64]
    g = torch.Generator().manual_seed(5)
    total = sum(lens)
    for pattern in ("rising", "falling", "spiky"):
        gain = torch.ones(total)
        if pattern == "rising":
            gain[:32], gain[700:732] = 1e-3, 1e-3
            gain[400:700] = 300.0
        elif pattern == "falling":
            gain[:32] = 500.0
            gain[32:700] = 1e-2
        else:
            gain[torch.randperm(total, generator=g)[:40]] = 2000.0
        case, kc, vc, ksc, vsc = _dynamic_case(workloads, lens, workloads.QWEN25_7B, seed=22, v_gain=gain)
        want = oracle.dynamic_int8_paged_attention_oracle(case.query, kc, vc, ksc, vsc, case.block_tables, lens)
        q, kcd, vcd, kscd, vscd, bt, sl = _dev(case.query, kc, vc, ksc, vsc, case.block_tables, case.seq_lens)
        for splits in (1, 4):
            out = kv.int8_paged_attention_dynamic(q.float(), kcd, vcd, kscd, vscd, bt, sl, num_splits=splits).cpu()
            scale = float(want.abs().max())
            assert max_abs(out, want) < 2e-3 * scale, (pattern, splits, max_abs(out, want), scale)
            assert cosine(out, want) > 0.9999
    assert kv.device_status() == 0


def test_dynamic_scale_attention_generic_path_and_write_chain(kv, workloads):
    """Shapes outside the tiled kernel (D=64, BS=8, group 4), and the whole chain on the device:
    reshape_and_cache_int8 writes the caches and scale caches that the attention then reads.  Parity unpinned (no
    CPU definition in the reference), as for the tests above."""
    from conftest import package

    ops = package("vllm_int8.vllm_int8_cache_ops")
    shape = workloads.LayerShape(8, 2, 64, 8)
    lens = [33, 9, 70]
    case, kc, vc, ksc, vsc = _dynamic_case(workloads, lens, shape, seed=23)
    want = oracle.dynamic_int8_paged_attention_oracle(case.query, kc, vc, ksc, vsc, case.block_tables, lens)
    q, kcd, vcd, kscd, vscd, bt, sl = _dev(case.query, kc, vc, ksc, vsc, case.block_tables, case.seq_lens)
    for splits in (None, 1, 3):
        _check(kv.int8_paged_attention_dynamic(q, kcd, vcd, kscd, vscd, bt, sl, num_splits=splits), want)
    # device chain on the tiled shape
    lens = [300, 77, 1]
    c = workloads.make_decode_case(lens, workloads.QWEN25_7B, seed=24)
    kc2, vc2, ks2, vs2 = ops.allocate_int8_kv_cache(c.num_blocks, 16, 4, 128, device="cuda")
    ops.reshape_and_cache_int8(c.key.cuda(), c.value.cuda(), kc2, vc2, ks2, vs2, c.slot_mapping.cuda())
    out = kv.int8_paged_attention_dynamic(c.query.cuda(), kc2, vc2, ks2, vs2, c.block_tables.cuda(), c.seq_lens.cuda())
    want2 = oracle.dynamic_int8_paged_attention_oracle(c.query, kc2.cpu(), vc2.cpu(), ks2.cpu(), vs2.cpu(),
                                                       c.block_tables, lens)
    _check(out, want2)
    # and it is close to the attention of the un-quantised K/V (the scheme's point): per-token scales beat 1e-2
    kf = torch.zeros(c.num_blocks * 16, 4, 128)
    vf = torch.zeros_like(kf)
    kf[c.slot_mapping], vf[c.slot_mapping] = c.key.float(), c.value.float()
    exact = oracle.float_paged_attention_oracle(c.query, kf.view(-1, 16, 4, 128), vf.view(-1, 16, 4, 128),
                                                c.block_tables, lens)
    assert max_abs(out.float().cpu(), exact) < 3e-2 and cosine(out.float().cpu(), exact) > 0.999
    assert kv.device_status() == 0


def test_vllm_call_sites_with_fake_engine_objects(kv, workloads):
    """do_kv_cache_update -> INT8 mirror write, forward -> INT8 attention, through the patched methods of a fake
    attention-implementation class, in all three modes."""
    from conftest import package

    sc, sh = package("vllm_int8.static_scales"), package("vllm_int8.vllm_shadow_cache_patch")
    ap, pool = package("vllm_int8.vllm_int8_attention_patch"), package("vllm_int8.cache_manager")
    lens = [300, 77]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=18)
    dev = "cuda"
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)

    class Meta:
        seq_lens = case.seq_lens.to(dev)
        block_table = case.block_tables.to(dev)
        num_actual_tokens = 2
        max_query_len = 1

    for mode in ("shadow", "takeover", "int8_only"):
        pool.clear_cache_pool()
        sc.set_static_scales(case.k_scale.repeat(28, 1), case.v_scale.repeat(28, 1))
        for d in (ap.ATTN_INT8_HITS, ap.ATTN_METRICS, ap.ATTN_COMPARE_COUNT, sh.WRITE_CALL_COUNT):
            d.clear()

        class Impl:
            def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
                pass

            def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                        output_block_scale=None):
                output[:2].copy_(want.to(output.dtype).to(output.device))  # stands in for the engine's bf16 attention
                return output

        class Layer:
            layer_name = "model.layers.5.self_attn.attn"

        sh.apply_shadow_cache_patch(Impl)
        ap.apply_int8_attention_patch(Impl, mode=mode)
        impl = Impl()
        native = torch.empty(case.num_blocks, 4, 16, 256, dtype=torch.bfloat16, device=dev)
        impl.do_kv_cache_update(Layer(), case.key.to(dev), case.value.to(dev), native, case.slot_mapping.to(dev))
        shadow = pool.get_layer_cache(Layer.layer_name)
        assert torch.equal(shadow.key_cache.cpu(), kc) and torch.equal(shadow.value_cache.cpu(), vc)
        padded_q = torch.zeros(4, 28, 128, dtype=torch.bfloat16, device=dev)
        padded_q[:2] = case.query.to(dev)
        out = torch.zeros(4, 28, 128, dtype=torch.bfloat16, device=dev)
        res = impl.forward(Layer(), padded_q, None, None, native, Meta(), out)
        _check(res[:2], want)
        if mode == "int8_only":
            assert ap.ATTN_INT8_HITS[Layer.layer_name] == 1 and ap.ATTN_INT8_STATS["last_batch"] == 2
            # the INT8-only forward reads nothing back on the host, so a decode step can be captured in a CUDA
            # graph (a host read of a device value during capture raises) and replayed
            out2 = torch.zeros(4, 28, 128, dtype=torch.bfloat16, device=dev)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                impl.forward(Layer(), padded_q, None, None, native, Meta(), out2)  # sizes this stream's workspace
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    impl.forward(Layer(), padded_q, None, None, native, Meta(), out2)
                out2.zero_()
                g.replay()
                stream.synchronize()
            _check(out2[:2], want)
            del g
        else:
            m = ap.ATTN_METRICS[Layer.layer_name][0]
            assert m["cosine"] > 0.9999 and m["relative_l2"] < 0.02
    pool.clear_cache_pool()
    sc.clear_static_scales()


def test_workspace_growth_keeps_captured_graphs_valid(kv, workloads):
    """A CUDA graph captured over a small call keeps the address of the split-KV workspace of that time.  A later,
    larger call makes the operator module switch to a bigger buffer; the old one must stay allocated, or the
    graph's partial rows would land in memory that now belongs to someone else.  Growth during a capture is
    refused with an explanation instead of allocating from the graph's private pool."""
    kv.release_workspaces()
    dev = "cuda"
    small, kc_s, vc_s = _case_on_gpu(kv, workloads, [600, 90], seed=61)
    want_small = oracle.int8_paged_attention_oracle(small.query, kc_s, vc_s, small.block_tables, [600, 90],
                                                    small.k_scale, small.v_scale)
    args_s = _dev(small.query, kc_s, vc_s, small.block_tables, small.seq_lens, small.k_scale, small.v_scale)
    out_s = torch.zeros(2, 28, 128, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        kv.int8_paged_attention(*args_s, num_splits=4, max_seq_len=600, out=out_s)  # sizes the workspace: 1 MiB
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            kv.int8_paged_attention(*args_s, num_splits=4, max_seq_len=600, out=out_s)
        # a call that needs more than the current buffer, inside a capture: refused, nothing allocated
        big, kc_b, vc_b = _case_on_gpu(kv, workloads, [3000] * 12, seed=62)
        args_b = _dev(big.query, kc_b, vc_b, big.block_tables, big.seq_lens, big.k_scale, big.v_scale)
        g2 = torch.cuda.CUDAGraph()
        with pytest.raises(RuntimeError, match="before capturing"):
            with torch.cuda.graph(g2, stream=stream):
                kv.int8_paged_attention(*args_b, num_splits=64, max_seq_len=3000)
        del g2
        # the same call eagerly: the module moves to a bigger buffer (12 * 28 * 64 rows of 528 B = 11 MB)
        out_b = kv.int8_paged_attention(*args_b, num_splits=64, max_seq_len=3000)
        stream.synchronize()
        _check(out_b, oracle.int8_paged_attention_oracle(big.query, kc_b, vc_b, big.block_tables, [3000] * 12,
                                                         big.k_scale, big.v_scale))
        # memory pressure of the kind that would reuse a freed megabyte, then the old graph again
        junk = [torch.full((1 << 20,), 0x7F, dtype=torch.uint8, device=dev) for _ in range(8)]
        out_s.zero_()
        g.replay()
        stream.synchronize()
        assert all(int(j[0]) == 0x7F and int(j[-1]) == 0x7F and int(j.min()) == 0x7F for j in junk)
    _check(out_s, want_small)
    del g
    kv.release_workspaces()
    assert kv.device_status() == 0


def test_long_parts_and_sink_plus_crowd_distributions(kv, workloads):
    """Parts of thousands of tokens, and the distribution real decoders produce: one 'sink' token far above a
    broad crowd of tokens that are individually tiny but carry most of the probability mass together."""
    lens = [8190, 1100, 2048, 37]
    case, kc, vc = _case_on_gpu(kv, workloads, lens, seed=20)
    args = lambda qq: _dev(qq, kc, vc, case.block_tables, case.seq_lens, case.k_scale, case.v_scale)
    want = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
    for splits in (1, 2, None):
        _check(kv.int8_paged_attention(*args(case.query), num_splits=splits), want)
    ks, _ = oracle.gather_paged_cache(kc, vc, case.block_tables, lens)
    for tok in (0, 4321):
        k_tok = oracle.dequant_per_head(ks[0][:, tok], case.k_scale, head_axis=0).repeat_interleave(7, dim=0)  # [Hq, D]
        base = case.query[0].float() * 0.05  # a flat crowd: all other scores within a fraction of a unit
        lo, hi = 0.0, 1.0
        for _ in range(20):  # bisect the sink strength so that the sink holds 5-15 % of the mass
            beta = 0.5 * (lo + hi)
            q_row = base + beta * k_tok
            k_all = oracle.dequant_per_head(ks[0], case.k_scale, head_axis=0)  # [Hkv, T, D]
            sc = torch.einsum("hgd,htd->hgt", q_row.reshape(4, 7, 128), k_all) / math.sqrt(128)
            share = torch.softmax(sc, dim=-1)[..., tok].mean()
            lo, hi = (beta, hi) if share < 0.10 else (lo, beta)
        q2 = case.query.clone()
        q2[0] = (base + beta * k_tok).to(q2.dtype)
        want2 = oracle.int8_paged_attention_oracle(q2, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
        for splits in (1, None):
            _check(kv.int8_paged_attention(*args(q2), num_splits=splits), want2)
    assert kv.device_status() == 0


def test_a_wait_that_cannot_finish_times_out_and_is_reported(kv, workloads):
    """Failure detection without a GPU fault: the bounded wait runs out, the status word says so, and the
    context keeps working."""
    from conftest import package

    assert kv.device_status() == 0
    assert kv.selftest_bounded_wait(attempts=200) == package("_lib").DEV_WAIT_TIMEOUT
    assert kv.device_status() == 0  # reading clears it
    g = load_golden("attn_97_256")
    _check(_run_int8(kv, g), g["out_chain_f32"], g["out_loop_bf16"])
