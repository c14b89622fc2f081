"""The CPU oracle against the reference's own outputs (fixtures made by tests/golden/make_golden.py).

This is the parity pin of the oracle: every restated function must reproduce what the reference's
Python code returned for the same seeded inputs — bit-exact for integer work, to fp32 round-off for
attention."""

import torch

import oracle
from conftest import load_golden, max_abs


def _fresh(t):
    return torch.zeros_like(t)


def test_static_quant_matches_reference_quant():
    g = load_golden("write_t37")
    q = oracle.static_quant_per_head(g["key"].permute(1, 0, 2)[None], g["k_scale"], head_axis=1)
    assert torch.equal(q, g["key_q_static"])


def test_cache_write_t37_bit_exact():
    g = load_golden("write_t37")
    kc, vc = _fresh(g["key_cache"]), _fresh(g["value_cache"])
    oracle.cache_write(g["key"], g["value"], kc, vc, g["slot_mapping"], g["k_scale"], g["v_scale"])
    assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])


def test_cache_write_n23_bit_exact():
    g = load_golden("write_n23")
    kc, vc = _fresh(g["key_cache"]), _fresh(g["value_cache"])
    oracle.cache_write(g["key"], g["value"], kc, vc, g["slot_mapping"], g["k_scale"], g["v_scale"])
    assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])


def test_real_activations_quant_bit_exact():
    g = load_golden("real_layer27")
    assert torch.equal(oracle.static_quant_per_head(g["k"], g["k_scale"], head_axis=1), g["k_q"])
    assert torch.equal(oracle.static_quant_per_head(g["v"], g["v_scale"], head_axis=1), g["v_q"])


def test_paged_layout_matches_reference():
    g = load_golden("paged_layout")
    kc, vc, bt, sl = oracle.build_paged_cache(g["k"], g["v"], 16)
    assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])
    assert torch.equal(bt, g["block_tables"]) and torch.equal(sl, g["seq_lens"])
    ks, vs = oracle.gather_paged_cache(kc, vc, bt, sl)
    assert torch.equal(torch.stack(ks), g["k"]) and torch.equal(torch.stack(vs), g["v"])


def _attention_case(name):
    g = load_golden(name)
    # slot mapping and write
    slots = oracle.slots_for_sequences(g["block_tables"], g["seq_lens"].tolist(), 16)
    assert torch.equal(slots, g["slot_mapping"])
    kc, vc = _fresh(g["key_cache"]), _fresh(g["value_cache"])
    oracle.cache_write(g["key"], g["value"], kc, vc, slots, g["k_scale"], g["v_scale"])
    assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])
    out = oracle.int8_paged_attention_oracle(
        g["query"], kc, vc, g["block_tables"], g["seq_lens"].tolist(), g["k_scale"], g["v_scale"]
    )
    assert max_abs(out, g["out_chain_f32"]) < 2e-6
    # the reference's loop reference rounds to bf16; the oracle rounded the same way must agree to 1 bf16 ulp
    assert max_abs(out.to(torch.bfloat16).float(), g["out_loop_bf16"].float()) <= 2 ** -8 * float(out.abs().max())


def test_attention_127_301():
    _attention_case("attn_127_301")


def test_attention_97_256():
    _attention_case("attn_97_256")


def test_quantize_q_definition_matches_the_reference_loop():
    """The optional INT8 query: the oracle, and the debug helper of the drop-in module that carries the reference's
    name, must both reproduce what the reference's torch_int8_paged_attention_reference(..., quantize_q=True)
    returned (src/triton_ops/int8_paged_attention.py:776-814), to one bf16 ulp."""
    from conftest import package

    helper = package("triton_ops.int8_paged_attention").torch_int8_paged_attention_reference
    for name in ("attn_127_301", "attn_97_256"):
        g = load_golden(name)
        want = g["out_loop_quantize_q_bf16"].float()
        ulp = 2 ** -8 * float(want.abs().max())
        out = oracle.int8_paged_attention_oracle(g["query"], g["key_cache"], g["value_cache"], g["block_tables"],
                                                 g["seq_lens"].tolist(), g["k_scale"], g["v_scale"], quantize_q=True)
        assert max_abs(out.to(torch.bfloat16).float(), want) <= ulp
        # the quantised query is not the plain one: the two references differ by more than rounding
        assert max_abs(want, g["out_loop_bf16"].float()) > 0
        got = helper(g["query"], g["key_cache"], g["value_cache"], g["block_tables"], g["seq_lens"], g["k_scale"],
                     g["v_scale"], quantize_q=True)
        assert got.dtype == torch.bfloat16 and max_abs(got.float(), want) <= ulp
        plain = helper(g["query"], g["key_cache"], g["value_cache"], g["block_tables"], g["seq_lens"], g["k_scale"],
                       g["v_scale"])
        assert max_abs(plain.float(), g["out_loop_bf16"].float()) <= ulp


def test_config1_chain():
    g = load_golden("config1")
    key, value = g["key"], g["value"]
    kc, vc = _fresh(g["key_cache"]), _fresh(g["value_cache"])
    oracle.cache_write(key[:512], value[:512], kc, vc, g["slot_mapping"][:512], g["k_scale"], g["v_scale"])
    out512 = oracle.int8_paged_attention_oracle(g["query"], kc, vc, g["block_tables"], [512], g["k_scale"], g["v_scale"])
    assert max_abs(out512, g["out_ctx512_f32"]) < 2e-6
    oracle.cache_write(key[512:], value[512:], kc, vc, g["slot_mapping"][512:], g["k_scale"], g["v_scale"])
    assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])
    out513 = oracle.int8_paged_attention_oracle(g["query"], kc, vc, g["block_tables"], [513], g["k_scale"], g["v_scale"])
    assert max_abs(out513, g["out_ctx513_f32"]) < 2e-6


def test_unquantised_attention_matches_reference_bf16_helper():
    g = load_golden("attn_127_301")
    lens = g["seq_lens"].tolist()
    Hkv, D = 4, 128
    nblk = g["key_cache"].shape[0]
    kc = torch.zeros(nblk, 16, Hkv, D, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    s = g["slot_mapping"]
    kc[s // 16, s % 16] = g["key"]
    vc[s // 16, s % 16] = g["value"]
    out = oracle.float_paged_attention_oracle(g["query"], kc, vc, g["block_tables"], lens)
    ref = g["out_unquantised_bf16"].float().reshape(out.shape)  # the helper returns [B, 1, Hq, D]
    assert max_abs(out.to(torch.bfloat16).float(), ref) <= 2 ** -8 * float(ref.abs().max())


def test_merge_of_partials_equals_unsplit():
    g = load_golden("attn_97_256")
    lens = g["seq_lens"].tolist()
    ks, vs = oracle.gather_paged_cache(g["key_cache"], g["value_cache"], g["block_tables"], lens)
    for b, T in enumerate(lens):
        k = oracle.dequant_per_head(ks[b], g["k_scale"], head_axis=0)
        v = oracle.dequant_per_head(vs[b], g["v_scale"], head_axis=0)
        full = oracle.decode_attention(g["query"][b], k, v)
        cuts = [0, 40, 40, 133, T]  # includes an empty part
        outs, lses = zip(*[
            oracle.partial_attention_with_lse(g["query"][b], k[:, a:z], v[:, a:z]) for a, z in zip(cuts[:-1], cuts[1:])
        ])
        merged = oracle.merge_partials(torch.stack(outs), torch.stack(lses))
        assert max_abs(merged, full) < 2e-6


def test_plain_c_quantiser_agrees_with_the_reference_vectors_and_the_torch_oracle():
    """Two independent restatements (C with nearbyintf on a binary32 quotient, PyTorch) and the reference's own
    outputs must give the same bytes, including ties, saturation and tiny scales."""
    from oracle import quant_c

    g = load_golden("write_t37")
    assert torch.equal(quant_c.static_quant(g["key"], g["k_scale"]), g["key_q_static"][0].permute(1, 0, 2))
    for name in ("write_t37", "write_n23", "attn_127_301"):
        g = load_golden(name)
        kc, vc = _fresh(g["key_cache"]), _fresh(g["value_cache"])
        quant_c.cache_write(g["key"], g["k_scale"], kc, g["slot_mapping"])
        quant_c.cache_write(g["value"], g["v_scale"], vc, g["slot_mapping"])
        assert torch.equal(kc, g["key_cache"]) and torch.equal(vc, g["value_cache"])
    r = load_golden("real_layer27")
    k_tm = r["k"].permute(0, 2, 1, 3).reshape(40, 4, 128)
    assert torch.equal(quant_c.static_quant(k_tm, r["k_scale"]), r["k_q"].permute(0, 2, 1, 3).reshape(40, 4, 128))
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(300, 4, 128, generator=gen) * 4
    x[::9] = torch.round(x[::9] * 2) / 2  # exact halves: ties at scale 1 and 0.5
    x[5] = 1e9
    x[6] = -1e9
    for scale in (torch.tensor([1.0, 0.5, 0.037, 1e-8]), torch.tensor([0.25, 2.0, 0.0123, 3.3])):
        for dtype in (torch.float32, torch.bfloat16, torch.float16):
            xs = x.to(dtype)
            for floor in (False, True):
                a = quant_c.static_quant(xs, scale, floor_scale=floor)
                b = oracle.static_quant_per_head(xs, scale, head_axis=1, floor_scale=floor)
                assert torch.equal(a, b)
