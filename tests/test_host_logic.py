"""Host-side behaviour that needs no GPU: the operators' argument checks, the drop-in modules' names and
signatures, the workload generators, and the partitioning helpers."""

import inspect

import pytest
import torch

import oracle
from conftest import package


def test_operators_reject_cpu_tensors_instead_of_falling_back(kv):
    """There is no CPU path behind the operators: CPU tensors fail the same assertion as in the reference."""
    k = torch.zeros(2, 4, 128, dtype=torch.bfloat16)
    kc = torch.zeros(2, 16, 4, 128, dtype=torch.int8)
    s = torch.ones(4)
    with pytest.raises(AssertionError):
        kv.int8_kv_cache_write(k, k, kc, kc.clone(), torch.zeros(2, dtype=torch.int64), s, s)
    q = torch.zeros(1, 28, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError):
        kv.int8_paged_attention(q, kc, kc, torch.zeros(1, 2, dtype=torch.int32), torch.ones(1, dtype=torch.int32), s, s)
    with pytest.raises(AssertionError):
        kv.bf16_paged_attention(q, kc.bfloat16(), kc.bfloat16(), torch.zeros(1, 2, dtype=torch.int32),
                                torch.ones(1, dtype=torch.int32))


REFERENCE_SIGNATURES = {
    # parameter names of the reference's public functions, in order
    ("triton_ops.int8_cache_write", "int8_kv_cache_write"):
        ["key", "value", "key_cache", "value_cache", "slot_mapping", "k_scale", "v_scale", "num_warps", "num_stages"],
    ("triton_ops.int8_cache_write", "torch_int8_kv_cache_write_reference"):
        ["key", "value", "key_cache", "value_cache", "slot_mapping", "k_scale", "v_scale"],
    ("triton_ops.int8_cache_write", "dequantize_paged_cache_for_debug"): ["cache", "scale"],
    ("triton_ops.int8_paged_attention", "int8_paged_attention"):
        ["query", "key_cache", "value_cache", "block_tables", "seq_lens", "k_scale", "v_scale",
         "quantize_q", "num_warps", "impl", "num_splits"],
    ("triton_ops.int8_paged_attention", "torch_int8_paged_attention_reference"):
        ["query", "key_cache", "value_cache", "block_tables", "seq_lens", "k_scale", "v_scale", "quantize_q"],
    ("triton_ops.bf16_paged_attention", "bf16_paged_attention"):
        ["query", "key_cache", "value_cache", "block_tables", "seq_lens"],
    ("vllm_int8.vllm_int8_cache_ops", "runtime_int8_cache_write"):
        ["key", "value", "key_cache", "value_cache", "slot_mapping", "k_scale", "v_scale"],
    ("vllm_int8.vllm_int8_cache_ops", "reshape_and_cache_int8"):
        ["key", "value", "key_cache", "value_cache", "k_scale_cache", "v_scale_cache", "slot_mapping"],
    ("vllm_int8.vllm_int8_cache_ops", "allocate_int8_kv_cache"):
        ["num_blocks", "block_size", "num_kv_heads", "head_dim", "device"],
    ("vllm_int8.vllm_int8_cache_ops", "dequantize_int8_cache"): ["cache", "scale_cache"],
    ("vllm_int8.vllm_int8_attention_patch", "_run_int8_attention"): ["layer", "query", "attn_metadata"],
    ("vllm_int8.vllm_int8_attention_patch", "_is_supported_decode"): ["query", "attn_metadata"],
}


@pytest.mark.parametrize("where,names", list(REFERENCE_SIGNATURES.items()))
def test_drop_in_modules_keep_the_reference_signatures(where, names):
    mod, fn = where
    f = getattr(package(mod), fn)
    got = list(inspect.signature(f).parameters)
    assert got[: len(names)] == names
    for extra in inspect.signature(f).parameters.values():
        if extra.name not in names:  # extensions must be optional keyword arguments
            assert extra.default is not inspect.Parameter.empty and extra.kind is inspect.Parameter.KEYWORD_ONLY
    sig = inspect.signature(package("triton_ops.int8_paged_attention").int8_paged_attention).parameters
    assert sig["impl"].default == "auto" and sig["num_splits"].default is None and sig["quantize_q"].default is False


def test_debug_helpers_in_drop_in_modules_agree_with_the_oracle():
    g = torch.Generator().manual_seed(0)
    key = torch.randn(20, 4, 128, generator=g).to(torch.bfloat16)
    value = torch.randn(20, 4, 128, generator=g).to(torch.bfloat16)
    ks, vs = torch.tensor([0.03, 0.02, 0.04, 0.05]), torch.tensor([0.02, 0.03, 0.01, 0.04])
    slots = torch.tensor(list(range(5, 24)) + [-1])
    w = package("triton_ops.int8_cache_write")
    kc, vc = torch.zeros(2, 16, 4, 128, dtype=torch.int8), torch.zeros(2, 16, 4, 128, dtype=torch.int8)
    w.torch_int8_kv_cache_write_reference(key, value, kc, vc, slots, ks, vs)
    kc_o, vc_o = torch.zeros_like(kc), torch.zeros_like(vc)
    oracle.cache_write(key, value, kc_o, vc_o, slots, ks, vs)
    assert torch.equal(kc, kc_o) and torch.equal(vc, vc_o)
    assert torch.equal(w.dequantize_paged_cache_for_debug(kc, ks), oracle.dequant_per_head(kc, ks, head_axis=2))
    a = package("triton_ops.int8_paged_attention")
    q = torch.randn(1, 28, 128, generator=g).to(torch.bfloat16)
    bt = torch.tensor([[0, 1]], dtype=torch.int32)
    out = a.torch_int8_paged_attention_reference(q, kc, vc, bt, torch.tensor([24]), ks, vs)
    want = oracle.int8_paged_attention_oracle(q, kc, vc, bt, [24], ks, vs)
    assert out.dtype == torch.bfloat16
    assert float((out.float() - want).abs().max()) < 1e-2


def test_decode_gate_and_cache_pool():
    patch = package("vllm_int8.vllm_int8_attention_patch")
    pool = package("vllm_int8.cache_manager")

    class Meta:
        pass

    m = Meta()
    m.seq_lens = torch.tensor([5, 9])
    m.block_table = torch.zeros(2, 3, dtype=torch.int32)
    m.num_actual_tokens = 2
    m.max_query_len = 1
    q = torch.zeros(4, 28, 128)  # padded query
    assert patch._is_supported_decode(q, m)
    m.max_query_len = 7
    assert not patch._is_supported_decode(q, m)  # prefill
    m.max_query_len = 1
    m.num_actual_tokens = 3
    assert not patch._is_supported_decode(q, m)
    assert not patch._is_supported_decode(q, None)
    assert not patch._is_supported_decode(q[0], m)
    pool.clear_cache_pool()
    entry = pool.allocate_layer_cache(layer_name="model.layers.3.self_attn.attn", num_blocks=4, block_size=16,
                                      num_kv_heads=4, head_dim=128, k_scale=torch.ones(4), v_scale=torch.ones(4),
                                      device="cpu")
    assert entry.key_cache.shape == (4, 16, 4, 128) and entry.key_cache.dtype == torch.int8
    assert int(entry.value_cache.abs().max()) == 0
    assert pool.has_layer_cache("model.layers.3.self_attn.attn") and pool.get_layer_cache("model.layers.3.self_attn.attn") is entry
    pool.clear_cache_pool()
    assert not pool.has_layer_cache("model.layers.3.self_attn.attn")


def test_workload_generators_are_seeded_and_shaped(workloads):
    a = workloads.config1_case(seed=0)
    b = workloads.config1_case(seed=0)
    c = workloads.config1_case(seed=1)
    assert torch.equal(a.key, b.key) and torch.equal(a.block_tables, b.block_tables) and not torch.equal(a.key, c.key)
    assert a.query.shape == (1, 28, 128) and a.key.shape == (513, 4, 128) and a.num_blocks == 64
    assert a.block_tables.shape == (1, 33) and len(set(a.block_tables[0].tolist())) == 33
    assert int(a.slot_mapping[512]) == int(a.block_tables[0, 32]) * 16
    # outlier channels: exactly four channels per head with ~8x the spread
    std = a.key.float().std(dim=0)  # [Hkv, D]
    assert ((std > 4).sum(dim=1) == 4).all()
    assert 0.4 < float(a.value.float().std()) < 0.6
    # calibrated scales saturate little: a few values beyond the calibration range clip at 127
    q = oracle.static_quant_per_head(a.key, a.k_scale, head_axis=1)
    assert int(q.abs().max()) == 127 and float((q.abs() == 127).float().mean()) < 1e-3
    key, value, slots, ks, vs, nb = workloads.prefill_write_case(2, 256, seed=3)
    assert key.shape == (512, 4, 128) and nb == 32
    live = slots[slots >= 0]
    assert live.unique().numel() == live.numel() and 0 < int((slots < 0).sum()) < 60


def test_head_batch_partition(kv):
    sh = package("sharding")
    for world, want_heads, want_batch in ((1, (0, 4), (0, 256)), (2, (2, 4), (0, 256)), (4, (3, 4), (0, 256)), (8, (3, 4), (128, 256))):
        shards = sh.head_batch_partition(world, 28, 4, 256)
        assert len(shards) == world
        last = shards[-1]
        assert last.kv_heads == want_heads and last.batch == want_batch
        assert last.q_heads == (want_heads[0] * 7, want_heads[1] * 7)
        covered = torch.zeros(4, 256, dtype=torch.int32)
        for s in shards:
            covered[s.kv_heads[0]:s.kv_heads[1], s.batch[0]:s.batch[1]] += 1
        assert int(covered.min()) == 1 and int(covered.max()) == 1
    with pytest.raises(ValueError):
        sh.head_batch_partition(8, 28, 4, 255)
    # the sharded views select exactly the owned heads and sequences
    q = torch.arange(6 * 28).reshape(6, 28, 1).float()
    kc = torch.zeros(3, 16, 4, 8)
    s = sh.head_batch_partition(8, 28, 4, 6)[5]
    qs, kcs, _, bts, sls, ks, _ = sh.shard_decode_inputs(s, q, kc, kc, torch.zeros(6, 2), torch.zeros(6), torch.arange(4.), torch.arange(4.))
    assert qs.shape == (3, 7, 1) and kcs.shape == (3, 16, 1, 8) and bts.shape == (3, 2) and sls.shape == (3,)
    assert float(ks[0]) == float(s.kv_heads[0]) and float(qs[0, 0, 0]) == float(s.batch[0] * 28 + s.q_heads[0])


def test_sequence_split_lengths(kv):
    sh = package("sharding")
    lens = [65536, 1000, 16, 1]
    total = [0] * 4
    for r in range(8):
        lo, hi, local = sh.sequence_split(lens, r, 8, 16)
        assert hi - lo == 512
        total = [a + b for a, b in zip(total, local)]
        if r > 0:
            assert local[2] == 0 and local[3] == 0
    assert total == lens
    assert sh.sequence_split([100], 1, 2, 16, blocks_per_rank=2) == (2, 4, [32])


def test_static_scales_lookup_and_native_page_dims(tmp_path):
    sc = package("vllm_int8.static_scales")
    sh = package("vllm_int8.vllm_shadow_cache_patch")
    k = torch.arange(28 * 4, dtype=torch.float32).reshape(28, 4) / 100 + 0.01
    path = tmp_path / "scales.pt"
    torch.save({"k_scale": k, "v_scale": k * 2, "k_amax": k * 127, "v_amax": k * 254}, path)
    sc.clear_static_scales()
    with pytest.raises(RuntimeError):
        sc.get_layer_scales("model.layers.3.self_attn.attn", "cpu")
    sc.load_static_scales(str(path))
    ks, vs = sc.get_layer_scales("model.layers.12.self_attn.attn", "cpu")
    assert torch.equal(ks, k[12]) and torch.equal(vs, 2 * k[12]) and ks.is_contiguous() and ks.dtype == torch.float32
    assert sc.extract_layer_idx("language_model.model.layers.27.self_attn.attn") == 27
    with pytest.raises(RuntimeError):
        sc.extract_layer_idx("lm_head")
    # the three native cache layouts of the engine
    assert sh._infer_native_page_dims(torch.empty(9, 4, 16, 256), 4) == (9, 16)
    assert sh._infer_native_page_dims(torch.empty(9, 2, 16, 4, 128), 4) == (9, 16)
    assert sh._infer_native_page_dims(torch.empty(2, 9, 32, 4, 128), 4) == (9, 32)
    with pytest.raises(ValueError):
        sh._infer_native_page_dims(torch.empty(9, 16), 4)
    sc.clear_static_scales()


def test_shadow_cache_patch_wiring_with_a_fake_engine_class():
    """The patched method runs the original first, allocates the layer's INT8 cache once from the native page
    geometry and the layer's scales, and hands the flattened slots to the write operator."""
    sc = package("vllm_int8.static_scales")
    sh = package("vllm_int8.vllm_shadow_cache_patch")
    pool = package("vllm_int8.cache_manager")
    pool.clear_cache_pool()
    sh.WRITE_CALL_COUNT.clear()
    sc.set_static_scales(torch.full((4, 2), 0.05), torch.full((4, 2), 0.07))
    calls = []

    class FakeImpl:
        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            calls.append("native")

    class Layer:
        layer_name = "model.layers.2.self_attn.attn"

    def fake_writer(key, value, kc, vc, slots, ks, vs):
        calls.append(("int8", tuple(kc.shape), slots.tolist(), float(ks[0]), float(vs[0])))

    key = torch.zeros(3, 2, 8)
    native = torch.zeros(5, 2, 16, 16)  # fused layout [blocks, Hkv, BS, 2D]
    sh.shadow_cache_update(Layer(), key, key, native, torch.tensor([[4], [5], [-1]]), writer=fake_writer)
    assert calls[-1] == ("int8", (5, 16, 2, 8), [4, 5, -1], pytest.approx(0.05), pytest.approx(0.07))
    assert sh.WRITE_CALL_COUNT[Layer.layer_name] == 1 and sh.NATIVE_CACHE_BYTES_BY_LAYER[Layer.layer_name] == native.numel() * 4
    first = pool.get_layer_cache(Layer.layer_name)
    sh.shadow_cache_update(Layer(), key, key, native, torch.tensor([6, 7, 8]), writer=fake_writer)
    assert pool.get_layer_cache(Layer.layer_name) is first and sh.WRITE_CALL_COUNT[Layer.layer_name] == 2
    with pytest.raises(AssertionError):
        sh.shadow_cache_update(Layer(), key, key, native, torch.tensor([6, 7]), writer=fake_writer)
    # class wrapping is idempotent and keeps the original call first (the INT8 write itself needs a GPU)
    assert sh.apply_shadow_cache_patch(FakeImpl) is FakeImpl
    patched = FakeImpl.do_kv_cache_update
    sh.apply_shadow_cache_patch(FakeImpl)
    assert FakeImpl.do_kv_cache_update is patched
    pool.clear_cache_pool()
    sc.clear_static_scales()


def test_attention_patch_falls_back_outside_decode_and_rejects_unknown_modes():
    ap = package("vllm_int8.vllm_int8_attention_patch")
    pool = package("vllm_int8.cache_manager")
    pool.clear_cache_pool()

    class FakeImpl:
        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output, output_scale=None,
                    output_block_scale=None):
            output.fill_(3.0)
            return output

    with pytest.raises(ValueError):
        ap.apply_int8_attention_patch(FakeImpl, mode="fast")
    ap.apply_int8_attention_patch(FakeImpl, mode="int8_only")
    with pytest.raises(RuntimeError):
        ap.apply_int8_attention_patch(FakeImpl, mode="shadow")

    class Layer:
        layer_name = "model.layers.0.self_attn.attn"

    out = torch.zeros(2, 28, 128)
    # no INT8 cache for the layer -> original forward
    res = FakeImpl().forward(Layer(), torch.zeros(2, 28, 128), None, None, None, None, out)
    assert res is out and float(out.min()) == 3.0 and ap.ATTN_INT8_HITS.get(Layer.layer_name, 0) == 0


def test_attention_call_site_passes_a_length_bound_instead_of_reading_seq_lens(monkeypatch):
    """The reference's operator reads seq_lens back on the host twice per call
    (src/triton_ops/int8_paged_attention.py:720-721); the call site here hands the operator an upper bound taken from
    the engine's metadata, or from the block table's width, so that no device value is read."""
    ap = package("vllm_int8.vllm_int8_attention_patch")
    pool = package("vllm_int8.cache_manager")
    pool.clear_cache_pool()
    seen = {}

    def fake_attention(query, kc, vc, block_tables, seq_lens, ks, vs, **kw):
        seen.update(kw, query_shape=tuple(query.shape), table_is_same=block_tables)
        return torch.zeros_like(query)

    monkeypatch.setattr(ap, "int8_paged_attention", fake_attention)

    class Layer:
        layer_name = "model.layers.3.self_attn.attn"

    pool.INT8_CACHE_POOL[Layer.layer_name] = pool.LayerInt8Cache(
        key_cache=torch.zeros(6, 16, 2, 8, dtype=torch.int8), value_cache=torch.zeros(6, 16, 2, 8, dtype=torch.int8),
        k_scale=torch.ones(2), v_scale=torch.ones(2))

    class Meta:
        seq_lens = torch.tensor([40, 17])
        block_table = torch.zeros(2, 5, dtype=torch.int32)
        num_actual_tokens = 2

    q = torch.zeros(4, 4, 8)
    ap._run_int8_attention(Layer(), q, Meta())
    assert seen["max_seq_len"] == 5 * 16 and seen["query_shape"] == (2, 4, 8) and seen["table_is_same"] is Meta.block_table
    Meta.max_seq_len = 40  # the engine's own bound wins when it is a host integer ...
    ap._run_int8_attention(Layer(), q, Meta())
    assert seen["max_seq_len"] == 40
    Meta.max_seq_len = 10 ** 6  # ... and never exceeds what the table can address
    ap._run_int8_attention(Layer(), q, Meta())
    assert seen["max_seq_len"] == 80
    Meta.max_seq_len = torch.tensor(40)  # a tensor would have to be read back: the table's width is used
    ap._run_int8_attention(Layer(), q, Meta())
    assert seen["max_seq_len"] == 80
    pool.clear_cache_pool()


def test_scale_calibration_accumulates_running_maxima(tmp_path):
    cal_mod = package("calibration")
    sc = package("vllm_int8.static_scales")
    g = torch.Generator().manual_seed(1)
    cal = cal_mod.ScaleCalibrator(num_layers=3, num_kv_heads=4)
    dumps = [{l: {"k": torch.randn(2, 4, 10, 128, generator=g).half() * (l + 1),
                  "v": torch.randn(2, 4, 10, 128, generator=g).half()} for l in (0, 2)} for _ in range(3)]
    for d in dumps:
        cal.observe_dump(d)
    out = cal.scales()
    for l in (0, 2):
        k_all = torch.cat([d[l]["k"] for d in dumps]).float()
        assert torch.equal(out["k_amax"][l], k_all.abs().amax(dim=(0, 2, 3)))
        assert torch.equal(out["k_scale"][l], (out["k_amax"][l] / 127.0).clamp_min(1e-6))
    assert torch.equal(out["k_scale"][1], torch.full((4,), 1e-6))  # a layer never observed floors at 1e-6
    # token-major observation ([T, Hkv, D], head axis 1) and the file round trip into the scale lookup
    cal.observe(1, torch.ones(5, 4, 8) * 2.54, torch.ones(5, 4, 8), head_axis=1)
    path = tmp_path / "scales.pt"
    cal.save(str(path))
    sc.load_static_scales(str(path))
    ks, vs = sc.get_layer_scales("model.layers.1.self_attn.attn", "cpu")
    assert torch.allclose(ks, torch.full((4,), 0.02)) and torch.allclose(vs, torch.full((4,), 1 / 127.0))
    sc.clear_static_scales()
