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
