"""GPU parity of the INT8 cache write, through the C ABI, against the oracle and the reference's
golden vectors.  The bar is bit-exact INT8 bytes and bit-exact placement (untouched bytes stay)."""

import pytest
import torch

import oracle
from conftest import load_golden

pytestmark = pytest.mark.gpu
CANARY = 0x55


def _gpu_write(kv, key, value, kc_shape, slots, ks, vs, fill=0, slot_dtype=None):
    dev = "cuda"
    kc = torch.full(kc_shape, fill, dtype=torch.int8, device=dev)
    vc = torch.full(kc_shape, fill, dtype=torch.int8, device=dev)
    s = slots.to(dev) if slot_dtype is None else slots.to(dev, slot_dtype)
    kv.int8_kv_cache_write(key.to(dev), value.to(dev), kc, vc, s, ks.to(dev), vs.to(dev))
    torch.cuda.synchronize()
    return kc.cpu(), vc.cpu()


@pytest.mark.parametrize("name", ["write_t37", "write_n23", "attn_127_301", "attn_97_256"])
def test_golden_cases_bit_exact(kv, name):
    g = load_golden(name)
    kc, vc = _gpu_write(kv, g["key"], g["value"], g["key_cache"].shape, g["slot_mapping"], g["k_scale"], g["v_scale"])
    assert torch.equal(kc, g["key_cache"])
    assert torch.equal(vc, g["value_cache"])


def test_runtime_entry_point_matches_golden(kv):
    from conftest import package

    rt = package("vllm_int8.vllm_int8_cache_ops")
    g = load_golden("write_n23")
    kc = torch.zeros(g["key_cache"].shape, dtype=torch.int8, device="cuda")
    vc = torch.zeros_like(kc)
    rt.runtime_int8_cache_write(g["key"].cuda(), g["value"].cuda(), kc, vc, g["slot_mapping"].cuda(),
                                g["k_scale"].cuda(), g["v_scale"].cuda())
    assert torch.equal(kc.cpu(), g["key_cache"]) and torch.equal(vc.cpu(), g["value_cache"])


def test_real_activations_fp16_input(kv):
    g = load_golden("real_layer27")
    k = g["k"].permute(0, 2, 1, 3).reshape(40, 4, 128).contiguous()  # [tokens, Hkv, D] fp16
    v = g["v"].permute(0, 2, 1, 3).reshape(40, 4, 128).contiguous()
    slots = torch.arange(40, dtype=torch.int64)
    kc, vc = _gpu_write(kv, k, v, (3, 16, 4, 128), slots, g["k_scale"], g["v_scale"])
    want_k = g["k_q"].permute(0, 2, 1, 3).reshape(40, 4, 128)
    want_v = g["v_q"].permute(0, 2, 1, 3).reshape(40, 4, 128)
    assert torch.equal(kc.reshape(48, 4, 128)[:40], want_k)
    assert torch.equal(vc.reshape(48, 4, 128)[:40], want_v)
    assert int(kc.reshape(48, 4, 128)[40:].abs().max()) == 0


def test_prefill_write_full_size_with_padding_slots(kv, workloads):
    """16384 tokens, permuted 1024-block pool, ~3% slots = -1; canary-filled caches show skipped rows."""
    key, value, slots, ks, vs, nb = workloads.prefill_write_case(8, 2048, seed=0)
    shape = (nb, 16, 4, 128)
    kc, vc = _gpu_write(kv, key, value, shape, slots, ks, vs, fill=CANARY)
    kc_o = torch.full(shape, CANARY, dtype=torch.int8)
    vc_o = torch.full(shape, CANARY, dtype=torch.int8)
    oracle.cache_write(key, value, kc_o, vc_o, slots, ks, vs)
    assert torch.equal(kc, kc_o) and torch.equal(vc, vc_o)
    skipped = int((slots < 0).sum())
    assert skipped > 0
    # every skipped token leaves one 4x128 row of canaries in each cache
    assert int((kc.reshape(-1, 512) == CANARY).all(dim=1).sum()) >= skipped


@pytest.mark.parametrize("dtype,heads,dim,tokens,bs", [
    (torch.bfloat16, 4, 128, 2048 + 37, 16),
    (torch.float16, 8, 128, 4099, 32),
    (torch.float32, 4, 128, 2500, 16),         # fp32 rows: four 16-byte pieces per unit
    (torch.bfloat16, 2, 64, 3000, 16),
    (torch.bfloat16, 16, 256, 2048, 16),
    (torch.float32, 3, 48, 2100, 16),          # units per token not a power of two: division instead of shifts
])
def test_large_writes_special_values_and_random_slot_order(kv, dtype, heads, dim, tokens, bs):
    """Thousands of tokens, several row widths and input types: int32 slots in random order over a pool larger than
    the write, padding slots, exact rounding ties, huge, infinite and NaN inputs (the quantiser's packed fast path has
    no range test of its own: saturation and the exact branch must come out right all the same), canaries around."""
    g = torch.Generator().manual_seed(tokens)
    key = torch.randn(tokens, heads, dim, generator=g).to(dtype)
    value = (torch.randn(tokens, heads, dim, generator=g) * 0.5).to(dtype)
    k_scale = torch.rand(heads, generator=g) * 0.02 + 0.01
    v_scale = torch.full((heads,), 0.0078125)  # 2^-7: every multiple of 2^-8 among the values is an exact tie
    special = torch.tensor([1e9, -1e9, float("inf"), float("-inf"), float("nan"), 0.0, -0.0, 3.0])
    if dtype == torch.float32:
        special[:2] = torch.tensor([3e38, -3e38])  # quotients far beyond the range in which the rounding trick is exact
    key[5, 0, :8] = special.to(dtype)
    value[7, 1, :8] = (torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, 126.5, -126.5, 127.5]) * 0.0078125).to(dtype)
    if dtype != torch.float16:  # quotients around -1.5 * 2^23 and -3 * 2^23, where the rounding constant's sum changes sign
        value[9, 0, :8] = (torch.tensor([-1.2e7, -1.3e7, -2e7, -2.5e7, -2.6e7, -3.4e7, 1.3e7, 2.6e7]) * 0.0078125).to(dtype)
    num_blocks = (tokens + bs - 1) // bs + 9
    perm = torch.randperm(num_blocks * bs, generator=g)[:tokens]
    slots = perm.to(torch.int32)
    slots[torch.rand(tokens, generator=g) < 0.02] = -1
    slots[9] = perm[9].to(torch.int32)  # the row of huge quotients is written, not padding
    shape = (num_blocks, bs, heads, dim)
    kc, vc = _gpu_write(kv, key, value, shape, slots, k_scale, v_scale, fill=CANARY)
    kc_o = torch.full(shape, CANARY, dtype=torch.int8)
    vc_o = torch.full(shape, CANARY, dtype=torch.int8)
    oracle.cache_write(key, value, kc_o, vc_o, slots.long(), k_scale, v_scale)
    assert torch.equal(kc, kc_o) and torch.equal(vc, vc_o)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("slot_dtype", [torch.int32, torch.int64])
def test_input_and_slot_dtypes(kv, dtype, slot_dtype):
    g = torch.Generator().manual_seed(3)
    T, H, D = 133, 4, 128
    key = (torch.randn(T, H, D, generator=g) * 2).to(dtype)
    value = torch.randn(T, H, D, generator=g).to(dtype)
    ks = torch.tensor([0.02, 0.031, 0.017, 0.05])
    vs = torch.tensor([0.011, 0.02, 0.03, 0.009])
    perm = torch.randperm(16 * 12, generator=g)[:T]
    perm[::17] = -1
    kc, vc = _gpu_write(kv, key, value, (12, 16, H, D), perm, ks, vs, fill=CANARY, slot_dtype=slot_dtype)
    kc_o = torch.full((12, 16, H, D), CANARY, dtype=torch.int8)
    vc_o = torch.full_like(kc_o, CANARY)
    oracle.cache_write(key, value, kc_o, vc_o, perm, ks, vs)
    assert torch.equal(kc, kc_o) and torch.equal(vc, vc_o)


def test_strided_views_and_odd_head_dim(kv):
    """vLLM hands the write views into a fused qkv buffer; odd head dims take the element path."""
    g = torch.Generator().manual_seed(9)
    T, H, D = 57, 2, 80
    fused = torch.randn(T, 3 * H * D + 5, generator=g).to(torch.bfloat16)
    key = fused[:, 5 : 5 + H * D].view(T, H, D)  # misaligned start, token stride != H*D
    value = fused[:, 5 + H * D : 5 + 2 * H * D].view(T, H, D)
    ks = torch.tensor([0.02, 0.04])
    vs = torch.tensor([0.03, 0.01])
    slots = torch.arange(T, dtype=torch.int64) + 3
    dev = "cuda"
    fused_d = fused.to(dev)
    key_d = fused_d[:, 5 : 5 + H * D].view(T, H, D)
    value_d = fused_d[:, 5 + H * D : 5 + 2 * H * D].view(T, H, D)
    kc = torch.zeros(8, 8, H, D, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    kv.int8_kv_cache_write(key_d, value_d, kc, vc, slots.to(dev), ks.to(dev), vs.to(dev))
    kc_o = torch.zeros(8, 8, H, D, dtype=torch.int8)
    vc_o = torch.zeros_like(kc_o)
    oracle.cache_write(key, value, kc_o, vc_o, slots, ks, vs)
    assert torch.equal(kc.cpu(), kc_o) and torch.equal(vc.cpu(), vc_o)
    # aligned strided view (vector path): D=128 slice of a wider buffer
    T, H, D = 64, 4, 128
    wide = torch.randn(T, 3 * H * D, generator=g).to(torch.bfloat16)
    wide_d = wide.to(dev)
    k2, v2 = wide[:, : H * D].view(T, H, D), wide[:, H * D : 2 * H * D].view(T, H, D)
    k2d, v2d = wide_d[:, : H * D].view(T, H, D), wide_d[:, H * D : 2 * H * D].view(T, H, D)
    ks = torch.tensor([0.02, 0.04, 0.03, 0.025])
    slots = torch.randperm(64, generator=g)
    kc = torch.zeros(4, 16, H, D, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    kv.int8_kv_cache_write(k2d, v2d, kc, vc, slots.to(dev), ks.to(dev), ks.to(dev))
    kc_o = torch.zeros(4, 16, H, D, dtype=torch.int8)
    vc_o = torch.zeros_like(kc_o)
    oracle.cache_write(k2, v2, kc_o, vc_o, slots, ks, ks)
    assert torch.equal(kc.cpu(), kc_o) and torch.equal(vc.cpu(), vc_o)


def test_rounding_ties_saturation_and_out_of_range_slots(kv):
    """Exact .5 quotients round to even, large values saturate at +-127, slots past the pool are skipped."""
    scale = torch.tensor([0.5, 0.25, 1.0, 2.0])
    base = torch.tensor([0.25, 0.75, 1.25, -0.25, -0.75, 63.25, 63.75, -63.75, 1e4, -1e4, 0.0, 31.875])
    key = base.repeat(11)[:128].reshape(1, 1, 128).repeat(6, 4, 1).to(torch.bfloat16)
    value = (-key).clone()
    slots = torch.tensor([0, 5, 17, 31, 32, 999], dtype=torch.int64)  # pool holds 32 slots
    kc, vc = _gpu_write(kv, key, value, (2, 16, 4, 128), slots, scale, scale, fill=CANARY)
    kc_o = torch.full((2, 16, 4, 128), CANARY, dtype=torch.int8)
    vc_o = torch.full_like(kc_o, CANARY)
    oracle.cache_write(key[:4], value[:4], kc_o, vc_o, slots[:4], scale, scale)
    assert torch.equal(kc, kc_o) and torch.equal(vc, vc_o)
    assert int(kc.max()) == 127 and int(kc.min()) == -127


def test_empty_and_argument_errors(kv):
    dev = "cuda"
    kc = torch.zeros(2, 16, 4, 128, dtype=torch.int8, device=dev)
    vc = torch.zeros_like(kc)
    s = torch.ones(4, device=dev)
    empty = torch.zeros(0, 4, 128, dtype=torch.bfloat16, device=dev)
    kv.int8_kv_cache_write(empty, empty, kc, vc, torch.zeros(0, dtype=torch.int64, device=dev), s, s)
    key = torch.zeros(3, 4, 128, dtype=torch.bfloat16, device=dev)
    with pytest.raises(AssertionError):
        kv.int8_kv_cache_write(key, key, kc, vc, torch.zeros(2, dtype=torch.int64, device=dev), s, s)
    with pytest.raises(AssertionError):
        kv.int8_kv_cache_write(key, key, kc.float(), vc, torch.zeros(3, dtype=torch.int64, device=dev), s, s)
    with pytest.raises(AssertionError):
        kv.int8_kv_cache_write(key, key, kc, vc, torch.zeros(3, dtype=torch.float32, device=dev), s, s)


def test_dynamic_per_token_head_write(kv):
    """The reference's alternative scheme: bit-exact against the restated kernel arithmetic, and the
    reference test's own bound (mean abs dequantisation error < 0.02; tests/test_vllm_int8_cache_ops.py).
    Parity unpinned: the reference defines this scheme only as a Triton kernel (no CPU definition to run), so the
    byte-level expectation is this repository's restatement of that kernel; the MAE bound is all the reference holds."""
    from conftest import package

    ops = package("vllm_int8.vllm_int8_cache_ops")
    g = torch.Generator().manual_seed(0)
    # D = 128, 64, 256, 512, 16 take the vector kernel (D / 16 lanes per row); 80 and 576 the general one
    for dtype, D in ((torch.bfloat16, 128), (torch.float16, 80), (torch.float32, 576), (torch.float16, 64),
                     (torch.float32, 256), (torch.bfloat16, 512), (torch.float32, 128), (torch.bfloat16, 16)):
        T, H = 23, 4
        key = torch.randn(T, H, D, generator=g).to(dtype)
        value = (torch.randn(T, H, D, generator=g) * 3).to(dtype)
        key[3, 1] = 0  # all-zero row: scale floors at 1e-6
        # exact ties: absmax 127 makes the scale exactly 1, so x.5 sits on a rounding boundary (half away from zero)
        ties = torch.tensor([127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5, 63.5, 0.25, -0.75, 3.0, -127.0, 8.5, -8.5])
        key[4, 2, :16] = ties.to(dtype)
        value[5, 0, :16] = (ties * 0.5).to(dtype)  # scale 0.5: the same quotients
        slots = torch.arange(7, 7 + T, dtype=torch.int64)
        slots[5] = -1
        kc, vc, ksc, vsc = ops.allocate_int8_kv_cache(32, 16, H, D, device="cuda")
        for t in (kc, vc):
            t.fill_(CANARY)
        ksc.fill_(-1.0)
        vsc.fill_(-1.0)
        ops.reshape_and_cache_int8(key.cuda(), value.cuda(), kc, vc, ksc, vsc, slots.cuda())
        kq, ks = oracle.dynamic_quant_per_token_head(key)
        vq, vs = oracle.dynamic_quant_per_token_head(value)
        kc_o = torch.full((32 * 16, H, D), CANARY, dtype=torch.int8)
        vc_o = torch.full_like(kc_o, CANARY)
        ks_o = torch.full((32 * 16, H), -1.0)
        vs_o = torch.full_like(ks_o, -1.0)
        live = slots >= 0
        kc_o[slots[live]], vc_o[slots[live]] = kq[live], vq[live]
        ks_o[slots[live]], vs_o[slots[live]] = ks[live], vs[live]
        assert torch.equal(kc.cpu().reshape(-1, H, D), kc_o) and torch.equal(vc.cpu().reshape(-1, H, D), vc_o)
        assert torch.equal(ksc.cpu().reshape(-1, H), ks_o) and torch.equal(vsc.cpu().reshape(-1, H), vs_o)
        deq = ops.dequantize_int8_cache(kc, ksc).cpu().reshape(-1, H, D)[slots[live]]
        assert float((deq - key[live].float()).abs().mean()) < 0.02
        assert ops.int8_cache_memory_bytes(kc, vc, ksc, vsc) == (2 * 32 * 16 * H * D, 2 * 32 * 16 * H * 4)
