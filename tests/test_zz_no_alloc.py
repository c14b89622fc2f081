"""The allocation-free attention entry point, called through the C ABI.

Some callers cannot give the library a split-KV workspace because they cannot allocate one: an engine
whose KV-cache pool already owns all free HBM, or a request loop in which cudaMalloc (a device-wide
synchronisation that may also fail) is off limits.  `int8kv_paged_attn_int8_static_ws` serves them from
a fixed buffer inside the library.  This file checks that it returns what the ordinary entry point
returns, on two calls in a row that reuse the buffer with different shapes, and that a shape whose
partial rows exceed the buffer is refused.  It is named so that pytest collects it last.
"""

import ctypes as C

import pytest
import torch

import oracle
from conftest import cosine, max_abs, package

pytestmark = pytest.mark.gpu
CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _args(lib_mod, q, kc, vc, bt, sl, ks, vs, out):
    B, Hq, D = q.shape
    return [
        _ptr(q), CODE[q.dtype], lib_mod.i64(q.stride()), B, Hq, kc.shape[2], D,
        _ptr(kc), _ptr(vc), lib_mod.i64(kc.stride()), lib_mod.i64(vc.stride()), kc.shape[0], kc.shape[1],
        _ptr(bt), int(bt.dtype == torch.int64), lib_mod.i64(bt.stride()), bt.shape[1],
        _ptr(sl), int(sl.dtype == torch.int64), int(sl.max()),
        _ptr(ks), _ptr(vs), _ptr(out), CODE[out.dtype], lib_mod.i64(out.stride()),
    ]


def _both_entry_points(lib_mod, lib, case, kc, vc, splits):
    dev = "cuda"
    q, kcd, vcd = case.query.to(dev), kc.to(dev), vc.to(dev)
    bt, sl = case.block_tables.to(dev), case.seq_lens.to(dev)
    ks, vs = case.k_scale.to(dev), case.v_scale.to(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, Hq, D = q.shape
    # existing entry point, workspace owned by the caller
    want = torch.empty_like(q)
    nbytes = lib.int8kv_workspace_bytes(B, Hq, D, max(splits, 1) if splits else lib.int8kv_max_splits())
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    rc = lib.int8kv_paged_attn_int8(*_args(lib_mod, q, kcd, vcd, bt, sl, ks, vs, want), splits, _ptr(ws), ws.numel(), 0, stream)
    assert rc == 0, lib_mod.status_str(rc)
    # allocation-free entry point: inputs and output only
    got = torch.full_like(q, float("nan"))
    rc = lib.int8kv_paged_attn_int8_static_ws(*_args(lib_mod, q, kcd, vcd, bt, sl, ks, vs, got), splits, 0, stream)
    assert rc == 0, lib_mod.status_str(rc)
    torch.cuda.synchronize()
    return got.float().cpu(), want.float().cpu()


def test_static_workspace_entry_point_matches_the_ordinary_one_twice_in_a_row():
    lib_mod = package("_lib")
    lib = lib_mod.load()
    wl = package("workloads")
    # two different shapes back to back: the second call reuses the buffer the first one filled
    for seed, lens, splits in ((31, [700, 45, 260, 1], 5), (32, [2048, 2048], 0)):
        case = wl.make_decode_case(lens, wl.QWEN25_7B, seed=seed)
        kc = torch.zeros(case.num_blocks, 16, 4, 128, dtype=torch.int8)
        vc = torch.zeros_like(kc)
        oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
        got, want = _both_entry_points(lib_mod, lib, case, kc, vc, splits)
        assert torch.isfinite(got).all()
        assert max_abs(got, want) <= 2e-2 and cosine(got, want) >= 0.9999
        ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale)
        assert max_abs(got, ref.to(torch.bfloat16).float()) <= 2e-2 and cosine(got, ref) >= 0.9999


def test_static_workspace_entry_point_refuses_what_does_not_fit():
    lib_mod = package("_lib")
    lib = lib_mod.load()
    dev = "cuda"
    B, Hq, Hkv, D, splits = 64, 64, 8, 128, 64  # 64*64*64 rows of 528 B = 138 MB of partial rows
    assert lib.int8kv_workspace_bytes(B, Hq, D, splits) > lib_mod.STATIC_WS_BYTES
    q = torch.zeros(B, Hq, D, dtype=torch.bfloat16, device=dev)
    kc = torch.zeros(4, 16, Hkv, D, dtype=torch.int8, device=dev)
    bt = torch.zeros(B, 128, dtype=torch.int32, device=dev)
    sl = torch.full((B,), 2048, dtype=torch.int32, device=dev)
    s = torch.ones(Hkv, device=dev)
    out = torch.full_like(q, 7.0)
    rc = lib.int8kv_paged_attn_int8_static_ws(*_args(lib_mod, q, kc, kc, bt, sl, s, s, out), splits, 0,
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == lib_mod.E_WORKSPACE and "workspace" in lib_mod.status_str(rc)
    torch.cuda.synchronize()
    assert float(out.float().min()) == 7.0  # nothing was launched
