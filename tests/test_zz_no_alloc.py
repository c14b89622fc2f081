"""The allocation-free attention entry point, called through the C ABI.

Some callers cannot give the library a split-KV workspace because they cannot allocate one: an engine
whose KV-cache pool already owns all free HBM, or a request loop in which cudaMalloc (a device-wide
synchronisation that may also fail) is off limits.  `int8kv_paged_attn_int8_static_ws` serves them from
a fixed buffer inside the library.  This file checks that it returns what the ordinary entry point
returns, on two calls in a row that reuse the buffer with different shapes, with the INT8-query option,
on a shape outside the tiled kernels and with parts planned on the device; that a shape whose partial
rows exceed the buffer is refused; and that the status word of that buffer, which is where a kernel
reports a wait that ran out, can be read (and cleared) without allocating.  It is named so that pytest
collects it last.
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


def _static_status(lib, clear=True):
    """The status word of the library's workspace, copied into a pinned host word by the library itself."""
    word = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    rc = lib.int8kv_static_ws_status(C.c_void_p(word.data_ptr()), int(clear), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    return int(word[0])


def _both_entry_points(lib_mod, lib, case, kc, vc, splits, flags=0):
    dev = "cuda"
    q, kcd, vcd = case.query.to(dev), kc.to(dev), vc.to(dev)
    bt, sl = case.block_tables.to(dev), case.seq_lens.to(dev)
    ks, vs = case.k_scale.to(dev), case.v_scale.to(dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    B, Hq, D = q.shape
    # existing entry point, workspace owned by the caller
    want = torch.empty_like(q)
    nbytes = lib.int8kv_workspace_bytes(B, Hq, D, splits if splits > 0 else lib.int8kv_max_splits())
    nbytes = max(nbytes, lib.int8kv_workspace_bytes_auto(B, Hq, kcd.shape[2], D, int(sl.max()), kcd.shape[1], 148))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    rc = lib.int8kv_paged_attn_int8(*_args(lib_mod, q, kcd, vcd, bt, sl, ks, vs, want), splits, _ptr(ws), ws.numel(), flags, stream)
    assert rc == 0, lib_mod.status_str(rc)
    # allocation-free entry point: inputs and output only
    got = torch.full_like(q, float("nan"))
    rc = lib.int8kv_paged_attn_int8_static_ws(*_args(lib_mod, q, kcd, vcd, bt, sl, ks, vs, got), splits, flags, stream)
    assert rc == 0, lib_mod.status_str(rc)
    torch.cuda.synchronize()
    assert _static_status(lib) == 0  # no wait ran out inside the library's buffer
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


def test_static_workspace_entry_point_options_and_other_shapes():
    """The INT8-query option, parts planned on the device (num_splits -1), and a layer shape outside the tiled
    kernels with the automatic count (where the rule of those kernels, not of the tiled ones, picks it)."""
    lib_mod = package("_lib")
    lib = lib_mod.load()
    wl = package("workloads")
    for seed, shape, lens, splits, flags in (
        (41, wl.QWEN25_7B, [700, 45, 260, 1], 0, lib_mod.FLAG_QUANTIZE_Q),
        (42, wl.QWEN25_7B, [700, 45, 260, 1, 2048], lib_mod.SPLITS_PLANNED, 0),
        (43, wl.LayerShape(8, 2, 64, 16), [900, 33, 260], 0, 0),
        (44, wl.LayerShape(8, 2, 64, 16), [900, 33, 260], 0, lib_mod.FLAG_QUANTIZE_Q),
    ):
        case = wl.make_decode_case(lens, shape, seed=seed)
        kc = torch.zeros(case.num_blocks, shape.block_size, shape.num_kv_heads, shape.head_dim, dtype=torch.int8)
        vc = torch.zeros_like(kc)
        oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
        got, want = _both_entry_points(lib_mod, lib, case, kc, vc, splits, flags)
        assert torch.isfinite(got).all()
        assert max_abs(got, want) <= 2e-2 and cosine(got, want) >= 0.9999
        ref = oracle.int8_paged_attention_oracle(case.query, kc, vc, case.block_tables, lens, case.k_scale, case.v_scale,
                                                 quantize_q=bool(flags & lib_mod.FLAG_QUANTIZE_Q))
        assert max_abs(got, ref.to(torch.bfloat16).float()) <= 2e-2 and cosine(got, ref) >= 0.9999


def test_static_workspace_status_word_reports_a_wait_that_ran_out():
    """The failure report of callers that own no workspace: the library's bounded-wait self-test, pointed at the
    library's own buffer, must show up in the word that int8kv_static_ws_status copies out; reading with `clear`
    resets it, and attention through the same buffer works afterwards.  The self-test kernel waits a bounded number
    of times for bytes that nothing sends and returns normally."""
    lib_mod = package("_lib")
    lib = lib_mod.load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    base = C.c_void_p()
    assert lib.int8kv_static_ws_address(C.byref(base)) == 0 and base.value
    _static_status(lib)  # start from a cleared word
    assert lib.int8kv_selftest_bounded_wait(base, lib_mod.STATIC_WS_BYTES, 200, stream) == 0
    assert _static_status(lib, clear=False) == lib_mod.DEV_WAIT_TIMEOUT  # reported, and kept without a clear
    assert _static_status(lib, clear=True) == lib_mod.DEV_WAIT_TIMEOUT
    assert _static_status(lib) == 0
    wl = package("workloads")
    case = wl.make_decode_case([300, 17], wl.QWEN25_7B, seed=45)
    kc = torch.zeros(case.num_blocks, 16, 4, 128, dtype=torch.int8)
    vc = torch.zeros_like(kc)
    oracle.cache_write(case.key, case.value, kc, vc, case.slot_mapping, case.k_scale, case.v_scale)
    got, want = _both_entry_points(lib_mod, lib, case, kc, vc, 4)
    assert max_abs(got, want) <= 2e-2 and cosine(got, want) >= 0.9999


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
