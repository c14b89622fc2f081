"""The C-ABI library on a machine without a GPU: it loads, exports every symbol the header declares, and its
host-only functions and argument validation behave (no kernel is launched here)."""

import ctypes as C
import re
from pathlib import Path

import pytest

from conftest import REPO, package

HEADER = REPO / "include" / "int8kv_b200.h"


@pytest.fixture(scope="module")
def lib():
    return package("_lib").load()


def declared_symbols():
    return sorted(set(re.findall(r"\b(int8kv_[a-z0-9_]+)\s*\(", HEADER.read_text())))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 12
    bound = set(package("_lib").EXPORTED_SYMBOLS)
    for n in names:
        assert hasattr(lib, n), n
        assert n in bound, f"{n} is declared in the header but has no ctypes signature"
    assert bound <= set(names)


def test_abi_version_and_status_strings(lib):
    text = HEADER.read_text()
    assert lib.int8kv_abi_version() == int(re.search(r"#define INT8KV_ABI_VERSION (\d+)", text).group(1))
    codes = {n: int(v) for n, v in re.findall(r"#define (INT8KV_E_[A-Z_]+) \((-\d+)\)", text)}
    assert len(codes) == 6
    seen = set()
    for name, code in codes.items():
        s = lib.int8kv_status_str(code).decode()
        assert s and s != "unknown status" and s not in seen
        seen.add(s)
    assert lib.int8kv_status_str(0).decode() == "ok"
    assert lib.int8kv_status_str(-99).decode() == "unknown status"


def test_workspace_sizing(lib):
    rf = lib.int8kv_partial_row_floats(128)
    assert rf == 132 and rf % 4 == 0
    assert lib.int8kv_partial_row_floats(64) == 68
    assert lib.int8kv_workspace_bytes(8, 28, 128, 1) == 16
    assert lib.int8kv_workspace_bytes(8, 28, 128, 4) == 4 * 8 * 28 * 132 * 4 + 16
    assert lib.int8kv_workspace_bytes(-1, 28, 128, 4) == -1
    n = lib.int8kv_workspace_bytes(8, 28, 128, 4)
    off = lib.int8kv_workspace_status_offset(n)
    assert off % 16 == 0 and n - 16 <= off + 16 <= n
    assert lib.int8kv_workspace_status_offset((1 << 20)) == (1 << 20) - 16


def test_automatic_workspace_covers_the_planned_path(lib):
    auto = lambda B, Hq, Hkv, seq: lib.int8kv_workspace_bytes_auto(B, Hq, Hkv, 128, seq, 16, 148)
    fixed = lambda B, Hq, Hkv, seq: lib.int8kv_workspace_bytes(B, Hq, 128, lib.int8kv_choose_splits(B, Hkv, seq, 16, 148))
    for B, Hq, Hkv, seq in ((1, 28, 4, 512), (8, 28, 4, 4096), (64, 28, 4, 8192), (256, 28, 4, 8192), (32, 64, 8, 65536),
                            (32, 8, 1, 65536), (2000, 28, 4, 8192)):
        assert auto(B, Hq, Hkv, seq) >= fixed(B, Hq, Hkv, seq)
    # one wave of items (1776 warps), seven query heads each, 132 floats per partial row, plus the sequence table
    assert auto(32, 7, 1, 65536) >= 1776 * 7 * 132 * 4 + 32 * 8 + 32
    # more sequences than a plan covers: exactly the fixed size
    assert auto(2000, 28, 4, 8192) == fixed(2000, 28, 4, 8192)
    assert auto(-1, 28, 4, 512) == -1 and auto(8, 30, 4, 512) == -1
    assert lib.int8kv_workspace_bytes_auto(0, 28, 4, 128, 512, 16, 148) == 16


def test_automatic_workspace_covers_the_untiled_kernels(lib):
    """Shapes the tiled kernels refuse (head_dim, block size or group) split by their own rule, one resident wave
    of warps; the automatic size has to hold that many partial rows whichever of the three refuses."""
    rows = lambda B, Hq, D, S: lib.int8kv_workspace_bytes(B, Hq, D, S)
    # head_dim 64, group 4: 16 warps per SM on 148 SMs over 64 x 8 items = 4 parts
    assert lib.int8kv_workspace_bytes_auto(64, 32, 8, 64, 2048, 16, 148) >= rows(64, 32, 64, 4)
    # block size 8 at head_dim 128, group 7: 12 warps per SM over 32 x 4 items = 13 parts
    assert lib.int8kv_workspace_bytes_auto(32, 28, 4, 128, 2048, 8, 148) >= rows(32, 28, 128, 13)
    # group 16 at head_dim 128: 8 warps per SM over 32 x 4 items = 9 parts
    assert lib.int8kv_workspace_bytes_auto(32, 64, 4, 128, 2048, 16, 148) >= rows(32, 64, 128, 9)
    # parts stay at least 128 tokens long
    assert lib.int8kv_workspace_bytes_auto(1, 32, 8, 64, 512, 16, 148) >= rows(1, 32, 64, 4)


def test_split_heuristic(lib):
    cap = lib.int8kv_max_splits()
    assert cap >= 16
    pick = lambda B, H, seq: lib.int8kv_choose_splits(B, H, seq, 16, 148)
    # enough (sequence, head) pairs for four waves of warps on 148 SMs: no split
    assert pick(4096, 4, 8192) == 1
    # a large ragged batch is still cut into a few parts per sequence for balance
    assert 4 <= pick(256, 4, 8192) <= 16
    # ... unless the sequences are short: parts below 32 tiles would mostly move partial rows
    assert pick(256, 4, 512) == 1
    # small calls: one resident wave of warps, never fewer than 2 tiles (32 tokens) per part
    assert pick(1, 4, 100) == 2
    assert pick(1, 4, 512) == 16 and pick(8, 4, 512) == 16
    assert pick(8, 4, 4096) == 32
    # long single sequence: many splits, bounded by the cap
    assert 32 <= pick(1, 4, 65536) <= cap
    for B in (1, 2, 4, 8):
        for seq in (512, 1024, 2048, 4096):
            s = pick(B, 4, seq)
            assert 1 <= s <= max(1, seq // 32) and (s & (s - 1)) == 0
    # monotone: more sequences never ask for more splits
    assert pick(8, 4, 4096) <= pick(1, 4, 4096)
    assert pick(0, 4, 4096) == 1


def test_argument_validation_returns_codes_before_any_launch(lib):
    _lib = package("_lib")
    st3, st4, st2 = _lib.i64([1, 1, 1]), _lib.i64([1, 1, 1, 1]), _lib.i64([1, 1])
    # cache write: negative sizes, bad dtype, null pointers
    assert lib.int8kv_cache_write(None, None, 0, -1, 4, 128, st3, st3, None, None, st4, st4, 1, 16, None, 1, None, None, None) == _lib.E_BAD_SHAPE
    assert lib.int8kv_cache_write(None, None, 7, 1, 4, 128, st3, st3, None, None, st4, st4, 1, 16, None, 1, None, None, None) == _lib.E_BAD_DTYPE
    assert lib.int8kv_cache_write(None, None, 0, 1, 4, 128, st3, st3, None, None, st4, st4, 1, 16, None, 1, None, None, None) == _lib.E_NULLPTR
    assert lib.int8kv_cache_write(None, None, 0, 0, 4, 128, st3, st3, None, None, st4, st4, 1, 16, None, 1, None, None, None) == _lib.OK
    # attention: Hq not a multiple of Hkv, bad dtype, null pointers, too many splits
    def attn(q_dtype=0, B=1, Hq=28, Hkv=4, splits=0, flags=0):
        return lib.int8kv_paged_attn_int8(None, q_dtype, st3, B, Hq, Hkv, 128, None, None, st4, st4, 4, 16, None, 0, st2, 4,
                                          None, 0, 64, None, None, None, 0, st3, splits, None, 0, flags, None)
    assert attn(Hq=30) == _lib.E_BAD_SHAPE
    assert attn(q_dtype=5) == _lib.E_BAD_DTYPE
    assert attn() == _lib.E_NULLPTR
    assert attn(B=0) == _lib.OK
    assert attn(splits=10 ** 6) == _lib.E_BAD_SHAPE
    assert attn(splits=-2) == _lib.E_BAD_SHAPE
    assert attn(splits=_lib.SPLITS_PLANNED) == _lib.E_NULLPTR  # -1 is a valid request; the null pointers are not
    # flags: the two defined bits pass validation (and then meet the null pointers), any other bit is refused
    assert attn(flags=_lib.FLAG_QUANTIZE_Q | _lib.FLAG_INPUTS_READY) == _lib.E_NULLPTR
    assert attn(flags=4) == _lib.E_BAD_SHAPE
    assert lib.int8kv_merge_partials(None, 0, 1, 28, 128, None, 0, st3, None) == _lib.E_BAD_SHAPE
    assert lib.int8kv_merge_partials(None, 2, 1, 28, 128, None, 0, st3, None) == _lib.E_NULLPTR
    assert lib.int8kv_paged_attn_bf16(None, 0, st3, 1, 28, 4, 128, None, None, 2, st4, st4, 4, 16, None, 0, st2, 4,
                                      None, 0, 64, None, 0, st3, 0, None, 0, 0, None) == _lib.E_BAD_DTYPE
    # the INT8 query option does not exist for float caches
    assert lib.int8kv_paged_attn_bf16(None, 0, st3, 1, 28, 4, 128, None, None, 0, st4, st4, 4, 16, None, 0, st2, 4,
                                      None, 0, 64, None, 0, st3, 0, None, 0, _lib.FLAG_QUANTIZE_Q, None) == _lib.E_UNSUPPORTED
    # dynamic-scale attention: scale caches are required
    def dyn(ksc, B=1):
        return lib.int8kv_paged_attn_int8_dynamic(None, 0, st3, B, 28, 4, 128, None, None, st4, st4, ksc, None, st3, st3,
                                                  4, 16, None, 0, st2, 4, None, 0, 64, None, 0, st3, 0, None, 0, 0, None)
    assert dyn(None) == _lib.E_NULLPTR
    assert dyn(None, B=0) == _lib.OK
    # the L-layer decode step: no layers is a no-op, a null array is refused, a failing layer is named
    failed = C.c_int(7)
    def layers_call(arr, n):
        return lib.int8kv_decode_step_layers(arr, n, C.byref(failed), 0, st3, st3, None, 0, 0, st3, 1, 28, 4, 128, st4, st4,
                                             4, 16, None, 0, st2, 4, None, 0, 64, 0, st3, 0, None, 0, 0, None)
    assert layers_call(None, 0) == _lib.OK and failed.value == -1
    assert layers_call(None, -1) == _lib.E_BAD_SHAPE
    assert layers_call(None, 2) == _lib.E_NULLPTR
    arr = (_lib.LayerArgs * 2)()  # all-null per-layer pointers: the first layer fails its own null check
    assert layers_call(arr, 2) == _lib.E_NULLPTR and failed.value == 0
    # peer exchange: layout size, and descriptors that cannot be right are refused before anything is launched
    rows = 32 * 64 * 132 * 4
    assert lib.int8kv_exchange_bytes(8, 32, 64, 128) == 256 + rows * 33 + 32 * 64 * 128 * 8  # staging + 2 slabs x 8 ranks x 8-byte pairs + output slab
    assert lib.int8kv_exchange_bytes(17, 32, 64, 128) == -1 and lib.int8kv_exchange_bytes(0, 32, 64, 128) == -1
    ex = _lib.Exchange(2, 0, (C.c_void_p * 16)(), 256 + 3 * 28 * 132 * 4 * 9 + 3 * 28 * 128 * 8)
    merge = lambda e: lib.int8kv_merge_exchanged(C.byref(e), 3, 28, 128, None, 0, st3, None, 0, None)
    assert merge(ex) == _lib.E_NULLPTR  # no buffers
    ex.peer_buffers[0], ex.peer_buffers[1] = 4096, 8192 + 16
    assert merge(ex) == _lib.E_WORKSPACE  # a buffer that is not 256-byte aligned
    ex.peer_buffers[1] = 8192
    assert merge(ex) == _lib.E_NULLPTR  # buffers fine, no output
    ex.buffer_bytes -= 1
    assert merge(ex) == _lib.E_WORKSPACE
    ex.rank = 2
    assert merge(ex) == _lib.E_BAD_SHAPE
    assert lib.int8kv_merge_exchanged(None, 3, 28, 128, None, 0, st3, None, 0, None) == _lib.E_NULLPTR
    # the library's own workspace: its accessors refuse null destinations before touching the device
    assert lib.int8kv_static_ws_status(None, 0, None) == _lib.E_NULLPTR
    assert lib.int8kv_static_ws_address(None) == _lib.E_NULLPTR


def test_error_type_carries_the_status(lib):
    _lib = package("_lib")
    with pytest.raises(_lib.Int8KVError) as e:
        _lib.check("int8kv_cache_write", _lib.E_WORKSPACE)
    assert e.value.code == _lib.E_WORKSPACE and "workspace" in str(e.value)
