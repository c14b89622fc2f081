"""ctypes binding of libint8kv_b200.so (the C ABI declared in include/int8kv_b200.h).

The library is loaded lazily from this directory.  If it is missing, it is built once with nvcc
when a compiler is available; otherwise loading raises — there is no CPU or eager fallback behind
the operators.
"""

from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_PKG_DIR = Path(__file__).resolve().parent
_LIB = None
_LOCK = threading.Lock()

ABI_VERSION = 2

OK = 0
E_NULLPTR, E_BAD_SHAPE, E_BAD_DTYPE, E_UNSUPPORTED, E_LAUNCH, E_WORKSPACE = -1, -2, -3, -4, -5, -6
DEV_WAIT_TIMEOUT = 1
DEV_SLOT_MISMATCH = 2
STATIC_WS_BYTES = 8 * 1024 * 1024
SPLITS_AUTO, SPLITS_PLANNED = 0, -1
FLAG_QUANTIZE_Q, FLAG_INPUTS_READY = 1, 2
PLAN_HEADER_TAG = 0x504C414E

BF16, FP16, FP32 = 0, 1, 2

_I64P = C.POINTER(C.c_int64)
_VP = C.c_void_p


class LayerArgs(C.Structure):
    """int8kv_layer_args of include/int8kv_b200.h: the per-layer pointers of int8kv_decode_step_layers."""

    _fields_ = [
        ("query", _VP), ("out", _VP), ("key", _VP), ("value", _VP),
        ("key_cache", _VP), ("value_cache", _VP), ("k_scale", _VP), ("v_scale", _VP),
    ]


EXCHANGE_BOTH_PHASES, EXCHANGE_MERGE_PHASE, EXCHANGE_GATHER_PHASE = 0, 1, 2  # int8kv_merge_exchanged_phase


class Exchange(C.Structure):
    """int8kv_exchange of include/int8kv_b200.h: the peer-mapped buffers of the sequence-parallel exchange."""

    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("peer_buffers", _VP * 16), ("buffer_bytes", C.c_int64)]


_SIGNATURES = {
    "int8kv_abi_version": (C.c_int, []),
    "int8kv_status_str": (C.c_char_p, [C.c_int]),
    "int8kv_partial_row_floats": (C.c_int, [C.c_int]),
    "int8kv_workspace_bytes": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "int8kv_workspace_bytes_auto": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int]),
    "int8kv_workspace_status_offset": (C.c_int64, [C.c_int64]),
    "int8kv_choose_splits": (C.c_int, [C.c_int, C.c_int, C.c_int64, C.c_int, C.c_int]),
    "int8kv_max_splits": (C.c_int, []),
    "int8kv_cache_write": (
        C.c_int,
        [_VP, _VP, C.c_int, C.c_int64, C.c_int, C.c_int, _I64P, _I64P, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _VP, _VP, _VP],
    ),
    "int8kv_paged_attn_int8": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, _VP, _VP, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_paged_attn_bf16": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, C.c_int, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_paged_attn_int8_partial": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, _VP, _VP,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_paged_attn_int8_static_ws": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, _VP, _VP, C.c_int, _I64P,
         C.c_int, C.c_int, _VP],
    ),
    "int8kv_cache_write_dynamic": (
        C.c_int,
        [_VP, _VP, C.c_int, C.c_int64, C.c_int, C.c_int, _I64P, _I64P, _VP, _VP, _I64P, _I64P, _VP, _VP, _I64P, _I64P,
         C.c_int64, C.c_int, _VP, C.c_int, _VP],
    ),
    "int8kv_paged_attn_int8_dynamic": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, _VP, _VP, _I64P, _I64P,
         C.c_int64, C.c_int, _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_decode_step": (
        C.c_int,
        [_VP, _VP, C.c_int, _I64P, _I64P, _VP, C.c_int,
         _VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, _VP, _VP, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_decode_step_layers": (
        C.c_int,
        [C.POINTER(LayerArgs), C.c_int, C.POINTER(C.c_int), C.c_int, _I64P, _I64P, _VP, C.c_int, C.c_int, _I64P,
         C.c_int, C.c_int, C.c_int, C.c_int, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_paged_attn_bf16_layers": (
        C.c_int,
        [C.POINTER(LayerArgs), C.c_int, C.POINTER(C.c_int), C.c_int, C.c_int, _I64P,
         C.c_int, C.c_int, C.c_int, C.c_int, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, C.c_int, _I64P,
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_static_ws_status": (C.c_int, [_VP, C.c_int, _VP]),
    "int8kv_static_ws_address": (C.c_int, [C.POINTER(_VP)]),
    "int8kv_exchange_bytes": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "int8kv_paged_attn_int8_partial_push": (
        C.c_int,
        [_VP, C.c_int, _I64P, C.c_int, C.c_int, C.c_int, C.c_int, _VP, _VP, _I64P, _I64P, C.c_int64, C.c_int,
         _VP, C.c_int, _I64P, C.c_int64, _VP, C.c_int, C.c_int64, _VP, _VP, C.POINTER(Exchange),
         C.c_int, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_merge_exchanged": (
        C.c_int, [C.POINTER(Exchange), C.c_int, C.c_int, C.c_int, _VP, C.c_int, _I64P, _VP, C.c_int64, _VP],
    ),
    "int8kv_merge_exchanged_phase": (
        C.c_int, [C.POINTER(Exchange), C.c_int, C.c_int, C.c_int, _VP, C.c_int, _I64P, _VP, C.c_int64, C.c_int, _VP],
    ),
    "int8kv_selftest_bounded_wait": (C.c_int, [_VP, C.c_int64, C.c_int, _VP]),
    "int8kv_merge_partials": (C.c_int, [_VP, C.c_int, C.c_int, C.c_int, C.c_int, _VP, C.c_int, _I64P, _VP]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)


def library_path() -> Path:
    override = os.environ.get("INT8KV_B200_LIB")
    return Path(override) if override else _PKG_DIR / "libint8kv_b200.so"


def load():
    """Return the loaded library (building it first if it does not exist and nvcc is present)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not path.exists():
            from . import build as _build

            _build.build()
        lib = C.CDLL(str(path))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means the library is stale
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.int8kv_abi_version() != ABI_VERSION:
            raise RuntimeError(
                f"{path} has ABI version {lib.int8kv_abi_version()}, the Python side expects {ABI_VERSION}; rebuild it"
            )
        _LIB = lib
        return lib


def status_str(code: int) -> str:
    return load().int8kv_status_str(int(code)).decode()


_I64_CACHE: dict = {}


def i64(values) -> "C.Array":
    """A ctypes int64 array of `values` (sizes or strides).  Arrays are immutable to the library and tensor
    geometries repeat from call to call, so they are built once per distinct tuple."""
    key = tuple(values)
    arr = _I64_CACHE.get(key)
    if arr is None:
        if len(_I64_CACHE) > 4096:
            _I64_CACHE.clear()
        arr = _I64_CACHE[key] = (C.c_int64 * len(key))(*[int(v) for v in key])
    return arr


class Int8KVError(RuntimeError):
    """A C-ABI entry point returned a negative status."""

    def __init__(self, fn: str, code: int):
        self.code = int(code)
        super().__init__(f"{fn} failed: {status_str(code)} (status {code})")


def check(fn: str, code: int) -> None:
    if code != OK:
        raise Int8KVError(fn, code)
