"""Loader of the plain-C quantiser oracle (oracle/quant_c.c); test infrastructure only.

`build()` compiles it with gcc into oracle/_build/ (git-ignored); the functions take and return torch CPU tensors.
"""

from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "_build" / "libquant_c.so"
_LIB = None


def build(force: bool = False) -> Path:
    src = _DIR / "quant_c.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        _SO.parent.mkdir(exist_ok=True)
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-fno-fast-math", "-o", str(_SO), str(src), "-lm"], check=True)
    return _SO


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(str(build()))
    return _LIB


def _p(t):
    return C.c_void_p(t.data_ptr())


def static_quant(x: torch.Tensor, scale: torch.Tensor, floor_scale: bool = False) -> torch.Tensor:
    """x [T, Hkv, D] any float dtype (promoted to fp32 like the reference), scale [Hkv] -> int8 [T, Hkv, D]."""
    xf = x.to(torch.float32).contiguous()
    s = scale.to(torch.float32).contiguous()
    q = torch.empty(xf.shape, dtype=torch.int8)
    T, H, D = xf.shape
    _lib().oracle_static_quant(_p(xf), _p(s), _p(q), C.c_int64(T), H, D, int(floor_scale))
    return q


def cache_write(x: torch.Tensor, scale: torch.Tensor, cache: torch.Tensor, slots: torch.Tensor, floor_scale: bool = True):
    xf = x.to(torch.float32).contiguous()
    s = scale.to(torch.float32).contiguous()
    sl = slots.to(torch.int64).contiguous()
    assert cache.is_contiguous() and cache.dtype == torch.int8
    T, H, D = xf.shape
    _lib().oracle_cache_write(_p(xf), _p(s), _p(cache), _p(sl), C.c_int64(T), H, D, C.c_int64(cache.shape[0]),
                              cache.shape[1], int(floor_scale))
