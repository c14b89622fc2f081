"""Host-side operators over the C ABI: INT8 KV cache write, INT8 paged decode attention, and the
BF16 paged-attention baseline.

Call signatures, argument meaning and error behaviour mirror the reference prototype's operator
modules (src/triton_ops/int8_cache_write.py:85-149, src/triton_ops/int8_paged_attention.py:683-769,
src/triton_ops/bf16_paged_attention.py:118-165): argument violations raise AssertionError, an
unknown `impl` raises ValueError, the write mutates the caches in place and returns None, attention
allocates and returns its output.  Everything runs asynchronously on the current CUDA stream.
PyTorch is used for device memory and streams only; all arithmetic happens in the CUDA library.
"""

from __future__ import annotations

import ctypes as C
import threading
from typing import Dict, Optional, Tuple

import torch

from . import _lib

_FLOAT_CODES = {torch.bfloat16: _lib.BF16, torch.float16: _lib.FP16, torch.float32: _lib.FP32}

# ---------------------------------------------------------------------------------------------------
# split-KV workspace: one growing buffer per (device, stream), owned by this module like the
# partial_out/partial_m/partial_l tensors that the reference allocates per call (:595-597)
# ---------------------------------------------------------------------------------------------------
_WS: Dict[Tuple[int, int], torch.Tensor] = {}
# Buffers that a larger one has replaced.  They are kept alive: a CUDA graph captured while one of them was current
# still holds its address, and handing that memory back to the allocator would let someone else's tensor land under
# the graph's partial rows.  Growth is geometric, so all retired buffers of a stream together are smaller than its
# current one.
_WS_RETIRED: Dict[Tuple[int, int], list] = {}
_WS_LOCK = threading.Lock()


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    with _WS_LOCK:
        buf = _WS.get(key)
        if buf is None or buf.numel() < nbytes:
            if torch.cuda.is_current_stream_capturing():
                # an allocation made now would come from the capturing graph's private pool and be handed out again
                # by later captures while this module still used it
                raise RuntimeError(
                    f"the split-KV workspace of this stream must grow to {nbytes} bytes during a CUDA-graph capture; "
                    "run the call once eagerly on this stream before capturing it")
            grow = max(nbytes, 1 << 20, 2 * buf.numel() if buf is not None else 0)
            if buf is not None:
                _WS_RETIRED.setdefault(key, []).append(buf)
            buf = torch.zeros(grow, dtype=torch.uint8, device=device)
            _WS[key] = buf
        return buf


def release_workspaces() -> None:
    """Drop every cached split-KV workspace, current and retired.  Only when no CUDA graph that was captured over
    calls of this module is going to be replayed any more: such a graph keeps using the addresses."""
    with _WS_LOCK:
        _WS.clear()
        _WS_RETIRED.clear()


def device_status(device=None) -> int:
    """Read (and clear) the status word the kernels set when a bounded wait ran out.

    Synchronises the device; meant for tests and debugging, not for the serving path.
    """
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _WS.get(key)
    if buf is None:
        return 0
    off = _lib.load().int8kv_workspace_status_offset(buf.numel())
    word = buf[off : off + 4].view(torch.int32)
    value = int(word.item())
    if value:
        word.zero_()
    return value


def selftest_bounded_wait(attempts: int = 200, device=None) -> int:
    """Launch the library's bounded-wait self-test (a warp waits `attempts` times for data that never comes) and
    return the status word afterwards: INT8KV_DEV_WAIT_TIMEOUT (1) is the expected answer.  Synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _workspace(device, 16)
    rc = _require_lib().int8kv_selftest_bounded_wait(ws.data_ptr(), ws.numel(), int(attempts), _stream_ptr(device))
    _lib.check("int8kv_selftest_bounded_wait", rc)
    return device_status(device)


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _as_f32_scale(scale: torch.Tensor) -> torch.Tensor:
    if scale.dtype != torch.float32:
        scale = scale.float()
    return scale.contiguous()


def _require_lib():
    return _lib.load()


def _flags(quantize_q: bool = False, inputs_ready: bool = False) -> int:
    return (_lib.FLAG_QUANTIZE_Q if quantize_q else 0) | (_lib.FLAG_INPUTS_READY if inputs_ready else 0)


# ---------------------------------------------------------------------------------------------------
# INT8 KV cache write
# ---------------------------------------------------------------------------------------------------
def int8_kv_cache_write(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    num_warps: int = 4,
    num_stages: int = 2,
) -> None:
    """Quantise key/value [T, Hkv, D] with static per-head scales and scatter them into the INT8 paged
    caches [num_blocks, BS, Hkv, D] at slot_mapping (slot = block*BS + offset; slot < 0 skips the token).

    `num_warps` / `num_stages` are accepted for call compatibility and ignored.
    """
    assert key.is_cuda and value.is_cuda
    assert key_cache.is_cuda and value_cache.is_cuda
    assert slot_mapping.is_cuda and k_scale.is_cuda and v_scale.is_cuda
    assert key.ndim == 3 and value.ndim == 3
    assert key_cache.ndim == 4 and value_cache.ndim == 4
    assert key.shape == value.shape and key_cache.shape == value_cache.shape
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    assert key.dtype in _FLOAT_CODES and value.dtype == key.dtype
    num_tokens, num_kv_heads, head_dim = key.shape
    num_blocks, block_size, cache_heads, cache_dim = key_cache.shape
    assert cache_heads == num_kv_heads and cache_dim == head_dim
    assert slot_mapping.ndim == 1 and slot_mapping.numel() == num_tokens
    assert k_scale.ndim == 1 and v_scale.ndim == 1
    assert k_scale.numel() == num_kv_heads and v_scale.numel() == num_kv_heads
    assert slot_mapping.dtype in (torch.int32, torch.int64)
    lib = _require_lib()
    k_scale = _as_f32_scale(k_scale)
    v_scale = _as_f32_scale(v_scale)
    if slot_mapping.stride(0) != 1:
        slot_mapping = slot_mapping.contiguous()
    rc = lib.int8kv_cache_write(
        key.data_ptr(), value.data_ptr(), _FLOAT_CODES[key.dtype],
        num_tokens, num_kv_heads, head_dim,
        _lib.i64(key.stride()), _lib.i64(value.stride()),
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        num_blocks, block_size,
        slot_mapping.data_ptr(), int(slot_mapping.dtype == torch.int64),
        k_scale.data_ptr(), v_scale.data_ptr(),
        _stream_ptr(key.device),
    )
    _lib.check("int8kv_cache_write", rc)


def reshape_and_cache_int8(
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    k_scale_cache: torch.Tensor,
    v_scale_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
) -> None:
    """Dynamic INT8 quantisation with one scale per (token, KV head): writes the INT8 rows into the paged
    caches and the fp32 scales into [num_blocks, BS, Hkv] scale caches at slot_mapping.  Signature and
    checks of the reference's vllm_int8/vllm_int8_cache_ops.py:134-210."""
    assert key.is_cuda and value.is_cuda and key_cache.is_cuda and value_cache.is_cuda and slot_mapping.is_cuda
    assert key.ndim == 3 and value.ndim == 3 and key.shape == value.shape
    num_tokens, num_kv_heads, head_dim = key.shape
    assert key_cache.ndim == 4 and value_cache.ndim == 4
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    assert k_scale_cache.dtype == torch.float32 and v_scale_cache.dtype == torch.float32
    assert slot_mapping.numel() == num_tokens
    num_blocks, block_size, cache_heads, cache_dim = key_cache.shape
    assert cache_heads == num_kv_heads and cache_dim == head_dim
    assert value_cache.shape == key_cache.shape
    assert tuple(k_scale_cache.shape) == (num_blocks, block_size, num_kv_heads)
    assert tuple(v_scale_cache.shape) == (num_blocks, block_size, num_kv_heads)
    assert key.dtype in _FLOAT_CODES and value.dtype == key.dtype
    assert slot_mapping.dtype in (torch.int32, torch.int64)
    lib = _require_lib()
    slot_mapping = slot_mapping.reshape(-1)
    if slot_mapping.stride(0) != 1:
        slot_mapping = slot_mapping.contiguous()
    rc = lib.int8kv_cache_write_dynamic(
        key.data_ptr(), value.data_ptr(), _FLOAT_CODES[key.dtype],
        num_tokens, num_kv_heads, head_dim,
        _lib.i64(key.stride()), _lib.i64(value.stride()),
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        k_scale_cache.data_ptr(), v_scale_cache.data_ptr(),
        _lib.i64(k_scale_cache.stride()), _lib.i64(v_scale_cache.stride()),
        num_blocks, block_size,
        slot_mapping.data_ptr(), int(slot_mapping.dtype == torch.int64),
        _stream_ptr(key.device),
    )
    _lib.check("int8kv_cache_write_dynamic", rc)


# ---------------------------------------------------------------------------------------------------
# paged decode attention
# ---------------------------------------------------------------------------------------------------
def _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens):
    assert query.is_cuda
    assert key_cache.is_cuda and value_cache.is_cuda
    assert block_tables.is_cuda and seq_lens.is_cuda
    assert query.ndim == 3 and key_cache.ndim == 4 and value_cache.ndim == 4
    assert block_tables.ndim == 2 and seq_lens.ndim == 1
    assert query.dtype in _FLOAT_CODES
    assert block_tables.dtype in (torch.int32, torch.int64)
    assert seq_lens.dtype in (torch.int32, torch.int64)
    B, Hq, D = query.shape
    _, block_size, Hkv, cache_D = key_cache.shape
    assert value_cache.shape == key_cache.shape
    assert cache_D == D and Hq % Hkv == 0
    assert block_tables.shape[0] == B and seq_lens.numel() == B
    assert key_cache.stride(-1) == 1 and value_cache.stride(-1) == 1
    return B, Hq, Hkv, D, block_size


def _max_seq_len(seq_lens, block_tables, block_size, max_seq_len, validate=True):
    """The reference checks seq_lens on the host (two device syncs, :720-723).  With `max_seq_len`
    given, no sync happens and the kernels clamp lengths to what the block table can address."""
    if max_seq_len is not None:
        return int(max_seq_len)
    if seq_lens.numel() == 0:
        return 0
    lo, hi = torch.aminmax(seq_lens)
    lo, hi = int(lo.item()), int(hi.item())
    if validate:
        assert lo > 0
        assert block_tables.shape[1] >= (hi + block_size - 1) // block_size
    return hi


_SM_COUNT: Dict[int, int] = {}


def _sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _SM_COUNT.get(idx)
    if n is None:
        n = _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def _plan_workspace(lib, device, B, Hq, Hkv, D, block_size, max_seq, num_splits, copies: int = 1):
    """(split argument for the library, workspace).  num_splits None = automatic (the library picks a count from the
    shape or, for large calls, plans the parts on the device from seq_lens), "planned" = always plan on the
    device, an int = exactly that many.  copies = 2: room for two layers' partial rows (chained layers)."""
    if num_splits is None or num_splits == "planned":
        splits = _lib.SPLITS_AUTO if num_splits is None else _lib.SPLITS_PLANNED
        nbytes = lib.int8kv_workspace_bytes_auto(B, Hq, Hkv, D, max_seq, block_size, _sm_count(device))
    else:
        splits = max(1, min(int(num_splits), lib.int8kv_max_splits()))
        nbytes = lib.int8kv_workspace_bytes(B, Hq, D, splits)
    if copies > 1:
        nbytes = copies * ((nbytes + 511) // 256 * 256)
    ws = _workspace(device, nbytes)
    return splits, ws


def last_split_plan(device=None):
    """(items, part length in 16-token tiles, waves aimed for) that a device-planned call on the current stream of
    `device` left in its workspace, or None if the bytes there are not a plan header (calls that are not planned
    may overwrite them with partial rows, or leave an older header in place).  Synchronises."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    with _WS_LOCK:
        buf = _WS.get(key)
    if buf is None:
        return None
    off = _require_lib().int8kv_workspace_status_offset(buf.numel()) - 16
    items, part, waves, tag = buf[off:off + 16].view(torch.int32).tolist()
    return (items, part, waves) if tag == _lib.PLAN_HEADER_TAG and items > 0 else None


def int8_paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    *,
    quantize_q: bool = False,
    num_warps: int = 4,
    impl: str = "auto",
    num_splits: Optional[int] = None,
    max_seq_len: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    inputs_ready: bool = False,
) -> torch.Tensor:
    """Decode attention of query [B, Hq, D] over an INT8 paged cache; returns [B, Hq, D] in query.dtype.

    impl: "auto", "v3" or "v4" are accepted (the reference's two kernel generations); one kernel
    family serves all of them here.  num_splits: None picks the KV split count from the shape, an int
    is honoured.  max_seq_len / out / inputs_ready are extensions: an upper bound of seq_lens that avoids
    the host synchronisation, a preallocated output, and the caller's promise that nothing the call reads
    is written by the kernel that precedes it on the stream (INT8KV_FLAG_INPUTS_READY: the call then
    overlaps that kernel's tail; same results).
    """
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    assert k_scale.is_cuda and v_scale.is_cuda
    assert k_scale.ndim == 1 and v_scale.ndim == 1
    assert k_scale.numel() == Hkv and v_scale.numel() == Hkv
    if impl not in ("auto", "v3", "v4"):
        raise ValueError(f"Unknown impl={impl!r}; expected 'auto', 'v3' or 'v4'")
    lib = _require_lib()
    k_scale = _as_f32_scale(k_scale)
    v_scale = _as_f32_scale(v_scale)
    max_seq = _max_seq_len(seq_lens, block_tables, block_size, max_seq_len)
    if out is None:
        out = torch.empty((B, Hq, D), device=query.device, dtype=query.dtype)
    else:
        assert out.shape == (B, Hq, D) and out.dtype in _FLOAT_CODES and out.is_cuda
    if B == 0:
        return out
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, max_seq, num_splits)
    rc = lib.int8kv_paged_attn_int8(
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), max_seq,
        k_scale.data_ptr(), v_scale.data_ptr(),
        out.data_ptr(), _FLOAT_CODES[out.dtype], _lib.i64(out.stride()),
        splits, ws.data_ptr(), ws.numel(),
        _flags(quantize_q, inputs_ready), _stream_ptr(query.device),
    )
    _lib.check("int8kv_paged_attn_int8", rc)
    return out


def int8_paged_attention_dynamic(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    k_scale_cache: torch.Tensor,
    v_scale_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    num_splits: Optional[int] = None,
    max_seq_len: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    inputs_ready: bool = False,
) -> torch.Tensor:
    """Decode attention over an INT8 paged cache whose scales are per (block, slot, head) — the caches that
    reshape_and_cache_int8 fills (k_scale_cache / v_scale_cache [num_blocks, BS, Hkv] fp32).  Returns [B, Hq, D] in
    query.dtype: the attention of `dequantize_int8_cache(key_cache, k_scale_cache)` and its V counterpart."""
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    assert k_scale_cache.is_cuda and v_scale_cache.is_cuda
    assert k_scale_cache.dtype == torch.float32 and v_scale_cache.dtype == torch.float32
    assert k_scale_cache.shape == key_cache.shape[:3] and v_scale_cache.shape == key_cache.shape[:3]
    lib = _require_lib()
    max_seq = _max_seq_len(seq_lens, block_tables, block_size, max_seq_len)
    if out is None:
        out = torch.empty((B, Hq, D), device=query.device, dtype=query.dtype)
    else:
        assert out.shape == (B, Hq, D) and out.dtype in _FLOAT_CODES and out.is_cuda
    if B == 0:
        return out
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, max_seq, num_splits)
    rc = lib.int8kv_paged_attn_int8_dynamic(
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        k_scale_cache.data_ptr(), v_scale_cache.data_ptr(),
        _lib.i64(k_scale_cache.stride()), _lib.i64(v_scale_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), max_seq,
        out.data_ptr(), _FLOAT_CODES[out.dtype], _lib.i64(out.stride()),
        splits, ws.data_ptr(), ws.numel(),
        _flags(False, inputs_ready), _stream_ptr(query.device),
    )
    _lib.check("int8kv_paged_attn_int8_dynamic", rc)
    return out


def bf16_paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    *,
    num_splits: Optional[int] = None,
    max_seq_len: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    inputs_ready: bool = False,
) -> torch.Tensor:
    """Decode attention over a bf16 (or fp16) paged cache: the same-run baseline for the INT8 path.

    Unlike the reference's baseline, which walks all block_tables.shape[1] blocks
    (src/triton_ops/bf16_paged_attention.py:155), only the blocks below seq_lens are read.
    """
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype in (torch.bfloat16, torch.float16) and value_cache.dtype == key_cache.dtype
    lib = _require_lib()
    max_seq = _max_seq_len(seq_lens, block_tables, block_size, max_seq_len, validate=False)
    if max_seq_len is None:
        max_seq = min(max_seq, block_tables.shape[1] * block_size)
    if out is None:
        out = torch.empty_like(query)
    else:
        assert out.shape == (B, Hq, D) and out.dtype in _FLOAT_CODES and out.is_cuda
    if B == 0:
        return out
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, max_seq, num_splits)
    rc = lib.int8kv_paged_attn_bf16(
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(), _FLOAT_CODES[key_cache.dtype],
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), max_seq,
        out.data_ptr(), _FLOAT_CODES[out.dtype], _lib.i64(out.stride()),
        splits, ws.data_ptr(), ws.numel(),
        _flags(False, inputs_ready), _stream_ptr(query.device),
    )
    _lib.check("int8kv_paged_attn_bf16", rc)
    return out


def int8_decode_step(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    slot_mapping: torch.Tensor,
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    *,
    max_seq_len: int,
    num_splits: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    inputs_ready: bool = False,
) -> torch.Tensor:
    """One layer's decode step in one library call: write the step's new K/V rows [B, Hkv, D] at slot_mapping,
    then attend with query [B, Hq, D] over the updated cache (seq_lens already count the new tokens).  Equivalent
    to int8_kv_cache_write followed by int8_paged_attention; `max_seq_len` is required, so the call never
    synchronises and can be captured in a CUDA graph."""
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    assert key.is_cuda and value.is_cuda and slot_mapping.is_cuda
    assert key.shape == (B, Hkv, D) and value.shape == key.shape
    assert key.dtype in _FLOAT_CODES and value.dtype == key.dtype
    assert slot_mapping.ndim == 1 and slot_mapping.numel() == B and slot_mapping.dtype in (torch.int32, torch.int64)
    assert k_scale.numel() == Hkv and v_scale.numel() == Hkv
    lib = _require_lib()
    k_scale = _as_f32_scale(k_scale)
    v_scale = _as_f32_scale(v_scale)
    if out is None:
        out = torch.empty((B, Hq, D), device=query.device, dtype=query.dtype)
    else:
        assert out.shape == (B, Hq, D) and out.dtype in _FLOAT_CODES and out.is_cuda
    if B == 0:
        return out
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    if slot_mapping.stride(0) != 1:
        slot_mapping = slot_mapping.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, int(max_seq_len), num_splits)
    rc = lib.int8kv_decode_step(
        key.data_ptr(), value.data_ptr(), _FLOAT_CODES[key.dtype], _lib.i64(key.stride()), _lib.i64(value.stride()),
        slot_mapping.data_ptr(), int(slot_mapping.dtype == torch.int64),
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), int(max_seq_len),
        k_scale.data_ptr(), v_scale.data_ptr(),
        out.data_ptr(), _FLOAT_CODES[out.dtype], _lib.i64(out.stride()),
        splits, ws.data_ptr(), ws.numel(),
        _flags(False, inputs_ready), _stream_ptr(query.device),
    )
    _lib.check("int8kv_decode_step", rc)
    return out


class DecodeStepLayers:
    """The decode step of L layers behind ONE library call, with the arguments marshalled once.

    A serving loop reuses the same buffers every step (the caches, and static input / output buffers exactly as
    under CUDA-graph replay), so everything the binding needs — L pointer records, strides, table geometry, the
    workspace — is fixed when this object is built; calling it costs one ctypes crossing and no per-layer Python.
    Arguments as int8_decode_step_layers.  The tensors are kept alive by the object; their contents may change
    between calls, their addresses may not.  Caches may be INT8 (keys / values: the step's new rows, or None for
    attention only) or bf16 / fp16 (attention only, no scales: the baseline).
    inputs_ready: no layer reads what an earlier layer of the call writes (INT8KV_FLAG_INPUTS_READY).  The object then
    holds a workspace of twice the ordinary size and the library chains the layers: one launch per layer, each
    carrying the previous layer's split-KV merge and starting its page stream under the previous layer's tail."""

    def __init__(self, queries, keys, values, key_caches, value_caches, slot_mapping, block_tables, seq_lens,
                 k_scales, v_scales, *, max_seq_len: int, num_splits: Optional[int] = None,
                 out: Optional[torch.Tensor] = None, inputs_ready: bool = False):
        L = len(key_caches)
        assert len(value_caches) == L and len(queries) == L
        assert (keys is None) == (values is None)
        fused = keys is not None
        if fused:
            assert len(keys) == L and len(values) == L and slot_mapping is not None
        if out is None:
            q0 = queries[0] if L else None
            shape = (L,) + (tuple(q0.shape) if L else (0, 0, 0))
            out = torch.empty(shape, device=block_tables.device, dtype=q0.dtype if L else torch.bfloat16)
        else:
            assert out.ndim == 4 and out.shape[0] == L and out.is_cuda and out.dtype in _FLOAT_CODES
        self.out = out
        self.num_layers = L
        self._args = None
        if L == 0:
            return
        q0, kc0, vc0 = queries[0], key_caches[0], value_caches[0]
        B, Hq, Hkv, D, block_size = _check_decode_args(q0, kc0, vc0, block_tables, seq_lens)
        assert out.shape[1:] == (B, Hq, D)
        if B == 0:
            return
        int8_cache = kc0.dtype == torch.int8
        assert int8_cache or (kc0.dtype in (torch.bfloat16, torch.float16) and not fused)
        if int8_cache:
            assert len(k_scales) == L and len(v_scales) == L
        lib = _require_lib()
        if seq_lens.stride(0) != 1:
            seq_lens = seq_lens.contiguous()
        if fused:
            assert slot_mapping.is_cuda and slot_mapping.ndim == 1 and slot_mapping.numel() == B
            assert slot_mapping.dtype in (torch.int32, torch.int64)
            if slot_mapping.stride(0) != 1:
                slot_mapping = slot_mapping.contiguous()
            k0, v0 = keys[0], values[0]
            assert k0.shape == (B, Hkv, D) and v0.shape == k0.shape
            assert k0.dtype in _FLOAT_CODES and v0.dtype == k0.dtype
        keep = [queries, keys, values, key_caches, value_caches, slot_mapping, block_tables, seq_lens, out]
        layers = (_lib.LayerArgs * L)()
        for l in range(L):
            q, kc, vc = queries[l], key_caches[l], value_caches[l]
            assert q.is_cuda and q.shape == q0.shape and q.dtype == q0.dtype and q.stride() == q0.stride()
            assert kc.dtype == kc0.dtype and vc.dtype == kc0.dtype and kc.is_cuda and vc.is_cuda
            assert kc.shape == kc0.shape and vc.shape == kc0.shape
            assert kc.stride() == kc0.stride() and vc.stride() == vc0.stride()
            assert out[l].stride() == out[0].stride()
            a = layers[l]
            a.query, a.out = q.data_ptr(), out[l].data_ptr()
            a.key_cache, a.value_cache = kc.data_ptr(), vc.data_ptr()
            if int8_cache:
                ks, vs = _as_f32_scale(k_scales[l]), _as_f32_scale(v_scales[l])
                assert ks.is_cuda and vs.is_cuda and ks.numel() == Hkv and vs.numel() == Hkv
                keep += [ks, vs]
                a.k_scale, a.v_scale = ks.data_ptr(), vs.data_ptr()
            if fused:
                k, v = keys[l], values[l]
                assert k.is_cuda and v.is_cuda and k.shape == k0.shape and v.shape == k0.shape
                assert k.dtype == k0.dtype and v.dtype == k0.dtype
                assert k.stride() == k0.stride() and v.stride() == v0.stride()
                a.key, a.value = k.data_ptr(), v.data_ptr()
        self._device = q0.device
        splits, ws = _plan_workspace(lib, q0.device, B, Hq, Hkv, D, block_size, int(max_seq_len), num_splits,
                                     copies=2 if inputs_ready and L > 1 else 1)
        self._ws_stream = torch.cuda.current_stream(q0.device).cuda_stream
        keep.append(ws)
        self._keep = keep
        self._failed = C.c_int(-1)
        zero3 = _lib.i64((0, 0, 0))
        common = (
            _FLOAT_CODES[q0.dtype], _lib.i64(q0.stride()),
            B, Hq, Hkv, D,
            _lib.i64(kc0.stride()), _lib.i64(vc0.stride()),
            kc0.shape[0], block_size,
            block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
            _lib.i64(block_tables.stride()), block_tables.shape[1],
            seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), int(max_seq_len),
            _FLOAT_CODES[out.dtype], _lib.i64(out[0].stride()),
            splits, ws.data_ptr(), ws.numel(), _flags(False, inputs_ready),
        )
        if int8_cache:
            self._name = "int8kv_decode_step_layers"
            self._fn = lib.int8kv_decode_step_layers
            self._args = (
                layers, L, C.byref(self._failed),
                _FLOAT_CODES[keys[0].dtype] if fused else 0,
                _lib.i64(keys[0].stride()) if fused else zero3, _lib.i64(values[0].stride()) if fused else zero3,
                slot_mapping.data_ptr() if fused else None, int(fused and slot_mapping.dtype == torch.int64),
            ) + common
        else:
            self._name = "int8kv_paged_attn_bf16_layers"
            self._fn = lib.int8kv_paged_attn_bf16_layers
            self._args = (layers, L, C.byref(self._failed), _FLOAT_CODES[kc0.dtype]) + common

    def __call__(self) -> torch.Tensor:
        """Enqueue the L layers on the current stream of the tensors' device and return `out` [L, B, Hq, D].
        The split-KV workspace belongs to the stream that was current when the object was built: call it there."""
        if self._args is None:
            return self.out
        stream = torch.cuda.current_stream(self._device).cuda_stream
        assert stream == self._ws_stream, "DecodeStepLayers must run on the stream it was built on"
        rc = self._fn(*self._args, stream)
        if rc != _lib.OK:
            raise _lib.Int8KVError(f"{self._name} (layer {self._failed.value})", rc)
        return self.out


def int8_decode_step_layers(
    queries,
    keys,
    values,
    key_caches,
    value_caches,
    slot_mapping: Optional[torch.Tensor],
    block_tables: torch.Tensor,
    seq_lens: torch.Tensor,
    k_scales,
    v_scales,
    *,
    max_seq_len: int,
    num_splits: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
    inputs_ready: bool = False,
) -> torch.Tensor:
    """The decode step of L layers in one library call (one binding crossing per model step instead of one per
    layer).  queries / keys / values: [L, B, ...] tensors or sequences of L same-shaped, same-strided tensors
    (keys = values = None: attention only); key_caches / value_caches: sequences of L caches of one shape and
    stride; k_scales / v_scales: [L, Hkv] or sequences of [Hkv].  Returns out [L, B, Hq, D].  Layer l computes
    exactly what int8_decode_step (or int8_paged_attention) computes for its arguments.  A loop that reuses its
    buffers should build a DecodeStepLayers once and call that instead."""
    return DecodeStepLayers(queries, keys, values, key_caches, value_caches, slot_mapping, block_tables, seq_lens,
                            k_scales, v_scales, max_seq_len=max_seq_len, num_splits=num_splits, out=out,
                            inputs_ready=inputs_ready)()


# ---------------------------------------------------------------------------------------------------
# partial attention + merge (sequence-parallel split across devices)
# ---------------------------------------------------------------------------------------------------
def partial_row_floats(head_dim: int) -> int:
    return _require_lib().int8kv_partial_row_floats(int(head_dim))


def int8_paged_attention_partial(
    query, key_cache, value_cache, block_tables, seq_lens, k_scale, v_scale,
    *, quantize_q: bool = False, num_splits: Optional[int] = None, max_seq_len: Optional[int] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Unmerged attention over the tokens this cache holds: fp32 rows [B, Hq, row] with
    row = [normalised out (D) | natural-log sum-exp | padding]; sequences with seq_len <= 0 give lse = -inf."""
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    lib = _require_lib()
    k_scale = _as_f32_scale(k_scale)
    v_scale = _as_f32_scale(v_scale)
    max_seq = _max_seq_len(seq_lens, block_tables, block_size, max_seq_len, validate=False)
    max_seq = min(max_seq, block_tables.shape[1] * block_size)
    rf = lib.int8kv_partial_row_floats(D)
    if out is None:
        out = torch.empty((B, Hq, rf), device=query.device, dtype=torch.float32)
    assert out.shape == (B, Hq, rf) and out.dtype == torch.float32 and out.is_contiguous()
    if B == 0:
        return out
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, max(max_seq, 1), num_splits)
    rc = lib.int8kv_paged_attn_int8_partial(
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), max_seq,
        k_scale.data_ptr(), v_scale.data_ptr(),
        out.data_ptr(),
        splits, ws.data_ptr(), ws.numel(),
        _flags(quantize_q), _stream_ptr(query.device),
    )
    _lib.check("int8kv_paged_attn_int8_partial", rc)
    return out


def int8_paged_attention_partial_push(
    query, key_cache, value_cache, block_tables, seq_lens, k_scale, v_scale, exchange,
    *, quantize_q: bool = False, num_splits: Optional[int] = None, max_seq_len: Optional[int] = None,
) -> None:
    """Unmerged attention over the tokens this cache holds, with the rows stored straight into every rank's exchange
    buffer (`exchange`: a _lib.Exchange describing the peer-mapped buffers, see sharding.PeerExchange) instead of
    being returned.  merge_exchanged, called behind it on the same stream, combines what all ranks pushed."""
    B, Hq, Hkv, D, block_size = _check_decode_args(query, key_cache, value_cache, block_tables, seq_lens)
    assert key_cache.dtype == torch.int8 and value_cache.dtype == torch.int8
    lib = _require_lib()
    k_scale = _as_f32_scale(k_scale)
    v_scale = _as_f32_scale(v_scale)
    max_seq = _max_seq_len(seq_lens, block_tables, block_size, max_seq_len, validate=False)
    max_seq = min(max_seq, block_tables.shape[1] * block_size)
    if seq_lens.stride(0) != 1:
        seq_lens = seq_lens.contiguous()
    splits, ws = _plan_workspace(lib, query.device, B, Hq, Hkv, D, block_size, max(max_seq, 1), num_splits)
    rc = lib.int8kv_paged_attn_int8_partial_push(
        query.data_ptr(), _FLOAT_CODES[query.dtype], _lib.i64(query.stride()),
        B, Hq, Hkv, D,
        key_cache.data_ptr(), value_cache.data_ptr(),
        _lib.i64(key_cache.stride()), _lib.i64(value_cache.stride()),
        key_cache.shape[0], block_size,
        block_tables.data_ptr(), int(block_tables.dtype == torch.int64),
        _lib.i64(block_tables.stride()), block_tables.shape[1],
        seq_lens.data_ptr(), int(seq_lens.dtype == torch.int64), max_seq,
        k_scale.data_ptr(), v_scale.data_ptr(),
        C.byref(exchange),
        splits, ws.data_ptr(), ws.numel(),
        _flags(quantize_q), _stream_ptr(query.device),
    )
    _lib.check("int8kv_paged_attn_int8_partial_push", rc)


def merge_exchanged(exchange, batch: int, num_q_heads: int, head_dim: int, dtype=torch.bfloat16,
                    out: Optional[torch.Tensor] = None, device=None, phase: int = _lib.EXCHANGE_BOTH_PHASES) -> torch.Tensor:
    """Wait (bounded, on the device) for every rank's pushed rows of the current step and merge them -> [B, Hq, D].
    A wait that runs out is reported through device_status().  phase: one of the two halves of the step
    (_lib.EXCHANGE_MERGE_PHASE, then _lib.EXCHANGE_GATHER_PHASE with the same `out`) instead of both."""
    lib = _require_lib()
    if out is None:
        out = torch.empty((batch, num_q_heads, head_dim), device=device, dtype=dtype)
    assert out.is_cuda and out.dtype in _FLOAT_CODES and out.shape == (batch, num_q_heads, head_dim)
    ws = _workspace(out.device, 16)
    rc = lib.int8kv_merge_exchanged_phase(
        C.byref(exchange), batch, num_q_heads, head_dim, out.data_ptr(), _FLOAT_CODES[out.dtype],
        _lib.i64(out.stride()), ws.data_ptr(), ws.numel(), int(phase), _stream_ptr(out.device),
    )
    _lib.check("int8kv_merge_exchanged_phase", rc)
    return out


def merge_partials(parts: torch.Tensor, head_dim: int, dtype=torch.bfloat16, out: Optional[torch.Tensor] = None):
    """parts: fp32 [R, B, Hq, row] partial rows (as produced above, one slab per rank) -> [B, Hq, D]."""
    assert parts.is_cuda and parts.dtype == torch.float32 and parts.ndim == 4 and parts.is_contiguous()
    lib = _require_lib()
    R, B, Hq, rf = parts.shape
    assert rf == lib.int8kv_partial_row_floats(head_dim)
    if out is None:
        out = torch.empty((B, Hq, head_dim), device=parts.device, dtype=dtype)
    assert out.dtype in _FLOAT_CODES
    rc = lib.int8kv_merge_partials(
        parts.data_ptr(), R, B, Hq, head_dim, out.data_ptr(), _FLOAT_CODES[out.dtype], _lib.i64(out.stride()),
        _stream_ptr(parts.device),
    )
    _lib.check("int8kv_merge_partials", rc)
    return out
