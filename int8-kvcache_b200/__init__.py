"""int8-kvcache_b200: B200-native (sm_100a) INT8 paged-KV decode kernels behind the operator
interface of the research prototype cjsmt/Int8-kvcache.

The directory name contains a hyphen, so import it with
`importlib.import_module("int8-kvcache_b200")`; sub-modules use relative imports.

    ops            int8_kv_cache_write / int8_paged_attention / bf16_paged_attention (+ partial/merge)
    triton_ops/    drop-in modules with the reference's module and function names
    vllm_int8/     drop-in cache-ops, cache-pool and attention call-site modules
    sharding       KV-head / batch partitioning and the cross-GPU sequence split
    workloads      seeded synthetic inputs shaped like the reference's benchmark configs
    csrc/          CUDA kernels and the C ABI (include/int8kv_b200.h)
"""

from . import _lib  # noqa: F401
from .ops import (  # noqa: F401
    bf16_paged_attention,
    device_status,
    last_split_plan,
    int8_paged_attention_dynamic,
    int8_decode_step,
    int8_decode_step_layers,
    DecodeStepLayers,
    int8_kv_cache_write,
    int8_paged_attention,
    int8_paged_attention_partial,
    int8_paged_attention_partial_push,
    merge_exchanged,
    merge_partials,
    partial_row_floats,
    release_workspaces,
    reshape_and_cache_int8,
    selftest_bounded_wait,
)

__all__ = [
    "int8_kv_cache_write",
    "int8_paged_attention",
    "bf16_paged_attention",
    "int8_paged_attention_partial",
    "int8_paged_attention_partial_push",
    "merge_exchanged",
    "int8_paged_attention_dynamic",
    "int8_decode_step",
    "int8_decode_step_layers",
    "DecodeStepLayers",
    "reshape_and_cache_int8",
    "merge_partials",
    "partial_row_floats",
    "device_status",
    "last_split_plan",
    "release_workspaces",
    "selftest_bounded_wait",
]
