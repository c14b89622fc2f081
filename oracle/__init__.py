"""CPU oracle for the INT8 paged-KV decode path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is the checker that the GPU kernels are compared against and the
CPU baseline that the benchmark times beside them.

The functions restate, in this project's own code, the arithmetic of the
reference prototype cjsmt/Int8-kvcache:

  * static symmetric per-KV-head INT8 quantisation      src/quant.py:37-40
  * per-head dequantisation                              src/quant.py:33-34
  * paged cache layout [num_blocks, block_size, Hkv, D]  src/paged_cache.py:4-59
  * slot_mapping scatter write                           src/triton_ops/int8_cache_write.py:152-183
  * fp32 decode attention with contiguous GQA groups     src/attention_ref.py:11-28
  * paged INT8 attention loop reference                  src/triton_ops/int8_paged_attention.py:776-814
  * optional per-head INT8 query (quantize_q)            src/triton_ops/int8_paged_attention.py:798-802
  * per-(slot, head) dequantisation                      vllm_int8/vllm_int8_cache_ops.py:250-256
  * split-KV partial merge                               src/triton_ops/int8_paged_attention.py:330-388

Parity pin: every function here is checked against outputs of the reference's
own Python code, generated in a container where the reference is importable
(tests/golden/make_golden.py) and committed as fixtures under tests/golden/.
"""

from .quant import (  # noqa: F401
    static_quant_per_head,
    dynamic_quant_per_token_head,
    dequant_per_head,
    SCALE_FLOOR,
)
from .paged_cache import (  # noqa: F401
    build_paged_cache,
    gather_paged_cache,
    cache_write,
    slots_for_sequences,
    random_block_tables,
)
from .attention_ref import (  # noqa: F401
    decode_attention,
    int8_paged_attention_oracle,
    quantize_query_per_head,
    float_paged_attention_oracle,
    dynamic_int8_paged_attention_oracle,
    partial_attention_with_lse,
    merge_partials,
)
