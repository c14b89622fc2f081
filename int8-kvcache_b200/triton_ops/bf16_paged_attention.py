"""Drop-in for the reference module src/triton_ops/bf16_paged_attention.py (the BF16 baseline)."""

from ..ops import bf16_paged_attention  # noqa: F401
