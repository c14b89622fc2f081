"""Drop-in replacements for the hot-path modules of the reference's `vllm_int8` package."""
