"""Drop-in replacements for the reference's `src/triton_ops` modules (same module and function names)."""
