"""Module path of the reference (fast_ops/flash_attention/flash_attention.py)."""
from fast_ops_b200.flash_attention.flash_attention import (  # noqa: F401
    FlashAttentionFunction,
    flash_attention_backward,
    flash_attention_forward,
    multi_head_attention,
)
