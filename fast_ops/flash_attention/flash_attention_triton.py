"""Module path of the reference's complete implementation
(fast_ops/flash_attention/flash_attention_triton.py): the same call names on the CUDA kernels."""
from fast_ops_b200.flash_attention.flash_attention_bshd import (  # noqa: F401
    flash_attn_bshd as flash_attn_triton,
    triton_dropout_mask,
)
