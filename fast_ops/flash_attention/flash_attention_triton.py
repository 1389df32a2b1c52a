"""Module path of the reference's complete implementation
(fast_ops/flash_attention/flash_attention_triton.py): the same call names on the CUDA kernels."""
from fast_ops_b200.flash_attention.flash_attention_bshd import (  # noqa: F401
    flash_attn_bshd as flash_attn_triton,
    triton_dropout_mask,
)


class FlashAttnTritonFunction:
    """Name of the reference's autograd function (flash_attention_triton.py:720); only `apply` is
    provided, with the reference's positional arguments (q, k, v, bias, causal, dropout_p,
    softmax_scale)."""

    apply = staticmethod(flash_attn_triton)
