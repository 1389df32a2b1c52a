from .flash_attention import (  # noqa: F401
    FlashAttentionFunction,
    dropout_mask,
    flash_attention_backward,
    flash_attention_forward,
    multi_head_attention,
    next_dropout_rng,
)
from .flash_attention_bshd import flash_attn_bshd, triton_dropout_mask  # noqa: F401
from .host import flash_attention_forward_host  # noqa: F401
