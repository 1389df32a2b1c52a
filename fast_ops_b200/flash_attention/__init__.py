from .flash_attention import (  # noqa: F401
    FlashAttentionFunction,
    flash_attention_backward,
    flash_attention_forward,
    multi_head_attention,
)
from .flash_attention_bshd import flash_attn_bshd  # noqa: F401
from .host import flash_attention_forward_host  # noqa: F401
