from .flash_attention import FlashAttentionFunction, flash_attention_forward, multi_head_attention  # noqa: F401
from .flash_attention_bshd import flash_attn_bshd  # noqa: F401
from .host import flash_attention_forward_host  # noqa: F401
