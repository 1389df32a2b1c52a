"""(B, S, H, D) entry point with the argument list of the reference's complete forward.

fast_ops/flash_attention/flash_attention_triton.py:720-731, :961 defines
`flash_attn_triton(q, k, v, bias=None, causal=False, dropout_p=0.0, softmax_scale=None)` on
(batch, seqlen, nheads, headdim) tensors.  This adapter feeds transposed views of the same
memory to the (B, H, S, D) kernel; bias and dropout are not implemented and raise.
"""
from __future__ import annotations

from typing import Optional

from torch import Tensor

from .flash_attention import flash_attention_forward


def flash_attn_bshd(q: Tensor, k: Tensor, v: Tensor, bias: Optional[Tensor] = None, causal: bool = False,
                    dropout_p: float = 0.0, softmax_scale: Optional[float] = None) -> Tensor:
    if bias is not None:
        raise RuntimeError("attention bias is not implemented in fast_ops_b200")
    if dropout_p != 0.0:
        raise RuntimeError("attention dropout is not implemented in fast_ops_b200")
    import torch

    o = torch.empty_like(q)  # the reference allocates O with q's layout (flash_attention_triton.py:773)
    flash_attention_forward(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal,
                            softmax_scale=softmax_scale, out=o.transpose(1, 2))
    return o
