"""(B, S, H, D) entry point with the argument list of the reference's complete implementation.

fast_ops/flash_attention/flash_attention_triton.py:720-731, :961 defines
`flash_attn_triton(q, k, v, bias=None, causal=False, dropout_p=0.0, softmax_scale=None)` on
(batch, seqlen, nheads, headdim) tensors, differentiable in q, k, v.  This adapter feeds
transposed views of the same memory to the (B, H, S, D) kernels, so nothing is copied.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from .flash_attention import _AttentionFunction, dropout_mask, flash_attention_forward, next_dropout_rng


def flash_attn_bshd(q: Tensor, k: Tensor, v: Tensor, bias: Optional[Tensor] = None, causal: bool = False,
                    dropout_p: float = 0.0, softmax_scale: Optional[float] = None) -> Tensor:
    """q: (B, Sq, H, D); k, v: (B, Sk, H, D); bias broadcastable to (B, H, Sq, Sk) with last two
    dimensions (1, Sk) or (Sq, Sk).  Returns a contiguous (B, Sq, H, D) tensor in q's dtype.  The
    dropout mask comes from the device's default generator, which every call advances by one index
    per attention probability, with or without dropout, as the reference does."""
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    # The reference advances the generator on every forward, dropout or not
    # (flash_attention_triton.py:780), so the offsets of later draws agree with a reference run.
    rng = next_dropout_rng(q.device, q.shape[0] * q.shape[2] * q.shape[1] * k.shape[1])
    # O has q's layout in both paths, as in the reference (flash_attention_triton.py:773)
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        ot, _ = _AttentionFunction.apply(qt, kt, vt, bool(causal), softmax_scale, bias, float(dropout_p), rng, True)
        return ot.transpose(1, 2)
    o = torch.empty((q.shape[0], q.shape[1], q.shape[2], q.shape[3]), dtype=q.dtype, device=q.device)
    flash_attention_forward(qt, kt, vt, causal=causal, softmax_scale=softmax_scale, out=o.transpose(1, 2),
                            bias=bias, dropout_p=float(dropout_p), rng=rng)
    return o


def triton_dropout_mask(dropout_p: float, batch_sz: int, n_heads: int, seqlen_q: int, seqlen_k: int,
                        device) -> Tensor:
    """Name and arguments of the reference's test helper (flash_attention_triton.py:699-717)."""
    return dropout_mask(dropout_p, batch_sz, n_heads, seqlen_q, seqlen_k, device)
