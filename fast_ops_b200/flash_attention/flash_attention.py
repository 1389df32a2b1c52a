"""FlashAttention forward with the reference's call signature.

Mirrors fast_ops/flash_attention/flash_attention.py of jfc4050/fast-ops:
`multi_head_attention(Q, K, V)` (:48-77) and `FlashAttentionFunction` (:28-45) keep their
names, argument meaning, (B, H, S, D) layout and error behaviour (a constraint violation
raises), except that `backward`, a placeholder that raises in the reference, is implemented.
The keyword-only extras (`causal`, `softmax_scale`, `return_lse`) follow the
reference's complete forward (flash_attention_triton.py:720-731); the default call is the
reference call.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple, Union

import torch
from torch import Tensor
from torch.autograd import Function

from .. import _lib


def _strides3(t: Tensor):
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


def _prepare_bias(bias: Optional[Tensor], Q: Tensor, N: int):
    """Checks a bias the way the reference does (flash_attention_triton.py:752-769) and returns
    (tensor kept alive, pointer, stride array, dtype code) for the C ABI."""
    if bias is None:
        return None, None, None, _lib.FO_F32
    B, H, M, _ = Q.shape
    if bias.dtype not in (Q.dtype, torch.float32):
        raise RuntimeError(f"bias must be float32 or have Q's dtype, got {bias.dtype}")
    if not bias.is_cuda or bias.device != Q.device:
        raise RuntimeError("bias must be on Q's device")
    if bias.dim() != 4:
        raise RuntimeError("bias must be 4-D, broadcastable to (B, H, M, N)")
    if bias.stride(-1) != 1:
        bias = bias.contiguous()
    if tuple(bias.shape[2:]) not in ((1, N), (M, N)):
        raise RuntimeError("Last 2 dimensions of bias must be (1, seqlen_k) or (seqlen_q, seqlen_k)")
    if bias.shape[0] not in (1, B) or bias.shape[1] not in (1, H):
        raise RuntimeError("bias batch and head dimensions must be 1 or match Q")
    bias = bias.expand(B, H, M, N)
    return bias, bias.data_ptr(), _strides3(bias), _lib.dtype_code(bias.dtype)


def next_dropout_rng(device: torch.device, count: int) -> Tuple[int, int]:
    """(seed, offset) of the device's default CUDA generator, whose offset is then advanced by
    `count` rounded up to a multiple of 4: the bookkeeping of the reference
    (flash_attention_triton.py:641-665, which edits the last two 64-bit words of the generator's
    state tensor: the same seed and offset), so that manual_seed() followed by the same sequence
    of calls gives the same masks."""
    device = torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    gen = torch.cuda.default_generators[index]
    seed, offset = int(gen.initial_seed()), int(gen.get_offset())
    gen.set_offset(offset + ((int(count) + 3) // 4) * 4)
    return seed, offset


def dropout_mask(dropout_p: float, batch: int, heads: int, seqlen_q: int, seqlen_k: int, device,
                 rng: Optional[Tuple[int, int]] = None) -> Tensor:
    """Boolean (B, H, M, N) keep mask of the attention dropout; with `rng=None` it draws (seed,
    offset) from the device's generator exactly as an attention call would
    (triton_dropout_mask, flash_attention_triton.py:699-717)."""
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("dropout_mask needs a CUDA device (there is no CPU path)")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    seed, offset = rng if rng is not None else next_dropout_rng(device, batch * heads * seqlen_q * seqlen_k)
    out = torch.empty((batch, heads, seqlen_q, seqlen_k), dtype=torch.uint8, device=device)
    rc = _lib.load().fo_dropout_mask(out.data_ptr(), batch, heads, seqlen_q, seqlen_k, float(dropout_p),
                                     seed & (2**64 - 1), offset & (2**64 - 1), device.index,
                                     _lib.current_stream_ptr(device))
    _lib.check(rc)
    return out.bool()


def flash_attention_forward(Q: Tensor, K: Tensor, V: Tensor, *, causal: bool = False,
                            softmax_scale: Optional[float] = None,
                            return_lse: bool = False,
                            out: Optional[Tensor] = None,
                            bias: Optional[Tensor] = None,
                            dropout_p: float = 0.0,
                            rng: Optional[Tuple[int, int]] = None) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    """O = softmax(scale * Q K^T [+ bias] [+ causal mask]) V on the CUDA device holding Q.

    `bias`: 4-D, fp32 or Q's dtype, last two dimensions (1, N) or (M, N), the first two 1 or
    (B, H); -inf entries mask.  `dropout_p` > 0 drops attention probabilities with the reference's
    counter-based mask; `rng` = (seed, offset) must then be given (see `next_dropout_rng`).

    Q: (B, H, M, D); K, V: (B, H, N, D); fp16 or bf16; D a multiple of 8 up to 128; the last dimension
    contiguous, the others with strides that are multiples of 8 elements (so (B, S, H, D)
    tensors viewed as (B, H, S, D) are accepted without a copy).  K and V may be expanded over the
    head dimension (stride 0: multi-query attention); the shared head is then read once per tile
    from the single copy.  Returns O (B, H, M, D) in
    Q's dtype, plus LSE (B, H, M) fp32 when `return_lse`.  `out`, if given, receives O: shape
    (B, H, M, D), Q's dtype and device, last dimension contiguous (any layout otherwise).
    """
    if not (isinstance(Q, Tensor) and isinstance(K, Tensor) and isinstance(V, Tensor)):
        raise RuntimeError("Q, K, V must be tensors")
    if Q.dim() != 4 or K.dim() != 4 or V.dim() != 4:
        raise RuntimeError("Q, K, V must be 4-D (B, H, S, D)")
    if not Q.is_cuda:
        raise RuntimeError("fast_ops_b200 attention needs CUDA tensors (there is no CPU path)")
    if K.device != Q.device or V.device != Q.device:
        raise RuntimeError("Q, K, V must be on the same device")
    if Q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"inputs must be float16 or bfloat16, got {Q.dtype}")
    if K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise RuntimeError("Q, K, V must have the same dtype")
    B, H, M, D = Q.shape
    if K.shape[0] != B or K.shape[1] != H or K.shape[3] != D or V.shape != K.shape:
        raise RuntimeError(f"shape mismatch: Q {tuple(Q.shape)}, K {tuple(K.shape)}, V {tuple(V.shape)}")
    N = K.shape[2]
    if D > 128 or D % 8 != 0:
        raise RuntimeError(f"head_dim must be a multiple of 8 and <= 128, got {D}")
    for name, t in (("Q", Q), ("K", K), ("V", V)):
        if t.stride(3) != 1:
            raise RuntimeError(f"{name}: the last dimension must be contiguous")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)

    if out is None:
        O = torch.empty((B, H, M, D), dtype=Q.dtype, device=Q.device)
    else:
        if out.shape != (B, H, M, D) or out.dtype != Q.dtype or out.device != Q.device or out.stride(3) != 1:
            raise RuntimeError("out must be (B, H, M, D) with Q's dtype and device and a contiguous last dimension")
        O = out
    lse = torch.empty((B, H, M), dtype=torch.float32, device=Q.device) if return_lse else None
    lib = _lib.load()
    if bias is None and dropout_p == 0.0:
        rc = lib.fo_flash_attn_fwd(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), lse.data_ptr() if return_lse else None,
            B, H, M, N, D, _strides3(Q), _strides3(K), _strides3(V), _strides3(O),
            _lib.dtype_code(Q.dtype), int(bool(causal)), scale, Q.device.index,
            _lib.current_stream_ptr(Q.device))
    else:
        if not 0.0 <= dropout_p < 1.0:
            raise RuntimeError(f"dropout_p must be in [0, 1), got {dropout_p}")
        if dropout_p > 0.0 and rng is None:
            raise RuntimeError("dropout needs rng=(seed, offset); see next_dropout_rng")
        seed, offset = rng if rng is not None else (0, 0)
        bias_t, bias_ptr, bias_strides, bias_code = _prepare_bias(bias, Q, N)
        rc = lib.fo_flash_attn_fwd_ex(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), lse.data_ptr() if return_lse else None,
            B, H, M, N, D, _strides3(Q), _strides3(K), _strides3(V), _strides3(O),
            _lib.dtype_code(Q.dtype), int(bool(causal)), scale,
            bias_ptr, bias_strides, bias_code, float(dropout_p), seed & (2**64 - 1), offset & (2**64 - 1),
            Q.device.index, _lib.current_stream_ptr(Q.device))
    _lib.check(rc)
    return (O, lse) if return_lse else O


def flash_attention_backward(dO: Tensor, Q: Tensor, K: Tensor, V: Tensor, O: Tensor, LSE: Tensor, *,
                             causal: bool = False,
                             softmax_scale: Optional[float] = None,
                             bias: Optional[Tensor] = None,
                             dropout_p: float = 0.0,
                             rng: Optional[Tuple[int, int]] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """(dQ, dK, dV) for the output gradient dO, from the forward's inputs, output O and LSE.

    `bias`, `dropout_p` and `rng` must be those of the forward call; no gradient is produced for
    the bias (as in the reference, flash_attention_triton.py:854).

    Shapes and dtypes as in `flash_attention_forward`; LSE is the (B, H, M) fp32 tensor that call
    returns with `return_lse=True`.  Semantics of the reference's complete backward
    (fast_ops/flash_attention/flash_attention_triton.py:832-958).
    """
    for name, t in (("dO", dO), ("Q", Q), ("K", K), ("V", V), ("O", O)):
        if not t.is_cuda or t.dim() != 4 or t.dtype != Q.dtype or t.device != Q.device:
            raise RuntimeError(f"{name} must be a 4-D CUDA tensor with Q's dtype and device")
        if t.stride(3) != 1:
            raise RuntimeError(f"{name}: the last dimension must be contiguous")
    if Q.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError(f"inputs must be float16 or bfloat16, got {Q.dtype}")
    B, H, M, D = Q.shape
    N = K.shape[2]
    if dO.shape != Q.shape or O.shape != Q.shape or V.shape != K.shape or K.shape[:2] != (B, H) or K.shape[3] != D:
        raise RuntimeError("shape mismatch between dO, Q, K, V, O")
    if LSE.shape != (B, H, M) or LSE.dtype != torch.float32 or not LSE.is_contiguous() or LSE.device != Q.device:
        raise RuntimeError("LSE must be a contiguous (B, H, M) float32 tensor on Q's device")
    scale = float(softmax_scale) if softmax_scale is not None else 1.0 / math.sqrt(D)
    if K.stride(1) == 0 or V.stride(1) == 0:
        # multi-query K/V expanded over the heads: the kernel writes one dK, dV per query head
        # (autograd sums them through the expand), so it needs per-head storage to read from too
        K, V = K.contiguous(), V.contiguous()
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    for t in (dQ, dK, dV):
        if t.stride(3) != 1:
            raise RuntimeError("gradient layout: the last dimension must be contiguous")
    dq_accum = torch.empty((B, H, M, D), dtype=torch.float32, device=Q.device)
    delta = torch.empty((B, H, M), dtype=torch.float32, device=Q.device)
    lib = _lib.load()
    if bias is None and dropout_p == 0.0:
        rc = lib.fo_flash_attn_bwd(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), dO.data_ptr(), LSE.data_ptr(),
            dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), dq_accum.data_ptr(), delta.data_ptr(),
            B, H, M, N, D, _strides3(Q), _strides3(K), _strides3(V), _strides3(O), _strides3(dO),
            _strides3(dQ), _strides3(dK), _strides3(dV),
            _lib.dtype_code(Q.dtype), int(bool(causal)), scale, Q.device.index, _lib.current_stream_ptr(Q.device))
    else:
        if dropout_p > 0.0 and rng is None:
            raise RuntimeError("dropout needs the forward's rng=(seed, offset)")
        seed, offset = rng if rng is not None else (0, 0)
        bias_t, bias_ptr, bias_strides, bias_code = _prepare_bias(bias, Q, N)
        rc = lib.fo_flash_attn_bwd_ex(
            Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), dO.data_ptr(), LSE.data_ptr(),
            dQ.data_ptr(), dK.data_ptr(), dV.data_ptr(), dq_accum.data_ptr(), delta.data_ptr(),
            B, H, M, N, D, _strides3(Q), _strides3(K), _strides3(V), _strides3(O), _strides3(dO),
            _strides3(dQ), _strides3(dK), _strides3(dV),
            _lib.dtype_code(Q.dtype), int(bool(causal)), scale,
            bias_ptr, bias_strides, bias_code, float(dropout_p), seed & (2**64 - 1), offset & (2**64 - 1),
            Q.device.index, _lib.current_stream_ptr(Q.device))
    _lib.check(rc)
    return dQ, dK, dV


class _AttentionFunction(Function):
    """Forward + backward with the keyword arguments carried as non-tensor inputs.

    `rng` is the (seed, offset) pair of the dropout mask, or None to draw it from the device's
    generator when `dropout_p` > 0; with `bshd_out` O is allocated as a (B, S, H, D) block and
    returned as its (B, H, S, D) view, so that the caller's transpose back is contiguous."""

    @staticmethod
    def forward(ctx, Q: Tensor, K: Tensor, V: Tensor, causal: bool, softmax_scale: Optional[float],
                bias: Optional[Tensor], dropout_p: float, rng: Optional[Tuple[int, int]] = None,
                bshd_out: bool = False):
        if rng is None and dropout_p > 0.0:
            # one index per attention probability (flash_attention_triton.py:780)
            rng = next_dropout_rng(Q.device, Q.shape[0] * Q.shape[1] * Q.shape[2] * K.shape[2])
        out = None
        if bshd_out:
            B, H, M, D = Q.shape
            out = torch.empty((B, M, H, D), dtype=Q.dtype, device=Q.device).transpose(1, 2)
        O, lse = flash_attention_forward(Q, K, V, causal=causal, softmax_scale=softmax_scale, return_lse=True,
                                         bias=bias, dropout_p=dropout_p, rng=rng, out=out)
        ctx.save_for_backward(Q, K, V, O, lse, bias)
        ctx.causal, ctx.softmax_scale, ctx.dropout_p, ctx.rng = causal, softmax_scale, dropout_p, rng
        ctx.mark_non_differentiable(lse)
        return O, lse

    @staticmethod
    def backward(ctx, dO: Tensor, _dlse):
        Q, K, V, O, lse, bias = ctx.saved_tensors
        if bias is not None and ctx.needs_input_grad[5]:
            raise RuntimeError("attention bias gradient is not supported")  # flash_attention_triton.py:854
        if dO.stride(3) != 1:
            dO = dO.contiguous()
        dQ, dK, dV = flash_attention_backward(dO, Q, K, V, O, lse, causal=ctx.causal,
                                              softmax_scale=ctx.softmax_scale, bias=bias,
                                              dropout_p=ctx.dropout_p, rng=ctx.rng)
        return dQ, dK, dV, None, None, None, None, None, None


class FlashAttentionFunction(Function):
    """fast_ops/flash_attention/flash_attention.py:28-45.  The reference's backward is a
    placeholder that raises; here it returns (dQ, dK, dV)."""

    @staticmethod
    def forward(ctx, Q: Tensor, K: Tensor, V: Tensor) -> Tensor:
        O, lse = flash_attention_forward(Q, K, V, return_lse=True)
        ctx.save_for_backward(Q, K, V, O, lse)
        return O

    @staticmethod
    def backward(ctx, dO: Tensor):
        Q, K, V, O, lse = ctx.saved_tensors
        if dO.stride(3) != 1:
            dO = dO.contiguous()
        return flash_attention_backward(dO, Q, K, V, O, lse)


def multi_head_attention(Q: Tensor, K: Tensor, V: Tensor, *, causal: bool = False,
                         softmax_scale: Optional[float] = None,
                         return_lse: bool = False,
                         bias: Optional[Tensor] = None,
                         dropout_p: float = 0.0) -> Union[Tensor, Tuple[Tensor, Tensor]]:
    """Drop-in for fast_ops.flash_attention.flash_attention.multi_head_attention (:48-77).

    :param Q: (B, H, M, D) query.  :param K: (B, H, N, D) key.  :param V: (B, H, N, D) value.
    :returns: (B, H, M, D), or (O, LSE) when `return_lse`.

    Limitations (violations raise RuntimeError), the reference's own: head_dim <= 128 and a
    multiple of 8 (the kernels are built for 64 and 128, other values run zero-padded in the next
    larger one); fp16 / bf16 inputs; last dimension
    contiguous.  The scale is 1/sqrt(D) unless `softmax_scale` is given.  `bias` and `dropout_p`
    as in `flash_attention_forward`; the dropout mask is drawn from the device's default generator.
    """
    if not causal and softmax_scale is None and not return_lse and bias is None and dropout_p == 0.0:
        return FlashAttentionFunction.apply(Q, K, V)
    if torch.is_grad_enabled() and (Q.requires_grad or K.requires_grad or V.requires_grad):
        O, lse = _AttentionFunction.apply(Q, K, V, bool(causal), softmax_scale, bias, float(dropout_p))
        return (O, lse) if return_lse else O
    rng = None
    if dropout_p > 0.0:
        rng = next_dropout_rng(Q.device, Q.shape[0] * Q.shape[1] * Q.shape[2] * K.shape[2])
    return flash_attention_forward(Q, K, V, causal=causal, softmax_scale=softmax_scale, return_lse=return_lse,
                                   bias=bias, dropout_p=float(dropout_p), rng=rng)
