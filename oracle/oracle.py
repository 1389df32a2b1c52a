"""ctypes front end of oracle/oracle.c (see that file for what each function restates).

The functions take and return torch CPU tensors so that tests can feed the oracle and the
CUDA path from the same seeded inputs.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")
_lib: Optional[ctypes.CDLL] = None

_DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def build(force: bool = False) -> str:
    """Compiles oracle.c with gcc (via the Makefile beside it) if the library is stale."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-C", _HERE, "-B", "_build/liboracle.so"], check=True)
    return _SO


def _load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        lib = ctypes.CDLL(_SO)
        lib.oracle_lion_step.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
            ctypes.c_double, ctypes.c_double, ctypes.c_double, ctypes.c_double]
        lib.oracle_lion_step.restype = None
        lib.oracle_attention_fwd.argtypes = [
            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
            ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        lib.oracle_attention_fwd.restype = None
        lib.oracle_attention_bwd.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 6 + [
            ctypes.c_float, ctypes.c_int, ctypes.c_int]
        lib.oracle_attention_bwd.restype = None
        lib.oracle_attention_ex.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_float] + [ctypes.c_void_p] * 7 + [
            ctypes.c_int] * 6 + [ctypes.c_float]
        lib.oracle_attention_ex.restype = None
        lib.oracle_dropout_mask.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_float, ctypes.c_uint64,
                                            ctypes.c_uint64]
        lib.oracle_dropout_mask.restype = None
        lib.oracle_num_threads.restype = ctypes.c_int
        lib.oracle_set_num_threads.argtypes = [ctypes.c_int]
        _lib = lib
    return _lib


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def set_num_threads(n: int) -> None:
    _load().oracle_set_num_threads(int(n))


def lion_step(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, lr: float,
              betas: Tuple[float, float], weight_decay: float) -> None:
    """One Lion step in place on CPU tensors (fast_ops/lion/lion_optimizer_ref.py:51-67)."""
    for t in (param, grad, exp_avg):
        if t.device.type != "cpu" or not t.is_contiguous():
            raise ValueError("oracle tensors must be contiguous CPU tensors")
    if param.dtype != grad.dtype:
        raise ValueError("param and grad must share a dtype")
    if not (param.numel() == grad.numel() == exp_avg.numel()):
        raise ValueError("size mismatch")
    _load().oracle_lion_step(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), param.numel(),
                             _DTYPE_CODE[param.dtype], _DTYPE_CODE[exp_avg.dtype],
                             float(lr), float(betas[0]), float(betas[1]), float(weight_decay))


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False,
                  softmax_scale: Optional[float] = None,
                  bh_range: Optional[Tuple[int, int]] = None,
                  row_range: Optional[Tuple[int, int, int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(scale * q k^T [+ causal mask]) v in fp32 on the CPU.

    q: (B,H,Sq,D), k/v: (B,H,Sk,D), any float dtype (upcast to fp32 first, as
    fast_ops/flash_attention/attention_ref.py:41-43 does).  Returns (out, lse), both fp32;
    out is (B,H,Sq,D), lse is (B,H,Sq).  With `bh_range=(b, e)` only the flattened
    (batch*head) slices b..e-1 are computed, and with `row_range=(begin, end, stride)` only
    those query rows of each slice; the rest of the outputs is left zero.
    """
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if softmax_scale is None:
        softmax_scale = 1.0 / (D ** 0.5)
    qf, kf, vf = (t.detach().to("cpu", torch.float32).contiguous() for t in (q, k, v))
    out = torch.zeros(B, H, Sq, D, dtype=torch.float32)
    lse = torch.zeros(B, H, Sq, dtype=torch.float32)
    b, e = bh_range if bh_range is not None else (0, B * H)
    r0, r1, rs = row_range if row_range is not None else (0, Sq, 1)
    _load().oracle_attention_fwd(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                 B, H, Sq, Sk, D, int(bool(causal)), float(softmax_scale), int(b), int(e),
                                 int(r0), int(r1), int(rs))
    return out, lse


def attention_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dout: torch.Tensor, causal: bool = False,
                  softmax_scale: Optional[float] = None,
                  bh_range: Optional[Tuple[int, int]] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dq, dk, dv) of softmax(scale * q k^T [+ causal mask]) v for the output gradient `dout`,
    in fp32 on the CPU: what autograd yields through fast_ops/flash_attention/attention_ref.py.
    Shapes as attention_fwd; with `bh_range` only those (batch*head) slices are filled."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if softmax_scale is None:
        softmax_scale = 1.0 / (D ** 0.5)
    qf, kf, vf, df = (t.detach().to("cpu", torch.float32).contiguous() for t in (q, k, v, dout))
    dq, dk, dv = torch.zeros_like(qf), torch.zeros_like(kf), torch.zeros_like(vf)
    lse = torch.zeros(B, H, Sq)
    delta = torch.zeros(B, H, Sq)
    b, e = bh_range if bh_range is not None else (0, B * H)
    _load().oracle_attention_bwd(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), df.data_ptr(), dq.data_ptr(),
                                 dk.data_ptr(), dv.data_ptr(), lse.data_ptr(), delta.data_ptr(), B, H, Sq, Sk, D,
                                 int(bool(causal)), float(softmax_scale), int(b), int(e))
    return dq, dk, dv


def dropout_mask(dropout_p: float, B: int, H: int, Sq: int, Sk: int, seed: int, offset: int) -> torch.Tensor:
    """Boolean (B,H,Sq,Sk) keep mask of the reference's attention dropout
    (fast_ops/flash_attention/flash_attention_triton.py:38-50 with the indices of :125, :217)."""
    keep = torch.empty(B, H, Sq, Sk, dtype=torch.uint8)
    _load().oracle_dropout_mask(keep.data_ptr(), keep.numel(), float(dropout_p), seed & (2**64 - 1),
                                offset & (2**64 - 1))
    return keep.bool()


def attention_ex(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, bias: Optional[torch.Tensor] = None,
                 keep_mask: Optional[torch.Tensor] = None, dropout_p: float = 0.0, causal: bool = False,
                 softmax_scale: Optional[float] = None, dout: Optional[torch.Tensor] = None):
    """Attention with additive bias and dropout in fp32 on the CPU
    (fast_ops/flash_attention/attention_ref.py:41-67 with `bias` and `dropout_mask`).

    q: (B,H,Sq,D), k/v: (B,H,Sk,D); bias broadcastable to (B,H,Sq,Sk); keep_mask boolean
    (B,H,Sq,Sk).  Returns (out, lse), or (out, lse, dq, dk, dv) when `dout` is given.
    """
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if softmax_scale is None:
        softmax_scale = 1.0 / (D ** 0.5)
    qf, kf, vf = (t.detach().to("cpu", torch.float32).contiguous() for t in (q, k, v))
    out = torch.zeros(B, H, Sq, D)
    lse = torch.zeros(B, H, Sq)
    bias_ptr, strides = None, None
    if bias is not None:
        bf = bias.detach().to("cpu", torch.float32)
        if bf.stride(-1) != 1:
            bf = bf.contiguous()
        bf = bf.expand(B, H, Sq, Sk)
        bias_ptr = bf.data_ptr()
        strides = (ctypes.c_int64 * 3)(bf.stride(0), bf.stride(1), bf.stride(2))
    keep_ptr = None
    if keep_mask is not None:
        km = keep_mask.detach().to("cpu", torch.uint8).expand(B, H, Sq, Sk).contiguous()
        keep_ptr = km.data_ptr()
    if dout is None:
        _load().oracle_attention_ex(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), bias_ptr, strides, keep_ptr,
                                    float(dropout_p), out.data_ptr(), lse.data_ptr(), None, None, None, None, None,
                                    B, H, Sq, Sk, D, int(bool(causal)), float(softmax_scale))
        return out, lse
    df = dout.detach().to("cpu", torch.float32).contiguous()
    dq, dk, dv = torch.zeros_like(qf), torch.zeros_like(kf), torch.zeros_like(vf)
    delta = torch.zeros(B, H, Sq)
    _load().oracle_attention_ex(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), bias_ptr, strides, keep_ptr,
                                float(dropout_p), out.data_ptr(), lse.data_ptr(), df.data_ptr(), dq.data_ptr(),
                                dk.data_ptr(), dv.data_ptr(), delta.data_ptr(),
                                B, H, Sq, Sk, D, int(bool(causal)), float(softmax_scale))
    return out, lse, dq, dk, dv

