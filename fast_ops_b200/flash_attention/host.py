"""Attention forward on HOST tensors: copies in, kernels and copies out are pipelined.

The reference API takes device tensors (fast_ops/flash_attention/flash_attention.py:48-77).  A
caller whose Q, K, V live in pinned host memory pays for three host-to-device copies and one
device-to-host copy per call; done one after the other they cost several times the kernel.
`flash_attention_forward_host` splits the (batch, head) grid into chunks (heads are independent)
and runs copy-in, kernel and copy-out of successive chunks on three streams, so the call takes
about as long as its largest copy direction.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
from torch import Tensor

from .flash_attention import flash_attention_forward

_workspaces: Dict[tuple, dict] = {}


def _workspace(device, dtype, hc, Sq, Sk, D, slots):
    key = (device.index, dtype, hc, Sq, Sk, D, slots)
    ws = _workspaces.get(key)
    if ws is None:
        mk = lambda s: [torch.empty((1, hc, s, D), dtype=dtype, device=device) for _ in range(slots)]  # noqa: E731
        ws = {"q": mk(Sq), "k": mk(Sk), "v": mk(Sk), "o": mk(Sq),
              "streams": [torch.cuda.Stream(device) for _ in range(3)]}
        _workspaces.clear()  # one live workspace: shapes rarely alternate
        _workspaces[key] = ws
    return ws


def flash_attention_forward_host(Q: Tensor, K: Tensor, V: Tensor, *, device: Optional[torch.device] = None,
                                 out: Optional[Tensor] = None, causal: bool = False,
                                 softmax_scale: Optional[float] = None, heads_per_chunk: int = 8,
                                 slots: int = 3) -> Tensor:
    """O = softmax(scale * Q K^T [+ mask]) V for contiguous (B, H, S, D) CPU tensors.

    Q, K, V (and `out`, if given) should be pinned; the result is a CPU tensor (pinned when
    allocated here).  The call returns after the current stream of `device` has been made to wait
    for the last copy-out, so stream-ordered work and CUDA events placed after it see the result;
    synchronise the stream before reading `out` on the host.
    """
    if Q.is_cuda or K.is_cuda or V.is_cuda:
        raise RuntimeError("flash_attention_forward_host takes CPU tensors; use flash_attention_forward")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise RuntimeError("host tensors must be contiguous (B, H, S, D)")
    if not torch.cuda.is_available():
        raise RuntimeError("fast_ops_b200 attention needs a CUDA device (there is no CPU path)")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B, H, Sq, D = Q.shape
    Sk = K.shape[2]
    if out is None:
        out = torch.empty((B, H, Sq, D), dtype=Q.dtype).pin_memory()
    hc = max(1, min(heads_per_chunk, H))
    while H % hc:
        hc -= 1
    ws = _workspace(device, Q.dtype, hc, Sq, Sk, D, slots)
    s_in, s_cmp, s_out = ws["streams"]
    cur = torch.cuda.current_stream(device)
    start = torch.cuda.Event()
    start.record(cur)
    for s in (s_in, s_cmp, s_out):
        s.wait_event(start)
    in_free = [None] * slots   # recorded when the kernel that read slot's inputs has finished
    out_free = [None] * slots  # recorded when slot's output has been copied out
    i = 0
    last = None
    for b in range(B):
        for h0 in range(0, H, hc):
            slot = i % slots
            dq, dk, dv, do = ws["q"][slot], ws["k"][slot], ws["v"][slot], ws["o"][slot]
            with torch.cuda.stream(s_in):
                if in_free[slot] is not None:
                    s_in.wait_event(in_free[slot])
                dq.copy_(Q[b:b + 1, h0:h0 + hc], non_blocking=True)
                dk.copy_(K[b:b + 1, h0:h0 + hc], non_blocking=True)
                dv.copy_(V[b:b + 1, h0:h0 + hc], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ready)
                if out_free[slot] is not None:
                    s_cmp.wait_event(out_free[slot])
                flash_attention_forward(dq, dk, dv, causal=causal, softmax_scale=softmax_scale, out=do)
                done = torch.cuda.Event()
                done.record(s_cmp)
                in_free[slot] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                out[b:b + 1, h0:h0 + hc].copy_(do, non_blocking=True)
                last = torch.cuda.Event()
                last.record(s_out)
                out_free[slot] = last
            i += 1
    cur.wait_event(last)
    return out
