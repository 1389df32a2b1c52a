"""FlashAttention backward on the GPU against the reference's autograd vectors and the CPU oracle.

The bar is the reference's own (tests/test_flash_attention_triton.py:132-142): the maximum
absolute error against the fp32 gradients must not exceed twice the error of a plain torch
implementation running in the same 16-bit precision.
"""
import numpy as np
import pytest
import torch

import fast_ops_b200._lib as L
import oracle
from fast_ops_b200.flash_attention import flash_attention_backward, flash_attention_forward, multi_head_attention
from helpers import DT, attention_dout, attention_inputs, golden_files, input_digest

pytestmark = pytest.mark.gpu


def torch_same_precision_grads(q, k, v, dout, causal):
    """Attention and its gradients with torch ops in the tensors' own 16-bit dtype."""
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    d = q.shape[-1]
    scores = torch.matmul(q, (k / d ** 0.5).transpose(-1, -2))
    if causal:
        mask = torch.triu(torch.ones(q.shape[2], k.shape[2], dtype=torch.bool, device=q.device), 1)
        scores = scores.masked_fill(mask, float("-inf"))
    out = torch.matmul(torch.softmax(scores, dim=-1), v)
    out.backward(dout)
    return q.grad, k.grad, v.grad


def run_backward(q, k, v, dout, causal, device):
    qd, kd, vd, dd = (t.to(device) for t in (q, k, v, dout))
    o, lse = flash_attention_forward(qd, kd, vd, causal=causal, return_lse=True)
    dq, dk, dv = flash_attention_backward(dd, qd, kd, vd, o, lse, causal=causal)
    torch.cuda.synchronize()
    assert L.device_status(device.index) == 0, "a kernel wait timed out"
    same = torch_same_precision_grads(qd, kd, vd, dd, causal)
    return (dq, dk, dv), same


def check(got, same, want, what):
    for name, g, s, w in zip(("dq", "dk", "dv"), got, same, want):
        err = (g.float().cpu() - w).abs().max().item()
        err_torch = (s.float().cpu() - w).abs().max().item()
        assert err <= 2 * err_torch + 1e-4, f"{what} {name}: error {err:.3e} vs same-precision torch {err_torch:.3e}"


@pytest.mark.parametrize("path", golden_files("attnbwd"), ids=lambda p: p.split("attnbwd_")[-1][:-4])
def test_backward_matches_reference_autograd_vectors(cuda_device, path):
    z = np.load(path)
    B, H, Sq, Sk, D = (int(x) for x in z["shape"])
    dt = DT[str(z["dtype"])]
    q, k, v = attention_inputs(int(z["seed"]), B, H, Sq, Sk, D, dt)
    dout = attention_dout(int(z["seed"]), B, H, Sq, D, dt)
    assert input_digest(q, k, v, dout) == str(z["input_sha256"])
    got, same = run_backward(q, k, v, dout, bool(z["causal"]), cuda_device)
    check(got, same, [torch.from_numpy(z[n]) for n in ("dq", "dk", "dv")], "reference vectors")


@pytest.mark.parametrize("case", [
    # B, H, Sq, Sk, D, dtype, causal
    (2, 3, 512, 512, 64, torch.bfloat16, True),
    (1, 2, 1024, 1024, 128, torch.bfloat16, True),
    (1, 2, 640, 640, 128, torch.float16, False),
    (1, 1, 129, 129, 64, torch.float16, True),
    (1, 2, 77, 513, 128, torch.bfloat16, False),
    (2, 1, 513, 77, 64, torch.bfloat16, True),
    (1, 1, 1, 1, 128, torch.bfloat16, True),
], ids=lambda c: "B%dH%dSq%dSk%dD%d_%s_%s" % (c[0], c[1], c[2], c[3], c[4], str(c[5])[6:], "causal" if c[6] else "full"))
def test_backward_matches_oracle(cuda_device, case):
    B, H, Sq, Sk, D, dtype, causal = case
    q, k, v = attention_inputs(4321 + Sq + Sk, B, H, Sq, Sk, D, dtype)
    dout = attention_dout(77 + Sq, B, H, Sq, D, dtype)
    want = oracle.attention_bwd(q, k, v, dout, causal=causal)
    got, same = run_backward(q, k, v, dout, causal, cuda_device)
    check(got, same, want, "oracle")


def test_autograd_through_the_reference_call(cuda_device):
    q, k, v = attention_inputs(5, 1, 2, 256, 256, 64, torch.bfloat16)
    dout = attention_dout(5, 1, 2, 256, 64, torch.bfloat16)
    want = oracle.attention_bwd(q, k, v, dout, causal=False)
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k, v))
    out = multi_head_attention(qd, kd, vd)  # three positional tensors, as in the reference
    out.backward(dout.to(cuda_device))
    same = torch_same_precision_grads(qd.detach(), kd.detach(), vd.detach(), dout.to(cuda_device), False)
    check((qd.grad, kd.grad, vd.grad), same, want, "autograd")
    # keyword form with a causal mask
    want_c = oracle.attention_bwd(q, k, v, dout, causal=True)
    for t in (qd, kd, vd):
        t.grad = None
    multi_head_attention(qd, kd, vd, causal=True).backward(dout.to(cuda_device))
    same_c = torch_same_precision_grads(qd.detach(), kd.detach(), vd.detach(), dout.to(cuda_device), True)
    check((qd.grad, kd.grad, vd.grad), same_c, want_c, "autograd causal")


def test_backward_multi_query_sums_over_heads(cuda_device):
    B, H, S, D = 1, 4, 256, 64
    gen = torch.Generator().manual_seed(41)
    q = torch.randn(B, H, S, D, generator=gen).bfloat16()
    k1, v1 = (torch.randn(B, 1, S, D, generator=gen).bfloat16() for _ in range(2))
    dout = torch.randn(B, H, S, D, generator=gen).bfloat16()
    dq, dk, dv = oracle.attention_bwd(q, k1.expand(B, H, S, D), v1.expand(B, H, S, D), dout, causal=True)
    want = (dq, dk.sum(1, keepdim=True), dv.sum(1, keepdim=True))
    qd, kd, vd = (t.to(cuda_device).requires_grad_(True) for t in (q, k1, v1))
    out = multi_head_attention(qd, kd.expand(B, H, S, D), vd.expand(B, H, S, D), causal=True)
    out.backward(dout.to(cuda_device))
    for name, g, w in zip(("dq", "dk", "dv"), (qd.grad, kd.grad, vd.grad), want):
        err = (g.float().cpu() - w).abs().max().item()
        assert err <= 0.03 * max(1.0, w.abs().max().item()), f"{name}: {err}"


@pytest.mark.parametrize("D", [32, 80, 96])
def test_backward_other_head_dims(cuda_device, D):
    B, H, Sq, Sk = 1, 2, 200, 300
    q, k, v = attention_inputs(70 + D, B, H, Sq, Sk, D, torch.bfloat16)
    dout = attention_dout(70 + D, B, H, Sq, D, torch.bfloat16)
    want = oracle.attention_bwd(q, k, v, dout, causal=True)
    got, same = run_backward(q, k, v, dout, True, cuda_device)
    check(got, same, want, f"D={D}")


def _bwd_ex(device, q, k, v, dout, causal, bias=None, p=0.0, rng=None):
    """Forward + backward with optional bias / dropout; returns (grads, same-precision torch grads, keep mask)."""
    from fast_ops_b200.flash_attention import dropout_mask

    qd, kd, vd, dd = (t.to(device) for t in (q, k, v, dout))
    bd = None if bias is None else bias.to(device)
    o, lse = flash_attention_forward(qd, kd, vd, causal=causal, return_lse=True, bias=bd, dropout_p=p, rng=rng)
    got = flash_attention_backward(dd, qd, kd, vd, o, lse, causal=causal, bias=bd, dropout_p=p, rng=rng)
    torch.cuda.synchronize()
    assert L.device_status(device.index) == 0, "a kernel wait timed out"
    keep = dropout_mask(p, q.shape[0], q.shape[1], q.shape[2], k.shape[2], device, rng=rng) if p > 0 else None
    # same-precision torch with the same bias and mask (tests/test_flash_attention_triton.py:107-117)
    qs, ks, vs = (t.clone().requires_grad_(True) for t in (qd, kd, vd))
    d = q.shape[-1]
    scores = torch.matmul(qs, (ks / d ** 0.5).transpose(-1, -2))
    if bd is not None:
        scores = (scores + bd).to(scores.dtype)
    if causal:
        mask = torch.triu(torch.ones(q.shape[2], k.shape[2], dtype=torch.bool, device=device), 1)
        scores = scores.masked_fill(mask, float("-inf"))
    attn = torch.softmax(scores, dim=-1)
    if keep is not None:
        attn = attn.masked_fill(~keep, 0.0)
    torch.matmul(attn, vs * (1.0 / (1.0 - p))).backward(dd)
    return got, (qs.grad, ks.grad, vs.grad), keep


@pytest.mark.parametrize("variant", ["plain", "vector_bias", "dropout"])
def test_backward_at_32_key_tiles(cuda_device, variant):
    """S = 4096, D = 128, bf16, causal: every query tile's dQ is the sum of up to 32 bulk
    reduce-adds from different CTAs (the small cases above stop at 8)."""
    B, H, S, D = 1, 2, 4096, 128
    q, k, v = attention_inputs(4096, B, H, S, S, D, torch.bfloat16)
    dout = attention_dout(4097, B, H, S, D, torch.bfloat16)
    bias, p, rng = None, 0.0, None
    if variant == "vector_bias":
        bias = torch.randn(1, H, 1, S, generator=torch.Generator().manual_seed(4098))
        bias[..., 5::23] = float("-inf")
    if variant == "dropout":
        p, rng = 0.17, (0, 16773120 + 4096 - (B * H * S * S) // 2 // 4 * 4)
    got, same, keep = _bwd_ex(cuda_device, q, k, v, dout, True, bias, p, rng)
    keep_cpu = None
    if p > 0:
        keep_cpu = oracle.dropout_mask(p, B, H, S, S, *rng)
        assert torch.equal(keep.cpu(), keep_cpu)
    want = oracle.attention_ex(q, k, v, bias=bias, keep_mask=keep_cpu, dropout_p=p, causal=True, dout=dout)
    check(got, same, want[2:], f"S=4096 {variant}")


def test_backward_at_the_long_context_length(cuda_device):
    """One head at S = 16384, D = 128, bf16, causal: the depth the benchmark times (128 key tiles;
    dQ of the last query tile is accumulated from 128 CTAs)."""
    B, H, S, D = 1, 1, 16384, 128
    q, k, v = attention_inputs(16384, B, H, S, S, D, torch.bfloat16)
    dout = attention_dout(16385, B, H, S, D, torch.bfloat16)
    want = oracle.attention_bwd(q, k, v, dout, causal=True)
    got, same = run_backward(q, k, v, dout, True, cuda_device)
    check(got, same, want, "S=16384")
