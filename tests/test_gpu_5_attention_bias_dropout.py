"""Attention with additive bias and dropout on the GPU, forward and backward, against the
reference's vectors (attention_ref with `bias` / `dropout_mask`, mask from the reference's own
mask kernel) and the CPU oracle.

Bars: the keep mask is bit-exact; outputs and gradients meet the reference's criterion
(tests/test_flash_attention_triton.py:132-142): maximum absolute error at most twice that of a
plain torch implementation running in the same 16-bit precision.
"""
import numpy as np
import pytest
import torch

import fast_ops_b200._lib as L
import oracle
from fast_ops.flash_attention.flash_attention_triton import flash_attn_triton, triton_dropout_mask
from fast_ops_b200.flash_attention import (
    dropout_mask,
    flash_attention_backward,
    flash_attention_forward,
    next_dropout_rng,
)
from helpers import DT, attention_dout, attention_inputs, golden_files, load_attention_ex_case

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["ws64", "ws"])
def impl(request):
    """Forces one of the two warp-specialised forward kernels (each has bias / dropout variants of
    its own; left alone the library picks by shape, which small tests would never vary)."""
    L.attn_configure(impl=request.param)
    yield request.param
    L.attn_configure(impl="auto")


def torch_same_precision(q, k, v, dout, causal, bias, keep, p):
    """Output and gradients with torch ops in the tensors' own 16-bit dtype
    (attention_ref with upcast=False, reorder_ops=True: tests/test_flash_attention_triton.py:107-117)."""
    q, k, v = (t.clone().requires_grad_(True) for t in (q, k, v))
    d = q.shape[-1]
    scores = torch.matmul(q, (k / d ** 0.5).transpose(-1, -2))
    if bias is not None:
        scores = (scores + bias).to(scores.dtype)
    if causal:
        mask = torch.triu(torch.ones(q.shape[2], k.shape[2], dtype=torch.bool, device=q.device), 1)
        scores = scores.masked_fill(mask, float("-inf"))
    attn = torch.softmax(scores, dim=-1)
    if keep is not None:
        attn = attn.masked_fill(~keep, 0.0)
    out = torch.matmul(attn, v * (1.0 / (1.0 - p)))
    out.backward(dout)
    return out.detach(), q.grad, k.grad, v.grad


def run_case(device, q, k, v, dout, causal, bias, p, rng, bias_dtype=torch.float32):
    qd, kd, vd, dd = (t.to(device) for t in (q, k, v, dout))
    bd = None if bias is None else bias.to(device=device, dtype=bias_dtype)
    o, lse = flash_attention_forward(qd, kd, vd, causal=causal, return_lse=True, bias=bd, dropout_p=p, rng=rng)
    dq, dk, dv = flash_attention_backward(dd, qd, kd, vd, o, lse, causal=causal, bias=bd, dropout_p=p, rng=rng)
    torch.cuda.synchronize()
    assert L.device_status(device.index) == 0, "a kernel wait timed out"
    keep = None
    if p > 0:
        B, H, Sq, _ = q.shape
        keep = dropout_mask(p, B, H, Sq, k.shape[2], device, rng=rng)
    same = torch_same_precision(qd, kd, vd, dd, causal, bd, keep, p)
    return (o, dq, dk, dv), lse, same, keep


def check(got, same, want, what, rows=None):
    names = ("out", "dq", "dk", "dv")
    for i, (name, g, s, w) in enumerate(zip(names, got, same, want)):
        g, s = g.float().cpu(), s.float().cpu()
        if rows is not None:
            r = rows[0] if name in ("out", "dq") else rows[1]
            g, s = g[:, :, r], s[:, :, r]
        err = (g - w).abs().max().item()
        err_torch = (s - w).abs().max().item()
        assert err <= 2 * err_torch + 1e-4, f"{what} {name}: error {err:.3e} vs same-precision torch {err_torch:.3e}"


@pytest.mark.parametrize("path", golden_files("attnex"), ids=lambda p: p.split("attnex_")[-1][:-4])
def test_bias_dropout_match_reference_vectors(cuda_device, impl, path):
    g, q, k, v, dout, bias, keep = load_attention_ex_case(path)
    p = float(g["dropout_p"])
    rng = (int(g["rng_seed"]), int(g["rng_offset"]))
    got, lse, same, keep_gpu = run_case(cuda_device, q, k, v, dout, bool(g["causal"]), bias, p, rng)
    if keep is not None:
        assert torch.equal(keep_gpu.cpu(), keep), "keep mask differs from the reference's mask kernel"
    want = [torch.from_numpy(g[n]) for n in ("out", "dq", "dk", "dv")]
    check(got, same, want, "reference vectors", rows=(g["rows_q"], g["rows_k"]))
    # LSE is that of the scores without dropout
    _, lse_o = oracle.attention_ex(q, k, v, bias=bias, causal=bool(g["causal"]))
    assert torch.allclose(lse.cpu(), lse_o, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("offset", [0, 16646144, 2**32 - 1000, 2**40 + 38813696 - 5000])
@pytest.mark.parametrize("seed", [0, 123, 2**33 + 7])
def test_dropout_mask_bit_exact(cuda_device, seed, offset):
    B, H, Sq, Sk = 2, 3, 130, 203
    got = dropout_mask(0.17, B, H, Sq, Sk, cuda_device, rng=(seed, offset))
    want = oracle.dropout_mask(0.17, B, H, Sq, Sk, seed, offset)
    assert torch.equal(got.cpu(), want)
    got = dropout_mask(0.5, 1, 1, 64, 64, cuda_device, rng=(seed, offset))
    assert torch.equal(got.cpu(), oracle.dropout_mask(0.5, 1, 1, 64, 64, seed, offset))


CASES = [
    # B, H, Sq, Sk, D, dtype, causal, bias code, bias dtype, dropout_p
    (2, 2, 512, 512, 128, torch.bfloat16, True, "1h1k", torch.float32, 0.0),
    (2, 2, 384, 384, 64, torch.float16, False, "b11k", torch.float16, 0.0),
    (1, 2, 300, 520, 128, torch.bfloat16, False, "1hqk", torch.bfloat16, 0.0),
    (2, 1, 257, 203, 64, torch.bfloat16, True, "b1qk", torch.float32, 0.0),   # odd row length: scalar loads
    (1, 2, 131, 77, 128, torch.float16, False, "1h1k", torch.float16, 0.0),
    (2, 2, 512, 512, 128, torch.bfloat16, True, None, None, 0.17),
    (1, 3, 260, 390, 64, torch.float16, False, None, None, 0.3),
    (2, 2, 384, 384, 128, torch.bfloat16, True, "b1qk", torch.float32, 0.17),
    (1, 2, 200, 333, 64, torch.bfloat16, False, "1h1k", torch.bfloat16, 0.1),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "B%dH%dSq%dSk%dD%d_%s_%s_%s_p%g" % (
    c[0], c[1], c[2], c[3], c[4], str(c[5])[6:], "causal" if c[6] else "full", c[7], c[9]))
def test_bias_dropout_match_oracle(cuda_device, impl, case):
    B, H, Sq, Sk, D, dtype, causal, code, bias_dtype, p = case
    q, k, v = attention_inputs(900 + Sq + Sk, B, H, Sq, Sk, D, dtype)
    dout = attention_dout(31 + Sq, B, H, Sq, D, dtype)
    bias = None
    if code is not None:
        shape = {"1h1k": (1, H, 1, Sk), "1hqk": (1, H, Sq, Sk), "b11k": (B, 1, 1, Sk), "b1qk": (B, 1, Sq, Sk)}[code]
        gen = torch.Generator().manual_seed(5 + Sq)
        bias = torch.randn(shape, generator=gen).to(bias_dtype).float()  # values exactly representable
        bias[..., 5::23] = float("-inf")
    # offsets next to a boundary between a kept and a dropped run of the hash, so that the mask
    # of a tensor this small has both
    rng = (0, 16773120 + 4096 - (B * H * Sq * Sk) // 2 // 4 * 4) if p > 0 else None
    got, lse, same, keep = run_case(cuda_device, q, k, v, dout, causal, bias, p, rng,
                                    bias_dtype=bias_dtype or torch.float32)
    keep_cpu = None
    if p > 0:
        keep_cpu = oracle.dropout_mask(p, B, H, Sq, Sk, *rng)
        assert torch.equal(keep.cpu(), keep_cpu)
        assert 0.05 < keep_cpu.float().mean().item() < 0.95
    out, lse_o, dq, dk, dv = oracle.attention_ex(q, k, v, bias=bias, keep_mask=keep_cpu, dropout_p=p, causal=causal,
                                                 dout=dout)
    check(got, same, (out, dq, dk, dv), "oracle")
    assert torch.allclose(lse.cpu(), lse_o, atol=2e-3, rtol=1e-3)


def _bias_of(code, B, H, Sq, Sk, seed, dtype=torch.float32):
    shape = {"1h1k": (1, H, 1, Sk), "1hqk": (1, H, Sq, Sk), "b11k": (B, 1, 1, Sk), "b1qk": (B, 1, Sq, Sk)}[code]
    gen = torch.Generator().manual_seed(seed)
    bias = torch.randn(shape, generator=gen).to(dtype).float()
    bias[..., 5::23] = float("-inf")
    return bias


def test_long_key_range_with_vector_bias_takes_the_128_key_kernel(cuda_device):
    """Nothing forced: a bias without dropout over more than 48 key tiles is where the library
    switches from the 64-key to the 128-key forward kernel.  Sk = 6272 is 49 tiles, not causal."""
    L.attn_configure(impl="auto")
    B, H, Sq, Sk, D = 1, 1, 384, 6272, 128
    q, k, v = attention_inputs(77, B, H, Sq, Sk, D, torch.bfloat16)
    dout = attention_dout(78, B, H, Sq, D, torch.bfloat16)
    bias = _bias_of("1h1k", B, H, Sq, Sk, 79)
    got, lse, same, _ = run_case(cuda_device, q, k, v, dout, False, bias, 0.0, None)
    out, lse_o, dq, dk, dv = oracle.attention_ex(q, k, v, bias=bias, causal=False, dout=dout)
    check(got, same, (out, dq, dk, dv), "49 key tiles, vector bias")
    assert torch.allclose(lse.cpu(), lse_o, atol=2e-3, rtol=1e-3)
    # and one tile fewer stays on the 64-key kernel: both sides of the switch agree with the oracle
    q2, k2, v2 = q, k[:, :, :6144].contiguous(), v[:, :, :6144].contiguous()
    bias2 = bias[..., :6144].contiguous()
    got2, lse2, same2, _ = run_case(cuda_device, q2, k2, v2, dout, False, bias2, 0.0, None)
    out2, lse_o2, dq2, dk2, dv2 = oracle.attention_ex(q2, k2, v2, bias=bias2, causal=False, dout=dout)
    check(got2, same2, (out2, dq2, dk2, dv2), "48 key tiles, vector bias")
    assert torch.allclose(lse2.cpu(), lse_o2, atol=2e-3, rtol=1e-3)


# The reference's own grid (tests/test_flash_attention_triton.py:24-37): seqlen 3072, head_dim 128,
# every bias shape, with and without dropout, with and without multi-query K/V.  Batch and heads
# are kept at 2 x 2 so that the CPU oracle stays within seconds per case.
REF_GRID = [(code, p, mq) for code in (None, "1h1k", "b11k", "1hqk", "b1qk") for p, mq in ((0.0, False), (0.17, True))]
REF_GRID += [(None, 0.17, False), ("1h1k", 0.17, False), ("1hqk", 0.0, True)]


@pytest.mark.parametrize("code,p,mq", REF_GRID, ids=lambda x: str(x))
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
def test_reference_grid_seqlen_3072(cuda_device, code, p, mq, causal):
    if causal != (code in (None, "1h1k", "b1qk")):
        pytest.skip("each bias shape runs with one mask setting, alternating")
    L.attn_configure(impl="auto")
    B, H, S, D = 2, 2, 3072, 128
    dtype = torch.bfloat16
    q, k, v = attention_inputs(3072 + len(str(code)), B, H, S, S, D, dtype)
    if mq:  # one K/V head shared by all query heads, expanded with stride 0 as the reference's tests do
        k, v = k[:, :1].expand(B, H, S, D), v[:, :1].expand(B, H, S, D)
    dout = attention_dout(3073, B, H, S, D, dtype)
    bias = None if code is None else _bias_of(code, B, H, S, S, 3074)
    rng = (0, 16773120 + 4096 - (B * H * S * S) // 2 // 4 * 4) if p > 0 else None
    dev = cuda_device
    qd, dd = q.to(dev), dout.to(dev)
    kd = k[:, :1].contiguous().to(dev).expand(B, H, S, D) if mq else k.to(dev)
    vd = v[:, :1].contiguous().to(dev).expand(B, H, S, D) if mq else v.to(dev)
    bd = None if bias is None else bias.to(dev)
    o, lse = flash_attention_forward(qd, kd, vd, causal=causal, return_lse=True, bias=bd, dropout_p=p, rng=rng)
    dq, dk, dv = flash_attention_backward(dd, qd, kd, vd, o, lse, causal=causal, bias=bd, dropout_p=p, rng=rng)
    torch.cuda.synchronize()
    assert L.device_status(dev.index) == 0, "a kernel wait timed out"
    keep = dropout_mask(p, B, H, S, S, dev, rng=rng) if p > 0 else None
    keep_cpu = None
    if p > 0:
        keep_cpu = oracle.dropout_mask(p, B, H, S, S, *rng)
        assert torch.equal(keep.cpu(), keep_cpu)
        assert 0.05 < keep_cpu.float().mean().item() < 0.95
    same = torch_same_precision(qd, kd.contiguous(), vd.contiguous(), dd, causal, bd, keep, p)
    want = oracle.attention_ex(q, k.contiguous(), v.contiguous(), bias=bias, keep_mask=keep_cpu, dropout_p=p,
                               causal=causal, dout=dout)
    check((o, dq, dk, dv), same, (want[0], want[2], want[3], want[4]), f"S=3072 {code} p={p} mq={mq}")
    assert torch.allclose(lse.cpu(), want[1], atol=2e-3, rtol=1e-3)


def test_bshd_entry_returns_q_layout_with_and_without_grad(cuda_device):
    """The reference allocates O with q's layout (flash_attention_triton.py:773): for ordinary
    contiguous (B, S, H, D) inputs `out.view(B, S, H * D)` must work in training and in eval."""
    B, S, H, D = 2, 200, 3, 64
    gen = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(B, S, H, D, generator=gen).half().to(cuda_device) for _ in range(3))
    assert q.is_contiguous()
    with torch.no_grad():
        o_eval = flash_attn_triton(q, k, v, None, True)
    qg = q.clone().requires_grad_(True)
    o_train = flash_attn_triton(qg, k, v, None, True)
    for o in (o_eval, o_train):
        assert o.shape == (B, S, H, D) and o.is_contiguous() and o.stride() == q.stride()
        o.view(B, S, H * D)
    assert torch.equal(o_eval, o_train.detach())
    o_train.sum().backward()
    assert qg.grad is not None and qg.grad.shape == q.shape


def test_generator_advances_on_every_bshd_forward(cuda_device):
    """increment_philox_state runs on every forward of the reference, with or without dropout
    (flash_attention_triton.py:780); later draws from the generator then match a reference run."""
    B, S, H, D = 1, 130, 2, 64
    q, k, v = (torch.randn(B, S, H, D, device=cuda_device, dtype=torch.float16) for _ in range(3))
    with torch.cuda.device(cuda_device):
        torch.cuda.manual_seed(5)
        before = next_dropout_rng(cuda_device, 0)
        flash_attn_triton(q, k, v)  # dropout_p = 0
        after = next_dropout_rng(cuda_device, 0)
    assert after[0] == before[0] and after[1] == before[1] + (B * H * S * S + 3) // 4 * 4


@pytest.mark.parametrize("code", ["1h1k", "b1qk"])
def test_fully_masked_rows_give_zero(cuda_device, code):
    """Bias of -inf everywhere (mask_all in tests/test_flash_attention_triton.py:86-87): the torch
    oracle gives NaN; this implementation defines O = 0, LSE = -inf and zero gradients."""
    B, H, S, D = 1, 2, 200, 64
    q, k, v = (t.to(cuda_device) for t in attention_inputs(3, B, H, S, S, D, torch.bfloat16))
    dout = attention_dout(3, B, H, S, D, torch.bfloat16).to(cuda_device)
    shape = {"1h1k": (1, H, 1, S), "b1qk": (B, 1, S, S)}[code]
    bias = torch.full(shape, float("-inf"), device=cuda_device)
    o, lse = flash_attention_forward(q, k, v, bias=bias, return_lse=True)
    assert torch.count_nonzero(o) == 0 and torch.all(lse == float("-inf"))
    dq, dk, dv = flash_attention_backward(dout, q, k, v, o, lse, bias=bias)
    for t in (dq, dk, dv):
        assert torch.count_nonzero(t) == 0
    # only some rows fully masked: the others are unaffected
    bias2 = torch.zeros(B, 1, S, S, device=cuda_device)
    bias2[:, :, 7] = float("-inf")
    o2, lse2 = flash_attention_forward(q, k, v, bias=bias2, return_lse=True)
    o_plain, lse_plain = flash_attention_forward(q, k, v, return_lse=True)
    rows = [r for r in range(S) if r != 7]
    assert torch.equal(o2[:, :, rows], o_plain[:, :, rows]) or torch.allclose(
        o2[:, :, rows].float(), o_plain[:, :, rows].float(), atol=1e-2)
    assert torch.count_nonzero(o2[:, :, 7]) == 0 and torch.all(lse2[:, :, 7] == float("-inf"))
    assert L.device_status(cuda_device.index) == 0


def test_reference_call_sequence_with_generator(cuda_device):
    """The flow of the reference's test (tests/test_flash_attention_triton.py:92-100): seed, call
    the (B, S, H, D) function with dropout, reseed, materialise the mask, compare with the oracle."""
    B, S, H, D, p = 2, 256, 2, 64, 0.17
    q, k, v = attention_inputs(8, B, H, S, S, D, torch.float16)
    dout = attention_dout(8, B, H, S, D, torch.float16)
    with torch.cuda.device(cuda_device):
        # start the generator next to a boundary of the hash so that the mask is mixed
        torch.cuda.manual_seed(0)
        next_dropout_rng(cuda_device, 16773120 + 4096 - B * H * S * S // 2)
        bias = torch.randn(1, H, 1, S, device=cuda_device)  # draws from the same generator: before the snapshot
        state = torch.cuda.get_rng_state(cuda_device)
        qs, ks, vs = (t.transpose(1, 2).to(cuda_device).requires_grad_(True) for t in (q, k, v))  # (B, S, H, D)
        out = flash_attn_triton(qs, ks, vs, bias, True, p)
        out.backward(dout.transpose(1, 2).to(cuda_device))
        after = next_dropout_rng(cuda_device, 0)
        torch.cuda.set_rng_state(state, cuda_device)
        keep = triton_dropout_mask(p, B, H, S, S, cuda_device)
        assert next_dropout_rng(cuda_device, 0) == after  # both advance the generator alike
    assert 0.05 < keep.float().mean().item() < 0.95
    want = oracle.attention_ex(q, k, v, bias=bias.cpu(), keep_mask=keep.cpu(), dropout_p=p, causal=True, dout=dout)
    got = (out.detach().transpose(1, 2), qs.grad.transpose(1, 2), ks.grad.transpose(1, 2), vs.grad.transpose(1, 2))
    same = torch_same_precision(*(t.to(cuda_device) for t in (q, k, v, dout)), True, bias, keep, p)
    check(got, same, (want[0], want[2], want[3], want[4]), "flash_attn_triton")
    # without grad the same call takes the forward-only path
    with torch.no_grad(), torch.cuda.device(cuda_device):
        torch.cuda.set_rng_state(state, cuda_device)
        out2 = flash_attn_triton(qs, ks, vs, bias, True, p)
    assert torch.equal(out2, out.detach())


def test_argument_errors(cuda_device):
    q, k, v = (t.to(cuda_device) for t in attention_inputs(1, 1, 2, 128, 128, 64, torch.bfloat16))
    with pytest.raises(RuntimeError, match="Last 2 dimensions of bias"):
        flash_attention_forward(q, k, v, bias=torch.zeros(1, 2, 64, 128, device=cuda_device))
    with pytest.raises(RuntimeError, match="float32 or have Q's dtype"):
        flash_attention_forward(q, k, v, bias=torch.zeros(1, 2, 1, 128, device=cuda_device, dtype=torch.float16))
    with pytest.raises(RuntimeError, match="4-D"):
        flash_attention_forward(q, k, v, bias=torch.zeros(128, device=cuda_device))
    with pytest.raises(RuntimeError, match="rng"):
        flash_attention_forward(q, k, v, dropout_p=0.1)
    with pytest.raises(RuntimeError, match="dropout_p"):
        flash_attention_forward(q, k, v, dropout_p=1.0, rng=(0, 0))
    # a bias that wants a gradient is refused in backward, as in the reference
    bias = torch.zeros(1, 2, 1, 128, device=cuda_device, requires_grad=True)
    qg = q.clone().requires_grad_(True)
    out = flash_attn_triton(qg.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), bias)
    with pytest.raises(RuntimeError, match="bias gradient"):
        out.sum().backward()
    # the C ABI rejects a bias of a third dtype and a negative stride
    lib = L.load()
    import ctypes
    s = (ctypes.c_int64 * 3)(128 * 64 * 2, 128 * 64, 64)
    bs = (ctypes.c_int64 * 3)(0, 0, 0)
    o = torch.empty_like(q)
    rc = lib.fo_flash_attn_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), None, 1, 2, 128, 128, 64,
                                  s, s, s, s, L.FO_BF16, 0, 0.125, q.data_ptr(), bs, L.FO_F16, 0.0, 0, 0,
                                  cuda_device.index, None)
    assert rc == -1 and b"bias" in lib.fo_last_error()  # FO_ERR_INVALID_ARGUMENT
    bs = (ctypes.c_int64 * 3)(0, -8, 0)
    rc = lib.fo_flash_attn_fwd_ex(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), None, 1, 2, 128, 128, 64,
                                  s, s, s, s, L.FO_BF16, 0, 0.125, q.data_ptr(), bs, L.FO_BF16, 0.0, 0, 0,
                                  cuda_device.index, None)
    assert rc == -1
