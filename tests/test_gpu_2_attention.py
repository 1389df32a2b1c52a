"""FlashAttention forward on the GPU against the reference's vectors and the CPU oracle.

Tolerances are the stated bars: max-abs 2e-3 for fp16 and 1e-2 for bf16 inputs against the
fp32 softmax(QK^T/sqrt(d))V of the reference.
"""
import numpy as np
import pytest
import torch

import fast_ops_b200._lib as L
import oracle
from fast_ops_b200.flash_attention import flash_attn_bshd, flash_attention_forward, multi_head_attention
from helpers import DT, attention_inputs, golden_files, input_digest

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}
LSE_TOL = 1e-3
IMPLS = ["ws", "ws64", "ws64p", "ws64s", "simple"]


@pytest.fixture(params=IMPLS)
def impl(request):
    L.attn_configure(impl=request.param)
    yield request.param
    L.attn_configure(impl="auto")


def run_gpu(q, k, v, device, **kw):
    out, lse = flash_attention_forward(q.to(device), k.to(device), v.to(device), return_lse=True, **kw)
    torch.cuda.synchronize()
    assert L.device_status(device.index) == 0, "a kernel wait timed out"
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("path", golden_files("attn"), ids=lambda p: p.split("attn_")[-1][:-4])
def test_attention_matches_reference_vectors(cuda_device, impl, path):
    z = np.load(path)
    B, H, Sq, Sk, D = (int(x) for x in z["shape"])
    in_dtype = DT[str(z["dtype"])]
    q, k, v = attention_inputs(int(z["seed"]), B, H, Sq, Sk, D, in_dtype)
    assert input_digest(q, k, v) == str(z["input_sha256"])
    # fp32 reference inputs run on the GPU as their fp16 cast (the reference's CPU config)
    run_dtype = torch.float16 if in_dtype == torch.float32 else in_dtype
    out, lse = run_gpu(q.to(run_dtype), k.to(run_dtype), v.to(run_dtype), cuda_device, causal=bool(z["causal"]))
    rows = torch.from_numpy(z["rows"])
    err = (out.float()[:, :, rows, :] - torch.from_numpy(z["out"])).abs().max().item()
    assert err <= TOL[run_dtype], f"max-abs error {err}"
    lse_tol = 5e-3 if in_dtype == torch.float32 else LSE_TOL  # the fp16 cast of fp32 inputs moves the scores
    assert (lse[:, :, rows] - torch.from_numpy(z["lse"])).abs().max().item() <= lse_tol


@pytest.mark.parametrize("case", [
    # B, H, Sq, Sk, D, dtype, causal
    (8, 12, 1024, 1024, 64, torch.bfloat16, True),     # GPT-2-small shape
    (1, 2, 2048, 2048, 128, torch.bfloat16, True),
    (1, 2, 2048, 2048, 128, torch.float16, False),
    (2, 3, 640, 640, 128, torch.float16, True),
    (1, 1, 129, 129, 64, torch.bfloat16, True),
    (1, 2, 1, 1, 128, torch.bfloat16, True),
    (1, 1, 77, 513, 64, torch.float16, False),
    (3, 1, 513, 77, 128, torch.bfloat16, True),
], ids=lambda c: "B%dH%dSq%dSk%dD%d_%s_%s" % (c[0], c[1], c[2], c[3], c[4], str(c[5])[6:], "causal" if c[6] else "full"))
def test_attention_matches_oracle(cuda_device, impl, case):
    B, H, Sq, Sk, D, dtype, causal = case
    q, k, v = attention_inputs(1234 + Sq + Sk, B, H, Sq, Sk, D, dtype)
    ref, ref_lse = oracle.attention_fwd(q, k, v, causal=causal)
    out, lse = run_gpu(q, k, v, cuda_device, causal=causal)
    err = (out.float() - ref).abs().max().item()
    assert err <= TOL[dtype], f"max-abs error {err}"
    assert (lse - ref_lse).abs().max().item() <= LSE_TOL


@pytest.mark.parametrize("kernel", ["ws64", "ws64p", "ws"])
def test_long_context_sample_against_oracle(cuda_device, kernel):
    """S = 16384, D = 128, bf16, causal (the long-context shape) on two heads, all rows checked."""
    L.attn_configure(impl=kernel)
    q, k, v = attention_inputs(99, 1, 2, 16384, 16384, 128, torch.bfloat16)
    ref, ref_lse = oracle.attention_fwd(q, k, v, causal=True)
    try:
        out, lse = run_gpu(q, k, v, cuda_device, causal=True)
    finally:
        L.attn_configure(impl="auto")
    assert (out.float() - ref).abs().max().item() <= TOL[torch.bfloat16]
    assert (lse - ref_lse).abs().max().item() <= LSE_TOL


def test_full_size_properties(cuda_device):
    """B=2, H=32, S=16384, D=128, bf16, causal: properties that need no oracle at this size (the
    kernel the library chooses by itself)."""
    L.attn_configure(impl="auto")
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    B, H, S, D = 2, 32, 16384, 128
    q, k, v = (torch.randn(B, H, S, D, generator=gen, device=cuda_device, dtype=torch.float32).bfloat16()
               for _ in range(3))
    o1, l1 = flash_attention_forward(q, k, v, causal=True, return_lse=True)
    o2, l2 = flash_attention_forward(q, k, v, causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert L.device_status(cuda_device.index) == 0
    assert torch.equal(o1, o2) and torch.equal(l1, l2), "two runs differ"
    # causal row 0 sees one key: O = V[0], LSE = scale * q0.k0
    assert torch.equal(o1[:, :, 0], v[:, :, 0])
    s00 = (q[:, :, 0].float() * k[:, :, 0].float()).sum(-1) / D ** 0.5
    assert torch.allclose(l1[:, :, 0], s00, atol=1e-3)
    # a head computed alone equals the same head inside the batch (no cross-talk between CTAs)
    b, h = 1, 17
    oa, la = flash_attention_forward(q[b:b + 1, h:h + 1], k[b:b + 1, h:h + 1], v[b:b + 1, h:h + 1], causal=True,
                                     return_lse=True)
    assert torch.equal(oa[0, 0], o1[b, h]) and torch.equal(la[0, 0], l1[b, h])
    # rows are convex combinations of V rows
    assert o1.float().abs().max() <= v.float().abs().max() * 1.01
    # the two kernels agree on a slice
    L.attn_configure(impl="simple")
    try:
        os_, ls_ = flash_attention_forward(q[:1, :2], k[:1, :2], v[:1, :2], causal=True, return_lse=True)
    finally:
        L.attn_configure(impl="auto")
    assert (os_.float() - o1[:1, :2].float()).abs().max().item() <= 1e-2
    assert (ls_ - l1[:1, :2]).abs().max().item() <= 1e-3


def test_strided_bshd_views_and_scale(cuda_device, impl):
    B, S, H, D = 2, 300, 3, 64
    gen = torch.Generator().manual_seed(8)
    q, k, v = (torch.randn(B, S, H, D, generator=gen).half() for _ in range(3))
    ref, _ = oracle.attention_fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=True,
                                  softmax_scale=0.2)
    out = flash_attn_bshd(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True, softmax_scale=0.2)
    torch.cuda.synchronize()
    assert out.shape == (B, S, H, D)
    assert (out.cpu().float().transpose(1, 2) - ref).abs().max().item() <= TOL[torch.float16]


def test_reference_call_signature_and_errors(cuda_device):
    q, k, v = attention_inputs(3, 1, 2, 256, 256, 64, torch.float16)
    qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
    out = multi_head_attention(qd, kd, vd)  # the reference's call: three positional tensors
    ref, _ = oracle.attention_fwd(q, k, v)
    assert out.dtype == torch.float16 and out.shape == q.shape
    assert (out.cpu().float() - ref).abs().max().item() <= TOL[torch.float16]
    with pytest.raises(RuntimeError):
        multi_head_attention(qd.float(), kd.float(), vd.float())
    with pytest.raises(RuntimeError):
        multi_head_attention(q, k, v)  # CPU tensors: no CPU path
    # a head_dim between the two kernel sizes, as a strided view: runs zero-padded
    out48 = multi_head_attention(qd[..., :48], kd[..., :48], vd[..., :48])
    ref48, _ = oracle.attention_fwd(q[..., :48], k[..., :48], v[..., :48])
    assert (out48.cpu().float() - ref48).abs().max().item() <= TOL[torch.float16]
    with pytest.raises(RuntimeError):
        multi_head_attention(qd[..., :44], kd[..., :44], vd[..., :44])  # not a multiple of 8
    with pytest.raises(RuntimeError):
        multi_head_attention(qd, kd[:, :1], vd)
    with pytest.raises(RuntimeError):
        bad = torch.randn(1, 2, 256, 136, device=cuda_device).half()
        multi_head_attention(bad, bad, bad)  # head_dim > 128


def test_host_pipelined_forward_matches_device_forward(cuda_device):
    from fast_ops_b200.flash_attention import flash_attention_forward_host

    q, k, v = attention_inputs(21, 2, 6, 512, 512, 64, torch.bfloat16)
    hq, hk, hv = (t.pin_memory() for t in (q, k, v))
    host_out = flash_attention_forward_host(hq, hk, hv, device=cuda_device, causal=True, heads_per_chunk=4)
    torch.cuda.synchronize()
    dev_out = flash_attention_forward(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=True)
    assert host_out.device.type == "cpu" and torch.equal(host_out, dev_out.cpu())
    # a second call reuses the workspace and the slots in a different order of completion
    host_out2 = flash_attention_forward_host(hq, hk, hv, device=cuda_device, causal=True, heads_per_chunk=1)
    torch.cuda.synchronize()
    assert torch.equal(host_out2, host_out)
    with pytest.raises(RuntimeError):
        flash_attention_forward_host(q.to(cuda_device), hk, hv)


def test_multi_query_expanded_kv(cuda_device, impl):
    """K and V with one head expanded over H query heads (stride 0), as the reference's tests
    build multi-query inputs (tests/test_flash_attention_triton.py:71-73)."""
    B, H, S, D = 2, 4, 300, 128
    gen = torch.Generator().manual_seed(31)
    q = torch.randn(B, H, S, D, generator=gen).bfloat16()
    k1, v1 = (torch.randn(B, 1, S, D, generator=gen).bfloat16() for _ in range(2))
    ref, ref_lse = oracle.attention_fwd(q, k1.expand(B, H, S, D), v1.expand(B, H, S, D), causal=True)
    kd, vd = k1.to(cuda_device).expand(B, H, S, D), v1.to(cuda_device).expand(B, H, S, D)
    assert kd.stride(1) == 0
    out, lse = flash_attention_forward(q.to(cuda_device), kd, vd, causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert (out.cpu().float() - ref).abs().max().item() <= TOL[torch.bfloat16]
    assert (lse.cpu() - ref_lse).abs().max().item() <= LSE_TOL


@pytest.mark.parametrize("D", [8, 32, 40, 80, 96, 120])
@pytest.mark.parametrize("causal", [False, True])
def test_other_head_dims_run_zero_padded(cuda_device, impl, D, causal):
    """The reference's contract is D <= 128, D % 8 == 0 (fast_ops/flash_attention/flash_attention.py:61-70);
    the kernels are built for 64 and 128 and take the others with TMA zero-fill."""
    B, H, Sq, Sk = 2, 2, 200, 333
    dtype = torch.bfloat16 if D % 16 else torch.float16
    q, k, v = attention_inputs(50 + D, B, H, Sq, Sk, D, dtype)
    want, lse_want = oracle.attention_fwd(q, k, v, causal=causal)
    out, lse = flash_attention_forward(q.to(cuda_device), k.to(cuda_device), v.to(cuda_device), causal=causal,
                                       return_lse=True)
    tol = 1e-2 if dtype == torch.bfloat16 else 2e-3
    assert (out.float().cpu() - want).abs().max().item() <= tol
    assert (lse.cpu() - lse_want).abs().max().item() <= 1e-3
