"""Pins the CPU oracle to vectors produced by the reference itself (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

import oracle
from helpers import DT, attention_inputs, from_bits, golden_files, input_digest, to_bits


@pytest.mark.parametrize("path", golden_files("lion"), ids=lambda p: p.split("lion_")[-1][:-4])
def test_lion_oracle_matches_reference_bit_for_bit(path):
    z = np.load(path)
    pd, md = DT[str(z["p_dtype"])], DT[str(z["m_dtype"])]
    lr, betas, wd = float(z["lr"]), tuple(float(b) for b in z["betas"]), float(z["weight_decay"])
    p = from_bits(z["p0"], pd)
    m = torch.zeros(p.numel(), dtype=md)
    for s in range(z["grads"].shape[0]):
        g = from_bits(z["grads"][s], pd)
        oracle.lion_step(p, g, m, lr, betas, wd)
        assert np.array_equal(to_bits(p), z["params"][s]), f"param differs at step {s}"
        assert np.array_equal(to_bits(m), z["exp_avgs"][s]), f"exp_avg differs at step {s}"


def test_lion_oracle_sign_of_zero_is_zero():
    # grad = 0 and momentum = 0: torch.sign(0) = 0, so only weight decay moves the parameter
    # (fast_ops/lion/lion_optimizer_ref.py:65), unlike the reference CUDA kernel's sign(0) = -1
    # (fast_ops/lion/lion_update.cu:10-13).
    p = torch.full((64,), 0.5, dtype=torch.float32)
    g = torch.zeros(64)
    m = torch.zeros(64, dtype=torch.bfloat16)
    oracle.lion_step(p, g, m, 1e-2, (0.9, 0.99), 0.0)
    assert torch.equal(p, torch.full((64,), 0.5))
    assert torch.equal(m.float(), torch.zeros(64))


@pytest.mark.parametrize("path", golden_files("attn"), ids=lambda p: p.split("attn_")[-1][:-4])
def test_attention_oracle_matches_reference(path):
    z = np.load(path)
    B, H, Sq, Sk, D = (int(x) for x in z["shape"])
    q, k, v = attention_inputs(int(z["seed"]), B, H, Sq, Sk, D, DT[str(z["dtype"])])
    assert input_digest(q, k, v) == str(z["input_sha256"]), "seeded inputs differ from the generator's"
    out, lse = oracle.attention_fwd(q, k, v, causal=bool(z["causal"]))
    rows = torch.from_numpy(z["rows"])
    # fp32 against fp32: only the summation order differs.
    assert torch.allclose(out[:, :, rows, :], torch.from_numpy(z["out"]), atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse[:, :, rows], torch.from_numpy(z["lse"]), atol=5e-6, rtol=1e-6)


def test_attention_oracle_bh_range_and_empty():
    q, k, v = attention_inputs(11, 2, 3, 40, 40, 64, torch.float32)
    full, lse = oracle.attention_fwd(q, k, v, causal=True)
    part, lse_p = oracle.attention_fwd(q, k, v, causal=True, bh_range=(2, 4))
    assert torch.equal(part.view(6, 40, 64)[2:4], full.view(6, 40, 64)[2:4])
    assert torch.equal(lse_p.view(6, 40)[2:4], lse.view(6, 40)[2:4])
    assert part.view(6, 40, 64)[:2].abs().sum() == 0 and part.view(6, 40, 64)[4:].abs().sum() == 0
    # causal row 0 attends to one key: out = v[0], lse = scaled score
    assert torch.allclose(full[:, :, 0], v[:, :, 0])
    assert torch.allclose(lse[:, :, 0], (q[:, :, 0] * k[:, :, 0]).sum(-1) / 8, atol=1e-6)


def test_oracle_thread_count_does_not_change_results():
    q, k, v = attention_inputs(12, 1, 2, 100, 100, 64, torch.float32)
    n0 = oracle.num_threads()
    a, la = oracle.attention_fwd(q, k, v)
    oracle.set_num_threads(1)
    b, lb = oracle.attention_fwd(q, k, v)
    oracle.set_num_threads(0)
    assert oracle.num_threads() == n0
    assert torch.equal(a, b) and torch.equal(la, lb)


def test_attention_oracle_row_sampling():
    q, k, v = attention_inputs(13, 1, 2, 50, 50, 64, torch.float32)
    full, lse = oracle.attention_fwd(q, k, v, causal=True)
    part, lse_p = oracle.attention_fwd(q, k, v, causal=True, row_range=(3, 47, 5))
    rows = list(range(3, 47, 5))
    assert torch.equal(part[:, :, rows], full[:, :, rows]) and torch.equal(lse_p[:, :, rows], lse[:, :, rows])
    mask = torch.ones(50, dtype=torch.bool)
    mask[rows] = False
    assert part[:, :, mask].abs().sum() == 0


@pytest.mark.parametrize("path", golden_files("attnbwd"), ids=lambda p: p.split("attnbwd_")[-1][:-4])
def test_attention_backward_oracle_matches_reference_autograd(path):
    from helpers import attention_dout

    z = np.load(path)
    B, H, Sq, Sk, D = (int(x) for x in z["shape"])
    dt = DT[str(z["dtype"])]
    q, k, v = attention_inputs(int(z["seed"]), B, H, Sq, Sk, D, dt)
    dout = attention_dout(int(z["seed"]), B, H, Sq, D, dt)
    assert input_digest(q, k, v, dout) == str(z["input_sha256"])
    dq, dk, dv = oracle.attention_bwd(q, k, v, dout, causal=bool(z["causal"]))
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        want = torch.from_numpy(z[name])
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4), f"{name}: {(got - want).abs().max()}"


@pytest.mark.parametrize("path", golden_files("attnex"), ids=lambda p: p.split("attnex_")[-1][:-4])
def test_attention_bias_dropout_oracle_matches_reference(path):
    """Bias and dropout: the oracle against attention_ref's forward and autograd gradients, and its
    restatement of the keep mask, bit for bit, against the reference's own mask kernel."""
    from helpers import load_attention_ex_case

    g, q, k, v, dout, bias, keep = load_attention_ex_case(path)
    B, H, Sq, Sk, D = (int(x) for x in g["shape"])
    p = float(g["dropout_p"])
    if keep is not None:
        mine = oracle.dropout_mask(p, B, H, Sq, Sk, int(g["rng_seed"]), int(g["rng_offset"]))
        assert torch.equal(mine, keep)
        assert 0 < int(keep.sum()) < keep.numel()
    out, lse, dq, dk, dv = oracle.attention_ex(q, k, v, bias=bias, keep_mask=keep, dropout_p=p,
                                               causal=bool(g["causal"]), dout=dout)
    rq, rk = g["rows_q"], g["rows_k"]
    for name, got, rows in (("out", out, rq), ("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rk)):
        want = torch.from_numpy(g[name])
        got = got[:, :, rows]
        assert torch.allclose(got, want, atol=2e-5, rtol=1e-4), f"{name}: {(got - want).abs().max()}"
    # forward-only entry gives the same output and LSE
    out2, lse2 = oracle.attention_ex(q, k, v, bias=bias, keep_mask=keep, dropout_p=p, causal=bool(g["causal"]))
    assert torch.equal(out2, out) and torch.equal(lse2, lse)


def test_attention_ex_oracle_reduces_to_plain_attention():
    q, k, v = attention_inputs(77, 1, 2, 70, 90, 64, torch.float32)
    out, lse = oracle.attention_fwd(q, k, v, causal=True)
    out2, lse2 = oracle.attention_ex(q, k, v, causal=True)
    assert torch.allclose(out, out2, atol=1e-6) and torch.allclose(lse, lse2, atol=1e-6)


def test_dropout_mask_oracle_statistics():
    """The reference's statistical criterion (tests/test_flash_attention_triton.py:203-246: over
    many generator offsets every element is kept about 1 - p of the time).  The hash keeps or
    drops long runs of consecutive indices, so the offsets here are spread over the whole
    32-bit index range instead of following one another."""
    p, B, H, Sq, Sk = 0.17, 1, 2, 32, 128
    trials = 2048
    total = torch.zeros(B, H, Sq, Sk)
    for t in range(trials):
        total += oracle.dropout_mask(p, B, H, Sq, Sk, 0, t * (2**32 // trials))
    frac = total / trials
    assert abs(frac.mean().item() - (1 - p)) < 0.01
    assert frac.min().item() > 0.75 and frac.max().item() < 0.91
