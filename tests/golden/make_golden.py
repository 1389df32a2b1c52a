"""Generates the golden vectors in this directory by running the REFERENCE implementations.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py /path/to/fast-ops [attention|attention_bwd|attention_ex|lion]

It imports fast_ops.flash_attention.attention_ref.attention_ref and
fast_ops.lion.lion_optimizer_ref.Lion from that checkout, feeds them seeded inputs and stores
inputs (or the seed and a digest of the inputs) and outputs as .npz files.  The tests only
read the .npz files; the reference is not needed to run them.

Lion vectors are produced single-threaded on sizes that are multiples of the CPU vector width,
because torch's CPU kernels treat the scalar `alpha` of add_ differently in their vectorised
body and in their scalar tail, and the tail's position depends on the thread count.
"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def bits(t: torch.Tensor) -> np.ndarray:
    """Raw storage of a tensor as a numpy array (uint16 for the 16-bit types)."""
    t = t.detach().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def attention_inputs(seed, B, H, Sq, Sk, D, dtype):
    """Q, K, V ~ N(0,1) in (B,H,S,D) layout from a seeded CPU generator, cast to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, Sq, D, generator=gen).to(dtype)
    k = torch.randn(B, H, Sk, D, generator=gen).to(dtype)
    v = torch.randn(B, H, Sk, D, generator=gen).to(dtype)
    return q, k, v


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(bits(t).tobytes())
    return h.hexdigest()


def make_attention(attention_ref):
    cases = [
        # name, seed, B, H, Sq, Sk, D, input dtype, causal, row stride of the stored sample
        ("c1_b2h4s256d64_f32_full", 0, 2, 4, 256, 256, 64, "f32", False, 4),
        ("s384d128_bf16_causal", 1, 1, 2, 384, 384, 128, "bf16", True, 3),
        ("s200d128_f16_causal_ragged", 2, 1, 2, 200, 200, 128, "f16", True, 1),
        ("s131d64_bf16_full_ragged", 3, 2, 1, 131, 131, 64, "bf16", False, 1),
        ("sq128sk320d64_f16_causal", 4, 1, 1, 128, 320, 64, "f16", True, 1),
        ("sq300sk100d128_bf16_full", 5, 1, 1, 300, 100, 128, "bf16", False, 1),
        ("s1024d64_bf16_causal", 6, 1, 2, 1024, 1024, 64, "bf16", True, 16),
    ]
    for name, seed, B, H, Sq, Sk, D, dt, causal, step in cases:
        q, k, v = attention_inputs(seed, B, H, Sq, Sk, D, DT[dt])
        # The reference takes (B,S,H,D); upcast=True makes it compute in fp32 and cast back
        # to the input dtype, so feed it fp32 copies of the (already rounded) inputs.
        qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
        out, attn = attention_ref(qf, kf, vf, causal=causal, upcast=True)
        out = out.transpose(1, 2).contiguous()  # (B,H,Sq,D)
        # LSE: the reference's torch path does not return it; rebuild it from the same scores
        # and check it against the attention matrix the reference did return.
        scores = torch.einsum("bhtd,bhsd->bhts", q.float() / (D ** 0.5), k.float())
        if causal:
            scores.masked_fill_(torch.triu(torch.ones(Sq, Sk, dtype=torch.bool), 1), float("-inf"))
        lse = torch.logsumexp(scores, dim=-1)
        assert torch.allclose(torch.exp(scores - lse[..., None]), attn, atol=2e-6), name
        rows = np.arange(0, Sq, step)
        np.savez_compressed(
            os.path.join(HERE, f"attn_{name}.npz"),
            seed=seed, shape=np.array([B, H, Sq, Sk, D]), dtype=dt, causal=causal,
            input_sha256=digest(q, k, v), rows=rows,
            out=out[:, :, rows, :].numpy(), lse=lse[:, :, rows].numpy())
        print("attention", name, out.shape, "stored rows", len(rows))


def make_attention_bwd(attention_ref):
    """Gradients through the reference's attention_ref by autograd, the way the reference's own
    tests obtain them (tests/test_flash_attention_triton.py:118-131)."""
    cases = [
        # name, seed, B, H, Sq, Sk, D, input dtype, causal
        ("s256d64_bf16_causal", 11, 1, 2, 256, 256, 64, "bf16", True),
        ("s200d128_f16_causal_ragged", 12, 1, 1, 200, 200, 128, "f16", True),
        ("sq130sk300d64_bf16_full", 13, 1, 2, 130, 300, 64, "bf16", False),
        ("s384d128_bf16_full", 14, 1, 1, 384, 384, 128, "bf16", False),
    ]
    for name, seed, B, H, Sq, Sk, D, dt, causal in cases:
        q, k, v = attention_inputs(seed, B, H, Sq, Sk, D, DT[dt])
        gen = torch.Generator().manual_seed(seed + 1000)
        dout = torch.randn(B, H, Sq, D, generator=gen).to(DT[dt])
        qf, kf, vf = (t.float().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        out, _ = attention_ref(qf, kf, vf, causal=causal, upcast=True)
        out.backward(dout.float().transpose(1, 2))
        np.savez_compressed(
            os.path.join(HERE, f"attnbwd_{name}.npz"),
            seed=seed, shape=np.array([B, H, Sq, Sk, D]), dtype=dt, causal=causal,
            input_sha256=digest(q, k, v, dout),
            dq=qf.grad.transpose(1, 2).contiguous().numpy(), dk=kf.grad.transpose(1, 2).contiguous().numpy(),
            dv=vf.grad.transpose(1, 2).contiguous().numpy())
        print("attention backward", name)


def reference_dropout_mask(ref_root, dropout_p, B, H, Sq, Sk, seed, offset):
    """Keep mask from the reference's own _dropout_mask_kernel
    (fast_ops/flash_attention/flash_attention_triton.py:668-696), run on the CPU by Triton's
    interpreter (TRITON_INTERPRET=1 is set in main() before triton is imported).  The
    interpreter leaves a Python float argument a float, on which the kernel's `.to()` fails, so
    dropout_p is handed over as the fp32 scalar the compiled kernel would receive."""
    import importlib.util

    import triton
    import triton.language as tl
    from triton.runtime.interpreter import TensorHandle

    spec = importlib.util.spec_from_file_location(
        "ref_flash_attention_triton", os.path.join(ref_root, "fast_ops/flash_attention/flash_attention_triton.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    p32 = tl.tensor(TensorHandle(np.array([dropout_p], dtype=np.float32), tl.float32), tl.float32)
    t = torch.empty((B, H, Sq, Sk), dtype=torch.int32)
    grid = (triton.cdiv(Sq, 128), B * H)
    mod._dropout_mask_kernel[grid](t, p32, Sq, Sk, seed, offset, 128, 128)
    return t.to(torch.bool)


def attention_ex_inputs(seed, B, H, Sq, Sk, D, dtype, bias_code):
    """Q, K, V as attention_inputs; dO and the fp32 bias from a second seeded generator.  The
    bias gets a few -inf (masking) entries, never a whole row."""
    q, k, v = attention_inputs(seed, B, H, Sq, Sk, D, dtype)
    gen = torch.Generator().manual_seed(seed + 1000)
    dout = torch.randn(B, H, Sq, D, generator=gen).to(dtype)
    bias = None
    if bias_code is not None:
        shape = {"1h1k": (1, H, 1, Sk), "1hqk": (1, H, Sq, Sk), "b11k": (B, 1, 1, Sk), "b1qk": (B, 1, Sq, Sk)}[bias_code]
        bias = torch.randn(shape, generator=gen)
        bias[..., 3::17] = float("-inf")
    return q, k, v, dout, bias


def make_attention_ex(attention_ref, ref_root):
    """Forward and autograd gradients of attention_ref with a bias and / or a dropout mask
    (fast_ops/flash_attention/attention_ref.py:50-51, :60-67), the mask made by the reference's
    mask kernel.  The reference's hash keeps or drops runs of up to ~10^6 consecutive element
    indices, so the offsets below are chosen next to a boundary of such a run (found by
    evaluating the hash) to get masks that contain both kept and dropped elements."""
    cases = [
        # name, seed, B, H, Sq, Sk, D, dtype, causal, bias shape code, dropout_p, rng seed, rng offset
        ("bias1h1k_s200d64_bf16_causal", 21, 2, 2, 200, 200, 64, "bf16", True, "1h1k", 0.0, 0, 0),
        ("biasb1qk_sq130sk300d128_f16_full", 22, 2, 2, 130, 300, 128, "f16", False, "b1qk", 0.0, 0, 0),
        ("bias1hqk_s256d128_bf16_causal", 23, 1, 2, 256, 256, 128, "bf16", True, "1hqk", 0.0, 0, 0),
        ("drop_s256d64_bf16_full", 24, 2, 2, 256, 256, 64, "bf16", False, None, 0.17, 0, 16646144),
        ("drop_biasb11k_s200d128_f16_causal", 25, 2, 3, 200, 200, 128, "f16", True, "b11k", 0.17, 0, 17700000),
    ]
    for name, seed, B, H, Sq, Sk, D, dt, causal, bias_code, p, rseed, roff in cases:
        q, k, v, dout, bias = attention_ex_inputs(seed, B, H, Sq, Sk, D, DT[dt], bias_code)
        keep = None
        if p > 0:
            keep = reference_dropout_mask(ref_root, p, B, H, Sq, Sk, rseed, roff)
            frac = keep.float().mean().item()
            assert 0.05 < frac < 0.95, (name, frac)
        qf, kf, vf = (t.float().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        out, _ = attention_ref(qf, kf, vf, causal=causal, bias=bias, dropout_p=p, dropout_mask=keep, upcast=True)
        out.backward(dout.float().transpose(1, 2))
        rq, rk = np.arange(0, Sq, 3), np.arange(0, Sk, 3)  # stored sample of rows
        np.savez_compressed(
            os.path.join(HERE, f"attnex_{name}.npz"),
            seed=seed, shape=np.array([B, H, Sq, Sk, D]), dtype=dt, causal=causal,
            bias_code="" if bias_code is None else bias_code,
            dropout_p=p, rng_seed=rseed, rng_offset=roff,
            keep_packed=np.zeros(0, np.uint8) if keep is None else np.packbits(keep.numpy()),
            input_sha256=digest(*([q, k, v, dout] + ([] if bias is None else [bias]))),
            rows_q=rq, rows_k=rk,
            out=out.detach().transpose(1, 2)[:, :, rq].contiguous().numpy(),
            dq=qf.grad.transpose(1, 2)[:, :, rq].contiguous().numpy(),
            dk=kf.grad.transpose(1, 2)[:, :, rk].contiguous().numpy(),
            dv=vf.grad.transpose(1, 2)[:, :, rk].contiguous().numpy())
        print("attention ex", name, "keep fraction", None if keep is None else round(frac, 3))


def make_lion(LionRef):
    n = 2048
    cases = [
        # name, p dtype, m dtype, lr, betas, wd, p std, g std
        ("bf16_bf16_c5like", "bf16", "bf16", 3e-5, (0.9, 0.99), 0.1, 0.02, 1e-3),
        ("f32_bf16_c4like", "f32", "bf16", 1e-4, (0.9, 0.99), 0.1, 0.02, 1e-3),
        ("f32_f32", "f32", "f32", 1e-4, (0.9, 0.99), 0.1, 0.02, 1e-3),
        ("f16_f16_reftest", "f16", "f16", 1e-3, (0.9, 0.99), 0.5, 1.0, 1.0),
        ("bf16_bf16_reftest", "bf16", "bf16", 1e-3, (0.9, 0.99), 0.0, 1.0, 1.0),
        ("bf16_f32", "bf16", "f32", 1e-4, (0.95, 0.98), 0.1, 0.02, 1e-3),
    ]
    steps = 4
    for name, pd, md, lr, betas, wd, pstd, gstd in cases:
        gen = torch.Generator().manual_seed(sum(map(ord, name)))
        p0 = (torch.randn(n, generator=gen) * pstd).to(DT[pd])
        grads = [(torch.randn(n, generator=gen) * gstd).to(DT[pd]) for _ in range(steps)]
        # Adversarial entries: zero gradient (sign(0) must be 0 on the first step), and
        # gradients chosen so that beta1*m + (1-beta1)*g lands on or next to zero.
        for g in grads:
            g[:16] = 0
        param = p0.clone().requires_grad_(True)
        opt = LionRef([param], lr=lr, betas=betas, weight_decay=wd)
        opt.state[param]["exp_avg"] = torch.zeros(n, dtype=DT[md])
        ps, ms = [], []
        for s in range(steps):
            g = grads[s]
            if s > 0:
                m = opt.state[param]["exp_avg"].float()
                cancel = (-(m * betas[0]) / (1 - betas[0])).to(DT[pd])
                g[16:272] = cancel[16:272]
                # one storage-type ulp to either side of the cancelling value
                g[272:400] = torch.nextafter(cancel[272:400].float(), torch.tensor(float("inf"))).to(DT[pd])
                g[400:528] = torch.nextafter(cancel[400:528].float(), torch.tensor(float("-inf"))).to(DT[pd])
            param.grad = g.clone()
            opt.step()
            ps.append(bits(param.data))
            ms.append(bits(opt.state[param]["exp_avg"]))
        np.savez_compressed(
            os.path.join(HERE, f"lion_{name}.npz"),
            p_dtype=pd, m_dtype=md, lr=lr, betas=np.array(betas), weight_decay=wd,
            p0=bits(p0), grads=np.stack([bits(g) for g in grads]), params=np.stack(ps),
            exp_avgs=np.stack(ms))
        print("lion", name, pd, md)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the jfc4050/fast-ops checkout> [all|attention|attention_bwd|"
                         "attention_ex|lion]")
    ref_root = sys.argv[1]
    os.environ["TRITON_INTERPRET"] = "1"  # the reference's mask kernel runs on the CPU
    sys.path.insert(0, ref_root)
    from fast_ops.flash_attention.attention_ref import attention_ref
    from fast_ops.lion.lion_optimizer_ref import Lion as LionRef

    torch.set_num_threads(1)
    only = sys.argv[2] if len(sys.argv) > 2 else "all"
    if only in ("all", "attention"):
        make_attention(attention_ref)
    if only in ("all", "attention_bwd"):
        make_attention_bwd(attention_ref)
    if only in ("all", "attention_ex"):
        make_attention_ex(attention_ref, ref_root)
    if only in ("all", "lion"):
        make_lion(LionRef)


if __name__ == "__main__":
    main()
