"""Shared test helpers: golden-file access, seeded inputs, ulp distances."""
import glob
import hashlib
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def golden_files(prefix):
    return sorted(glob.glob(os.path.join(GOLDEN, prefix + "_*.npz")))


def from_bits(a: np.ndarray, dtype: torch.dtype) -> torch.Tensor:
    """Inverse of the generator's `bits`: raw storage -> torch tensor."""
    if dtype in (torch.float16, torch.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).view(dtype)
    return torch.from_numpy(a.copy())


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def attention_inputs(seed, B, H, Sq, Sk, D, dtype):
    """The generator's input recipe: Q, K, V ~ N(0,1), (B,H,S,D), seeded CPU generator."""
    gen = torch.Generator().manual_seed(int(seed))
    q = torch.randn(B, H, Sq, D, generator=gen).to(dtype)
    k = torch.randn(B, H, Sk, D, generator=gen).to(dtype)
    v = torch.randn(B, H, Sk, D, generator=gen).to(dtype)
    return q, k, v


def attention_ex_inputs(seed, B, H, Sq, Sk, D, dtype, bias_code):
    """The generator's recipe for the bias / dropout cases: Q, K, V as above, dO and an fp32 bias
    (with a few -inf entries) from a second seeded generator."""
    q, k, v = attention_inputs(seed, B, H, Sq, Sk, D, dtype)
    gen = torch.Generator().manual_seed(int(seed) + 1000)
    dout = torch.randn(B, H, Sq, D, generator=gen).to(dtype)
    bias = None
    if bias_code:
        shape = {"1h1k": (1, H, 1, Sk), "1hqk": (1, H, Sq, Sk), "b11k": (B, 1, 1, Sk), "b1qk": (B, 1, Sq, Sk)}[bias_code]
        bias = torch.randn(shape, generator=gen)
        bias[..., 3::17] = float("-inf")
    return q, k, v, dout, bias


def load_attention_ex_case(path):
    """(golden dict, q, k, v, dout, bias, keep mask or None) of one attnex_*.npz file, with the
    regenerated inputs checked against the stored digest."""
    g = np.load(path)
    B, H, Sq, Sk, D = (int(x) for x in g["shape"])
    q, k, v, dout, bias = attention_ex_inputs(int(g["seed"]), B, H, Sq, Sk, D, DT[str(g["dtype"])], str(g["bias_code"]))
    assert input_digest(*([q, k, v, dout] + ([] if bias is None else [bias]))) == str(g["input_sha256"])
    keep = None
    if float(g["dropout_p"]) > 0:
        keep = torch.from_numpy(np.unpackbits(g["keep_packed"])[: B * H * Sq * Sk].reshape(B, H, Sq, Sk).astype(bool))
    return g, q, k, v, dout, bias, keep


def input_digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        h.update(to_bits(t).tobytes())
    return h.hexdigest()


def ordered_int(t: torch.Tensor) -> torch.Tensor:
    """Maps a float tensor to integers whose difference is the distance in ulps of its dtype."""
    if t.dtype == torch.float32:
        i = t.detach().cpu().contiguous().view(torch.int32).to(torch.int64)
        return torch.where(i < 0, -(i & 0x7FFFFFFF), i)
    i = t.detach().cpu().contiguous().view(torch.int16).to(torch.int64)
    return torch.where(i < 0, -(i & 0x7FFF), i)


def ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    assert a.dtype == b.dtype
    return (ordered_int(a) - ordered_int(b)).abs()


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 ulps (the unit the parity bar is stated in), for any float dtype."""
    return (ordered_int(a.float().bfloat16()) - ordered_int(b.float().bfloat16())).abs()


def attention_dout(seed, B, H, Sq, D, dtype):
    """The generator's recipe for the output gradient of the backward vectors."""
    gen = torch.Generator().manual_seed(int(seed) + 1000)
    return torch.randn(B, H, Sq, D, generator=gen).to(dtype)
