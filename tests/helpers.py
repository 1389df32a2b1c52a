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
