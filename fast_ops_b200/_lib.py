"""Loads the C-ABI library (libfast_ops_b200.so) and declares its entry points for ctypes.

There is no fallback: if the library is missing and cannot be built, or a call fails, the
caller gets a RuntimeError.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
# FO_B200_LIB points the loader at another build of the same library (kernel tuning).
LIB_PATH = os.environ.get("FO_B200_LIB") or os.path.join(_HERE, "libfast_ops_b200.so")

FO_F16, FO_BF16, FO_F32 = 0, 1, 2

_lock = threading.Lock()
_lib = None

_c = ctypes
_PTR = _c.c_void_p
_I64P = _c.POINTER(_c.c_int64)

# name -> (restype, argtypes); mirrors include/fast_ops_b200.h
SIGNATURES = {
    "fo_version": (_c.c_int, []),
    "fo_last_error": (_c.c_char_p, []),
    "fo_device_status": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_int), _c.c_int]),
    "fo_flash_attn_fwd": (_c.c_int, [_PTR, _PTR, _PTR, _PTR, _PTR,
                                     _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                     _I64P, _I64P, _I64P, _I64P,
                                     _c.c_int, _c.c_int, _c.c_float, _c.c_int, _PTR]),
    "fo_attn_configure": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int]),
    "fo_flash_attn_bwd": (_c.c_int, [_PTR] * 11 + [_c.c_int] * 5 + [_I64P] * 8 +
                          [_c.c_int, _c.c_int, _c.c_float, _c.c_int, _PTR]),
    "fo_flash_attn_fwd_ex": (_c.c_int, [_PTR, _PTR, _PTR, _PTR, _PTR,
                                        _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                        _I64P, _I64P, _I64P, _I64P,
                                        _c.c_int, _c.c_int, _c.c_float,
                                        _PTR, _I64P, _c.c_int, _c.c_float, _c.c_uint64, _c.c_uint64,
                                        _c.c_int, _PTR]),
    "fo_flash_attn_bwd_ex": (_c.c_int, [_PTR] * 11 + [_c.c_int] * 5 + [_I64P] * 8 +
                             [_c.c_int, _c.c_int, _c.c_float,
                              _PTR, _I64P, _c.c_int, _c.c_float, _c.c_uint64, _c.c_uint64,
                              _c.c_int, _PTR]),
    "fo_dropout_mask": (_c.c_int, [_PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_float,
                                   _c.c_uint64, _c.c_uint64, _c.c_int, _PTR]),
    "fo_lion_update": (_c.c_int, [_PTR, _PTR, _PTR, _c.c_int64, _c.c_int, _c.c_int, _c.c_int,
                                  _c.c_double, _c.c_double, _c.c_double, _c.c_double, _c.c_int, _PTR]),
    "fo_lion_multi_tensor_step": (_c.c_int, [_c.POINTER(_PTR), _c.POINTER(_PTR), _c.POINTER(_PTR), _I64P, _c.c_int,
                                             _c.c_int, _c.c_int, _c.c_int,
                                             _c.c_double, _c.c_double, _c.c_double, _c.c_double, _c.c_int, _PTR]),
    "fo_lion_multi_tensor_step_noalloc": (_c.c_int, [_c.POINTER(_PTR), _c.POINTER(_PTR), _c.POINTER(_PTR), _I64P,
                                                     _c.c_int, _c.c_int, _c.c_int, _c.c_int,
                                                     _c.c_double, _c.c_double, _c.c_double, _c.c_double,
                                                     _c.c_int, _PTR]),
    "fo_lion_flat_step": (_c.c_int, [_PTR, _PTR, _PTR, _c.c_int64, _c.c_int64, _c.c_int, _c.c_int, _c.c_int,
                                     _c.c_double, _c.c_double, _c.c_double, _c.c_double, _c.c_int, _PTR]),
    "fo_lion_flat_step_push": (_c.c_int, [_PTR, _PTR, _PTR, _c.c_int64, _c.c_int64, _c.POINTER(_PTR), _c.c_int,
                                          _c.c_int, _c.c_int, _c.c_int,
                                          _c.c_double, _c.c_double, _c.c_double, _c.c_double, _c.c_int, _PTR]),
    "fo_lion_clear_cache": (_c.c_int, []),
    "fo_launch_count": (_c.c_int64, []),
    "fo_debug_wait_timeout": (_c.c_int, [_c.c_int, _PTR, _c.c_int, _PTR]),
    "fo_debug_set_attn_trace": (_c.c_int, [_PTR]),
    "fo_debug_attn_trace_shape": (_c.c_int, [_c.POINTER(_c.c_int), _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "fo_debug_umma_tile": (_c.c_int, [_PTR, _PTR, _PTR, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _PTR]),
}


def load() -> ctypes.CDLL:
    """Returns the loaded library, building it first if the file is missing (needs nvcc).  An
    existing library is loaded as it is, even when sources are newer: rebuild with
    `python -m fast_ops_b200.build` after editing them."""
    global _lib
    if _lib is not None:  # the common case, without the lock
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            from . import build as _build

            try:
                _build.build()
            except Exception as exc:  # no nvcc, compile error, ...
                raise RuntimeError(
                    f"fast_ops_b200: {LIB_PATH} is missing and could not be built ({exc}); "
                    "run `python -m fast_ops_b200.build` where nvcc is available") from exc
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here means header and library disagree
            fn.restype = restype
            fn.argtypes = argtypes
        _apply_env_options(lib)
        _lib = lib
        return lib


ATTN_IMPLS = {"auto": 0, "simple": 1, "ws": 2, "ws64": 3, "ws64p": 4, "ws64s": 5}


def attn_configure(impl=None, ping_pong=None, head_group=None) -> None:
    """Process-wide options of the attention forward (C-ABI fo_attn_configure); None leaves an
    option unchanged.  impl: "auto" | "simple" | "ws" | "ws64" | "ws64p" | "ws64s"; ping_pong: bool; head_group: heads
    scheduled together for L2 reuse, 0 = automatic."""
    check(load().fo_attn_configure(-1 if impl is None else ATTN_IMPLS[impl],
                                   -1 if ping_pong is None else int(bool(ping_pong)),
                                   -1 if head_group is None else int(head_group)))


def _apply_env_options(lib) -> None:
    """FO_ATTN_IMPL / FO_ATTN_PINGPONG / FO_ATTN_HEAD_GROUP are read once, when the library is
    loaded (the library itself reads no environment variable)."""
    impl = os.environ.get("FO_ATTN_IMPL")
    pp = os.environ.get("FO_ATTN_PINGPONG")
    hg = os.environ.get("FO_ATTN_HEAD_GROUP")
    if impl is not None and impl not in ATTN_IMPLS:
        raise RuntimeError(f"FO_ATTN_IMPL must be one of {sorted(ATTN_IMPLS)}, got {impl!r}")
    lib.fo_attn_configure(-1 if impl is None else ATTN_IMPLS[impl], -1 if pp is None else int(int(pp) != 0),
                          -1 if hg is None else int(hg))


def check(rc: int) -> None:
    """Turns a non-zero status into RuntimeError carrying the library's message."""
    if rc != 0:
        msg = load().fo_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"fast_ops_b200 error {rc}: {msg}")


def dtype_code(dtype) -> int:
    import torch

    try:
        return {torch.float16: FO_F16, torch.bfloat16: FO_BF16, torch.float32: FO_F32}[dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype}") from None


def current_stream_ptr(device) -> int:
    """Raw cudaStream_t of torch's current stream on `device` (the cheap accessor when this torch
    has it: constructing a torch.cuda.Stream object costs a few microseconds per call)."""
    import torch

    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        index = device.index if isinstance(device, torch.device) else int(device)
        if index is None:
            index = torch.cuda.current_device()
        return raw(index)
    return torch.cuda.current_stream(device).cuda_stream


def device_status(device_index: int, reset: bool = False) -> int:
    out = ctypes.c_int(0)
    check(load().fo_device_status(int(device_index), ctypes.byref(out), int(reset)))
    return out.value
