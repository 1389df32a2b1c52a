"""The C-ABI library loads without a GPU and exports exactly what include/fast_ops_b200.h declares."""
import ctypes
import os
import re

import fast_ops_b200._lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fast_ops_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fo_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("fo_flash_attn_fwd", "fo_lion_update", "fo_lion_multi_tensor_step", "fo_lion_flat_step",
                 "fo_last_error", "fo_device_status"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(L.LIB_PATH) if os.path.exists(L.LIB_PATH) else L.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_signatures_cover_the_header():
    assert sorted(L.SIGNATURES) == declared_functions()


def test_version_and_error_text_need_no_gpu():
    lib = L.load()
    assert lib.fo_version() >= 100
    assert lib.fo_last_error() == b""
    # argument validation happens before any CUDA call
    rc = lib.fo_lion_update(None, None, None, 8, L.FO_BF16, L.FO_F16, L.FO_BF16, 1e-4, 0.9, 0.99, 0.0, 0, None)
    assert rc == -1 and b"same dtype" in lib.fo_last_error()
    s = (ctypes.c_int64 * 3)(0, 0, 0)
    rc = lib.fo_flash_attn_fwd(1, 1, 1, 1, None, 1, 1, 128, 128, 100, s, s, s, s, L.FO_BF16, 0, 0.1, 0, None)
    assert rc == -1 and b"head_dim" in lib.fo_last_error()
    rc = lib.fo_flash_attn_fwd(1, 1, 1, 1, None, 1, 1, 128, 128, 130, s, s, s, s, L.FO_BF16, 0, 0.1, 0, None)
    assert rc == -1


def test_bias_and_dropout_arguments_are_validated_without_a_gpu():
    lib = L.load()
    s = (ctypes.c_int64 * 3)(0, 0, 0)
    common = (1, 1, 1, 1, None, 1, 1, 128, 128, 64, s, s, s, s, L.FO_BF16, 0, 0.125)
    rc = lib.fo_flash_attn_fwd_ex(*common, None, None, L.FO_F32, 1.0, 0, 0, 0, None)
    assert rc == -1 and b"dropout_p" in lib.fo_last_error()
    rc = lib.fo_flash_attn_fwd_ex(*common, 16, s, L.FO_F16, 0.0, 0, 0, 0, None)
    assert rc == -1 and b"bias must be fp32" in lib.fo_last_error()
    rc = lib.fo_flash_attn_fwd_ex(*common, 16, None, L.FO_F32, 0.0, 0, 0, 0, None)
    assert rc == -1 and b"strides" in lib.fo_last_error()
    rc = lib.fo_dropout_mask(None, 1, 1, 8, 8, 0.5, 0, 0, 0, None)
    assert rc == -1
    rc = lib.fo_dropout_mask(16, 1, 1, 8, 8, 0.0, 0, 0, 0, None)
    assert rc == -1 and b"dropout_p" in lib.fo_last_error()


def test_attention_options_are_validated_without_a_gpu():
    lib = L.load()
    assert lib.fo_attn_configure(-1, -1, -1) == 0  # leaves everything as it is
    assert lib.fo_attn_configure(6, -1, -1) == -1 and b"impl" in lib.fo_last_error()
    assert lib.fo_attn_configure(-1, 2, -1) == -1 and b"ping_pong" in lib.fo_last_error()
    assert lib.fo_attn_configure(-1, -1, -2) == -1 and b"head_group" in lib.fo_last_error()
    L.attn_configure(impl="ws", ping_pong=False, head_group=3)
    L.attn_configure(impl="auto", ping_pong=True, head_group=0)
