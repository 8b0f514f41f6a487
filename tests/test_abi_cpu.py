"""CPU tests of the drop-in boundary: the library builds (nvcc cross-compiles), loads without a GPU,
exports every symbol include/kiln_b200.h declares, and refuses to run without an sm_100 device."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "kiln_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_lib):
    L = ctypes.CDLL(built_lib)
    names = _declared()
    assert {"kb_attn_self", "kb_attn_cross", "kb_attn_nag", "kb_qk_prep", "kb_status", "kb_attn_selfcheck", "kb_init"} <= set(names)
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/kiln_b200.h but not exported"


def test_error_strings_and_sizes(built_lib):
    import kiln_b200
    L = kiln_b200.lib()
    assert L.kb_version() >= 100
    for code in range(0, -9, -1):
        assert L.kb_error_string(code).decode() not in ("", "unknown error")
    assert L.kb_error_string(-99).decode() == "unknown error"
    # scratch = fp16 staging copies, 256-byte aligned (only what needs norm/RoPE for fp16 inputs, everything otherwise), plus,
    # for single-context calls, room for the balanced schedule's partial results: per SM two streams of (128 x 128 + 2 x 128)
    # floats and two flags (148 SMs are assumed where no device can be asked)
    F16, BF16, F32 = kiln_b200.KB_F16, kiln_b200.KB_BF16, kiln_b200.KB_F32
    split = 148 * 2 * (128 * 128 + 256) * 4 + 1280
    assert kiln_b200.workspace_bytes(4096, 4096, 16, F16, True, True) == 2 * 4096 * 2048 * 2 + split
    assert kiln_b200.workspace_bytes(4096, 4096, 16, BF16, True, True) == 3 * 4096 * 2048 * 2 + split
    assert kiln_b200.workspace_bytes(100, 7, 2, F16, True, False) == 100 * 256 * 2 + split
    assert kiln_b200.workspace_bytes(100, 7, 2, F16) == split
    assert kiln_b200.workspace_bytes(1, 1, 1, F16, True, True) == 512 + split
    # NAG adds the cross-head norm exchange: [12 query tiles][16 heads][2 column halves][2][128] floats + 12 counters (256-byte aligned)
    assert kiln_b200.workspace_bytes(1536, 512, 16, F32, n_ctx=2) == (1536 + 4 * 512) * 2048 * 2 + 12 * 16 * 2048 + 256
    assert kiln_b200.workspace_bytes(1536, 512, 16, F16, n_ctx=2) == 12 * 16 * 2048 + 256


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_no_device_fails_loudly(built_lib):
    """There is no CPU fallback: without a device every launch entry point returns KB_ERR_DEVICE."""
    import kiln_b200
    L = kiln_b200.lib()
    assert L.kb_init() == -6
    buf = (ctypes.c_char * 4096)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    a = ctypes.c_void_p((p.value + 255) & ~255)
    assert L.kb_attn_self(a, a, a, a, None, None, None, None, 1, 1, 1, 128, 128, 128, 128, 0, 0, 1e-6, None, 0, None) == -6
    assert L.kb_attn_nag(a, a, None, a, a, 1, 0, a, a, 1, 0, 5.0, 2.5, 0.25, 1, 1, 128, 128, 128, 0, 0, 1e-6, None, 0, None) == -6
    with pytest.raises(kiln_b200.KilnError):
        kiln_b200.check_status()
