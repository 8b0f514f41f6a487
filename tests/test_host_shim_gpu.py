"""The C++ op-set shim (kiln_b200/host/gpu_ops.cpp) through its C trampolines: same names, argument
meaning and error behaviour as the reference's attention()/attention16()/rmsnorm()/rope_half()."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from golden_inputs import gen
from util_gpu import assert_close, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def shim(built_lib):
    from kiln_b200 import build
    S = ctypes.CDLL(build.build_host())
    ws = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    S.kbh_set_context.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    S.kbh_set_context(None, ctypes.c_void_p(ws.data_ptr()), ws.numel())
    S._ws = ws
    return S


P = lambda t: ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("case", gen.ATTN_CASES, ids=[c[0] for c in gen.ATTN_CASES])
def test_attention_and_attention16_vs_reference_golden(shim, golden, case):
    name, Tq, Tk, npad, H = case
    q, k, v = gen.attn_inputs(case)
    ld = H * 128
    dq, dk, dv = dev(q), dev(k), dev(v)                       # fp32, as the engine holds them
    err = ctypes.create_string_buffer(256)
    o32 = torch.zeros(Tq, ld, device="cuda")
    assert shim.kbh_attention(P(o32), ld, P(dq), ld, P(dk), ld, P(dv), ld, Tq, Tk, H, 128, 0, npad, 1, err, 256) == 0, err.value
    o16 = torch.zeros(Tq, ld, device="cuda", dtype=torch.float16)
    assert shim.kbh_attention(P(o16), ld, P(dq), ld, P(dk), ld, P(dv), ld, Tq, Tk, H, 128, 0, npad, 0, err, 256) == 0, err.value
    torch.cuda.synchronize()
    assert_close(o32.cpu().numpy(), golden[f"{name}/ref_attn"], f"shim attention {name}")
    assert_close(o16.float().cpu().numpy(), golden[f"{name}/tfa_f16"].astype(np.float32), f"shim attention16 {name} vs tfa::k_flash")


def test_errors_become_exceptions(shim):
    t = torch.zeros(64, 256, device="cuda")
    err = ctypes.create_string_buffer(256)
    assert shim.kbh_attention(P(t), 256, P(t), 256, P(t), 256, P(t), 256, 64, 64, 4, 64, 0, 0, 0, err, 256) == -1
    assert b"unsupported head size" in err.value              # the reference's message (engine/src/kernels.cu:870)
    assert shim.kbh_attention(P(t), 256, P(t), 256, P(t), 256, P(t), 256, 64, 64, 2, 128, 1, 0, 1, err, 256) == -1
    assert b"causal" in err.value
    assert shim.kbh_attention(P(t), 256, P(t), 250, P(t), 256, P(t), 256, 64, 64, 2, 128, 0, 0, 1, err, 256) == -1


def test_rmsnorm_rope_in_place_fp32_vs_reference_golden(shim, golden):
    x, w_bits, H = gen.norm_inputs()
    T = x.shape[0]
    c, s = oracle.cosmos_rope(6, 8)
    ref = oracle.rope_half(golden["rmsnorm/out"], T, H, c, s)   # the reference kernel's norm output, then its RoPE arithmetic
    dx = dev(x)
    dw = torch.from_numpy(w_bits.view(np.int16)).cuda()
    err = ctypes.create_string_buffer(256)
    assert shim.kbh_rmsnorm_rope(P(dx), P(dw), T, H, ctypes.c_float(1e-6), P(dev(c)), P(dev(s)), err, 256) == 0, err.value
    torch.cuda.synchronize()
    np.testing.assert_allclose(dx.cpu().numpy(), ref, rtol=1e-5, atol=2e-6)
