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


def test_linear16_epilogues_and_heads(shim):
    """linear16 with the engine's Epi16 values and the fused head form, against the oracle; an ineligible weight throws."""
    M, N, K, H = 150, 256, 128, 2
    x = oracle.round16(oracle.randn(500, M * K), 0).reshape(M, K)
    w = oracle.round16(oracle.randn(501, N * K) * np.float32(0.05), 0).reshape(N, K)
    gate = oracle.randn(502, N)
    resid = oracle.randn(503, M * N).reshape(M, N)
    dx, dw = dev(x).half(), dev(w).half()
    err = ctypes.create_string_buffer(256)
    f = ctypes.c_float
    for epi in range(4):
        c32 = epi in (0, 3)
        c = dev(resid).clone() if epi == 3 else torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32 if c32 else torch.float16)
        assert shim.kbh_linear16(P(c), N, P(dx), M, P(dw), N, K, epi, P(dev(gate)) if epi == 3 else None, None, None, None, 0, f(0),
                                 err, 256) == 0, err.value
        torch.cuda.synchronize()
        ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None)
        assert np.abs(c.float().cpu().numpy() - ref).max() <= 2e-4 + 2.0 ** -10 * np.abs(ref).max(), epi
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(504, 128), 1)
    bits = (nw.view(np.uint32) >> 16).astype(np.uint16)
    cos, sin = oracle.cosmos_rope(10, 15)
    y = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
    assert shim.kbh_linear16(P(y), N, P(dx), M, P(dw), N, K, 4, None, P(dev(bits.view(np.int16))), P(dev(cos)), P(dev(sin)), 150, f(1e-6),
                             err, 256) == 0, err.value
    torch.cuda.synchronize()
    assert_close(y.float().cpu().numpy(), oracle.linear_heads16(x, w, H, bits, cos, sin), "shim linear16_heads")
    assert shim.kbh_linear16(P(y), N, P(dx), M, P(dw), 192, K, 1, None, None, None, None, 0, f(0), err, 256) == -1
    assert b"eligible" in err.value


def test_enqueue_cost_from_cpp(shim):
    """Host cost of one call from C++ (no Python in the loop): printed with -s; the bound only guards against regressions
    of an order of magnitude (a DiT step makes ~100 calls of 30-150 us of device time each)."""
    Tq, Tk, H = 1536, 64, 16
    q = torch.randn(Tq, H * 128, device="cuda").half()
    k = torch.randn(Tk, H * 128, device="cuda").half()
    v = torch.randn(Tk, H * 128, device="cuda").half()
    out = torch.empty_like(q)
    shim.kbh_enqueue_cost_us.restype = ctypes.c_double
    shim.kbh_enqueue_cost_us.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int] * 5
    shim.kbh_enqueue_cost_us(P(out), P(q), P(k), P(v), Tq, Tk, 0, H, 20)                  # warm-up
    us = shim.kbh_enqueue_cost_us(P(out), P(q), P(k), P(v), Tq, Tk, 0, H, 200)
    print(f"\nhost cost per kb_attn_cross call from C++: {us:.2f} us (200 calls, device time ~8 us each)")
    assert 0 < us < 100
