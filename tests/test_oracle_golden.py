"""CPU tests: the oracle (oracle/kiln_oracle.c) against the golden vectors produced by the
reference's own kernels on a B200 (tests/golden/ref_fixtures.npz) and against torch on CPU."""
import os

import numpy as np
import pytest
import torch

import oracle
from golden_inputs import gen


def _digest_ok(golden, key, *arrays):
    assert str(golden[key]) == gen.digest(*arrays), f"{key}: regenerated inputs differ from the fixture's (libm?)"


def test_randn_matches_torch():
    # reference: engine/src/pipeline.cu:16-64 claims torch.randn's CPU stream; equal up to libm rounding
    for seed, n in [(0, 16), (7, 1000), (123456789, 100003), (3, 4096 * 2048 // 64)]:
        torch.manual_seed(seed)
        t = torch.randn(n).numpy()
        o = oracle.randn(seed, n)
        np.testing.assert_allclose(o, t, rtol=0, atol=2e-6)
    with pytest.raises(ValueError):
        oracle.randn(1, 8)


def test_round16_matches_torch():
    x = np.concatenate([oracle.randn(5, 4096) * 3, np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 6e-8, 5.96e-8, 3e38, -1e-40], np.float32)])
    assert np.array_equal(oracle.round16(x, 0), torch.from_numpy(x).half().float().numpy())
    assert np.array_equal(oracle.round16(x, 1), torch.from_numpy(x).bfloat16().float().numpy())


@pytest.mark.parametrize("case", gen.ATTN_CASES, ids=[c[0] for c in gen.ATTN_CASES])
def test_attention_vs_reference_fp32_kernel(golden, case):
    name, Tq, Tk, npad, H = case
    q, k, v = gen.attn_inputs(case)
    _digest_ok(golden, f"{name}/digest", q, k, v)
    ref = golden[f"{name}/ref_attn"]                      # bench/tfa_test.cu ref_attn, run on a B200
    o32 = oracle.attention(q, k, v, H, npad, acc64=False)
    o64 = oracle.attention(q, k, v, H, npad, acc64=True)
    # same arithmetic, different libm / FMA contraction / expf: a few ulp of the fp32 sums (outputs are O(1))
    np.testing.assert_allclose(o32, ref, rtol=1e-5, atol=5e-6)
    np.testing.assert_allclose(o64, ref, rtol=1e-5, atol=5e-6)
    # the reference's tensor-core kernel sits within the path's tolerance of the oracle
    tfa = golden[f"{name}/tfa_f16"].astype(np.float32)
    assert np.abs(tfa - o64).max() <= 2e-3
    assert np.abs(tfa - o64).sum() / np.abs(o64).sum() <= 1e-3


def test_attention_npad_equals_explicit_zero_keys():
    # the analytic rule (engine/src/gpu.h:149-151) must equal really appending npad zero keys
    H, Tq, Tk, npad = 2, 33, 26, 70
    q = oracle.randn(1, Tq * H * 128).reshape(Tq, -1)
    k = oracle.randn(2, Tk * H * 128).reshape(Tk, -1)
    v = oracle.randn(3, Tk * H * 128).reshape(Tk, -1)
    kz = np.concatenate([k, np.zeros((npad, H * 128), np.float32)])
    vz = np.concatenate([v, np.zeros((npad, H * 128), np.float32)])
    np.testing.assert_allclose(oracle.attention(q, k, v, H, npad), oracle.attention(q, kz, vz, H, 0), rtol=0, atol=1e-6)


def test_attention_vs_torch_sdpa():
    H, Tq, Tk = 3, 50, 77
    q = oracle.randn(4, Tq * H * 128).reshape(Tq, -1)
    k = oracle.randn(5, Tk * H * 128).reshape(Tk, -1)
    v = oracle.randn(6, Tk * H * 128).reshape(Tk, -1)
    t = lambda a, T: torch.from_numpy(a).double().view(T, H, 128).transpose(0, 1)
    ref = torch.nn.functional.scaled_dot_product_attention(t(q, Tq), t(k, Tk), t(v, Tk)).transpose(0, 1).reshape(Tq, -1).float().numpy()
    np.testing.assert_allclose(oracle.attention(q, k, v, H), ref, rtol=0, atol=1e-6)


def test_rmsnorm_vs_reference_kernel(golden):
    x, w_bits, H = gen.norm_inputs()
    _digest_ok(golden, "rmsnorm/digest", x, w_bits)
    np.testing.assert_allclose(oracle.rmsnorm(x, w_bits, H), golden["rmsnorm/out"], rtol=2e-6, atol=1e-7)


def test_rope_vs_reference_kernel(golden):
    x, Hp, Wp, H = gen.rope_inputs()
    _digest_ok(golden, "rope/digest", x)
    c, s = oracle.cosmos_rope(Hp, Wp)
    assert np.array_equal(c, golden["rope/cos"]) and np.array_equal(s, golden["rope/sin"])   # cosmos_rope, engine/src/dit.cu:196-215
    np.testing.assert_allclose(oracle.rope_half(x, Hp * Wp, H, c, s), golden["rope/out"], rtol=0, atol=1e-6)
    # first 22 frequency pairs are the temporal ones: identity for an image
    assert np.all(c[:, :22] == 1) and np.all(s[:, :22] == 0)


def test_nag_vs_reference_kernel(golden):
    zp, zn = gen.nag_inputs()
    _digest_ok(golden, "nag/digest", zp, zn)
    for i, (s, tau, alpha) in enumerate(gen.NAG_PARAMS):
        np.testing.assert_allclose(oracle.nag(zp, zn, s, tau, alpha, acc64=False), golden[f"nag/f32_{i}"], rtol=2e-6, atol=1e-7)
        np.testing.assert_allclose(oracle.nag(zp, zn, s, tau, alpha, acc64=True), golden[f"nag/f32_{i}"], rtol=1e-5, atol=1e-6)
        # fp16 rows: the kernel reads fp16, computes in fp32, rounds once (engine/src/dit.cu:289-292)
        zp16, zn16 = oracle.round16(zp, 0), oracle.round16(zn, 0)
        o16 = oracle.round16(oracle.nag(zp16, zn16, s, tau, alpha, acc64=False), 0)
        g16 = golden[f"nag/f16_{i}"].astype(np.float32)
        assert np.mean(o16 != g16) < 0.01 and np.abs(o16 - g16).max() <= 2e-3   # at most a rounding tie apart


def test_nag_identities():
    zp, zn = gen.nag_inputs()
    np.testing.assert_allclose(oracle.nag(zp, zn, 1.0, 2.5, 0.25), zp, rtol=1e-6, atol=1e-7)   # s=1: g = Z+
    np.testing.assert_allclose(oracle.nag(zp, zn, 5.0, 2.5, 0.0), zp, rtol=0, atol=0)          # alpha=0: Z+
    out = oracle.nag(zp, zn, 5.0, 2.5, 1.0)                                                    # alpha=1: clamped g
    ratio = np.abs(out).sum(1) / np.abs(zp).sum(1)
    assert np.all(ratio <= 2.5 * (1 + 1e-5))


# ---------------------------------------------------------------- the fp16 GEMM behind the projections
def _gemm_gen():
    import importlib.util
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "make_ref_gemm_fixtures.py")
    spec = importlib.util.spec_from_file_location("make_ref_gemm_fixtures", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_linear16_oracle_vs_reference_kernel_golden():
    """ko_linear16 against the outputs of the reference's tc16::k_gemm16 (all four epilogues). The reference sums each
    32-wide k tile in fp16 before flushing to fp32, so it is the less exact side: the bound is that tile error."""
    ggen = _gemm_gen()
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gemm_fixtures.npz"))
    for case in ggen.GEMM_CASES:
        name, M, N, K = case
        x, w, gate, resid = ggen.gemm_inputs(case)
        for ename, epi in ggen.EPIS.items():
            ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None)
            got = g[f"{name}/{ename}"].astype(np.float32)
            scale = np.abs(gate).max() if epi == 3 else 1.0
            bound = (2.0 ** -11 * np.sqrt(K / 32) * 4.0 + 2.0 ** -9 * np.abs(ref).max()) * scale
            assert np.abs(got - ref).max() <= bound, (name, ename, np.abs(got - ref).max(), bound)
            assert np.abs(got - ref).sum() / np.abs(ref).sum() <= 1e-3, (name, ename)


def test_attention_bwd_oracle_vs_reference_fixture():
    """ko_attention_bwd (fp64) against the outputs of the reference's attention_bwd (engine/src/train.cu:216-242: fp32 cuBLAS
    SGEMMs) recorded on a B200, and against central differences of the forward oracle."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_ref_bwd_fixtures", os.path.join(os.path.dirname(__file__), "golden", "make_ref_bwd_fixtures.py"))
    bgen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bgen)
    path = os.path.join(os.path.dirname(__file__), "golden", "ref_bwd_fixtures.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/ref_bwd_fixtures.npz has not been generated (tests/golden/make_ref_bwd_fixtures.py on a B200)")
    golden = np.load(path)
    n = bgen.KEEP_HEADS * 128
    for case in bgen.BWD_CASES:
        name, Tq, Tk, npad = case
        q, k, v, dout = bgen.bwd_inputs(case)
        outs = oracle.attention_bwd(q[:, :n], k[:, :n], v[:, :n], dout[:, :n], bgen.KEEP_HEADS, npad)   # heads are independent
        for gname, o in zip(("dq", "dk", "dv"), outs):
            g = golden[f"{name}/{gname}"]
            assert np.abs(o - g).max() <= 2e-5 * max(1.0, float(np.abs(g).max())), f"{name}/{gname}: {np.abs(o - g).max():.3e}"
    rng = np.random.default_rng(0)
    q, k, v, do = (rng.standard_normal((r, 128)).astype(np.float32) for r in (5, 7, 7, 5))
    for npad in (0, 3):
        dq, dk, dv = oracle.attention_bwd(q, k, v, do, 1, npad)
        f = lambda q, k, v: float((oracle.attention(q, k, v, 1, npad).astype(np.float64) * do).sum())
        for which, arr, grad in ((0, q, dq), (1, k, dk), (2, v, dv)):
            a, b = arr.copy(), arr.copy()
            a[2, 17] += 1e-2
            b[2, 17] -= 1e-2
            args_a, args_b = [q, k, v], [q, k, v]
            args_a[which], args_b[which] = a, b
            assert abs((f(*args_a) - f(*args_b)) / 2e-2 - grad[2, 17]) <= 2e-4
