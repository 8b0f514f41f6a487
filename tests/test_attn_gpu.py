"""GPU parity tests of the sm_100a kernels, called through the C ABI, against the CPU oracle
(fp64-accumulating restatement of the reference arithmetic) on the same seeded inputs.
Tolerance: max-abs <= 2e-3 and mean-relative <= 1e-3 (util_gpu.TOL_*)."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from golden_inputs import gen
from util_gpu import DT, assert_close, assert_close_bf16_storage, dev, sample_rows, seeded

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kb(built_lib):
    import kiln_b200
    assert kiln_b200.lib().kb_init() == 0, "sm_100 device and the CUDA library are required (there is no fallback)"
    return kiln_b200


def _ws(kb, rows_q, rows_k, H, kind, norm=False, n_ctx=1):
    n = kb.workspace_bytes(rows_q, rows_k, H, DT[kind], norm, norm, n_ctx)
    return torch.empty(max(n, 16), dtype=torch.uint8, device="cuda") if n else None


def _self(kb, q, k, v, B, T, H, kind, out_kind=None, **kw):
    out = torch.full((B * T, H * 128), float("nan"), device="cuda", dtype=torch.float32 if out_kind == "f32" else DT[kind])
    kw.setdefault("workspace", _ws(kb, B * T, B * T, H, kind, "qn_w" in kw or "rope_cos" in kw))
    kb.attn_self(out, dev(q, kind), dev(k, kind), dev(v, kind), B, T, H, **kw)
    assert kb.check_status() == 0
    return out.float().cpu().numpy()


def _cross(kb, q, k, v, Tq, Tk, npad, H, kind, out_kind=None):
    out = torch.full((Tq, H * 128), float("nan"), device="cuda", dtype=torch.float32 if out_kind == "f32" else DT[kind])
    kb.attn_cross(out, dev(q, kind), dev(k, kind), dev(v, kind), Tq, Tk, npad, H, workspace=_ws(kb, Tq, Tk, H, kind))
    assert kb.check_status() == 0
    return out.float().cpu().numpy()


def test_selfcheck(kb):
    L = kb.lib()
    ws = torch.empty(L.kb_selfcheck_workspace_bytes(), dtype=torch.uint8, device="cuda")
    err = ctypes.c_float(-1)
    rc = L.kb_attn_selfcheck(ctypes.c_void_p(ws.data_ptr()), ws.numel(), ctypes.byref(err), None)
    assert rc == 0 and 0 <= err.value <= 2e-3


# ---------------------------------------------------------------- golden fixtures (the reference's own kernels)
@pytest.mark.parametrize("case", gen.ATTN_CASES, ids=[c[0] for c in gen.ATTN_CASES])
def test_vs_reference_kernels_golden(kb, golden, case):
    name, Tq, Tk, npad, H = case
    q, k, v = gen.attn_inputs(case)                         # fp16-exact values, the harness's distribution
    out16 = _cross(kb, q, k, v, Tq, Tk, npad, H, "f16")
    out32 = _cross(kb, q, k, v, Tq, Tk, npad, H, "f16", "f32")
    assert_close(out32, golden[f"{name}/ref_attn"], f"{name} vs ref_attn")
    assert_close(out16, golden[f"{name}/ref_attn"], f"{name} fp16 out vs ref_attn")
    # against the reference's tensor-core kernel (what attention16 returns): both round to fp16
    assert_close(out16, golden[f"{name}/tfa_f16"].astype(np.float32), f"{name} vs tfa::k_flash")


# ---------------------------------------------------------------- self-attention
@pytest.mark.parametrize("T,H,kind", [(1, 1, "f16"), (7, 2, "bf16"), (128, 1, "f16"), (129, 2, "f16"), (256, 1, "bf16"),
                                      (257, 3, "f16"), (300, 2, "bf16"), (1000, 16, "f16")])
def test_self_small_full_oracle(kb, T, H, kind):
    q, k, v = (seeded(s, T, H * 128, kind) for s in (1, 2, 3))
    ref = oracle.attention(q, k, v, H)
    assert_close(_self(kb, q, k, v, 1, T, H, kind, "f32"), ref, f"self T={T} H={H} {kind} fp32 out")
    if kind == "f16":
        assert_close(_self(kb, q, k, v, 1, T, H, kind), ref, f"self T={T} H={H} fp16 out")
    else:
        assert_close_bf16_storage(_self(kb, q, k, v, 1, T, H, kind), ref, f"self T={T} H={H} bf16 out")


@pytest.mark.parametrize("T,kind", [(1536, "f16"), (3456, "bf16"), (4096, "bf16")])
def test_self_full_size_sampled_rows(kb, T, kind):
    """Benchmark configurations 1, 4 (one image, no norm) and 5 at full size; the oracle runs on sampled query rows."""
    H = 16
    q, k, v = (seeded(s, T, H * 128, kind) for s in (1, 2, 3))
    out = _self(kb, q, k, v, 1, T, H, kind, "f32")
    rows = sample_rows(T, 48)
    ref = oracle.attention(q[rows], k, v, H)
    assert_close(out[rows], ref, f"self T={T} {kind} sampled rows")
    # every row is a convex combination of V rows
    vmin, vmax = v.min(0), v.max(0)
    assert np.all(out >= vmin - 1e-3) and np.all(out <= vmax + 1e-3)


def test_self_batch_and_strides(kb):
    """B=2 (the CFG batch) equals two B=1 calls; Q, K, V as quarters of one [R, 4D] buffer (engine/src/dit.cu:387-388)."""
    T, H, B, kind = 384, 4, 2, "f16"
    D = H * 128
    big = dev(seeded(9, B * T, 4 * D, kind), kind)
    q, k, v, a = big[:, :D], big[:, D:2 * D], big[:, 2 * D:3 * D], big[:, 3 * D:]
    kb.attn_self(a, q, k, v, B, T, H)
    assert kb.check_status() == 0
    for b in range(B):
        sl = slice(b * T, (b + 1) * T)
        one = torch.empty(T, D, device="cuda", dtype=torch.float16)
        kb.attn_self(one, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), 1, T, H)
        assert torch.equal(one, a[sl])
        ref = oracle.attention(q[sl].float().cpu().numpy(), k[sl].float().cpu().numpy(), v[sl].float().cpu().numpy(), H)
        assert_close(a[sl].float().cpu().numpy(), ref, f"batched self b={b}")


def test_fp32_inputs_as_the_engine_holds_them(kb):
    """Q, K, V in fp32 (engine/src/dit.cu:429-430) with fp16 output: the attention16() contract."""
    T, Tk, H = 300, 77, 4
    q, k, v = (oracle.randn(s, n * H * 128).reshape(n, H * 128) for s, n in ((1, T), (2, Tk), (3, Tk)))
    out = torch.empty(T, H * 128, device="cuda", dtype=torch.float16)
    ws = torch.empty(kb.workspace_bytes(T, Tk, H, torch.float32), dtype=torch.uint8, device="cuda")
    kb.attn_cross(out, dev(q), dev(k), dev(v), T, Tk, 512 - Tk, H, workspace=ws)
    assert kb.check_status() == 0
    assert_close(out.float().cpu().numpy(), oracle.attention(q, k, v, H, 512 - Tk), "fp32 in, fp16 out")


def test_self_deterministic_and_head_independent(kb):
    T, H, kind = 700, 8, "bf16"
    q, k, v = (seeded(s, T, H * 128, kind) for s in (4, 5, 6))
    a = _self(kb, q, k, v, 1, T, H, kind)
    b = _self(kb, q, k, v, 1, T, H, kind)
    assert np.array_equal(a, b)                           # no atomics, no timing dependence (reference: README "--repeat")
    one = _self(kb, q[:, 256:384].copy(), k[:, 256:384].copy(), v[:, 256:384].copy(), 1, T, 1, kind)
    assert np.array_equal(one, a[:, 256:384])


def test_self_linear_in_v_and_key_permutation(kb):
    T, H, kind = 512, 2, "f16"
    q, k, v1, v2 = (seeded(s, T, H * 128, kind) for s in (1, 2, 3, 4))
    o1 = _self(kb, q, k, v1, 1, T, H, kind, "f32")
    o2 = _self(kb, q, k, v2, 1, T, H, kind, "f32")
    vs = oracle.round16(0.5 * v1 - 0.25 * v2, 0)
    o3 = _self(kb, q, k, vs, 1, T, H, kind, "f32")
    assert np.abs(o3 - (0.5 * o1 - 0.25 * o2)).max() < 2e-3
    perm = np.random.RandomState(0).permutation(T)
    o4 = _self(kb, q, k[perm], v1[perm], 1, T, H, kind, "f32")
    assert np.abs(o4 - o1).max() < 1e-3


def test_self_large_scores_rescale_path(kb):
    """Scores far apart between key blocks force the running-max rescale of O; RMS-normalised q/k with
    weights of 1-3 reach this range (bench/tfa_test.cu:37-41 uses 1.5 sigma)."""
    T, H, kind = 640, 2, "f16"
    q = seeded(1, T, H * 128, kind, 3.0)
    k = seeded(2, T, H * 128, kind, 3.0)
    k[384:] *= 2.0                                        # later blocks dominate: max jumps by far more than 2^8
    k = oracle.round16(k, 0)
    v = seeded(3, T, H * 128, kind)
    assert_close(_self(kb, q, k, v, 1, T, H, kind, "f32"), oracle.attention(q, k, v, H), "rescale path")


# ---------------------------------------------------------------- fused Q/K RMSNorm + RoPE
def _norm_rope_ref(x, w_bits, H, T, c, s):
    """fp32 reference order: rmsnorm, then rope per batch element (engine/src/dit.cu:464-468); no rounding."""
    y = oracle.rmsnorm(x, w_bits, H)
    B = x.shape[0] // T
    return np.concatenate([oracle.rope_half(y[b * T:(b + 1) * T], T, H, c, s) for b in range(B)])


@pytest.mark.parametrize("Hp,Wp,B,kind", [(6, 8, 1, "f16"), (12, 20, 2, "bf16")])
def test_self_with_norm_rope_small(kb, Hp, Wp, B, kind):
    T, H = Hp * Wp, 4
    q, k, v = (seeded(s, B * T, H * 128, kind) for s in (1, 2, 3))
    wq = oracle.round16(1 + 0.02 * oracle.randn(7, 128), 1)
    wk = oracle.round16(1 + 0.02 * oracle.randn(8, 128), 1)
    bits = lambda w: (w.view(np.uint32) >> 16).astype(np.uint16)
    c, s = oracle.cosmos_rope(Hp, Wp)
    qn = _norm_rope_ref(q, bits(wq), H, T, c, s)
    kn = _norm_rope_ref(k, bits(wk), H, T, c, s)
    ref = np.concatenate([oracle.attention(qn[b * T:(b + 1) * T], kn[b * T:(b + 1) * T], v[b * T:(b + 1) * T], H) for b in range(B)])
    out = _self(kb, q, k, v, B, T, H, kind, "f32", qn_w=dev(wq).bfloat16(), kn_w=dev(wk).bfloat16(), rope_cos=dev(c), rope_sin=dev(s))
    assert_close(out, ref, f"norm+rope self {Hp}x{Wp} B={B} {kind}")


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_q_norm_only_strided_many_items(kb, kind):
    """The cross-attention call pattern on a self-sized problem: Q gets RMSNorm, K arrives normalised; Q/K/V are column
    slices of one buffer, the token count is ragged and there are more work items (160) than SMs."""
    Hp, Wp, H = 45, 50, 16
    T = Hp * Wp
    big = seeded(1, T, 3 * H * 128, kind)
    q, k, v = big[:, :H * 128], big[:, H * 128:2 * H * 128], big[:, 2 * H * 128:]
    wq = oracle.round16(1 + 0.05 * oracle.randn(7, 128), 1)
    bits = (wq.view(np.uint32) >> 16).astype(np.uint16)
    dbig = dev(big, kind)
    dq, dk, dv = dbig[:, :H * 128], dbig[:, H * 128:2 * H * 128], dbig[:, 2 * H * 128:]
    out = torch.full((T, H * 128), float("nan"), device="cuda", dtype=torch.float32)
    kb.attn_self(out, dq, dk, dv, 1, T, H, qn_w=dev(wq).bfloat16(), workspace=_ws(kb, T, T, H, kind, norm=True))
    assert kb.check_status() == 0
    rows = sample_rows(T, 40)
    qn = oracle.rmsnorm(np.ascontiguousarray(q), bits, H)
    assert_close(out.cpu().numpy()[rows], oracle.attention(qn[rows], k, v, H), f"Q norm only {kind}")


def test_qk_prep_vs_reference_kernels_golden(kb, golden):
    """The pre-pass alone against the reference's k_rmsnorm_warp and k_rope_half outputs (fp32 in, as the engine keeps Q/K)."""
    x, w_bits, H = gen.norm_inputs()
    w = torch.from_numpy(w_bits.view(np.int16)).cuda().view(torch.bfloat16)
    out = torch.empty(x.shape, device="cuda", dtype=torch.float16)
    kb.qk_prep(out, dev(x), x.shape[0], H, x.shape[0], w=w)
    ref = golden["rmsnorm/out"]
    assert np.abs(out.float().cpu().numpy() - ref).max() <= np.abs(ref).max() * 2.0 ** -11 + 1e-6     # one fp16 rounding
    x, Hp, Wp, H = gen.rope_inputs()
    out = torch.empty(x.shape, device="cuda", dtype=torch.float16)
    kb.qk_prep(out, dev(x), x.shape[0], H, Hp * Wp, rope_cos=dev(golden["rope/cos"]), rope_sin=dev(golden["rope/sin"]))
    ref = golden["rope/out"]
    assert np.abs(out.float().cpu().numpy() - ref).max() <= np.abs(ref).max() * 2.0 ** -11 + 1e-6
    assert kb.check_status() == 0


def test_self_config4_full_size(kb):
    """Benchmark configuration 4: bf16, B=2, T=3456 (48x72 patches), per-head Q/K RMSNorm (1 + N(0,0.02)) and 3D RoPE."""
    Hp, Wp, B, H, kind = 48, 72, 2, 16, "bf16"
    T = Hp * Wp
    q, k, v = (seeded(s, B * T, H * 128, kind) for s in (1, 2, 3))
    wq = oracle.round16(1 + 0.02 * oracle.randn(7, 128), 1)
    wk = oracle.round16(1 + 0.02 * oracle.randn(8, 128), 1)
    bits = lambda w: (w.view(np.uint32) >> 16).astype(np.uint16)
    c, s = oracle.cosmos_rope(Hp, Wp)
    out = _self(kb, q, k, v, B, T, H, kind, "f32", qn_w=dev(wq).bfloat16(), kn_w=dev(wk).bfloat16(), rope_cos=dev(c), rope_sin=dev(s))
    kn = _norm_rope_ref(k, bits(wk), H, T, c, s)
    for b in range(B):
        rows = sample_rows(T, 24, seed=b)
        qn_rows = _norm_rope_ref(q[b * T:(b + 1) * T], bits(wq), H, T, c, s)[rows]
        ref = oracle.attention(qn_rows, kn[b * T:(b + 1) * T], v[b * T:(b + 1) * T], H)
        assert_close(out[b * T:(b + 1) * T][rows], ref, f"config 4 b={b}")


# ---------------------------------------------------------------- cross-attention
@pytest.mark.parametrize("Tk,npad", [(1, 0), (1, 511), (16, 496), (26, 486), (77, 0), (127, 385), (128, 384), (129, 0), (256, 256), (512, 0)])
@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_cross_lengths(kb, Tk, npad, kind):
    """Benchmark configuration 2 shapes: reference semantics (Tk = valid, npad = L - valid) and -inf masking (npad = 0)."""
    Tq, H = 1536, 16
    q = seeded(4, Tq, H * 128, kind)
    k, v = seeded(5, 512, H * 128, kind), seeded(6, 512, H * 128, kind)
    out = _cross(kb, q, k, v, Tq, Tk, npad, H, kind, "f32")
    rows = sample_rows(Tq, 40)
    assert_close(out[rows], oracle.attention(q[rows], k[:Tk], v[:Tk], H, npad), f"cross Tk={Tk} npad={npad} {kind}")


def test_cross_config2_seeded_valid_length(kb):
    Tq, H, L = 1536, 16, 512
    valid = int(np.random.RandomState(2).randint(16, L + 1))
    q, k, v = seeded(4, Tq, H * 128, "f16"), seeded(5, L, H * 128, "f16"), seeded(6, L, H * 128, "f16")
    k[valid:] = 0
    v[valid:] = 0                                          # the padded context rows really are zero (engine/src/gpu.h:149-151)
    rows = sample_rows(Tq, 40)
    ref_pad = oracle.attention(q[rows], k[:valid], v[:valid], H, L - valid)
    out = _cross(kb, q, k, v, Tq, valid, L - valid, H, "f16")
    assert_close(out[rows], ref_pad, f"config 2 reference semantics valid={valid}")
    # analytic padding == attending to the explicit zero rows
    out_explicit = _cross(kb, q, k, v, Tq, L, 0, H, "f16")
    assert np.abs(out_explicit - out).max() <= 1e-3
    out_mask = _cross(kb, q, k, v, Tq, valid, 0, H, "f16")
    assert_close(out_mask[rows], oracle.attention(q[rows], k[:valid], v[:valid], H, 0), "config 2 -inf masking")


def test_cross_ragged_queries_do_not_write_past_end(kb):
    Tq, Tk, H = 1000, 77, 2
    q, k, v = seeded(1, Tq, H * 128, "f16"), seeded(2, Tk, H * 128, "f16"), seeded(3, Tk, H * 128, "f16")
    buf = torch.full((Tq + 64, H * 128), 7.0, device="cuda", dtype=torch.float16)      # canary rows after the output
    kb.attn_cross(buf[:Tq], dev(q, "f16"), dev(k, "f16"), dev(v, "f16"), Tq, Tk, 0, H)
    assert kb.check_status() == 0
    assert torch.all(buf[Tq:] == 7.0)
    assert_close(buf[:Tq].float().cpu().numpy(), oracle.attention(q, k, v, H), "ragged cross 1000x77")


# ---------------------------------------------------------------- NAG
def _nag(kb, q, kp, vp, Tp, npp, kn, vn, Tn, npn, s, tau, alpha, Tq, H, kind, out_kind="f32"):
    out = torch.full((Tq, H * 128), float("nan"), device="cuda", dtype=torch.float32 if out_kind == "f32" else DT[kind])
    kb.attn_nag(out, dev(q, kind), dev(kp, kind), dev(vp, kind), Tp, npp, dev(kn, kind), dev(vn, kind), Tn, npn, s, tau, alpha, Tq, H,
                workspace=_ws(kb, Tq, max(Tp, Tn), H, kind, n_ctx=2))
    assert kb.check_status() == 0
    return out.float().cpu().numpy()


def _nag_ref(q, kp, vp, Tp, npp, kn, vn, Tn, npn, s, tau, alpha, H):
    zp = oracle.attention(q, kp[:Tp], vp[:Tp], H, npp)
    zn = oracle.attention(q, kn[:Tn], vn[:Tn], H, npn)
    return oracle.nag(zp, zn, s, tau, alpha), zp


@pytest.mark.parametrize("Tq,H,Tp,Tn,kind,s", [(200, 2, 77, 26, "f16", 5.0), (130, 1, 16, 300, "bf16", 5.0), (257, 4, 512, 1, "f16", 6.0),
                                                (300, 8, 129, 128, "f16", 5.0), (520, 3, 40, 200, "bf16", 5.0), (1536, 16, 333, 45, "f16", 5.0), (1536, 16, 333, 45, "f16", 6.0),
                                                (1536, 16, 512, 512, "bf16", 5.0)])
def test_nag(kb, Tq, H, Tp, Tn, kind, s):
    """Benchmark configuration 3: reference default s=5 (engine/src/models.h:80) and s=6 (the "z+ + 5 (z+ - z-)" wording of the same formula), tau=2.5, alpha=0.25."""
    L = 512
    q = seeded(7, Tq, H * 128, kind)
    kp, vp, kn, vn = (seeded(sd, L, H * 128, kind) for sd in (8, 9, 10, 11))
    ref, _ = _nag_ref(q, kp, vp, Tp, L - Tp, kn, vn, Tn, L - Tn, s, 2.5, 0.25, H)
    out = _nag(kb, q, kp, vp, Tp, L - Tp, kn, vn, Tn, L - Tn, s, 2.5, 0.25, Tq, H, kind)
    assert_close(out, ref, f"NAG Tq={Tq} H={H} Tp={Tp} Tn={Tn} {kind} s={s}")
    # 16-bit output takes the other kernel form (two query tiles per item, positive then negative context)
    out16 = _nag(kb, q, kp, vp, Tp, L - Tp, kn, vn, Tn, L - Tn, s, 2.5, 0.25, Tq, H, kind, out_kind=kind)
    (assert_close if kind == "f16" else assert_close_bf16_storage)(out16, ref, f"NAG 16-bit out Tq={Tq} H={H} Tp={Tp} Tn={Tn} {kind} s={s}")


def test_nag_identities_and_clamp(kb):
    Tq, H, L, kind = 384, 16, 512, "f16"
    q = seeded(7, Tq, H * 128, kind)
    kp, vp, kn, vn = (seeded(sd, L, H * 128, kind) for sd in (8, 9, 10, 11))
    zp = _cross(kb, q, kp, vp, Tq, 100, 412, H, kind, "f32")
    a0 = _nag(kb, q, kp, vp, 100, 412, kn, vn, 60, 452, 5.0, 2.5, 0.0, Tq, H, kind)     # alpha = 0 -> Z+
    assert np.abs(a0 - zp).max() <= 1e-5
    s1 = _nag(kb, q, kp, vp, 100, 412, kn, vn, 60, 452, 1.0, 2.5, 0.25, Tq, H, kind)    # s = 1 -> g = Z+
    assert np.abs(s1 - zp).max() <= 1e-5
    same = _nag(kb, q, kp, vp, 100, 412, kp, vp, 100, 412, 5.0, 2.5, 0.25, Tq, H, kind)  # Z- = Z+ -> g = Z+
    assert np.abs(same - zp).max() <= 1e-4
    a1 = _nag(kb, q, kp, vp, 100, 412, kn, vn, 60, 452, 9.0, 1.0, 1.0, Tq, H, kind)     # alpha = 1, tau = 1: |out|_1 <= |Z+|_1 per token
    assert np.all(np.abs(a1).sum(1) <= np.abs(zp).sum(1) * (1 + 1e-4))
    det = _nag(kb, q, kp, vp, 100, 412, kn, vn, 60, 452, 9.0, 1.0, 1.0, Tq, H, kind)
    assert np.array_equal(a1, det)


# ---------------------------------------------------------------- errors come back as codes, nothing runs
def test_argument_errors(kb):
    L = kb.lib()
    t = torch.zeros(256, 256, device="cuda", dtype=torch.float16)
    P = lambda x: ctypes.c_void_p(x.data_ptr())
    args = dict(B=1, T=256, H=2)
    assert L.kb_attn_self(None, P(t), P(t), P(t), None, None, None, None, 1, 256, 2, 256, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -1
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), None, None, None, None, 1, 0, 2, 256, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -1
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), None, None, None, None, 1, 256, 2, 252, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -2
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), None, None, None, None, 1, 256, 4, 256, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -3
    assert L.kb_attn_self(P(t), ctypes.c_void_p(t.data_ptr() + 2), P(t), P(t), None, None, None, None, 1, 256, 2, 256, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -2
    w = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), P(w), None, None, None, 1, 256, 2, 256, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -4
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), None, None, None, None, 1, 256, 2, 256, 256, 256, 256, 1, 1, 1e-6, None, 0, None) == -4   # bf16 needs staging
    small = torch.empty(1024, dtype=torch.uint8, device="cuda")
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), P(w), None, None, None, 1, 256, 2, 256, 256, 256, 256, 0, 0, 1e-6, P(small), 1024, None) == -4
    assert L.kb_attn_nag(P(t), P(t), None, P(t), P(t), 10, 0, P(t), P(t), 10, 0, 5.0, 2.5, 0.25, 256, 65, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -3
    assert L.kb_attn_nag(P(t), P(t), None, P(t), P(t), 10, 0, P(t), P(t), 10, 0, 5.0, 2.5, 0.25, 256, 2, 256, 256, 256, 0, 0, 1e-6, None, 0, None) == -4   # NAG always needs its scratch
    assert kb.check_status() == 0
    with pytest.raises(kb.KilnError):
        kb.attn_cross(t, t, t, t, 256, 0, 0, 2)


# ---------------------------------------------------------------- the exact variants the benchmark step times
def _bits(w):
    return (w.view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("T,B,Hp,Wp", [(4096, 1, 64, 64), (3456, 2, 48, 72)])
def test_self_benchmark_variant_bf16_in_bf16_out_norm_rope(kb, T, B, Hp, Wp):
    """kb_attn_self exactly as bench.py calls it: bf16 Q/K/V as thirds of one buffer, per-head Q/K RMSNorm, 3D RoPE,
    bf16 OUTPUT (staged in shared memory and written by TMA stores), full size; also the same call with fp16 output.
    Both sizes take the balanced schedule (items cut across SMs, partial results merged)."""
    H, kind = 16, "bf16"
    D = H * 128
    big = seeded(21, B * T, 3 * D, kind)
    q, k, v = (np.ascontiguousarray(big[:, i * D:(i + 1) * D]) for i in range(3))
    wq = oracle.round16(1 + 0.02 * oracle.randn(7, 128), 1)
    wk = oracle.round16(1 + 0.02 * oracle.randn(8, 128), 1)
    c, s = oracle.cosmos_rope(Hp, Wp)
    dbig = dev(big, kind)
    ws = _ws(kb, B * T, B * T, H, kind, norm=True)
    kn = _norm_rope_ref(k, _bits(wk), H, T, c, s)
    refs = []
    for b in range(B):
        rows = sample_rows(T, 24, seed=b)
        qn_rows = _norm_rope_ref(q[b * T:(b + 1) * T], _bits(wq), H, T, c, s)[rows]
        refs.append((rows + b * T, oracle.attention(qn_rows, kn[b * T:(b + 1) * T], v[b * T:(b + 1) * T], H)))
    pick = np.concatenate([r for r, _ in refs])
    ref = np.concatenate([x for _, x in refs])
    for out_dt in (torch.bfloat16, torch.float16):
        out = torch.full((B * T, D), float("nan"), device="cuda", dtype=out_dt)
        kb.attn_self(out, dbig[:, :D], dbig[:, D:2 * D], dbig[:, 2 * D:], B, T, H, qn_w=dev(wq).bfloat16(), kn_w=dev(wk).bfloat16(),
                     rope_cos=dev(c), rope_sin=dev(s), workspace=ws)
        assert kb.check_status() == 0
        o = out.float().cpu().numpy()
        assert not np.isnan(o).any()
        if out_dt == torch.bfloat16:
            assert_close_bf16_storage(o[pick], ref, f"benchmark self T={T} B={B} bf16 out")
        else:
            assert_close(o[pick], ref, f"benchmark self T={T} B={B} fp16 out")


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("Tq,Tp,Tn,s", [(130, 512, 512, 5.0), (300, 333, 45, 6.0), (1536, 512, 512, 6.0), (1536, 333, 45, 5.0),
                                         (4096, 512, 512, 5.0), (4096, 333, 45, 5.0)])
def test_nag_benchmark_variant_qnorm_16bit_out(kb, kind, Tq, Tp, Tn, s):
    """kb_attn_nag exactly as bench.py calls it: fused Q RMSNorm (qn_w), 16-bit inputs, 16-BIT OUTPUT (blend staged in
    shared memory, TMA stores), H = 16, full 512-key contexts (npad = 0) and ragged ones with analytic padding."""
    H, L = 16, 512
    q = seeded(31, Tq, H * 128, kind)
    kp, vp, kn, vn = (seeded(sd, L, H * 128, kind) for sd in (32, 33, 34, 35))
    wq = oracle.round16(1 + 0.02 * oracle.randn(36, 128), 1)
    rows = sample_rows(Tq, 40)
    qn = oracle.rmsnorm(q, _bits(wq), H)[rows]
    ref, _ = _nag_ref(qn, kp, vp, Tp, L - Tp, kn, vn, Tn, L - Tn, s, 2.5, 0.25, H)
    ws = torch.empty(kb.workspace_bytes(Tq, L, H, DT[kind], True, False, n_ctx=2), dtype=torch.uint8, device="cuda")
    for out_dt in (DT[kind], torch.float32):
        out = torch.full((Tq, H * 128), float("nan"), device="cuda", dtype=out_dt)
        kb.attn_nag(out, dev(q, kind), dev(kp, kind), dev(vp, kind), Tp, L - Tp, dev(kn, kind), dev(vn, kind), Tn, L - Tn, s, 2.5, 0.25, Tq, H,
                    qn_w=dev(wq).bfloat16(), workspace=ws)
        assert kb.check_status() == 0
        o = out.float().cpu().numpy()
        assert not np.isnan(o).any()
        what = f"benchmark NAG Tq={Tq} Tp={Tp} Tn={Tn} s={s} {kind} out={out_dt}"
        if out_dt == torch.bfloat16:
            assert_close_bf16_storage(o[rows], ref, what)
        else:
            assert_close(o[rows], ref, what)


@pytest.mark.parametrize("T,H,B,kind", [(2560, 16, 1, "f16"), (2000, 3, 1, "bf16"), (4096, 2, 1, "bf16"), (2000, 2, 2, "f16")])
def test_balanced_schedule_equals_whole_items(kb, T, H, B, kind):
    """The balanced (item, key block) schedule, taken when the workspace has room for partial results, against the
    whole-items schedule of the same call without that room, and against the oracle: items cut across two or more SMs
    (2 heads x 4096 tokens: an item spans five SMs), ragged token counts, a batch. (The library takes the balanced schedule
    only when it saves more than eight key-block steps on the slowest SM: all four cases do.)"""
    q, k, v = (seeded(s, B * T, H * 128, kind) for s in (41, 42, 43))
    dq, dk, dv = dev(q, kind), dev(k, kind), dev(v, kind)
    full = torch.empty(kb.workspace_bytes(B * T, B * T, H, DT[kind]), dtype=torch.uint8, device="cuda")
    stage_only = kb.workspace_bytes(B * T, B * T, H, DT[kind]) - kb.workspace_bytes(0, 0, H, DT[kind])
    small = full[:stage_only] if stage_only else None
    outs = []
    for ws in (full, small):
        o = torch.full((B * T, H * 128), float("nan"), device="cuda", dtype=torch.float32)
        kb.attn_self(o, dq, dk, dv, B, T, H, workspace=ws)
        assert kb.check_status() == 0
        outs.append(o.cpu().numpy())
    # a part that starts in the middle of the keys takes its own running maximum, so its fp16 weights P = 2^(s - m) round
    # differently from the whole-item run's: agreement to a fraction of the tolerance, not to the bit
    assert np.abs(outs[0] - outs[1]).max() <= 5e-4
    for b in range(B):
        rows = sample_rows(T, 24, seed=b)
        sl = slice(b * T, (b + 1) * T)
        assert_close(outs[0][sl][rows], oracle.attention(q[sl][rows], k[sl], v[sl], H), f"balanced schedule T={T} H={H} b={b}")
    again = torch.empty(B * T, H * 128, device="cuda", dtype=torch.float32)
    kb.attn_self(again, dq, dk, dv, B, T, H, workspace=full)
    assert kb.check_status() == 0
    assert np.array_equal(again.cpu().numpy(), outs[0])     # merge order is fixed: bit-identical repeat


def test_alignment_of_weights_and_tables_is_an_error_code(kb):
    """Norm weights and RoPE tables are read with 16-byte vector loads: a pointer that is not 16-byte aligned must come
    back as KB_ERR_ALIGN from the host-side checks; nothing is launched."""
    L = kb.lib()
    t = torch.zeros(256, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    tab = torch.zeros(256 * 64 + 8, device="cuda", dtype=torch.float32)
    ws = torch.empty(8 << 20, dtype=torch.uint8, device="cuda")
    P = lambda x, off=0: ctypes.c_void_p(x.data_ptr() + off)
    self_args = lambda qn, kn, c, s: (P(t), P(t), P(t), P(t), qn, kn, c, s, 1, 256, 2, 256, 256, 256, 256, 1, 1, 1e-6, P(ws), ws.numel(), None)
    assert L.kb_attn_self(*self_args(P(w, 2), None, None, None)) == -2
    assert L.kb_attn_self(*self_args(None, P(w, 8), None, None)) == -2
    assert L.kb_attn_self(*self_args(None, None, P(tab, 4), P(tab))) == -2
    assert L.kb_attn_self(*self_args(None, None, P(tab), P(tab, 8))) == -2
    assert L.kb_attn_self(*self_args(P(w), P(w, 16), P(tab), P(tab, 32))) == 0
    assert L.kb_attn_nag(P(t), P(t), P(w, 2), P(t), P(t), 10, 0, P(t), P(t), 10, 0, 5.0, 2.5, 0.25, 256, 2, 256, 256, 256, 1, 1, 1e-6,
                         P(ws), ws.numel(), None) == -2
    assert L.kb_qk_prep(P(t), 256, 1, P(t), 256, 1, 256, 2, 256, P(w, 2), 1e-6, None, None, None) == -2
    assert L.kb_qk_prep(P(t), 256, 1, P(t), 256, 1, 256, 2, 256, None, 1e-6, P(tab, 4), P(tab), None) == -2
    assert L.kb_attn_self(P(t), P(t), P(t), P(t), None, None, None, None, 1, 1, 5000, 256, 256, 256, 256, 1, 1, 1e-6, P(ws), ws.numel(), None) == -3
    assert kb.check_status() == 0
