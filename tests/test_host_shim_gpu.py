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


def _bits(w):
    return (w.view(np.uint32) >> 16).astype(np.uint16)


def test_fused_self_attention16_engine_buffers(shim):
    """self_attention16: the engine's fp32 Q/K/V quarters of one [R, 4D] buffer (engine/src/dit.cu:387-388) with the per-head
    norm weights and the RoPE tables, B = 2, fp16 out - one call for rmsnorm x2 + rope_half x2 per image + attention16."""
    Hp, Wp, B, H = 9, 14, 2, 4
    T, D = Hp * Wp, 4 * 128
    big = oracle.randn(700, B * T * 4 * D).reshape(B * T, 4 * D)
    wq = oracle.round16(1 + 0.02 * oracle.randn(701, 128), 1)
    wk = oracle.round16(1 + 0.02 * oracle.randn(702, 128), 1)
    c, s = oracle.cosmos_rope(Hp, Wp)
    dbig = dev(big)
    out = torch.full((B * T, D), float("nan"), device="cuda", dtype=torch.float16)
    err = ctypes.create_string_buffer(256)
    q_ptr = ctypes.c_void_p(dbig.data_ptr())
    k_ptr = ctypes.c_void_p(dbig.data_ptr() + D * 4)
    v_ptr = ctypes.c_void_p(dbig.data_ptr() + 2 * D * 4)
    dwq, dwk = dev(_bits(wq).view(np.int16)), dev(_bits(wk).view(np.int16))
    assert shim.kbh_self_attention16(P(out), D, q_ptr, k_ptr, v_ptr, 4 * D, B, T, H, P(dwq), P(dwk), P(dev(c)), P(dev(s)), ctypes.c_float(1e-6),
                                     err, 256) == 0, err.value
    torch.cuda.synchronize()
    q, k, v = (np.ascontiguousarray(big[:, i * D:(i + 1) * D]) for i in range(3))
    nr = lambda x, w: np.concatenate([oracle.rope_half(oracle.rmsnorm(x[b * T:(b + 1) * T], _bits(w), H), T, H, c, s) for b in range(B)])
    qn, kn = nr(q, wq), nr(k, wk)
    ref = np.concatenate([oracle.attention(qn[b * T:(b + 1) * T], kn[b * T:(b + 1) * T], v[b * T:(b + 1) * T], H) for b in range(B)])
    assert_close(out.float().cpu().numpy(), ref, "shim self_attention16")


def test_fused_nag_attention16_and_qkv_projection(shim):
    """nag_attention16 (rmsnorm(Q) + attention16 x2 + k_nag in one call, engine/src/dit.cu:476-487) and linear16_qkv (the three
    projections + norm + RoPE of engine/src/dit.cu:461-468 in one launch) against the oracle chains."""
    Tq, H, L, Tp, Tn = 200, 4, 512, 77, 26
    D = H * 128
    q = oracle.randn(710, Tq * D).reshape(Tq, D)
    ctx = [oracle.randn(711 + i, L * D).reshape(L, D) for i in range(4)]
    wq = oracle.round16(1 + 0.02 * oracle.randn(715, 128), 1)
    out = torch.full((Tq, D), float("nan"), device="cuda", dtype=torch.float16)
    err = ctypes.create_string_buffer(256)
    f = ctypes.c_float
    dctx = [dev(x) for x in ctx]
    assert shim.kbh_nag_attention16(P(out), D, P(dev(q)), D, P(dev(_bits(wq).view(np.int16))), P(dctx[0]), P(dctx[1]), Tp, L - Tp, P(dctx[2]), P(dctx[3]),
                                    Tn, L - Tn, D, f(5.0), f(2.5), f(0.25), Tq, H, f(1e-6), err, 256) == 0, err.value
    torch.cuda.synchronize()
    qn = oracle.rmsnorm(q, _bits(wq), H)
    zp = oracle.attention(qn, ctx[0][:Tp], ctx[1][:Tp], H, L - Tp)
    zn = oracle.attention(qn, ctx[2][:Tn], ctx[3][:Tn], H, L - Tn)
    assert_close(out.float().cpu().numpy(), oracle.nag(zp, zn, 5.0, 2.5, 0.25), "shim nag_attention16")

    M, K = 150, 256
    x = oracle.round16(oracle.randn(720, M * K), 0).reshape(M, K)
    ws = [oracle.round16(oracle.randn(721 + i, D * K) * np.float32(0.05), 0).reshape(D, K) for i in range(3)]
    wk = oracle.round16(1 + 0.02 * oracle.randn(725, 128), 1)
    cos, sin = oracle.cosmos_rope(10, 15)
    ys = [torch.full((M, D), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
    dws = [dev(w).half() for w in ws]
    assert shim.kbh_linear16_qkv(P(ys[0]), P(ys[1]), P(ys[2]), D, P(dev(x).half()), M, P(dws[0]), P(dws[1]), P(dws[2]), D, K,
                                 P(dev(_bits(wq).view(np.int16))), P(dev(_bits(wk).view(np.int16))), P(dev(cos)), P(dev(sin)), 150, f(1e-6), err, 256) == 0, err.value
    torch.cuda.synchronize()
    assert_close(ys[0].float().cpu().numpy(), oracle.linear_heads16(x, ws[0], H, _bits(wq), cos, sin), "shim linear16_qkv q")
    assert_close(ys[1].float().cpu().numpy(), oracle.linear_heads16(x, ws[1], H, _bits(wk), cos, sin), "shim linear16_qkv k")
    ref_v = oracle.linear16(x, ws[2], 1)
    assert np.abs(ys[2].float().cpu().numpy() - ref_v).max() <= 2e-4 + 2.0 ** -10 * np.abs(ref_v).max()


def test_ineligible_attention_falls_through_to_the_engines_exact_path(shim):
    """attention() forwards to the fused kernels only what the reference's own fast path takes; a causal call (the text
    encoder) or Dh = 64 (the adapter) goes to the exact path the engine registered, as in the reference's dispatcher
    (engine/src/kernels.cu:830-866); rmsnorm with no weight normalises with weight 1 (engine/src/kernels.cu:650-673)."""
    t = torch.zeros(64, 256, device="cuda")
    err = ctypes.create_string_buffer(256)
    before = shim.kbh_register_exact_probe(1)
    assert shim.kbh_attention(P(t), 256, P(t), 256, P(t), 256, P(t), 256, 64, 64, 2, 128, 1, 0, 1, err, 256) == 0      # causal
    assert shim.kbh_attention(P(t), 256, P(t), 256, P(t), 256, P(t), 256, 64, 64, 4, 64, 0, 0, 1, err, 256) == 0       # Dh = 64
    assert shim.kbh_register_exact_probe(0) == before + 2
    assert shim.kbh_attention(P(t), 256, P(t), 256, P(t), 256, P(t), 256, 64, 64, 2, 128, 1, 0, 1, err, 256) == -1     # nothing registered: throws
    x = oracle.randn(730, 40 * 128).reshape(40, 128)
    dx = dev(x)
    assert shim.kbh_rmsnorm_only(P(dx), None, 40, ctypes.c_float(1e-6), err, 256) == 0, err.value
    torch.cuda.synchronize()
    np.testing.assert_allclose(dx.cpu().numpy(), oracle.rmsnorm(x, None, 1), rtol=1e-5, atol=2e-6)


def _bf16(seed, rows, cols, amp):
    a = oracle.round16(oracle.randn(seed, max(rows * cols, 16))[:rows * cols] * np.float32(amp), 1).reshape(rows, cols)
    return a, dev(_bits(a).view(np.int16))


def test_linear16_with_unmerged_loras(shim):
    """linear16 on a weight that carries two LoRAs (engine/src/kernels.cu:578-596): the shim stacks and converts them, forms
    t = x A_cat^T in the context's workspace and adds t B_cat^T inside the GEMM — every Epi16 against the oracle's restatement
    of that sequence; then the q/k/v form with LoRAs on q and v."""
    M, N, K, H = 150, 256, 128, 2
    x = oracle.round16(oracle.randn(800, M * K), 0).reshape(M, K)
    w = oracle.round16(oracle.randn(801, N * K) * np.float32(0.05), 0).reshape(N, K)
    gate = oracle.randn(802, N)
    resid = oracle.randn(803, M * N).reshape(M, N)
    (a1, da1), (b1, db1) = _bf16(804, 12, K, 0.05), _bf16(805, N, 12, 0.05)      # rank 12 + 16 = 28 -> padded to 32
    (a2, da2), (b2, db2) = _bf16(806, 16, K, 0.05), _bf16(807, N, 16, 0.05)
    loras = [(a1, b1, 2.0), (a2, b2, -1.25)]
    t_ref, b_ref = oracle.lora_operands(x, loras)
    dx, dw = dev(x).half(), dev(w).half()
    a_cat = torch.full((32, K), float("nan"), device="cuda", dtype=torch.float16)
    b_cat = torch.full((N, 32), float("nan"), device="cuda", dtype=torch.float16)
    err = ctypes.create_string_buffer(256)
    f = ctypes.c_float
    shim.kbh_linear16_lora.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, f, ctypes.c_void_p,
                                       ctypes.c_int, ctypes.c_void_p, f, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    for epi in range(4):
        c32 = epi in (0, 3)
        c = dev(resid).clone() if epi == 3 else torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32 if c32 else torch.float16)
        assert shim.kbh_linear16_lora(P(c), N, P(dx), M, P(dw), N, K, epi, P(dev(gate)) if epi == 3 else None, P(da1), 12, P(db1), 2.0,
                                      P(da2), 16, P(db2), -1.25, P(a_cat), P(b_cat), err, 256) == 0, err.value
        torch.cuda.synchronize()
        ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None, lora=(t_ref, b_ref))
        # t is rounded to fp16 on both sides from sums in different orders: one fp16 step of t times |B| summed over the rank
        assert np.abs(c.float().cpu().numpy() - ref).max() <= 2e-3 + 2.0 ** -10 * np.abs(ref).max(), epi
    assert np.array_equal(b_cat[:, :28].float().cpu().numpy(), b_ref) and not b_cat[:, 28:].float().abs().sum().item()
    assert not a_cat[28:].float().abs().sum().item()

    # q/k/v in one launch, LoRA on q (rank 16) and v (rank 8), none on k
    D = H * 128
    ws = [oracle.round16(oracle.randn(810 + i, D * K) * np.float32(0.05), 0).reshape(D, K) for i in range(3)]
    dws = [dev(a).half() for a in ws]
    wq, wk = (oracle.round16(1.0 + 0.05 * oracle.randn(820 + i, 128), 1) for i in range(2))
    cos, sin = oracle.cosmos_rope(10, 15)
    (aq, daq), (bq, dbq) = _bf16(830, 16, K, 0.05), _bf16(831, D, 16, 0.05)
    (av, dav), (bv, dbv) = _bf16(832, 8, K, 0.05), _bf16(833, D, 8, 0.05)
    packs = []
    for da, db, r, s in ((daq, dbq, 16, 1.5), (dav, dbv, 8, 3.0)):
        ac = torch.empty((r, K), device="cuda", dtype=torch.float16)
        bc = torch.empty((D, r), device="cuda", dtype=torch.float16)
        assert shim.kbh_pack_lora(P(ac), P(bc), D, K, P(da), r, P(db), f(s), err, 256) == 0, err.value
        packs.append((ac, bc, r))
    ys = [torch.full((M, D), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
    assert shim.kbh_linear16_qkv_lora(P(ys[0]), P(ys[1]), P(ys[2]), D, P(dx), M, P(dws[0]), P(dws[1]), P(dws[2]), D, K,
                                      P(dev(_bits(wq).view(np.int16))), P(dev(_bits(wk).view(np.int16))), P(dev(cos)), P(dev(sin)), 150, f(1e-6),
                                      P(packs[0][0]), P(packs[0][1]), 16, P(packs[1][0]), P(packs[1][1]), 8, err, 256) == 0, err.value
    torch.cuda.synchronize()
    tq, bqc = oracle.lora_operands(x, [(aq, bq, 1.5)])
    yq = oracle.rmsnorm(oracle.linear16(x, ws[0], 0, lora=(tq, bqc)), _bits(wq), H, 1e-6)
    yq = oracle.round16(oracle.rope_half(yq, M, H, cos, sin), 0)
    assert_close(ys[0].float().cpu().numpy(), yq, "shim linear16_qkv q with LoRA")
    assert_close(ys[1].float().cpu().numpy(), oracle.linear_heads16(x, ws[1], H, _bits(wk), cos, sin), "shim linear16_qkv k")
    tv, bvc = oracle.lora_operands(x, [(av, bv, 3.0)])
    ref_v = oracle.linear16(x, ws[2], 1, lora=(tv, bvc))
    assert np.abs(ys[2].float().cpu().numpy() - ref_v).max() <= 2e-3 + 2.0 ** -10 * np.abs(ref_v).max()


def test_cross_kv16_then_nag_attention_on_the_cache(shim):
    """cross_kv16 (the body of the engine's cache_context loop, engine/src/dit.cu:228-230) for a prompt and a NAG negative
    context, against the oracle's linear + rmsnorm + linear."""
    H, KD, L = 2, 1024, 77
    D = H * 128
    ctx = oracle.randn(900, L * KD).reshape(L, KD)
    wk, wv = (oracle.round16(oracle.randn(901 + j, D * KD) * np.float32(1.0 / 32), 0).reshape(D, KD) for j in range(2))
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(903, 128), 1)
    k16 = torch.full((L, D), float("nan"), device="cuda", dtype=torch.float16)
    v16 = torch.full((L, D), float("nan"), device="cuda", dtype=torch.float16)
    err = ctypes.create_string_buffer(256)
    assert shim.kbh_cross_kv16(P(k16), P(v16), D, P(dev(ctx)), L, P(dev(wk).half()), P(dev(wv).half()), D, KD, P(dev(_bits(nw).view(np.int16))),
                               ctypes.c_float(1e-6), err, 256) == 0, err.value
    torch.cuda.synchronize()
    x16 = oracle.round16(ctx, 0)
    k_ref = oracle.round16(oracle.rmsnorm(oracle.linear16(x16, wk, 0), _bits(nw), H, 1e-6), 0)
    v_ref = oracle.linear16(x16, wv, 1)
    assert np.all(np.abs(k16.float().cpu().numpy() - k_ref) <= 2.0 ** -10 * np.abs(k_ref) + 1e-4)
    assert np.all(np.abs(v16.float().cpu().numpy() - v_ref) <= 2.0 ** -10 * np.abs(v_ref) + 1e-4)


def test_attention_bwd_through_the_shim(shim):
    """attention_bwd with the trainer's signature (engine/src/train.cu:216): fp32 rows in and out, scratch from the context."""
    Tq, Tk, npad, H = 150, 26, 486, 2
    D = H * 128
    q, k = (oracle.round16(oracle.randn(940 + i, r * D) * np.float32(1.5), 0).reshape(r, D) for i, r in enumerate((Tq, Tk)))
    v, do = (oracle.round16(oracle.randn(942 + i, r * D), 0).reshape(r, D) for i, r in enumerate((Tk, Tq)))
    outs = [torch.full((r, D), float("nan"), device="cuda") for r in (Tq, Tk, Tk)]
    err = ctypes.create_string_buffer(256)
    assert shim.kbh_attention_bwd(P(outs[0]), P(outs[1]), P(outs[2]), P(dev(q)), P(dev(k)), P(dev(v)), P(dev(do)), Tq, Tk, npad, H, err, 256) == 0, err.value
    torch.cuda.synchronize()
    for name, o, r in zip(("dq", "dk", "dv"), outs, oracle.attention_bwd(q, k, v, do, H, npad)):
        assert_close(o.cpu().numpy(), r, f"shim attention_bwd {name}")
