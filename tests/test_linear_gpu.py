"""GPU parity tests of the fp16 projection GEMM (kb_linear16) through the C ABI, against the CPU oracle
(fp64-accumulating restatement of the reference's linear16) and the reference kernel's own golden outputs.

Tolerances: the GEMM accumulates exact fp16 x fp16 products in fp32, so fp32 outputs are held to
1e-5 * sqrt(K) * scale; fp16 outputs to one fp16 rounding step (2^-10 |ref|) on top. The fused head
epilogue is held to the attention path's tolerance (2e-3 max-abs, 1e-3 mean-relative)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle
from util_gpu import assert_close, dev, sample_rows, seeded

pytestmark = pytest.mark.gpu

_HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_ref_gemm_fixtures", os.path.join(_HERE, "golden", "make_ref_gemm_fixtures.py"))
ggen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(ggen)


@pytest.fixture(scope="module")
def kb(built_lib):
    import kiln_b200
    assert kiln_b200.lib().kb_init() == 0, "sm_100 device and the CUDA library are required (there is no fallback)"
    return kiln_b200


@pytest.fixture(scope="module")
def gemm_golden():
    return np.load(os.path.join(_HERE, "golden", "ref_gemm_fixtures.npz"))


def _run(kb, x, w, epi, gate=None, resid=None, ldc_pad=0, **kw):
    from kiln_b200 import ops
    M, N = x.shape[0], w.shape[0]
    c32 = epi in (ops.EPI_F32, ops.EPI_RESID)
    full = torch.full((M, N + ldc_pad), float("nan"), device="cuda", dtype=torch.float32 if c32 else torch.float16)
    c = full[:, :N]
    if epi == ops.EPI_RESID:
        c.copy_(dev(resid))
    ops.linear16(c, dev(x, "f16"), dev(w, "f16"), epi, gate=None if gate is None else dev(gate), **kw)
    assert kb.check_status() == 0
    if ldc_pad:
        assert torch.isnan(full[:, N:].float()).all(), "wrote outside the output columns"
    return c.float().cpu().numpy()


def _close(out, ref, K, what, f16_out):
    scale = max(1.0, float(np.abs(ref).max()))
    d = np.abs(out.astype(np.float64) - ref.astype(np.float64))
    bound = 1e-5 * np.sqrt(K) * scale + (np.abs(ref) * 2.0 ** -10 + 1e-7 if f16_out else 0.0)
    assert not np.isnan(out).any(), f"{what}: NaN"
    assert np.all(d <= bound), f"{what}: worst excess {np.max(d - bound):.3e} (max err {d.max():.3e})"


@pytest.mark.parametrize("case", ggen.GEMM_CASES, ids=[c[0] for c in ggen.GEMM_CASES])
def test_epilogues_vs_oracle_and_reference_golden(kb, gemm_golden, case):
    from kiln_b200 import ops
    name, M, N, K = case
    x, w, gate, resid = ggen.gemm_inputs(case)
    for ename, epi in ggen.EPIS.items():
        out = _run(kb, x, w, epi, gate=gate if epi == ops.EPI_RESID else None, resid=resid, ldc_pad=8)
        ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None)
        _close(out, ref, K, f"{name}/{ename} vs oracle", epi in (1, 2))
        # the reference kernel sums each 32-wide k tile in fp16: hold it (and so us against it) to that error
        g = gemm_golden[f"{name}/{ename}"].astype(np.float32)
        tile_err = 2.0 ** -11 * np.sqrt(K / 32) * 4.0
        assert np.abs(out - g).max() <= tile_err + 2.0 ** -9 * np.abs(g).max(), f"{name}/{ename} vs reference kernel: {np.abs(out - g).max():.3e}"


def test_resid_without_gate(kb):
    from kiln_b200 import ops
    x, w = seeded(11, 70, 128, "f16"), seeded(12, 128, 128, "f16", 0.05)
    resid = oracle.randn(13, 70 * 128).reshape(70, 128)
    out = _run(kb, x, w, ops.EPI_RESID, resid=resid)
    _close(out, oracle.linear16(x, w, 3, None, resid), 128, "resid, no gate", False)


def _heads_inputs(M, H, K, seed):
    x = seeded(seed, M, K, "f16")
    w = seeded(seed + 1, H * 128, K, "f16", 1.0 / np.sqrt(K))
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(seed + 2, 128), 1)
    return x, w, nw, (nw.view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("H", [3, 4], ids=["single_cta_tiles", "cta_pair_tiles"])
@pytest.mark.parametrize("norm,rope", [(True, True), (True, False), (False, True), (False, False)])
def test_heads_epilogue(kb, norm, rope, H):
    """The q / k projection with the per-head RMSNorm and RoPE fused, against the engine's chain of separate ops."""
    from kiln_b200 import ops
    Hp, Wp, B, K = 9, 13, 3, 320                             # 117 tokens per image, 3 images: rope row = r % 117
    M = B * Hp * Wp
    x, w, nw, nbits = _heads_inputs(M, H, K, 40)
    cos, sin = oracle.cosmos_rope(Hp, Wp)
    kw = {}
    if norm:
        kw["head_w"] = dev(nw).to(torch.bfloat16)
    if rope:
        kw["rope_cos"], kw["rope_sin"] = dev(cos), dev(sin)
    out = _run(kb, x, w, ops.EPI_HEADS16, ldc_pad=16, **kw)
    ref = oracle.linear_heads16(x, w, H, nbits if norm else None, np.tile(cos, (B, 1)) if rope else None, np.tile(sin, (B, 1)) if rope else None)
    assert_close(out, ref, f"heads16 norm={norm} rope={rope}")
    # tighter: the only differences are fp32 summation order and one fp16 rounding
    assert np.abs(out - ref).max() <= 2.0 ** -10 * np.abs(ref).max() + 1e-4


def test_dit_projection_sizes_sampled_rows(kb):
    """4096 tokens x 2048 -> 2048 (512 tiles, several per CTA): oracle on sampled rows at the full K and N."""
    from kiln_b200 import ops
    M, N, K = 4096, 2048, 2048
    x, w, nw, nbits = _heads_inputs(M, N // 128, K, 60)
    rows = sample_rows(M, 24, 5)
    out = _run(kb, x, w, ops.EPI_F32)
    _close(out[rows], oracle.linear16(x[rows], w, 0), K, "4096x2048x2048 fp32", False)
    cos, sin = oracle.cosmos_rope(64, 64)
    outh = _run(kb, x, w, ops.EPI_HEADS16, head_w=dev(nw).to(torch.bfloat16), rope_cos=dev(cos), rope_sin=dev(sin))
    y = oracle.rmsnorm(oracle.linear16(x[rows], w, 0), nbits, N // 128)
    refh = oracle.round16(oracle.rope_half(y, len(rows), N // 128, cos[rows], sin[rows]), 0)
    assert_close(outh[rows], refh, "4096x2048x2048 heads16")
    # MLP shapes: K = 8192 down-projection into the residual stream, GELU up-projection on a ragged M
    xm = seeded(70, 300, 8192, "f16", 0.5)
    wm = seeded(71, 256, 8192, "f16", 0.01)
    resid = oracle.randn(72, 300 * 256).reshape(300, 256)
    gate = oracle.randn(73, 256)
    _close(_run(kb, xm, wm, ops.EPI_RESID, gate=gate, resid=resid), oracle.linear16(xm, wm, 3, gate, resid), 8192, "K=8192 resid", False)
    _close(_run(kb, xm, wm, ops.EPI_GELU16), oracle.linear16(xm, wm, 2), 8192, "K=8192 gelu16", True)


def test_linearity_full_size(kb):
    """Size-independent property at the full DiT size: (a X1 + b X2) W^T = a X1 W^T + b X2 W^T with exactly
    representable scalings, so the three fp32 results agree to summation rounding."""
    from kiln_b200 import ops
    M, N, K = 4096, 2048, 2048
    g = torch.Generator(device="cuda").manual_seed(7)
    x1 = (torch.randint(-8, 9, (M, K), device="cuda", generator=g).half()) / 8
    x2 = (torch.randint(-8, 9, (M, K), device="cuda", generator=g).half()) / 8
    w = (torch.randint(-8, 9, (N, K), device="cuda", generator=g).half()) / 64
    outs = []
    for xx in (x1, x2, x1 * 2 + x2 * 0.5):
        c = torch.empty((M, N), device="cuda", dtype=torch.float32)
        ops.linear16(c, xx.contiguous(), w, ops.EPI_F32)
        outs.append(c)
    assert kb.check_status() == 0
    # every product is a multiple of 2^-10 and every partial sum stays below 2^10: fp32 sums are exact
    assert torch.equal(outs[2], outs[0] * 2 + outs[1] * 0.5)
    assert torch.equal(outs[0], (x1.double() @ w.double().T).float())


def test_projection_feeds_attention(kb):
    """Fused projections -> attention with fp16 operands and no workspace equals fp32 projections ->
    attention entry point doing norm + RoPE itself."""
    from kiln_b200 import ops
    Hp, Wp, H, K = 12, 16, 2, 256
    T = Hp * Wp
    x = seeded(80, T, K, "f16")
    ws = [seeded(81 + i, H * 128, K, "f16", 1.5 / np.sqrt(K)) for i in range(3)]
    nq = oracle.round16(1.0 + 0.05 * oracle.randn(90, 128), 1)
    nk = oracle.round16(1.0 + 0.05 * oracle.randn(91, 128), 1)
    cos, sin = oracle.cosmos_rope(Hp, Wp)
    dx, dcos, dsin = dev(x, "f16"), dev(cos), dev(sin)
    q = torch.empty((T, H * 128), device="cuda", dtype=torch.float16)
    k, v = torch.empty_like(q), torch.empty_like(q)
    ops.linear16(q, dx, dev(ws[0], "f16"), ops.EPI_HEADS16, head_w=dev(nq).to(torch.bfloat16), rope_cos=dcos, rope_sin=dsin)
    ops.linear16(k, dx, dev(ws[1], "f16"), ops.EPI_HEADS16, head_w=dev(nk).to(torch.bfloat16), rope_cos=dcos, rope_sin=dsin)
    ops.linear16(v, dx, dev(ws[2], "f16"), ops.EPI_F16)
    out = torch.empty((T, H * 128), device="cuda", dtype=torch.float32)
    ops.attn_self(out, q, k, v, 1, T, H)                     # fp16, no norm, no RoPE: no staging pass, no workspace
    assert kb.check_status() == 0
    bits = lambda a: (a.view(np.uint32) >> 16).astype(np.uint16)
    qr = oracle.linear_heads16(x, ws[0], H, bits(nq), cos, sin)
    kr = oracle.linear_heads16(x, ws[1], H, bits(nk), cos, sin)
    vr = oracle.linear16(x, ws[2], 1)
    assert_close(out.cpu().numpy(), oracle.attention(qr, kr, vr, H), "projection -> attention chain")


def test_argument_errors(kb):
    import ctypes
    L = kb.lib()
    a = torch.zeros((128, 128), device="cuda", dtype=torch.float16)
    c = torch.zeros((128, 128), device="cuda", dtype=torch.float32)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def call(C=c, ldc=128, A=a, lda=128, W=a, ldw=128, M=128, N=128, K=128, epi=0, gate=None, hw=None, cos=None, sin=None, T=0):
        return L.kb_linear16(p(C), ldc, p(A), lda, p(W), ldw, M, N, K, epi, gate, hw, cos, sin, T, 1e-6, None)

    assert call() == 0
    assert call(M=0) == 0
    assert call(N=60) == -3 and call(N=64, epi=3) == -3 and call(N=64, epi=4) == -3 and call(K=32) == -3 and call(lda=64) == -3   # KB_ERR_SHAPE
    assert call(epi=5) == -1 and call(epi=0, gate=p(c)) == -1                     # KB_ERR_ARG
    assert call(epi=4, cos=p(c), sin=None) == -1 and call(epi=4, cos=p(c), sin=p(c), T=0) == -1
    assert call(lda=132) == -2 and call(ldc=130) == -2                            # KB_ERR_ALIGN
    assert L.kb_linear16(ctypes.c_void_p(a.data_ptr() + 2), 128, p(a), 128, p(a), 128, 128, 128, 128, 1, None, None, None, None, 0,
                         1e-6, None) == -2
    assert kb.check_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (129, 256, 64), (257, 512, 128), (128, 256, 192), (640, 384, 64), (2, 256, 2048)],
                         ids=["one_row", "pair_second_cta_one_row", "pair_ragged", "pair_not_taken_m128", "single_n384", "two_rows_long_k"])
def test_edge_shapes_every_epilogue(kb, M, N, K):
    """Smallest and raggedest shapes of both tile shapes (CTA pair: N % 256 == 0 and M > 128; single CTA otherwise), with a
    padded row stride: every epilogue against the oracle, nothing written outside the M x N window."""
    from kiln_b200 import ops
    x = seeded(200 + M, M, K, "f16")
    w = seeded(201 + N, N, K, "f16", 1.0 / np.sqrt(K))
    gate = oracle.randn(202, max(N, 16))[:N].copy()
    resid = oracle.randn(203, max(M * N, 16))[:M * N].reshape(M, N).copy()
    for epi in (ops.EPI_F32, ops.EPI_F16, ops.EPI_GELU16, ops.EPI_RESID):
        out = _run(kb, x, w, epi, gate=gate if epi == ops.EPI_RESID else None, resid=resid, ldc_pad=8)
        ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None)
        _close(out, ref, K, f"{M}x{N}x{K} epi {epi}", epi in (1, 2))
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(204, 128), 1)
    bits = (nw.view(np.uint32) >> 16).astype(np.uint16)
    T = 7                                                    # table shorter than M: rows wrap (batched images)
    cos, sin = (a[5:5 + T].copy() for a in oracle.cosmos_rope(4, 8))
    out = _run(kb, x, w, ops.EPI_HEADS16, ldc_pad=8, head_w=dev(nw).to(torch.bfloat16), rope_cos=dev(cos), rope_sin=dev(sin))
    reps = (M + T - 1) // T
    ref = oracle.linear_heads16(x, w, N // 128, bits, np.tile(cos, (reps, 1))[:M], np.tile(sin, (reps, 1))[:M])
    # fp32 summation order and one fp16 rounding are the only differences: a one-ulp disagreement is the worst case
    assert not np.isnan(out).any()
    assert np.all(np.abs(out - ref) <= 2.0 ** -10 * np.abs(ref) + 1e-4), f"{M}x{N}x{K} heads16: {np.abs(out - ref).max():.3e}"


@pytest.mark.parametrize("M,H,K", [(300, 2, 128), (333, 3, 192), (4096, 16, 2048)], ids=["pair_tiles", "single_tiles", "dit_size"])
def test_qkv_one_launch_equals_three_calls(kb, M, H, K):
    """kb_linear16_qkv: q and k with their own norm weights and RoPE, v plain — bit-identical to three kb_linear16 calls."""
    from kiln_b200 import ops
    N = H * 128
    side = int(np.sqrt(M))
    dx = dev(seeded(300, M, K, "f16"), "f16")
    ws = [dev(seeded(301 + i, N, K, "f16", 1.0 / np.sqrt(K)), "f16") for i in range(3)]
    nws = [dev(oracle.round16(1.0 + 0.05 * oracle.randn(310 + i, 128), 1)).to(torch.bfloat16) for i in range(2)]
    cos, sin = (dev(a) for a in oracle.cosmos_rope(side, side))          # table shorter than M: rows wrap
    one = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.linear16_qkv(one, dx, ws, head_ws=(nws[0], nws[1], None), rope_on=(True, True, False), rope_cos=cos, rope_sin=sin)
    three = [torch.empty((M, N), device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.linear16(three[0], dx, ws[0], ops.EPI_HEADS16, head_w=nws[0], rope_cos=cos, rope_sin=sin)
    ops.linear16(three[1], dx, ws[1], ops.EPI_HEADS16, head_w=nws[1], rope_cos=cos, rope_sin=sin)
    ops.linear16(three[2], dx, ws[2], ops.EPI_F16)
    assert kb.check_status() == 0
    for i in range(3):
        assert torch.equal(one[i], three[i]), f"projection {i} differs from its own launch"


def test_qkv_argument_errors(kb):
    import ctypes
    L = kb.lib()
    a = torch.zeros((128, 128), device="cuda", dtype=torch.float16)
    vp3 = ctypes.c_void_p * 3
    ptrs = vp3(a.data_ptr(), a.data_ptr(), a.data_ptr())
    none3 = vp3(None, None, None)
    on = (ctypes.c_int * 3)(1, 1, 0)
    off = (ctypes.c_int * 3)(0, 0, 0)
    args = lambda C=ptrs, W=ptrs, hw=none3, r=off, cos=None: (C, 128, ctypes.c_void_p(a.data_ptr()), 128, W, 128, 128, 128, 128, hw, r, cos, cos, 128, 1e-6, None)
    assert L.kb_linear16_qkv(*args()) == 0
    assert L.kb_linear16_qkv(*args(r=on)) == -1                                   # RoPE asked for without tables
    assert L.kb_linear16_qkv(*args(W=vp3(a.data_ptr(), None, a.data_ptr()))) == -1
    assert L.kb_linear16_qkv(*args(C=vp3(a.data_ptr(), a.data_ptr() + 2, a.data_ptr()))) == -2
    assert kb.check_status() == 0


def _lora_device_operands(kb, x16, loras, pad_to):
    """A_cat / B_cat packed on the device by kb_lora_pack, the stacked rank padded with zero rows / columns to a multiple of
    `pad_to`, and t = x . A_cat^T by the narrow fp16 epilogue."""
    from kiln_b200 import ops
    K, N = loras[0][0].shape[1], loras[0][1].shape[0]
    R = sum(a.shape[0] for a, _, _ in loras)
    Rp = (R + pad_to - 1) // pad_to * pad_to
    ac = torch.zeros((Rp, K), device="cuda", dtype=torch.float16)
    bc = torch.zeros((N, Rp), device="cuda", dtype=torch.float16)
    o = 0
    for a, b, s in loras:
        ops.lora_pack(ac[o:], 0, dev(a).to(torch.bfloat16), 1.0)
        ops.lora_pack(bc, o, dev(b).to(torch.bfloat16), s)
        o += a.shape[0]
    t = torch.full((x16.shape[0], Rp), float("nan"), device="cuda", dtype=torch.float16)
    ops.linear16(t, x16, ac, ops.EPI_F16)
    return t, bc, R


@pytest.mark.parametrize("case", [c for c in ggen.GEMM_CASES if c[0] in ggen.LORA_CASES], ids=[c[0] for c in ggen.GEMM_CASES if c[0] in ggen.LORA_CASES])
@pytest.mark.parametrize("pad_to", [8, 64], ids=["rank_as_is", "rank_padded_to_k_step"])
def test_lora_second_product_vs_oracle_and_reference_golden(kb, gemm_golden, case, pad_to):
    """The engine's unmerged LoRA path (linear16, engine/src/kernels.cu:578-596): operands packed, t = x A_cat^T, then
    acc = x W^T + t B_cat^T under every epilogue — against the oracle and against the reference kernel's own outputs."""
    from kiln_b200 import ops
    name, M, N, K = case
    x, w, gate, resid = ggen.gemm_inputs(case)
    loras = ggen.lora_inputs(case)
    t_ref, b_ref = oracle.lora_operands(x, loras)
    dx = dev(x, "f16")
    t, bc, R = _lora_device_operands(kb, dx, loras, pad_to)
    assert kb.check_status() == 0
    # packed operand: a rounding of a product of two exact values — bit-exact against the oracle and the reference's kernel
    assert np.array_equal(bc[:, :R].float().cpu().numpy(), b_ref), "B_cat differs from the oracle"
    assert np.array_equal(bc[:, :R].cpu().numpy().view(np.uint16), gemm_golden[f"{name}/lora_b"][:, :R].view(np.uint16)), "B_cat differs from k_lora_pack"
    assert not t[:, R:].float().abs().sum().item(), "padding columns of t are not zero"
    tn = t[:, :R].float().cpu().numpy()
    _close(tn, t_ref, K, f"{name} t vs oracle", True)
    _close(tn, gemm_golden[f"{name}/lora_t"][:, :R].astype(np.float32), K, f"{name} t vs the reference's product", True)
    for ename, epi in ggen.EPIS.items():
        c32 = epi in (ops.EPI_F32, ops.EPI_RESID)
        full = torch.full((M, N + 8), float("nan"), device="cuda", dtype=torch.float32 if c32 else torch.float16)
        c = full[:, :N]
        if epi == ops.EPI_RESID:
            c.copy_(dev(resid))
        ops.linear16(c, dx, dev(w, "f16"), epi, gate=dev(gate) if epi == ops.EPI_RESID else None, lora=(t, bc))
        assert kb.check_status() == 0
        assert torch.isnan(full[:, N:].float()).all(), "wrote outside the output columns"
        out = c.float().cpu().numpy()
        # the oracle gets the t this library produced, so that only the second product itself is compared here
        ref = oracle.linear16(x, w, epi, gate if epi == 3 else None, resid if epi == 3 else None, lora=(tn, b_ref))
        _close(out, ref, K + R, f"{name}/lora_{ename} vs oracle", epi in (1, 2))
        g = gemm_golden[f"{name}/lora_{ename}"].astype(np.float32)
        tile_err = 2.0 ** -11 * np.sqrt((K + R) / 32) * 4.0
        assert np.abs(out - g).max() <= tile_err + 2.0 ** -9 * np.abs(g).max(), f"{name}/lora_{ename} vs reference kernel: {np.abs(out - g).max():.3e}"


@pytest.mark.parametrize("M,N,K,K2", [(300, 512, 128, 8), (300, 512, 128, 72), (70, 384, 64, 128), (4096, 2048, 2048, 32)],
                         ids=["pair_tiles_rank8", "pair_tiles_partial_k_step", "single_tiles_two_k_steps", "dit_size_rank32"])
def test_second_product_shapes(kb, M, N, K, K2):
    """Second product of any width that is a multiple of 8, on both tile shapes, in a padded buffer (the columns past K2
    hold NaN and must not be read): sampled rows against the oracle."""
    from kiln_b200 import ops
    x, w = seeded(400, M, K, "f16"), seeded(401, N, K, "f16", 1.0 / np.sqrt(K))
    t, b = seeded(402, M, K2, "f16"), seeded(403, N, K2, "f16", 1.0 / np.sqrt(K2))
    tf = torch.full((M, K2 + 8), float("nan"), device="cuda", dtype=torch.float16)
    bf = torch.full((N, K2 + 16), float("nan"), device="cuda", dtype=torch.float16)
    tf[:, :K2].copy_(dev(t, "f16")); bf[:, :K2].copy_(dev(b, "f16"))
    c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float32)
    ops.linear16(c, dev(x, "f16"), dev(w, "f16"), ops.EPI_F32, lora=(tf[:, :K2], bf[:, :K2]))
    assert kb.check_status() == 0
    rows = sample_rows(M, 24)
    ref = oracle.linear16(x[rows], w, 0, lora=(t[rows], b))
    _close(c[torch.as_tensor(rows, device="cuda")].cpu().numpy(), ref, K + K2, f"{M}x{N}x{K}+{K2}", False)


@pytest.mark.parametrize("M,H,K", [(300, 2, 128), (333, 3, 192)], ids=["pair_tiles", "single_tiles"])
def test_qkv_lora_one_launch_equals_three_calls(kb, M, H, K):
    """kb_linear16_qkv_lora with a different rank per projection (none on v) — bit-identical to three kb_linear16_lora /
    kb_linear16 calls, and the head epilogue sees the LoRA-adjusted value (checked against the oracle on q)."""
    from kiln_b200 import ops
    N = H * 128
    x = seeded(500, M, K, "f16")
    dx = dev(x, "f16")
    wn = [seeded(501 + i, N, K, "f16", 1.0 / np.sqrt(K)) for i in range(3)]
    ws = [dev(a, "f16") for a in wn]
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(510, 128), 1)
    nws = [dev(nw).to(torch.bfloat16), None]
    cos_n, sin_n = oracle.cosmos_rope(20, 15)
    cos, sin = dev(cos_n), dev(sin_n)
    ranks = [16, 40, 0]
    tn = [seeded(520 + i, M, r, "f16") if r else None for i, r in enumerate(ranks)]
    bn = [seeded(530 + i, N, r, "f16", 0.2) if r else None for i, r in enumerate(ranks)]
    loras = [None if r == 0 else (dev(tn[i], "f16"), dev(bn[i], "f16")) for i, r in enumerate(ranks)]
    one = [torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.linear16_qkv(one, dx, ws, head_ws=(nws[0], nws[1], None), rope_on=(True, True, False), rope_cos=cos, rope_sin=sin, loras=loras)
    three = [torch.empty((M, N), device="cuda", dtype=torch.float16) for _ in range(3)]
    ops.linear16(three[0], dx, ws[0], ops.EPI_HEADS16, head_w=nws[0], rope_cos=cos, rope_sin=sin, lora=loras[0])
    ops.linear16(three[1], dx, ws[1], ops.EPI_HEADS16, head_w=nws[1], rope_cos=cos, rope_sin=sin, lora=loras[1])
    ops.linear16(three[2], dx, ws[2], ops.EPI_F16)
    assert kb.check_status() == 0
    for i in range(3):
        assert torch.equal(one[i], three[i]), f"projection {i} differs from its own launch"
    # q: rmsnorm and rope of (x W^T + t B^T), the order of engine/src/dit.cu:461-468 with a LoRA on the projection
    y = oracle.linear16(x, wn[0], 0, lora=(tn[0], bn[0]))
    bits = (nw.view(np.uint32) >> 16).astype(np.uint16)
    y = oracle.rmsnorm(y, bits, H, 1e-6)
    reps = (M + cos_n.shape[0] - 1) // cos_n.shape[0]                    # table shorter than M: rows wrap
    y = oracle.round16(oracle.rope_half(y, M, H, np.tile(cos_n, (reps, 1))[:M], np.tile(sin_n, (reps, 1))[:M]), 0)
    out = one[0].float().cpu().numpy()
    assert np.all(np.abs(out - y) <= 2.0 ** -10 * np.abs(y) + 1e-4), f"q with LoRA: {np.abs(out - y).max():.3e}"


@pytest.mark.parametrize("N", [8, 24, 72, 200], ids=lambda n: f"n{n}")
def test_narrow_outputs_of_the_store_epilogues(kb, N):
    """Output widths that are no multiple of the 128-column tile (the stacked rank of a LoRA down-projection): the three
    store epilogues against the oracle, nothing written past column N."""
    from kiln_b200 import ops
    M, K = 333, 192
    x, w = seeded(600, M, K, "f16"), seeded(601 + N, N, K, "f16", 1.0 / np.sqrt(K))
    for epi in (ops.EPI_F32, ops.EPI_F16, ops.EPI_GELU16):
        out = _run(kb, x, w, epi, ldc_pad=136)
        _close(out, oracle.linear16(x, w, epi), K, f"N={N} epi {epi}", epi in (1, 2))


def test_lora_argument_errors(kb):
    import ctypes
    L = kb.lib()
    a = torch.zeros((128, 128), device="cuda", dtype=torch.float16)
    c = torch.zeros((128, 128), device="cuda", dtype=torch.float32)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def call(A2=p(a), lda2=128, W2=p(a), ldw2=128, K2=32):
        return L.kb_linear16_lora(p(c), 128, p(a), 128, p(a), 128, A2, lda2, W2, ldw2, K2, 128, 128, 128, 0, None, None, None, None, 0, 1e-6, None)

    assert call() == 0 and call(K2=0, A2=None, W2=None) == 0
    assert call(A2=None) == -1 and call(W2=None) == -1 and call(K2=-8) == -1      # KB_ERR_ARG
    assert call(K2=12) == -3 and call(lda2=16) == -3                              # KB_ERR_SHAPE
    assert call(lda2=132) == -2 and call(A2=ctypes.c_void_p(a.data_ptr() + 2)) == -2   # KB_ERR_ALIGN
    assert L.kb_lora_pack(p(a), 128, 120, p(a), 4, 16, 1.0, None) == -1           # columns past the row stride
    assert kb.check_status() == 0


@pytest.mark.parametrize("L,src", [(26, "f32"), (77, "f32"), (512, "f32"), (300, "f16"), (40, "bf16")], ids=lambda v: str(v))
def test_cross_kv_producer_feeds_cross_attention(kb, L, src):
    """kb_cross_kv: K = rmsnorm(ctx Wk^T) and V = ctx Wv^T of a [L, 1024] context as fp16 in one GEMM launch — against the oracle's
    restatement of Dit::cache_context (engine/src/dit.cu:228-230), then through kb_attn_cross against the oracle's attention on the
    oracle's K and V (the engine's order: cache_context, then attention16 with npad zero keys, dit.cu:476-481)."""
    from kiln_b200 import ops
    H, KD = 3, 1024
    N = H * 128
    kind = {"f32": None, "f16": "f16", "bf16": "bf16"}[src]
    ctx = oracle.randn(700 + L, L * KD).reshape(L, KD)
    if kind:
        ctx = oracle.round16(ctx, 0 if kind == "f16" else 1)
    wk, wv = (seeded(710 + j, N, KD, "f16", 1.0 / np.sqrt(KD)) for j in range(2))
    nw = oracle.round16(1.0 + 0.05 * oracle.randn(712, 128), 1)
    bits = (nw.view(np.uint32) >> 16).astype(np.uint16)
    k16 = torch.full((L, N + 8), float("nan"), device="cuda", dtype=torch.float16)
    v16 = torch.full((L, N + 8), float("nan"), device="cuda", dtype=torch.float16)
    ops.cross_kv(k16[:, :N], v16[:, :N], dev(ctx, kind), dev(wk, "f16"), dev(wv, "f16"), kn_w=dev(nw).to(torch.bfloat16))
    assert kb.check_status() == 0
    assert torch.isnan(k16[:, N:].float()).all() and torch.isnan(v16[:, N:].float()).all(), "wrote outside the output columns"
    x16 = oracle.round16(ctx, 0)                                     # the GEMM reads the context as fp16
    k_ref = oracle.round16(oracle.rmsnorm(oracle.linear16(x16, wk, 0), bits, H, 1e-6), 0)
    v_ref = oracle.linear16(x16, wv, 1)
    ko, vo = k16[:, :N].float().cpu().numpy(), v16[:, :N].float().cpu().numpy()
    assert np.all(np.abs(ko - k_ref) <= 2.0 ** -10 * np.abs(k_ref) + 1e-4), f"K: {np.abs(ko - k_ref).max():.3e}"
    assert np.all(np.abs(vo - v_ref) <= 2.0 ** -10 * np.abs(v_ref) + 1e-4), f"V: {np.abs(vo - v_ref).max():.3e}"
    Tq, npad = 200, 512 - L if L < 512 else 0
    q = seeded(720, Tq, N, "f16")
    out = torch.empty((Tq, N), device="cuda", dtype=torch.float32)
    kb.attn_cross(out, dev(q, "f16"), k16[:, :N], v16[:, :N], Tq, L, npad, H)
    assert kb.check_status() == 0
    assert_close(out.cpu().numpy(), oracle.attention(q, k_ref, v_ref, H, npad), f"cross-attention on produced K/V, L={L}")
