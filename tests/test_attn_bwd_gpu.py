"""GPU parity tests of the attention backward (kb_attn_bwd) through the C ABI: against the fp64 CPU oracle (a restatement of
the reference's attention_bwd, engine/src/train.cu:216-242), against the reference's own outputs (golden fixture and, where
the reference is compiled, a live run), and through size-independent properties at the full DiT size.

Tolerance: the attention path's bar, max-abs <= 2e-3 and mean-relative <= 1e-3, against the oracle on the operands the tensor cores
see (inputs rounded once to fp16). Against the REFERENCE'S outputs, which come from unrounded fp32 inputs through fp32 SGEMMs, the
max-abs bound is taken relative to the gradient's scale (2e-3 * max|ref|, gradients there reach 3.9): rounding q, k, v and dout to
fp16 alone moves those gradients by up to 2.8e-3 (6e-4 mean-relative; measured with the fp64 oracle), which no fp16-operand kernel
can avoid; the forward outputs, convex combinations of V, never met this because their scale is 1."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle
from util_gpu import assert_close, dev, sample_rows, seeded

pytestmark = pytest.mark.gpu

_HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_ref_bwd_fixtures", os.path.join(_HERE, "golden", "make_ref_bwd_fixtures.py"))
bgen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bgen)


@pytest.fixture(scope="module")
def kb(built_lib):
    import kiln_b200
    assert kiln_b200.lib().kb_init() == 0, "sm_100 device and the CUDA library are required (there is no fallback)"
    return kiln_b200


def _run(kb, q, k, v, dout, B, Tq, Tk, npad, H, kind=None, pad=8):
    """Outputs live in padded, NaN-filled buffers: nothing may be written outside the [rows, H*128] window."""
    D = H * 128
    outs = [torch.full((B * T, D + pad), float("nan"), device="cuda") for T in (Tq, Tk, Tk)]
    kb.attn_bwd(outs[0][:, :D], outs[1][:, :D], outs[2][:, :D], dev(q, kind), dev(k, kind), dev(v, kind), dev(dout, kind), B, Tq, Tk, npad, H)
    assert kb.check_status() == 0
    for o in outs:
        assert torch.isnan(o[:, D:]).all(), "wrote outside the output columns"
    return [o[:, :D].cpu().numpy() for o in outs]


@pytest.mark.parametrize("Tq,Tk,H,npad,kind", [(128, 128, 1, 0, None), (200, 77, 2, 435, None), (300, 300, 3, 0, "f16"), (130, 257, 2, 0, "bf16"),
                                               (1, 3, 1, 0, None), (257, 26, 4, 486, "f16"), (640, 384, 2, 0, None)],
                         ids=["one_tile", "cross_pad", "ragged_self_f16", "ragged_bf16", "single_row", "cross_pad_f16", "many_blocks"])
def test_small_cases_vs_oracle(kb, Tq, Tk, H, npad, kind):
    D = H * 128
    q, k = seeded(40, Tq, D, kind or "f16", 1.5), seeded(41, Tk, D, kind or "f16", 1.5)
    v, dout = seeded(42, Tk, D, kind or "f16"), seeded(43, Tq, D, kind or "f16")
    if kind is None:                                               # fp32 inputs that are not fp16-exact: the staging rounds them
        q, k, v, dout = (a + np.float32(1e-4) * oracle.randn(44 + i, a.size).reshape(a.shape) for i, a in enumerate((q, k, v, dout)))
    dq, dk, dv = _run(kb, q, k, v, dout, 1, Tq, Tk, npad, H, kind)
    r16 = lambda a: oracle.round16(a, 0) if kind != "bf16" else a  # the kernels see the fp16 rounding of fp32 inputs (bf16 -> fp16 is exact here only by value range)
    rq, rk, rv = oracle.attention_bwd(r16(q), r16(k), r16(v), r16(dout), H, npad)
    assert_close(dq, rq, f"dq {Tq}x{Tk}x{H} npad {npad}")
    assert_close(dk, rk, f"dk {Tq}x{Tk}x{H} npad {npad}")
    assert_close(dv, rv, f"dv {Tq}x{Tk}x{H} npad {npad}")


def test_batch_equals_per_image_calls(kb):
    B, T, H = 2, 200, 2
    D = H * 128
    q, k, v, dout = (seeded(50 + i, B * T, D, "f16", 1.5 if i < 2 else 1.0) for i in range(4))
    both = _run(kb, q, k, v, dout, B, T, T, 0, H, "f16")
    for b in range(B):
        sl = slice(b * T, (b + 1) * T)
        one = _run(kb, q[sl], k[sl], v[sl], dout[sl], 1, T, T, 0, H, "f16")
        for name, x, y in zip(("dq", "dk", "dv"), both, one):
            assert np.array_equal(x[sl], y), f"{name} of image {b} differs from its own call"


@pytest.mark.parametrize("case", bgen.BWD_CASES, ids=[c[0] for c in bgen.BWD_CASES])
def test_vs_reference_golden(kb, case):
    """The reference's attention_bwd outputs (fp32 SGEMM path, 16 heads) on the same seeded inputs."""
    golden = np.load(os.path.join(_HERE, "golden", "ref_bwd_fixtures.npz"))
    name, Tq, Tk, npad = case
    q, k, v, dout = bgen.bwd_inputs(case)
    outs = _run(kb, q, k, v, dout, 1, Tq, Tk, npad, bgen.H)
    n = bgen.KEEP_HEADS * 128
    for gname, o in zip(("dq", "dk", "dv"), outs):
        g = golden[f"{name}/{gname}"]
        assert_close(o[:, :n], g, f"{name}/{gname} vs the reference's attention_bwd", max_abs=2e-3 * max(1.0, float(np.abs(g).max())))


def test_properties_at_the_dit_size(kb):
    """4096 tokens x 16 heads (the trainer's self-attention call at a 1024 x 1024 image, train.cu:344): (1) sampled query rows of
    dq against the oracle with the full K/V; (2) doubling dout doubles every gradient (every rounding scales by a power of two,
    except where a dS entry is an fp16 subnormal: held to 2e-5); (3) repeat runs are bit-identical; (4) one head's dk / dv rows
    against the oracle on all 4096 queries."""
    T, H = 4096, 16
    D = H * 128
    q, k = seeded(60, T, D, "f16", 1.5), seeded(61, T, D, "f16", 1.5)
    v, dout = seeded(62, T, D, "f16"), seeded(63, T, D, "f16")
    dq, dk, dv = _run(kb, q, k, v, dout, 1, T, T, 0, H, "f16", pad=0)
    dq2, dk2, dv2 = _run(kb, q, k, v, 2.0 * dout, 1, T, T, 0, H, "f16", pad=0)
    for name, a2, a1 in (("dq", dq2, dq), ("dk", dk2, dk), ("dv", dv2, dv)):
        assert np.abs(a2 - 2 * a1).max() <= 2e-5, f"{name} is not linear in dout: {np.abs(a2 - 2 * a1).max():.3e}"
    dq3, dk3, dv3 = _run(kb, q, k, v, dout, 1, T, T, 0, H, "f16", pad=0)
    assert np.array_equal(dq3, dq) and np.array_equal(dk3, dk) and np.array_equal(dv3, dv), "repeat run differs"
    rows = sample_rows(T, 12)
    rq, _, _ = oracle.attention_bwd(q[rows], k, v, dout[rows], H, 0, key_rows=(0, 0))
    assert_close(dq[rows], rq, "dq rows at 4096 tokens")
    h = 5
    cs = slice(h * 128, (h + 1) * 128)
    j0, j1 = 4000, 4096                                                # the last key block, through all 32 query blocks
    _, rk, rv = oracle.attention_bwd(q[:, cs], k[:, cs], v[:, cs], dout[:, cs], 1, 0, key_rows=(j0, j1))
    assert_close(dk[j0:j1, cs], rk, "dk rows of one head at 4096 tokens")
    assert_close(dv[j0:j1, cs], rv, "dv rows of one head at 4096 tokens")


def test_equal_keys_give_zero_dq(kb):
    """Rows of dS sum to zero (k_dsoftmax, train.cu:124-131): with every key equal, dq = dS K / sqrt(128) vanishes."""
    Tq, Tk, H = 130, 200, 2
    D = H * 128
    q, dout, v = seeded(70, Tq, D, "f16", 1.5), seeded(71, Tq, D, "f16"), seeded(72, Tk, D, "f16")
    k = np.tile(seeded(73, 1, D, "f16"), (Tk, 1))
    dq, dk, dv = _run(kb, q, k, v, dout, 1, Tq, Tk, 0, H, "f16")
    assert np.abs(dq).max() <= 2e-3, f"{np.abs(dq).max():.3e}"


def test_argument_errors(kb):
    import ctypes
    L = kb.lib()
    a = torch.zeros((128, 128), device="cuda", dtype=torch.float16)
    o = torch.zeros((128, 128), device="cuda")
    ws = torch.zeros(L.kb_attn_bwd_workspace_bytes(1, 128, 128, 1, 0) + 256, device="cuda", dtype=torch.uint8)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def call(dq=p(o), q=p(a), Tq=128, ld=128, w=p(ws), wb=ws.numel(), npad=0):
        return L.kb_attn_bwd(dq, p(o), p(o), q, p(a), p(a), p(a), 1, Tq, 128, npad, 1, ld, 128, 128, 128, 128, 128, 128, 0, w, wb, None)

    assert call() == 0
    assert call(dq=None) == -1 and call(q=None) == -1 and call(Tq=0) == -1 and call(npad=-1) == -1
    assert call(ld=64) == -3 and call(ld=132) == -2
    assert call(w=None) == -4 and call(wb=1024) == -4
    assert kb.check_status() == 0
