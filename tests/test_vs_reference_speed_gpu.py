"""The reference's own CUDA kernels (compiled for sm_100a into oracle/_ref by oracle/build.py) timed beside this
library's on the same GPU, same shapes, in one process. Skipped when oracle/_ref was not built. Run with -s to see
the numbers; the assertions only hold the ordering (this library at least twice as fast at the DiT sizes).

    python -m pytest tests/test_vs_reference_speed_gpu.py -m gpu -s
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF):
        pytest.skip("oracle/_ref/libkiln_ref.so not built (needs the reference tree at build time)")
    R = ctypes.CDLL(REF)
    vp, i = ctypes.c_void_p, ctypes.c_int
    R.kref_time_linear16.restype = ctypes.c_float
    R.kref_time_linear16.argtypes = [vp, i, vp, vp, i, i, i, i, vp, i, i]
    R.kref_time_tfa_f16.restype = ctypes.c_float
    R.kref_time_tfa_f16.argtypes = [vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, i]
    return R


@pytest.fixture(scope="module")
def kb(built_lib):
    import kiln_b200
    assert kiln_b200.lib().kb_init() == 0
    return kiln_b200


def _timed(fn, warm=3, reps=10):
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


@pytest.mark.parametrize("M,N,K", [(4096, 2048, 2048), (4096, 8192, 2048), (4096, 2048, 8192)])
def test_linear16_vs_reference_gemm(kb, ref, M, N, K):
    from kiln_b200 import ops
    x = torch.randn(M, K, device="cuda").half()
    w = (torch.randn(N, K, device="cuda") * 0.02).half()
    c = torch.empty(M, N, device="cuda", dtype=torch.float16)
    ours = _timed(lambda: ops.linear16(c, x, w, ops.EPI_F16))
    theirs = ref.kref_time_linear16(c.data_ptr(), N, x.data_ptr(), w.data_ptr(), M, N, K, 1, None, 3, 10) * 1e3
    assert kb.check_status() == 0 and theirs > 0
    fl = 2.0 * M * N * K
    print(f"\nlinear16 {M}x{N}x{K} fp16 out: this library {ours:.1f} us ({fl / ours / 1e6:.0f} TFLOP/s), "
          f"reference tc16::k_gemm16 {theirs:.1f} us ({fl / theirs / 1e6:.0f} TFLOP/s), ratio {theirs / ours:.1f}x")
    assert theirs > 2.0 * ours


@pytest.mark.parametrize("Tq,Tk,npad", [(4096, 4096, 0), (4096, 26, 486)])
def test_attention16_vs_reference_flash(kb, ref, Tq, Tk, npad):
    H = 16
    q = torch.randn(Tq, H * 128, device="cuda") * 1.5                  # the reference kernel takes fp32 and converts while staging
    k = torch.randn(Tk, H * 128, device="cuda") * 1.5
    v = torch.randn(Tk, H * 128, device="cuda")
    out = torch.empty(Tq, H * 128, device="cuda", dtype=torch.float16)
    q16, k16, v16 = q.half(), k.half(), v.half()
    ours = _timed(lambda: kb.attn_cross(out, q16, k16, v16, Tq, Tk, npad, H))
    ws = torch.empty(max(16, kb.workspace_bytes(Tq, Tk, H, torch.float32)), dtype=torch.uint8, device="cuda")
    ours32 = _timed(lambda: kb.attn_cross(out, q, k, v, Tq, Tk, npad, H, workspace=ws))
    ld = H * 128
    theirs = ref.kref_time_tfa_f16(out.data_ptr(), ld, q.data_ptr(), ld, k.data_ptr(), ld, v.data_ptr(), ld, Tq, Tk, H, npad, 3, 10) * 1e3
    assert kb.check_status() == 0 and theirs > 0
    fl = 4.0 * Tq * (Tk + npad) * 128 * H
    print(f"\nattention16 Tq={Tq} Tk={Tk} npad={npad}: this library {ours:.1f} us on fp16 operands, {ours32:.1f} us from the engine's fp32 "
          f"activations (staging pass included), reference tfa::k_flash {theirs:.1f} us; {fl / ours / 1e6:.0f} vs {fl / theirs / 1e6:.0f} TFLOP/s")
    if Tk >= 1024:
        assert theirs > 2.0 * ours32


@pytest.mark.parametrize("Tq,Tk,npad", [(4096, 4096, 0), (1536, 1536, 0), (4096, 77, 435)], ids=["self_4096", "self_1536", "cross_77_of_512"])
def test_attention_bwd_vs_reference(kb, ref, Tq, Tk, npad):
    """kb_attn_bwd (all its launches, fp32 inputs as the trainer holds them) beside the reference's attention_bwd
    (engine/src/train.cu:216-242: fp32 cuBLAS SGEMMs with P and dP in the arena) on the same GPU."""
    H, D = 16, 2048
    ref.kref_engine_init.argtypes = [ctypes.c_size_t, ctypes.c_char_p, ctypes.c_int]
    ref.kref_attention_bwd.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_char_p, ctypes.c_int]
    err = ctypes.create_string_buffer(512)
    assert ref.kref_engine_init(3 << 30, err, 512) == 0, err.value
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    rn = lambda r: torch.randn(r, D, device="cuda", generator=g)
    q, k, v, do = rn(Tq), rn(Tk), rn(Tk), rn(Tq)
    mine = [torch.empty(Tq, D, device="cuda"), torch.empty(Tk, D, device="cuda"), torch.empty(Tk, D, device="cuda")]
    theirs = [torch.empty_like(t) for t in mine]
    ws = torch.empty(kb.lib().kb_attn_bwd_workspace_bytes(1, Tq, Tk, H, kb.KB_F32), dtype=torch.uint8, device="cuda")
    P = lambda t: ctypes.c_void_p(t.data_ptr())

    def run_ref():
        assert ref.kref_attention_bwd(P(theirs[0]), P(theirs[1]), P(theirs[2]), P(q), P(k), P(v), P(do), Tq, Tk, npad, err, 512) == 0, err.value

    t_ours = _timed(lambda: kb.attn_bwd(mine[0], mine[1], mine[2], q, k, v, do, 1, Tq, Tk, npad, H, workspace=ws))
    t_ref = _timed(run_ref, warm=1, reps=3)
    assert kb.check_status() == 0
    flop = 10.0 * Tq * Tk * 128 * H
    worst = max(float((a - b).abs().max() / b.abs().max().clamp_min(1.0)) for a, b in zip(mine, theirs))
    print(f"\nattention backward {Tq}x{Tk} (npad {npad}): ours {t_ours:.1f} us ({flop / t_ours / 1e6:.0f} TFLOP/s of the five products), "
          f"reference {t_ref:.1f} us, {t_ref / t_ours:.1f}x; worst difference relative to the gradient's scale {worst:.2e}")
    assert t_ours < t_ref
    assert worst <= 2e-3
