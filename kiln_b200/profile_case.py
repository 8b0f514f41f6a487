"""Runs one kernel family a few times on seeded inputs, for profilers and quick timing.

    python -m kiln_b200.profile_case --case self|cross|nag|prep [--tokens 4096] [--batch 1] [--heads 16]
                                     [--ctx 512] [--dtype f16|bf16] [--norm] [--reps 5]
    python -m kiln_b200.profile_case --case linear [--tokens 4096] [--n 2048] [--k 2048] [--epi f16|f32|gelu16|resid|heads16]
    python -m kiln_b200.profile_case --case block [--tokens 4096] [--heads 16]

Prints the average CUDA-event time per call and the algorithmic TFLOP/s (4*Tq*Tk*128*H per attention, 2*M*N*K per
linear layer). `block` is the self-attention half of a DiT block (engine/src/dit.cu:461-471): q, k, v projections,
attention, output projection into the fp32 residual stream, once with the fused head epilogue feeding attention
directly and once the way the engine orders it (fp32 projections, then norm + RoPE inside the attention call).
Under `ncu`, select the kernel with -k regex:attn_fwd_kernel (qk_prep_kernel, gemm16_kernel) and skip warm-up launches with -s.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import kiln_b200 as kb  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="self", choices=["self", "cross", "nag", "prep", "linear", "block"])
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epi", default="f16", choices=["f32", "f16", "gelu16", "resid", "heads16"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--norm", action="store_true", help="Q/K RMSNorm (+ RoPE for self) through the staging pre-pass")
    ap.add_argument("--cublas", action="store_true", help="linear: also time torch.matmul on the same operands")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warm", type=int, default=2)
    a = ap.parse_args()
    assert kb.lib().kb_init() == 0
    if a.case in ("linear", "block"):
        return linear_cases(a)
    dt = torch.float16 if a.dtype == "f16" else torch.bfloat16
    T, B, H, L = a.tokens, a.batch, a.heads, a.ctx
    D = H * 128
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g).to(dt)
    q, k, v = rn(B * T, D), rn(B * T, D), rn(B * T, D)
    out = torch.empty(B * T, D, device="cuda", dtype=dt)
    w = torch.ones(128, device="cuda", dtype=torch.bfloat16) if a.norm else None
    cos = sin = None
    if a.norm and a.case in ("self", "prep"):
        side = int(round(T ** 0.5))
        assert side * side == T, "--norm with RoPE wants a square token grid"
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle"))
        cos = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
        sin = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
    ws = torch.empty(max(16, kb.workspace_bytes(B * T, B * max(T, L), H, dt, True, True, n_ctx=2)), dtype=torch.uint8, device="cuda")
    kp, vp, kn, vn = rn(L, D), rn(L, D), rn(L, D), rn(L, D)
    if a.case == "self":
        fn = lambda: kb.attn_self(out, q, k, v, B, T, H, qn_w=w, kn_w=w, rope_cos=cos, rope_sin=sin, workspace=ws)
        flop = 4.0 * T * T * 128 * H * B
    elif a.case == "cross":
        fn = lambda: kb.attn_cross(out[:T], q[:T], kp, vp, T, L, 0, H, qn_w=w, workspace=ws)
        flop = 4.0 * T * L * 128 * H
    elif a.case == "nag":
        fn = lambda: kb.attn_nag(out[:T], q[:T], kp, vp, L, 0, kn, vn, L, 0, 5.0, 2.5, 0.25, T, H, qn_w=w, workspace=ws)
        flop = 8.0 * T * L * 128 * H
    else:
        st = torch.empty(B * T, D, device="cuda", dtype=torch.float16)
        fn = lambda: kb.qk_prep(st, q, B * T, H, T, w=w, rope_cos=cos, rope_sin=sin)
        flop = 0.0
    for _ in range(a.warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / a.reps * 1e3
    assert kb.check_status() == 0
    print(f"case={a.case} tokens={T} batch={B} heads={H} ctx={L} dtype={a.dtype} norm={a.norm}: {us:.1f} us/call"
          + (f", {flop / us / 1e6:.1f} TFLOP/s" if flop else f", {B * T * D * (q.element_size() + 2) / us / 1e3:.0f} GB/s"))


def timed(fn, warm, reps):
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


def linear_cases(a):
    from kiln_b200 import ops
    T, H = a.tokens, a.heads
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    rn = lambda r, c, amp=1.0: (torch.randn(r, c, device="cuda", generator=g) * amp).half()
    hw = torch.ones(128, device="cuda", dtype=torch.bfloat16)
    cos = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
    sin = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
    if a.case == "linear":
        M, N, K = T, a.n, a.k
        epi = {"f32": ops.EPI_F32, "f16": ops.EPI_F16, "gelu16": ops.EPI_GELU16, "resid": ops.EPI_RESID, "heads16": ops.EPI_HEADS16}[a.epi]
        nset = 4                                            # distinct operand sets so that weights do not stay in L2 between calls
        xs, wts = [rn(M, K) for _ in range(nset)], [rn(N, K, 0.02) for _ in range(nset)]
        c = torch.zeros(M, N, device="cuda", dtype=torch.float32 if epi in (ops.EPI_F32, ops.EPI_RESID) else torch.float16)
        kw = dict(head_w=hw, rope_cos=cos, rope_sin=sin) if epi == ops.EPI_HEADS16 else {}
        it = [0]

        def fn():
            it[0] = (it[0] + 1) % nset
            ops.linear16(c, xs[it[0]], wts[it[0]], epi, **kw)
        us = timed(fn, a.warm, a.reps)
        assert kb.check_status() == 0
        print(f"case=linear M={M} N={N} K={K} epi={a.epi}: {us:.1f} us/call, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
        if a.cublas and epi == ops.EPI_F16:                 # the library GEMM on the same operands, for scale

            def mm():
                it[0] = (it[0] + 1) % nset
                torch.matmul(xs[it[0]], wts[it[0]].T, out=c)
            us = timed(mm, a.warm, a.reps)
            print(f"  cuBLAS (torch.matmul) fp16: {us:.1f} us/call, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
        return
    D = H * 128
    x = rn(T, D)
    wq, wk, wv, wo = (rn(D, D, 0.02) for _ in range(4))
    resid = torch.zeros(T, D, device="cuda", dtype=torch.float32)
    gate = torch.ones(D, device="cuda")
    q16, k16, v16, o16 = (torch.empty(T, D, device="cuda", dtype=torch.float16) for _ in range(4))
    q32, k32, v32 = (torch.empty(T, D, device="cuda", dtype=torch.float32) for _ in range(3))
    ws = torch.empty(max(16, kb.workspace_bytes(T, T, H, torch.float32, True, True)), dtype=torch.uint8, device="cuda")

    def fused():
        ops.linear16(q16, x, wq, ops.EPI_HEADS16, head_w=hw, rope_cos=cos, rope_sin=sin)
        ops.linear16(k16, x, wk, ops.EPI_HEADS16, head_w=hw, rope_cos=cos, rope_sin=sin)
        ops.linear16(v16, x, wv, ops.EPI_F16)
        kb.attn_self(o16, q16, k16, v16, 1, T, H)
        ops.linear16(resid, o16, wo, ops.EPI_RESID, gate=gate)

    def fused_one_launch():
        ops.linear16_qkv([q16, k16, v16], x, [wq, wk, wv], head_ws=(hw, hw, None), rope_on=(True, True, False), rope_cos=cos, rope_sin=sin)
        kb.attn_self(o16, q16, k16, v16, 1, T, H)
        ops.linear16(resid, o16, wo, ops.EPI_RESID, gate=gate)

    def engine_order():
        ops.linear16(q32, x, wq, ops.EPI_F32)
        ops.linear16(k32, x, wk, ops.EPI_F32)
        ops.linear16(v32, x, wv, ops.EPI_F32)
        kb.attn_self(o16, q32, k32, v32, 1, T, H, qn_w=hw, kn_w=hw, rope_cos=cos, rope_sin=sin, workspace=ws)
        ops.linear16(resid, o16, wo, ops.EPI_RESID, gate=gate)

    flop = 4.0 * T * T * 128 * H + 4 * 2.0 * T * D * D
    for name, fn in (("q, k, v in one launch", fused_one_launch), ("fused head epilogue", fused), ("engine order", engine_order)):
        us = timed(fn, a.warm, a.reps)
        assert kb.check_status() == 0
        print(f"case=block tokens={T} heads={H} [{name}]: {us:.1f} us/block-half, {flop / us / 1e6:.1f} TFLOP/s")


if __name__ == "__main__":
    main()
