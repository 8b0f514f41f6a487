"""Runs one kernel family a few times on seeded inputs, for profilers and quick timing.

    python -m kiln_b200.profile_case --case self|cross|nag|prep [--tokens 4096] [--batch 1] [--heads 16]
                                     [--ctx 512] [--dtype f16|bf16] [--norm] [--reps 5]

Prints the average CUDA-event time per call and the algorithmic TFLOP/s (4*Tq*Tk*128*H per attention).
Under `ncu`, select the kernel with -k regex:attn_fwd_kernel (or qk_prep_kernel) and skip warm-up launches with -s.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import kiln_b200 as kb  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="self", choices=["self", "cross", "nag", "prep"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"])
    ap.add_argument("--norm", action="store_true", help="Q/K RMSNorm (+ RoPE for self) through the staging pre-pass")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warm", type=int, default=2)
    a = ap.parse_args()
    assert kb.lib().kb_init() == 0
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


if __name__ == "__main__":
    main()
