"""kb_attn_self_static: self-attention for callers that have no workspace to give and may not allocate
(an engine whose arena is already full, a plugin handed only inputs and outputs). The staging scratch is
a fixed 32 MiB array inside the library, so this test checks, through the C ABI, that
  * two calls in a row (the second must not be disturbed by what the first left in the array) give what
    kb_attn_self gives with a caller-owned workspace, within the suite's tolerance;
  * the call leaves the driver's free-memory figure where it was (nothing was allocated behind the caller's back);
  * a problem that does not fit the array is refused with KB_ERR_STATIC_SCRATCH and launches nothing.
This file sorts last on purpose: a run that stops at the first failure has then run everything else."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from util_gpu import TOL_MAX_ABS, TOL_MEAN_REL, dev, errors, seeded

pytestmark = pytest.mark.gpu

KB_ERR_STATIC_SCRATCH = -9
P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())


def _both(L, kb, seed, B, Hp, Wp, H, kind):
    """Run kb_attn_self (caller workspace) and kb_attn_self_static on the same seeded bf16/fp16 inputs with Q/K norm + RoPE."""
    T = Hp * Wp
    dt = {"bf16": torch.bfloat16, "f16": torch.float16}[kind]
    code = {"bf16": kb.KB_BF16, "f16": kb.KB_F16}[kind]
    q, k, v = (dev(seeded(seed + i, B * T, H * 128, kind), kind) for i in range(3))
    wq = dev(1 + 0.02 * oracle.randn(seed + 3, 128)).to(torch.bfloat16)
    wk = dev(1 + 0.02 * oracle.randn(seed + 4, 128)).to(torch.bfloat16)
    c, s = (dev(a) for a in oracle.cosmos_rope(Hp, Wp))
    ld = H * 128
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(kb.workspace_bytes(B * T, B * T, H, dt, True, True), dtype=torch.uint8, device="cuda")
    ref = torch.full((B * T, ld), float("nan"), device="cuda", dtype=dt)
    rc = L.kb_attn_self(P(ref), P(q), P(k), P(v), P(wq), P(wk), P(c), P(s), B, T, H, ld, ld, ld, ld, code, code, 1e-6, P(ws), ws.numel(), stream)
    assert rc == 0
    out = torch.full((B * T, ld), float("nan"), device="cuda", dtype=dt)
    rc = L.kb_attn_self_static(P(out), P(q), P(k), P(v), P(wq), P(wk), P(c), P(s), B, T, H, ld, ld, ld, ld, code, code, 1e-6, stream)
    assert rc == 0, kb.lib().kb_error_string(rc)
    assert kb.check_status() == 0
    return out.float().cpu().numpy(), ref.float().cpu().numpy()


def test_static_scratch_matches_workspace_entry_point_twice(built_lib):
    import kiln_b200 as kb
    L = kb.lib()
    assert L.kb_init() == 0
    # first call: 24x32 patches, B=2, bf16 -> 3 staged tensors of 6 MiB; second call: a smaller, differently shaped
    # problem in fp16, so stale rows of the first call sit right behind the rows the second one uses
    for seed, B, Hp, Wp, H, kind in [(100, 2, 24, 32, 16, "bf16"), (200, 1, 17, 23, 8, "f16")]:
        out, ref = _both(L, kb, seed, B, Hp, Wp, H, kind)
        assert not np.isnan(out).any()
        e_max, e_rel, _ = errors(out, ref)
        assert e_max <= TOL_MAX_ABS and e_rel <= TOL_MEAN_REL, f"static vs workspace entry point: max_abs {e_max:.3e} mean_rel {e_rel:.3e}"
        assert np.array_equal(out, ref)          # same kernels, same schedule (whole items per SM at these sizes), same bytes


def test_static_scratch_call_allocates_nothing(built_lib):
    """Free device memory as the driver reports it is the same before and after a call (all tensors exist beforehand,
    the entry point was used before, and nothing else allocates in between)."""
    import kiln_b200 as kb
    L = kb.lib()
    assert L.kb_init() == 0
    T, H = 768, 16
    ld = H * 128
    q, k, v = (dev(seeded(300 + i, T, ld, "bf16"), "bf16") for i in range(3))
    w = dev(1 + 0.02 * oracle.randn(303, 128)).to(torch.bfloat16)
    c, s = (dev(a) for a in oracle.cosmos_rope(24, 32))
    out = torch.empty(T, ld, device="cuda", dtype=torch.bfloat16)
    call = lambda: L.kb_attn_self_static(P(out), P(q), P(k), P(v), P(w), P(w), P(c), P(s), 1, T, H, ld, ld, ld, ld, kb.KB_BF16, kb.KB_BF16, 1e-6, None)
    assert call() == 0                             # first use on this device: looks up the array's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    assert call() == 0
    assert call() == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert kb.check_status() == 0


def test_static_scratch_refuses_oversize(built_lib):
    import kiln_b200 as kb
    L = kb.lib()
    assert L.kb_init() == 0
    T, H = 4096, 16                               # bf16 staging = 3 x 16 MiB > 32 MiB
    t = torch.zeros(T, H * 128, device="cuda", dtype=torch.bfloat16)
    out = torch.full((T, H * 128), 3.0, device="cuda", dtype=torch.bfloat16)
    rc = L.kb_attn_self_static(P(out), P(t), P(t), P(t), None, None, None, None, 1, T, H, 2048, 2048, 2048, 2048, kb.KB_BF16, kb.KB_BF16, 1e-6, None)
    assert rc == KB_ERR_STATIC_SCRATCH
    assert b"built-in buffer" in L.kb_error_string(rc)
    torch.cuda.synchronize()
    assert torch.all(out == 3.0)                  # nothing ran
    # fp16 inputs without norm/RoPE need no staging at all and are accepted at any size
    th = torch.zeros(T, H * 128, device="cuda", dtype=torch.float16)
    oh = torch.empty_like(th)
    assert L.kb_attn_self_static(P(oh), P(th), P(th), P(th), None, None, None, None, 1, T, H, 2048, 2048, 2048, 2048, kb.KB_F16, kb.KB_F16, 1e-6, None) == 0
    # a head count that would overflow the size arithmetic is refused before anything is computed from it
    assert L.kb_attn_self_static(P(oh), P(th), P(th), P(th), None, None, None, None, 1, 16, 1 << 24, 2048, 2048, 2048, 2048, kb.KB_F16, kb.KB_F16, 1e-6, None) == -3
    assert kb.check_status() == 0
