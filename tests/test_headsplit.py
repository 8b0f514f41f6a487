"""Head split at batch 1: the sharding arithmetic and gather-then-blend semantics on CPU (gloo, 2 ranks),
the multi-peer epilogue on one GPU (two "peer" buffers on the same device), the stand-alone NAG combine
against the reference's k_nag golden outputs, and — where two GPUs are visible — the real thing under torchrun."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from golden_inputs import gen
from util_gpu import assert_close, assert_close_bf16_storage, dev, seeded  # noqa: F401

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gloo_rank(rank, world, port, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle as orc
    from kiln_b200.headsplit import plan
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    H, T, L = 4, 40, 30
    full = {n: orc.randn(s, r * H * 128).reshape(r, H * 128) for n, s, r in (("q", 1, T), ("kp", 2, L), ("vp", 3, L), ("kn", 4, L), ("vn", 5, L))}
    hl, h0, col0 = plan(H, world, rank)
    sl = slice(col0, col0 + hl * 128)
    zp = orc.attention(full["q"][:, sl], full["kp"][:, sl], full["vp"][:, sl], hl, 7)
    zn = orc.attention(full["q"][:, sl], full["kn"][:, sl], full["vn"][:, sl], hl, 3)
    # what the kernels exchange: per token the L1 norms of Z+ and of g = s Z+ - (s - 1) Z- over the LOCAL heads,
    # summed over ranks (2 floats per token and rank); the blend then runs on the local columns only
    s_, tau, alpha = 5.0, 2.5, 0.25
    g = s_ * zp - (s_ - 1.0) * zn
    norms = torch.from_numpy(np.stack([np.abs(zp).sum(1), np.abs(g).sum(1)]).astype(np.float64))
    dist.all_reduce(norms)
    ratio = norms[1].numpy() / np.maximum(norms[0].numpy(), 1e-12)
    kk = np.where(ratio > tau, tau / ratio, 1.0)[:, None]
    mine = (alpha * kk * g + (1 - alpha) * zp).astype(np.float32)
    gp = [torch.zeros(T, hl * 128) for _ in range(world)]
    gb = [torch.zeros(T, hl * 128) for _ in range(world)]
    dist.all_gather(gp, torch.from_numpy(zp))
    dist.all_gather(gb, torch.from_numpy(mine))
    zp_full, blended = torch.cat(gp, 1).numpy(), torch.cat(gb, 1).numpy()      # rank r's block lands at columns r*hl*128
    ref_p = orc.attention(full["q"], full["kp"], full["vp"], H, 7)
    ref = orc.nag(ref_p, orc.attention(full["q"], full["kn"], full["vn"], H, 3), s_, tau, alpha)
    out[rank] = (float(np.abs(zp_full - ref_p).max()), float(np.abs(blended - ref).max()))
    dist.destroy_process_group()


def test_headsplit_norm_exchange_then_local_blend_gloo_cpu():
    """Two CPU ranks: per-rank heads, the per-token norms summed over ranks, NAG blend on the local columns, all-gather of the
    blended column blocks == unsplit result."""
    from kiln_b200.headsplit import plan
    assert plan(16, 8, 3) == (2, 6, 768) and plan(16, 1, 0) == (16, 0, 0)
    with pytest.raises(ValueError):
        plan(16, 3, 0)
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_gloo_rank, args=(world, 29533, out), nprocs=world, join=True)
        for r in range(world):
            assert out[r][0] < 1e-6 and out[r][1] < 2e-6


@pytest.mark.gpu
def test_nag_combine_vs_reference_golden(built_lib, golden):
    import kiln_b200 as kb
    zp, zn = gen.nag_inputs()
    for i, (s, tau, alpha) in enumerate(gen.NAG_PARAMS):
        a = dev(zp)
        kb.nag_combine(a, dev(zn), s, tau, alpha)
        np.testing.assert_allclose(a.cpu().numpy(), golden[f"nag/f32_{i}"], rtol=2e-5, atol=1e-6)       # k_nag<float>
        a16 = dev(zp).half()
        kb.nag_combine(a16, dev(zn).half(), s, tau, alpha)
        g16 = golden[f"nag/f16_{i}"].astype(np.float32)                                                  # k_nag<__half>
        o16 = a16.float().cpu().numpy()
        assert np.mean(o16 != g16) < 0.01 and np.abs(o16 - g16).max() <= 2e-3
    # strided rows (a slice of a wider buffer) and bf16
    big = dev(seeded(3, 50, 4096, "bf16"), "bf16")
    a, n = big[:, :2048], big[:, 2048:]
    ref = oracle.nag(a.float().cpu().numpy(), n.float().cpu().numpy(), 5.0, 2.5, 0.25)
    kb.nag_combine(a, n, 5.0, 2.5, 0.25)
    assert_close_bf16_storage(a.float().cpu().numpy(), ref, "strided bf16 combine")
    assert kb.check_status() == 0


@pytest.mark.gpu
def test_push_epilogue_two_peer_buffers_on_one_gpu(built_lib):
    """The head-split epilogue with both "peers" on this GPU: local heads 4..7 of 8 land at columns 512.. of both
    buffers, other columns stay untouched, both counters reach the expected arrivals and the bounded wait passes."""
    import kiln_b200 as kb
    L = kb.lib()
    T, H, hl, col0, kind = 300, 8, 4, 512, "f16"
    D = H * 128
    q, k, v = (seeded(s, T, hl * 128, kind) for s in (1, 2, 3))
    bufs = [torch.full((T, D), 9.0, device="cuda", dtype=torch.float16) for _ in range(2)]
    ctrs = torch.zeros(2, 32, dtype=torch.int64, device="cuda")                     # one 64-bit counter per peer, apart
    kb.attn_push([b.data_ptr() for b in bufs], [ctrs[i].data_ptr() for i in range(2)], col0, dev(q, kind), dev(k, kind), dev(v, kind),
                 1, T, T, 0, hl, D, kb.KB_F16)
    assert L.kb_push_arrivals_per_call(1, T, hl, 2) == 2 * hl * 3      # what a counter sees when BOTH ranks of a pair have pushed
    expect = hl * 3                                                     # here only one producer runs: its 12 tiles
    kb.wait_arrivals(ctrs[0].data_ptr(), expect)
    kb.wait_arrivals(ctrs[1].data_ptr(), expect)
    assert kb.check_status() == 0
    assert ctrs[0, 0].item() == expect and ctrs[1, 0].item() == expect
    ref = oracle.attention(q, k, v, hl)
    for b in bufs:
        assert_close(b[:, col0:col0 + hl * 128].float().cpu().numpy(), ref, "pushed tile")
        assert torch.all(b[:, :col0] == 9.0) and torch.all(b[:, col0 + hl * 128:] == 9.0)
    assert torch.equal(bufs[0], bufs[1])


@pytest.mark.gpu
def test_bounded_wait_runs_out_and_is_reported(built_lib):
    """Failure detection without a GPU fault: a wait for arrivals that never come gives up at its limit (2 s), the kernel
    returns normally with the time-out bit in the device status word, kb_status reports KB_ERR_TIMEOUT once and clears it,
    and the context stays usable (the next attention call is correct)."""
    import time
    import kiln_b200 as kb
    from kiln_b200.ops import KilnError
    assert kb.lib().kb_init() == 0
    assert kb.check_status() == 0
    ctr = torch.zeros(1, dtype=torch.int64, device="cuda")             # nothing will ever bump it
    t0 = time.time()
    kb.wait_arrivals(ctr.data_ptr(), 1)
    with pytest.raises(KilnError) as ei:
        kb.check_status()
    assert ei.value.code == -7                                           # KB_ERR_TIMEOUT
    assert 1.5 < time.time() - t0 < 10.0, "the wait must end at its own limit"
    assert kb.check_status() == 0                                        # read and cleared
    T, H = 200, 2
    q, k, v = (oracle.round16(oracle.randn(900 + i, T * H * 128), 0).reshape(T, H * 128) for i in range(3))
    out = torch.empty(T, H * 128, device="cuda", dtype=torch.float32)
    kb.attn_self(out, dev(q, "f16"), dev(k, "f16"), dev(v, "f16"), 1, T, H)
    assert kb.check_status() == 0
    assert_close(out.cpu().numpy(), oracle.attention(q, k, v, H), "attention after a reported time-out")


@pytest.mark.gpu
def test_nag_push_epilogue_and_exchange_counters_on_one_gpu(built_lib):
    """kb_attn_nag_push with both "peers" on this GPU and all heads local: the norms and the counters go to both exchange
    areas, the blended tiles to both output buffers; results equal kb_attn_nag; a second call (epoch 2) reuses the areas
    without clearing anything (the counters only grow)."""
    import kiln_b200 as kb
    L = kb.lib()
    Tq, H, Lc, Tp, Tn, kind = 300, 4, 512, 77, 26, "bf16"
    D = H * 128
    q = seeded(7, Tq, D, kind)
    kp, vp, kn, vn = (seeded(s, Lc, D, kind) for s in (8, 9, 10, 11))
    wq = oracle.round16(1 + 0.02 * oracle.randn(12, 128), 1)
    dw = dev(wq).bfloat16()
    dq, dkp, dvp, dkn, dvn = (dev(a, kind) for a in (q, kp, vp, kn, vn))
    ws = torch.empty(kb.workspace_bytes(Tq, Lc, H, torch.bfloat16, True, False, n_ctx=2), dtype=torch.uint8, device="cuda")
    ref = torch.empty(Tq, D, device="cuda", dtype=torch.bfloat16)
    kb.attn_nag(ref, dq, dkp, dvp, Tp, Lc - Tp, dkn, dvn, Tn, Lc - Tn, 5.0, 2.5, 0.25, Tq, H, qn_w=dw, workspace=ws)
    xb = L.kb_nag_exchange_bytes(Tq, H)
    n_qt = (Tq + 127) // 128
    flag_off = L.kb_nag_exchange_counter_offset(Tq, H)
    xch = [torch.zeros(xb, dtype=torch.uint8, device="cuda") for _ in range(2)]
    bufs = [torch.full((Tq, 2 * D), 9.0, device="cuda", dtype=torch.bfloat16) for _ in range(2)]      # the heads land at columns D..2D
    ctrs = torch.zeros(2, 32, dtype=torch.int64, device="cuda")
    for epoch in (1, 2):
        for b in bufs:
            b[:, D:] = 9.0
        kb.attn_nag_push([b.data_ptr() for b in bufs], [ctrs[i].data_ptr() for i in range(2)], [x.data_ptr() for x in xch],
                         [x.data_ptr() + flag_off for x in xch], 0, D, 0, H, epoch, dq, dkp, dvp, Tp, Lc - Tp, dkn, dvn, Tn, Lc - Tn,
                         5.0, 2.5, 0.25, Tq, H, 2 * D, kb.KB_BF16, qn_w=dw, workspace=ws)
        assert kb.check_status() == 0
        for i, b in enumerate(bufs):
            assert torch.equal(b[:, D:], ref), f"epoch {epoch} buffer {i}"
            assert torch.all(b[:, :D] == 9.0)
            flags = xch[i][flag_off:flag_off + 4 * n_qt].view(torch.int32)
            assert torch.all(flags == epoch * H)
            assert ctrs[i, 0].item() == epoch * H * n_qt
    out = ref.float().cpu().numpy()
    qn = oracle.rmsnorm(q, (wq.view(np.uint32) >> 16).astype(np.uint16), H)
    zp = oracle.attention(qn, kp[:Tp], vp[:Tp], H, Lc - Tp)
    zn = oracle.attention(qn, kn[:Tn], vn[:Tn], H, Lc - Tn)
    assert_close_bf16_storage(out, oracle.nag(zp, zn, 5.0, 2.5, 0.25), "NAG with fused Q norm, bf16 out")


def _one_rank_reuse(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import kiln_b200 as kb
    from kiln_b200 import headsplit
    from kiln_b200.ops import KilnError
    torch.cuda.set_device(0)
    T, H = 300, 4
    hs = headsplit.HeadSplit(T, H, torch.float16)
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    q, k, v = (torch.randn(T, H * 128, device="cuda", generator=g).half() for _ in range(3))
    a = hs.attention(0, q, k, v, T).clone()
    hs.release(0)
    b = hs.attention(0, q, k, v, T).clone()                   # the buffer was released: the push goes ahead
    assert kb.check_status() == 0 and torch.equal(a, b)
    hs.attention(0, q, k, v, T, wait=False)                   # NOT released: the bounded wait in front of this push runs out
    try:
        kb.check_status()
        out["timeout"] = False
    except KilnError as e:
        out["timeout"] = e.code == -7
    hs.release(0); hs.release(0)
    torch.cuda.synchronize()
    out["ok"] = True
    dist.destroy_process_group()


@pytest.mark.gpu
def test_buffer_reuse_protocol_one_rank(built_lib):
    """The release / wait hand-shake that guards a gathered buffer against the next push, on one GPU with a one-rank
    group: a released buffer is pushed into again at once; a push into a buffer nobody released waits, gives up at its
    limit and is reported as KB_ERR_TIMEOUT (no hang, the context stays usable)."""
    from kiln_b200.headsplit import reuse_target
    assert reuse_target(3, 8) == 24
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_one_rank_reuse, args=(1, 29541, out), nprocs=1, join=True)
        assert out.get("ok") and out.get("timeout")


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_headsplit_two_gpus_torchrun(built_lib):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    launch = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1"]
    # parity against the CPU oracle (sampled rows, two calls in a row), then timing + agreement with the single-GPU kernels
    r = subprocess.run(launch + ["--master-port", "29517", os.path.join(ROOT, "tests", "headsplit_rank.py"), "1536"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "HEADSPLIT PARITY OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
    r = subprocess.run(launch + ["--master-port", "29518", "-m", "kiln_b200.headsplit_bench", "--tokens", "1536", "--reps", "3", "--check"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
