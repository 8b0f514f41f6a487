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
from util_gpu import assert_close, assert_close_bf16_storage, dev, seeded

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
    gp = [torch.zeros(T, hl * 128) for _ in range(world)]
    gn = [torch.zeros(T, hl * 128) for _ in range(world)]
    dist.all_gather(gp, torch.from_numpy(zp))
    dist.all_gather(gn, torch.from_numpy(zn))
    zp_full, zn_full = torch.cat(gp, 1).numpy(), torch.cat(gn, 1).numpy()     # rank r's block lands at columns r*hl*128
    blended = orc.nag(zp_full, zn_full, 5.0, 2.5, 0.25)
    ref_p = orc.attention(full["q"], full["kp"], full["vp"], H, 7)
    ref = orc.nag(ref_p, orc.attention(full["q"], full["kn"], full["vn"], H, 3), 5.0, 2.5, 0.25)
    out[rank] = (float(np.abs(zp_full - ref_p).max()), float(np.abs(blended - ref).max()))
    dist.destroy_process_group()


def test_headsplit_gather_then_blend_gloo_cpu():
    """Two CPU ranks: per-rank heads, all-gather of column blocks, NAG blend on the gathered full rows == unsplit result."""
    from kiln_b200.headsplit import plan
    assert plan(16, 8, 3) == (2, 6, 768) and plan(16, 1, 0) == (16, 0, 0)
    with pytest.raises(ValueError):
        plan(16, 3, 0)
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_gloo_rank, args=(world, 29533, out), nprocs=world, join=True)
        for r in range(world):
            assert out[r][0] < 1e-6 and out[r][1] < 1e-6


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
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_headsplit_two_gpus_torchrun(built_lib):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", "-m", "kiln_b200.headsplit_bench", "--tokens", "1536", "--reps", "3", "--check"]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
