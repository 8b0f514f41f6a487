#!/usr/bin/env python
"""Benchmark of the DiT attention path: one "step" = the attention calls of one DiT forward of one image.

Workload (fixed): 1024x1024 image -> 4096 tokens, 16 heads x 128, 28 blocks; per block
  * self-attention with per-head Q/K RMSNorm and 3D RoPE          (kb_attn_self,  137.44 GFLOP)
  * NAG cross-attention to a positive and a negative 512-token context with Q RMSNorm
    (kb_attn_nag: both cross-attentions and the combine in one kernel, 34.36 GFLOP)
bf16 activations in HBM, fp16 tensor-core operands, fp32 accumulation; seeded synthetic N(0,1) inputs.
FLOPs are algorithmic: 4*Tq*Tk*128*H per attention, the count the reference's own harness uses.
Every block has its own buffers (28 x 109 MB), so consecutive launches never find their inputs in L2.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --all-configs                     # one JSON line per benchmark configuration (1 GPU)
    python bench.py --case self|cross|nag|prep|linear|block|bwd [--tokens T] [--batch B] [--ctx L] [--valid V] [--dtype f16|bf16]
                    [--norm] [--reps R] [--warm W]    # one kernel family a few times: what the profiler captures run

N > 1 (under torchrun): one image per GPU, no communication on the data path ("weak" scaling); the line then also carries
a `headsplit` object: batch 1 with the 16 heads split over the N GPUs (fused push / norm exchange against local + ncclAllGather).
--impl reference: the reference has no CPU implementation of this path, so the arm times the CPU
restatement of its arithmetic (oracle/, OpenMP over all host cores) on a bounded sample of the
same workload. One JSON line goes to stdout.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

T, H, L, BLOCKS, D = 4096, 16, 512, 28, 2048
FLOP_SELF = 4.0 * T * T * 128 * H
FLOP_CROSS = 4.0 * T * L * 128 * H
FLOP_STEP = BLOCKS * (FLOP_SELF + 2 * FLOP_CROSS)
WORKLOAD = "anima-dit attention step: 1024x1024 -> 4096 tokens, 16x128 heads, 28 blocks x (self-attn + Q/K RMSNorm + 3D RoPE, NAG cross-attn to 2x512-token contexts), bf16"
METRIC = "attention TFLOP/s per DiT step (4096 tokens)"


def cosmos_rope_table(Hp, Wp):
    """cos/sin tables [Hp*Wp, 64] of the DiT's 3D RoPE for one image (engine/src/dit.cu:196-215): of the 64 rotation pairs
    the first 22 belong to the time axis (identity for an image), 21 to the row and 21 to the column of the patch, with
    frequencies 1 / (10000 * 4^(42/40))^(2j/42) in single precision."""
    import numpy as np
    dim_h, dim_t = 42, 44
    theta = np.float32(10000.0 * 4.0 ** (dim_h / (dim_h - 2)))
    hf = (np.float32(1.0) / np.power(theta, (2 * np.arange(dim_h // 2, dtype=np.float32)) / np.float32(dim_h))).astype(np.float32)
    t = np.arange(Hp * Wp)
    ang_h = (t // Wp).astype(np.float32)[:, None] * hf[None, :]
    ang_w = (t % Wp).astype(np.float32)[:, None] * hf[None, :]
    c = np.ones((Hp * Wp, 64), np.float32)
    s = np.zeros((Hp * Wp, 64), np.float32)
    c[:, dim_t // 2:dim_t // 2 + 21], s[:, dim_t // 2:dim_t // 2 + 21] = np.cos(ang_h), np.sin(ang_h)
    c[:, dim_t // 2 + 21:], s[:, dim_t // 2 + 21:] = np.cos(ang_w), np.sin(ang_w)
    return c, s


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d.get("bf16_tflops_sustained"), d.get("bf16_tflops"), d.get("hbm_gbs"), "measured"
    return 1400.0, 1590.0, 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs (read-only queries)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = self.proc.communicate()[0]
        rows, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                rows.append((float(f[0]), float(f[2])))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load = those drawing at least 60 % of the highest power seen
        pmax = max((p for _, p in rows), default=0.0)
        load = [c for c, p in rows if p >= 0.6 * pmax]
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(rows), "samples_under_load": len(load), "power_w_max": pmax}


# ------------------------------------------------------------------------------------------------ reference arm
def cpu_sample(seconds_target=12.0):
    """Times the CPU restatement of the reference arithmetic on a slice of the workload: self-attention of the
    first `rows` query tokens of one block against all 4096 keys, all 16 heads. Returns (TFLOP/s, cores, rows, secs)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import oracle
    oracle.set_threads(os.cpu_count() or 1)
    k = oracle.round16(oracle.randn(2, T * D), 1).reshape(T, D)
    v = oracle.round16(oracle.randn(3, T * D), 1).reshape(T, D)
    q = oracle.round16(oracle.randn(1, T * D), 1).reshape(T, D)
    rows = 64
    t0 = time.perf_counter()
    oracle.attention(q[:rows], k, v, H, acc64=False)
    dt = time.perf_counter() - t0
    rows = int(min(T, max(64, rows * seconds_target / max(dt, 1e-3))))
    reps, dt = 0, 0.0
    t0 = time.perf_counter()
    while dt < seconds_target and reps < 64:          # whole-block passes until ~seconds_target of CPU work
        oracle.attention(q[:rows], k, v, H, acc64=False)
        reps += 1
        dt = time.perf_counter() - t0
    return 4.0 * rows * reps * T * 128 * H / dt / 1e12, oracle.max_threads(), rows * reps, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    oracle.set_threads(os.cpu_count() or 1)       # a launcher may have exported OMP_NUM_THREADS=1: the arm uses every host core
    k = oracle.round16(oracle.randn(2, T * D), 1).reshape(T, D)
    v = oracle.round16(oracle.randn(3, T * D), 1).reshape(T, D)
    q = oracle.round16(oracle.randn(1, T * D), 1).reshape(T, D)
    # size one step's sample for ~2 s so that K + W steps end within a few minutes
    t0 = time.perf_counter()
    oracle.attention(q[:32], k, v, H, acc64=False)
    rows = int(min(T, max(32, 32 * 2.0 / max(time.perf_counter() - t0, 1e-3))))
    for _ in range(args.warmup):
        oracle.attention(q[:rows], k, v, H, acc64=False)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.attention(q[:rows], k, v, H, acc64=False)
    dt = (time.perf_counter() - t0) / args.steps
    tflops = 4.0 * rows * T * 128 * H / dt / 1e12
    sample = f"per step: self-attention of {rows} of 4096 query tokens x 4096 keys x 16 heads of one block (fp32, two-pass, OpenMP); ms_per_step extrapolates to the full 4.81 TFLOP step"
    gpu_ref = reference_kernels_on_gpu(args)
    line = {"impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": FLOP_STEP / (tflops * 1e12) * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD},
            "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": oracle.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    if gpu_ref is not None:
        line["reference_kernels_on_this_gpu"] = gpu_ref
    print(json.dumps(line), flush=True)


def reference_kernels_on_gpu(args):
    """The reference has no CPU attention: its implementation of this path IS its CUDA kernels. Where those were compiled from the
    reference tree (oracle/_ref/libkiln_ref.so) and a GPU is present, time them on this GPU in the engine's own order for one DiT
    block (engine/src/dit.cu:464-487: rmsnorm(Q), rmsnorm(K), rope_half(Q), rope_half(K), attention16; rmsnorm(Q), attention16 to
    the positive and to the negative context, k_nag) on the engine's fp32 activations, and report the step as 28 such blocks. An
    extra field beside the CPU arm, not the arm's value. Returns None when the library or a GPU is missing."""
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so")
    if not os.path.exists(ref_path):
        return None
    try:
        import ctypes
        import torch
        if not torch.cuda.is_available():
            return None
        R = ctypes.CDLL(ref_path)
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(dev)
        g = torch.Generator(device=dev)
        g.manual_seed(11)
        rn = lambda r: torch.randn(r, D, device=dev, generator=g)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        cf = ctypes.c_float
        nset = 6                                                   # rotating fp32 operand sets: 6 x 3 x 33.5 MB, more than L2
        sets = [(rn(T), rn(T), rn(T), rn(T)) for _ in range(nset)]
        ctx = [rn(L) for _ in range(4)]
        w = (torch.ones(128, device=dev) * 1.0).to(torch.bfloat16)
        cos_h, sin_h = cosmos_rope_table(64, 64)
        cos, sin = torch.from_numpy(cos_h).to(dev), torch.from_numpy(sin_h).to(dev)
        a16 = torch.empty(T, D, device=dev, dtype=torch.float16)
        n16 = torch.empty(T, D, device=dev, dtype=torch.float16)

        def block(i):
            q, k, v, q2 = sets[i % nset]
            R.kref_rmsnorm(P(q), P(q), P(w), T * H, 128, cf(1e-6))
            R.kref_rmsnorm(P(k), P(k), P(w), T * H, 128, cf(1e-6))
            R.kref_rope_half(P(q), T, H, 128, P(cos), P(sin))
            R.kref_rope_half(P(k), T, H, 128, P(cos), P(sin))
            R.kref_tfa_f16(P(a16), D, P(q), D, P(k), D, P(v), D, T, T, H, 0)
            R.kref_rmsnorm(P(q2), P(q2), P(w), T * H, 128, cf(1e-6))
            R.kref_tfa_f16(P(a16), D, P(q2), D, P(ctx[0]), D, P(ctx[1]), D, T, L, H, 0)
            R.kref_tfa_f16(P(n16), D, P(q2), D, P(ctx[2]), D, P(ctx[3]), D, T, L, H, 0)
            R.kref_nag_f16(P(a16), P(n16), T, D, cf(5.0), cf(2.5), cf(0.25))

        for i in range(3):
            block(i)
        torch.cuda.synchronize()
        nblk = 12
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(nblk):
            block(i)
        e1.record()
        torch.cuda.synchronize()
        if R.kref_sync() != 0:
            return None
        ms_block = e0.elapsed_time(e1) / nblk
        return {"kind": "reference", "ms_per_step": ms_block * BLOCKS, "value": FLOP_STEP / (ms_block * BLOCKS * 1e-3) / 1e12, "unit": "TFLOP/s",
                "what": "the reference's own CUDA kernels (tfa::k_flash, k_rmsnorm_warp, k_rope_half, k_nag<half>; engine/src/tcflash.cuh, "
                        "kernels.cu, dit.cu) compiled for sm_100a, run in the engine's order on fp32 activations: %d blocks timed with CUDA "
                        "events on the legacy stream, the step taken as %d blocks" % (nblk, BLOCKS)}
    except Exception as e:                                          # an extra: never let it take the arm down
        print(f"# reference kernels on the GPU: skipped ({type(e).__name__}: {e})", file=sys.stderr)
        return None


# ------------------------------------------------------------------------------------------------ our arm
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import kiln_b200 as kb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rc = kb.lib().kb_init()
    if rc != 0:
        raise kb.KilnError(rc, "kb_init")
    dev = torch.device("cuda", local)
    bf = torch.bfloat16
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)

    def randn(*shape):
        return torch.randn(*shape, device=dev, generator=g, dtype=torch.float32).to(bf)

    cos, sin = (torch.from_numpy(a).to(dev) for a in cosmos_rope_table(64, 64))
    blocks = []
    for _ in range(BLOCKS):
        qkv = randn(T, 3 * D)                       # Q, K, V as thirds of one buffer, like the engine's [R, 4D] scratch
        blk = {"q": qkv[:, :D], "k": qkv[:, D:2 * D], "v": qkv[:, 2 * D:], "a": torch.empty(T, D, device=dev, dtype=bf),
               "q2": randn(T, D), "a2": torch.empty(T, D, device=dev, dtype=bf),
               "kp": randn(L, D), "vp": randn(L, D), "kn": randn(L, D), "vn": randn(L, D),
               "wq": (1 + 0.02 * torch.randn(128, device=dev, generator=g)).to(bf), "wk": (1 + 0.02 * torch.randn(128, device=dev, generator=g)).to(bf),
               "wq2": (1 + 0.02 * torch.randn(128, device=dev, generator=g)).to(bf)}
        blocks.append(blk)
    ws_bytes = max(kb.workspace_bytes(T, T, H, bf, True, True), kb.workspace_bytes(T, L, H, bf, True, False, n_ctx=2))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)

    def block_calls(b):
        kb.attn_self(b["a"], b["q"], b["k"], b["v"], 1, T, H, qn_w=b["wq"], kn_w=b["wk"], rope_cos=cos, rope_sin=sin, workspace=ws)
        kb.attn_nag(b["a2"], b["q2"], b["kp"], b["vp"], L, 0, b["kn"], b["vn"], L, 0, 5.0, 2.5, 0.25, T, H, qn_w=b["wq2"], workspace=ws)

    def step():
        for b in blocks:
            block_calls(b)
    LAUNCHES_PER_STEP = BLOCKS * 4                  # (staging pre-pass + attention kernel) x (self, NAG)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    assert kb.check_status() == 0
    # One step = 112 launches of 8-130 us each: captured once into a CUDA graph and replayed, so that the timed region holds the
    # kernels and not the host's enqueue gaps between them (the library allocates nothing per call, so its calls capture as they
    # are; the cooperative launches capture too). --no-graph times the eager calls.
    eager_step, graphed = step, False
    if not args.no_graph:
        try:
            cg = torch.cuda.CUDAGraph()
            cap_stream = torch.cuda.Stream()
            cap_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cap_stream):
                # thread-local capture mode: the process group's watchdog thread may query its events meanwhile
                with torch.cuda.graph(cg, stream=cap_stream, capture_error_mode="thread_local"):
                    eager_step()
            torch.cuda.current_stream().wait_stream(cap_stream)
            cg.replay()
            torch.cuda.synchronize()
            assert kb.check_status() == 0
            step, graphed = cg.replay, True
        except Exception as e:                                   # capture not possible here: time the eager calls and say so
            print(f"# CUDA graph capture failed ({type(e).__name__}: {e}); timing eager calls", file=sys.stderr)
            torch.cuda.synchronize()
            step = eager_step
    # ---- the timed region: exactly K steps between barriers, device time by CUDA events, max over ranks; repeated
    # REPEATS times so that the line carries a spread, `value` is the median region
    REPEATS = 5
    sampler = ClockSampler(local) if rank == 0 else None
    regions = []
    for _ in range(REPEATS):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        regions.append(ms / args.steps)
    clocks = sampler.stop() if sampler else None
    assert kb.check_status() == 0
    ms_per_step = statistics.median(regions)
    value = world * FLOP_STEP / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel: per-launch CUDA events on the launch stream (library's ProfScope hooks), taken
    # over a separate pass of the same steps that lasts at least 2 s, with its own clock record. The event pairs add a
    # little to every launch, so avg_launch_us is slightly pessimistic against the launches inside `value`.
    prof_sampler = ClockSampler(local) if rank == 0 else None
    tot = {"attn": [0.0, 0], "nag": [0.0, 0], "prep": [0.0, 0]}
    t_start, prof_steps = time.perf_counter(), 0
    chunk = max(1, min(8192 // LAUNCHES_PER_STEP, 32))
    while time.perf_counter() - t_start < 2.0 or prof_steps < args.steps:
        kb.prof_enable(True)
        for _ in range(chunk):
            eager_step()                                              # the library's event pairs are recorded by eager calls only
        for key, cat in (("attn", kb.PROF_ATTENTION), ("nag", kb.PROF_NAG), ("prep", kb.PROF_NORM_ROPE)):
            ms_c, n_c = kb.prof_read(cat)
            tot[key][0] += ms_c
            tot[key][1] += n_c
        kb.prof_enable(False)
        prof_steps += chunk
    prof_clocks = prof_sampler.stop() if prof_sampler else None
    attn_ms, attn_n = tot["attn"]
    nag_ms, nag_n = tot["nag"]
    prep_ms, prep_n = tot["prep"]
    sustained, burst, hbm, src = read_peaks()
    achieved = FLOP_SELF / (attn_ms / attn_n * 1e-3) / 1e12
    # which peak the run justifies: the burst figure when the SM clock stayed near its maximum with no power cap active
    # (a short kernel at full clock), the sustained figure when the pass ran clock-limited like the seconds-long GEMM loop
    mhz = (prof_clocks or {}).get("sm_mhz")
    mhz_max = (prof_clocks or {}).get("sm_max_mhz")
    at_burst_clock = bool(mhz and mhz_max and mhz >= 0.9 * mhz_max and "sw_power_cap" not in (prof_clocks or {}).get("reasons", []))
    peak = burst if at_burst_clock else sustained
    roofline = {"bound": "tensor", "kernel": "attn_fwd_kernel<MODE_PAIR> (self-attention, 4096x4096x16 heads)", "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{src} {'bf16_tflops (burst): the pass ran at ' + str(mhz) + ' MHz, no power cap' if at_burst_clock else 'bf16_tflops_sustained: the pass ran clock- or power-limited'}",
                "frac_burst": achieved / burst, "frac_sustained": achieved / sustained,
                "traffic": None, "avg_launch_us": attn_ms / attn_n * 1e3, "launches_timed": attn_n, "pass_seconds": time.perf_counter() - t_start,
                "time_x_sm_mhz": (attn_ms / attn_n * 1e3) * mhz if mhz else None, "clocks": prof_clocks,
                "other_kernels": {"nag_attn_us": nag_ms / nag_n * 1e3, "nag_tflops": 2 * FLOP_CROSS / (nag_ms / nag_n * 1e-3) / 1e12,
                                  "staging_prepass_us": prep_ms / prep_n * 1e3}}
    traffic_file = os.path.join(ROOT, "profiles", "attn_pair_traffic.json")
    if os.path.exists(traffic_file):
        roofline["traffic"] = json.load(open(traffic_file)).get("dram_bytes_per_launch_T4096")

    # ---- the metric's other token counts (1536 = 32x48 and 3456 = 48x72 patches): the same self-attention call, kernel
    # time per launch from the same hooks (rotating input sets larger than L2)
    other_tokens = {}
    if rank == 0:
        for (hp, wp) in ((32, 48), (48, 72)):
            tt = hp * wp
            c_t, s_t = (torch.from_numpy(a).to(dev) for a in cosmos_rope_table(hp, wp))
            nset = max(2, int(200e6 // (tt * 3 * D * 2)) + 1)
            sets = [randn(tt, 3 * D) for _ in range(nset)]
            o_t = torch.empty(tt, D, device=dev, dtype=bf)
            call = lambda i: kb.attn_self(o_t, sets[i % nset][:, :D], sets[i % nset][:, D:2 * D], sets[i % nset][:, 2 * D:], 1, tt, H,
                                          qn_w=blocks[0]["wq"], kn_w=blocks[0]["wk"], rope_cos=c_t, rope_sin=s_t, workspace=ws)
            for i in range(3):
                call(i)
            kb.prof_enable(True)
            for i in range(40):
                call(i)
            k_ms, k_n = kb.prof_read(kb.PROF_ATTENTION)
            p_ms, p_n = kb.prof_read(kb.PROF_NORM_ROPE)
            kb.prof_enable(False)
            us = k_ms / k_n * 1e3
            other_tokens[str(tt)] = {"self_attn_kernel_us": us, "tflops": 4.0 * tt * tt * 128 * H / us / 1e6, "frac_burst": 4.0 * tt * tt * 128 * H / us / 1e6 / burst,
                                     "staging_prepass_us": p_ms / p_n * 1e3, "ms_per_28_blocks": 28 * (us + p_ms / p_n * 1e3) / 1e3}
            del sets
        assert kb.check_status() == 0

    # ---- end to end through the C ABI with HOST buffers: every block's inputs come from pinned host memory and
    # both attention outputs go back to the host, inside the timed region; copies overlap compute on side streams
    NSLOT = 2
    # per step the host sends what changes per step: every block's Q/K/V and cross Q. The cross-attention K/V of the two text
    # contexts stay resident on the GPU, as the engine caches them per image (engine/src/dit.cu:217-234).
    pin_in = [{k2: torch.empty_like(blocks[i][k2], device="cpu").pin_memory() for k2 in ("q2",)} for i in range(NSLOT)]
    pin_qkv = [torch.empty(T, 3 * D, dtype=bf).pin_memory() for _ in range(NSLOT)]
    pin_out = [(torch.empty(T, D, dtype=bf).pin_memory(), torch.empty(T, D, dtype=bf).pin_memory()) for _ in range(NSLOT)]
    for i in range(NSLOT):
        pin_qkv[i].copy_(torch.cat([blocks[i]["q"], blocks[i]["k"], blocks[i]["v"]], 1))
        for k2 in pin_in[i]:
            pin_in[i][k2].copy_(blocks[i][k2])
    slots = []
    for i in range(NSLOT):
        qkv = torch.empty(T, 3 * D, device=dev, dtype=bf)
        s = dict(blocks[i])
        s.update({"qkv": qkv, "q": qkv[:, :D], "k": qkv[:, D:2 * D], "v": qkv[:, 2 * D:], "a": torch.empty(T, D, device=dev, dtype=bf),
                  "a2": torch.empty(T, D, device=dev, dtype=bf)})
        s["q2"] = torch.empty_like(blocks[i]["q2"])
        slots.append(s)
    h2d_bytes = BLOCKS * (pin_qkv[0].numel() + sum(t_.numel() for t_ in pin_in[0].values())) * 2
    d2h_bytes = BLOCKS * 2 * T * D * 2
    s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    ev_in = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_done = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_out = [torch.cuda.Event() for _ in range(NSLOT)]

    def e2e_step():
        for i in range(BLOCKS):
            sl = i % NSLOT
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[sl])                      # the slot's previous compute has read its inputs
                slots[sl]["qkv"].copy_(pin_qkv[sl], non_blocking=True)
                for k2 in pin_in[sl]:
                    slots[sl][k2].copy_(pin_in[sl][k2], non_blocking=True)
                ev_in[sl].record(s_in)
            s_main.wait_event(ev_in[sl])
            s_main.wait_event(ev_out[sl])                         # the slot's previous outputs have left
            block_calls(slots[sl])
            ev_done[sl].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[sl])
                pin_out[sl][0].copy_(slots[sl]["a"], non_blocking=True)
                pin_out[sl][1].copy_(slots[sl]["a2"], non_blocking=True)
                ev_out[sl].record(s_out)
        s_main.wait_stream(s_out)

    e2e_steps = max(1, min(args.steps, 5))
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    assert kb.check_status() == 0
    e2e = {"value": world * FLOP_STEP / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
           "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
           "note": "all 28 blocks' Q/K/V and cross Q copied from pinned host memory and both outputs copied back every step (text-context K/V "
                   "resident, as the engine caches them per image); bound by the host-to-device copy path (PCIe / host memory, shared by "
                   "all ranks of a node): %.1f GB/s per GPU here" % ((h2d_bytes + d2h_bytes) / e2e_s / 1e9)}

    hs_result = None
    if world > 1 and H % world == 0:
        # configuration 5B: batch 1, the 16 heads split over the GPUs (peer stores only; no TMA multicast anywhere)
        from kiln_b200 import headsplit_bench
        hs_result = headsplit_bench.measure(T, H, L, reps=20, check=True)
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms_per_step, "regions": {"n": REPEATS, "ms_per_step": regions, "spread": (max(regions) - min(regions)) / ms_per_step},
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f16 tensor-core operands, f32 accumulate (bf16 in HBM)", "data": "synthetic",
                "config": {"workload": WORKLOAD, "images_per_gpu": 1, "flop_per_step_per_gpu": FLOP_STEP,
                           "l2": "28 distinct per-block buffer sets (3 GB) cycle through: inputs larger than L2",
                           "launch": "one CUDA graph of the step's 112 launches, replayed" if graphed else "eager calls through the C ABI"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": args.steps * LAUNCHES_PER_STEP, "roofline": roofline,
                "other_token_counts": other_tokens}
        if hs_result is not None:
            line["headsplit"] = hs_result
        if world == 1:
            tf, cores, rows, secs = cpu_sample()
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": f"self-attention of {rows} query rows (passes over one block's 4096 tokens) x 4096 keys x 16 heads, fp32 two-pass CPU restatement with OpenMP, {secs:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ per-config report
def run_all_configs(args):
    """The five benchmark configurations on one GPU: time and accuracy of this library next to the reference's own
    kernels (tfa::k_flash, k_rmsnorm_warp, k_rope_half, k_nag compiled for sm_100a into oracle/_ref/, when present) and
    the CPU oracle on sampled query rows. One JSON line per case on stdout."""
    import ctypes
    import numpy as np
    import torch
    import kiln_b200 as kb
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    assert kb.lib().kb_init() == 0
    dev = "cuda"
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so")
    R = ctypes.CDLL(ref_path) if os.path.exists(ref_path) else None
    if R is not None:
        R.kref_time_tfa_f16.restype = ctypes.c_float
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    cf = ctypes.c_float
    sustained, burst, hbm, src = read_peaks()
    NSET = 6                                                    # rotating input sets: more than L2 for every case below

    def seeded(seed, rows, kind):
        return oracle.round16(oracle.randn(seed, rows * D), kind).reshape(rows, D)

    def timed(fn, reps=20, warm=3):
        for i in range(warm):
            fn(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for i in range(reps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3                 # us

    def graph_us(fn, n=20, replays=5):
        """Per-call device time with the host out of the picture: n calls captured in one CUDA graph, replayed."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(0)                                               # attributes, status word: before the capture
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for i in range(n):
                    fn(i)
            g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            side.synchronize()
            e0.record(side)
            for _ in range(replays):
                g.replay()
            e1.record(side)
            side.synchronize()
        torch.cuda.current_stream().wait_stream(side)
        return e0.elapsed_time(e1) / (n * replays) * 1e3        # us

    def errs(out, ref):
        d = np.abs(out.astype(np.float64) - ref.astype(np.float64))
        return {"max_abs": float(d.max()), "mean_rel": float(d.sum() / np.abs(ref).sum()),
                "rel_l2": float(np.sqrt((d * d).sum() / (ref.astype(np.float64) ** 2).sum()))}

    def rows_sample(Tq, n=48):
        return np.array(sorted(set([0, 127, 128, Tq - 1] + list(np.random.RandomState(0).randint(0, Tq, n)))), np.int64)

    def emit(rec):
        print(json.dumps(rec), flush=True)

    def attention_case(name, kind, Tq, Tk_rows, Tk, npad, flop):
        dt = torch.float16 if kind == 0 else torch.bfloat16
        q, k, v = seeded(1, Tq, kind), seeded(2, Tk_rows, kind), seeded(3, Tk_rows, kind)
        sets = [tuple(torch.from_numpy(a).to(dev).to(dt).clone() for a in (q, k, v)) for _ in range(NSET)]
        out = torch.empty(Tq, D, device=dev, dtype=dt)
        ws = torch.empty(max(16, kb.workspace_bytes(Tq, Tk_rows, H, dt)), dtype=torch.uint8, device=dev)
        us = timed(lambda i: kb.attn_cross(out, *sets[i % NSET], Tq, Tk, npad, H, workspace=ws))
        # kernel-only time from the library's per-launch event pairs: short kernels are otherwise hidden behind the
        # host cost of a Python/ctypes call (argument marshalling + three tensor-map encodes), which a C++ caller does not pay
        kb.prof_enable(True)
        for i in range(10):
            kb.attn_cross(out, *sets[i % NSET], Tq, Tk, npad, H, workspace=ws)
        k_ms, k_n = kb.prof_read(kb.PROF_ATTENTION)
        s_ms, s_n = kb.prof_read(kb.PROF_NORM_ROPE)
        kb.prof_enable(False)
        g_us = graph_us(lambda i: kb.attn_cross(out, *sets[i % NSET], Tq, Tk, npad, H, workspace=ws))
        out32 = torch.empty(Tq, D, device=dev, dtype=torch.float32)
        kb.attn_cross(out32, *sets[0], Tq, Tk, npad, H, workspace=ws)
        assert kb.check_status() == 0
        rows = rows_sample(Tq)
        ref = oracle.attention(q[rows], k[:Tk], v[:Tk], H, npad)
        rec = {"case": name, "dtype": "f16" if kind == 0 else "bf16", "Tq": Tq, "Tk": Tk, "npad": npad, "ours_us": us,
               "ours_kernel_us": k_ms / k_n * 1e3, "ours_staging_us": (s_ms / s_n * 1e3) if s_n else 0.0, "ours_graph_us": g_us,
               "ours_tflops": flop / us / 1e6, "frac_of_burst_peak": flop / us / 1e6 / burst,
               "hbm_gbs": (2 * Tq + 2 * Tk) * D * 2 / us / 1e3, "err_fp32_out": errs(out32.cpu().numpy()[rows], ref),
               "err_16bit_out": errs(out.float().cpu().numpy()[rows], ref)}
        if R is not None:
            f32 = [tuple(t.float() for t in st) for st in sets[:2]]
            o16 = torch.empty(Tq, D, device=dev, dtype=torch.float16)
            rus = timed(lambda i: R.kref_tfa_f16(P(o16), D, P(f32[i % 2][0]), D, P(f32[i % 2][1]), D, P(f32[i % 2][2]), D, Tq, Tk, H, npad), reps=10)
            # both without host cost: ours replayed from a CUDA graph, the reference kernel launched back to back from C
            rloop = R.kref_time_tfa_f16(P(o16), D, P(f32[0][0]), D, P(f32[0][1]), D, P(f32[0][2]), D, Tq, Tk, H, npad, 3, 20) * 1e3
            rec.update({"reference_tfa_us": rus, "reference_tfa_tflops": flop / rus / 1e6, "speedup_vs_reference_kernel": rus / us,
                        "reference_tfa_loop_us": rloop, "speedup_device_time": rloop / g_us,
                        "reference_tfa_err": errs(o16.float().cpu().numpy()[rows], ref)})
        emit(rec)

    # config 1: self-attention fp16, 1536 tokens
    attention_case("cfg1 self 1536 fp16", 0, 1536, 1536, 1536, 0, 4.0 * 1536 * 1536 * 128 * H)
    # config 2: cross-attention fp16, L = 512 padded context: reference semantics (npad = L - valid) and -inf masking (npad = 0)
    draw = int(np.random.RandomState(2).randint(16, 513))
    for valid in (16, 26, 77, 256, 512, draw):
        attention_case(f"cfg2 cross valid={valid} zero-key padding (reference)", 0, 1536, 512, valid, 512 - valid, 4.0 * 1536 * valid * 128 * H)
        if valid < 512:
            attention_case(f"cfg2 cross valid={valid} masked padding", 0, 1536, 512, valid, 0, 4.0 * 1536 * valid * 128 * H)
    # config 3: NAG fp16, two contexts with independent seeded valid lengths, s = 5 (reference default) and s = 6 (the same formula written as z+ + 5 (z+ - z-))
    rs = np.random.RandomState(3)
    vp_len, vn_len = int(rs.randint(16, 513)), int(rs.randint(16, 513))
    Tq = 1536
    q = seeded(7, Tq, 0)
    ctx = [seeded(sd, 512, 0) for sd in (8, 9, 10, 11)]
    dq = torch.from_numpy(q).to(dev).half()
    dctx = [torch.from_numpy(a).to(dev).half() for a in ctx]
    ws = torch.empty(kb.workspace_bytes(Tq, 512, H, torch.float16, n_ctx=2), dtype=torch.uint8, device=dev)
    rows = rows_sample(Tq)
    zp = oracle.attention(q[rows], ctx[0][:vp_len], ctx[1][:vp_len], H, 512 - vp_len)
    zn = oracle.attention(q[rows], ctx[2][:vn_len], ctx[3][:vn_len], H, 512 - vn_len)
    for sc in (5.0, 6.0):
        out = torch.empty(Tq, D, device=dev, dtype=torch.float16)
        out32 = torch.empty(Tq, D, device=dev, dtype=torch.float32)
        fn = lambda o: kb.attn_nag(o, dq, dctx[0], dctx[1], vp_len, 512 - vp_len, dctx[2], dctx[3], vn_len, 512 - vn_len, sc, 2.5, 0.25, Tq, H, workspace=ws)
        us = timed(lambda i: fn(out))
        fn(out32)
        assert kb.check_status() == 0
        ref = oracle.nag(zp, zn, sc, 2.5, 0.25)
        flop = 4.0 * Tq * (vp_len + vn_len) * 128 * H
        rec = {"case": f"cfg3 NAG s={sc} valid+={vp_len} valid-={vn_len}", "dtype": "f16", "ours_us": us, "ours_tflops": flop / us / 1e6,
               "hbm_gbs": (2 * Tq + 2 * (vp_len + vn_len)) * D * 2 / us / 1e3, "err_fp32_out": errs(out32.cpu().numpy()[rows], ref),
               "err_16bit_out": errs(out.float().cpu().numpy()[rows], ref)}
        if R is not None:
            qf, cf32 = dq.float(), [t.float() for t in dctx]
            a16, n16 = torch.empty(Tq, D, device=dev, dtype=torch.float16), torch.empty(Tq, D, device=dev, dtype=torch.float16)
            def ref_nag(i):
                R.kref_tfa_f16(P(a16), D, P(qf), D, P(cf32[0]), D, P(cf32[1]), D, Tq, vp_len, H, 512 - vp_len)
                R.kref_tfa_f16(P(n16), D, P(qf), D, P(cf32[2]), D, P(cf32[3]), D, Tq, vn_len, H, 512 - vn_len)
                R.kref_nag_f16(P(a16), P(n16), Tq, D, cf(sc), cf(2.5), cf(0.25))
            rus = timed(ref_nag, reps=10)
            rec.update({"reference_unfused_us": rus, "speedup_vs_reference_kernels": rus / us, "reference_err": errs(a16.float().cpu().numpy()[rows], ref)})
        emit(rec)
    # config 4: full-step self-attention bf16, B=2, 3456 tokens (48x72), Q/K RMSNorm (1 + N(0, 0.02)) + 3D RoPE; one call, x28 for the step
    Hp, Wp, B = 48, 72, 2
    Tt = Hp * Wp
    bfk = 1
    q, k, v = seeded(1, B * Tt, bfk), seeded(2, B * Tt, bfk), seeded(3, B * Tt, bfk)
    wq = oracle.round16(1 + 0.02 * oracle.randn(7, 128), 1)
    wk = oracle.round16(1 + 0.02 * oracle.randn(8, 128), 1)
    bits = lambda w: (w.view(np.uint32) >> 16).astype(np.uint16)
    c, s_ = oracle.cosmos_rope(Hp, Wp)
    sets = [tuple(torch.from_numpy(a).to(dev).bfloat16().clone() for a in (q, k, v)) for _ in range(3)]
    dwq, dwk = torch.from_numpy(wq).to(dev).bfloat16(), torch.from_numpy(wk).to(dev).bfloat16()
    dc, ds = torch.from_numpy(c).to(dev), torch.from_numpy(s_).to(dev)
    ws = torch.empty(kb.workspace_bytes(B * Tt, B * Tt, H, torch.bfloat16, True, True), dtype=torch.uint8, device=dev)
    out = torch.empty(B * Tt, D, device=dev, dtype=torch.bfloat16)
    out32 = torch.empty(B * Tt, D, device=dev, dtype=torch.float32)
    call = lambda o, st: kb.attn_self(o, *st, B, Tt, H, qn_w=dwq, kn_w=dwk, rope_cos=dc, rope_sin=ds, workspace=ws)
    us = timed(lambda i: call(out, sets[i % 3]))
    call(out32, sets[0])
    assert kb.check_status() == 0
    flop = 4.0 * Tt * Tt * 128 * H * B
    nr = lambda x, w: np.concatenate([oracle.rope_half(oracle.rmsnorm(x[b * Tt:(b + 1) * Tt], bits(w), H), Tt, H, c, s_) for b in range(B)])
    kn = nr(k, wk)
    rows = rows_sample(Tt, 24)
    qn = nr(q, wq)
    ref = np.concatenate([oracle.attention(qn[b * Tt:(b + 1) * Tt][rows], kn[b * Tt:(b + 1) * Tt], v[b * Tt:(b + 1) * Tt], H) for b in range(B)])
    pick = np.concatenate([rows + b * Tt for b in range(B)])
    rec = {"case": "cfg4 self B=2 3456 tokens bf16 + Q/K RMSNorm + 3D RoPE (one block; a step is 28 of these)", "dtype": "bf16", "ours_us": us,
           "ours_ms_per_28_blocks": us * 28 / 1e3, "ours_tflops": flop / us / 1e6, "frac_of_sustained_peak": flop / us / 1e6 / sustained,
           "err_fp32_out": errs(out32.cpu().numpy()[pick], ref), "err_bf16_out": errs(out.float().cpu().numpy()[pick], ref)}
    if R is not None:
        qf, kf, vf = (t.float() for t in sets[0])
        wqb = torch.from_numpy(bits(wq).view(np.int16)).to(dev)
        wkb = torch.from_numpy(bits(wk).view(np.int16)).to(dev)
        o16 = torch.empty(B * Tt, D, device=dev, dtype=torch.float16)
        q2, k2 = qf.clone(), kf.clone()
        def ref_block(i):
            q2.copy_(qf); k2.copy_(kf)                               # the reference ops work in place
            R.kref_rmsnorm(P(q2), P(q2), P(wqb), B * Tt * H, 128, cf(1e-6))
            R.kref_rmsnorm(P(k2), P(k2), P(wkb), B * Tt * H, 128, cf(1e-6))
            for b in range(B):
                qb, kb_, vb, ob = q2[b * Tt:], k2[b * Tt:], vf[b * Tt:], o16[b * Tt:]
                R.kref_rope_half(P(qb), Tt, H, 128, P(dc), P(ds))
                R.kref_rope_half(P(kb_), Tt, H, 128, P(dc), P(ds))
                R.kref_tfa_f16(P(ob), D, P(qb), D, P(kb_), D, P(vb), D, Tt, Tt, H, 0)
        rus = timed(ref_block, reps=5, warm=2)
        copy_us = timed(lambda i: (q2.copy_(qf), k2.copy_(kf)), reps=5, warm=2)
        rec.update({"reference_unfused_us": rus - copy_us, "speedup_vs_reference_kernels": (rus - copy_us) / us,
                    "reference_err": errs(o16.float().cpu().numpy()[pick], ref)})
    emit(rec)
    # config 5 is the default bench run (python bench.py); other token counts of the metric:
    for T_ in (1536, 3456, 4096):
        attention_case(f"self {T_} tokens bf16 (metric token count)", 1, T_, T_, T_, 0, 4.0 * T_ * T_ * 128 * H)


# ------------------------------------------------------------------------------------------------ single cases
def run_case(a):
    """One kernel family a few times on seeded inputs, for profilers and quick timing: prints the average CUDA-event time per
    call and the algorithmic TFLOP/s (4*Tq*Tk*128*H per attention, 2*M*N*K per linear layer). `cross` takes --valid real keys of
    a --ctx padded context (zero-key padding, the engine's semantics); `block` is the self-attention half of a DiT block
    (engine/src/dit.cu:461-471): q, k, v projections, attention, output projection into the fp32 residual stream, once with
    the fused head epilogue feeding attention directly and once the way the engine orders it. Under ncu, select the kernel
    with -k regex:attn_fwd_kernel (qk_prep_kernel, gemm16_kernel) and skip the warm-up launches with -s."""
    import torch
    import kiln_b200 as kb
    assert kb.lib().kb_init() == 0
    if a.case in ("linear", "block"):
        return linear_cases(a)
    if a.case == "bwd":
        return bwd_case(a)
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
        cos = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
        sin = torch.zeros(T, 64, device="cuda").uniform_(-1, 1, generator=g)
    ws = torch.empty(max(16, kb.workspace_bytes(B * T, B * max(T, L), H, dt, True, True, n_ctx=2)), dtype=torch.uint8, device="cuda")
    kp, vp, kn, vn = rn(L, D), rn(L, D), rn(L, D), rn(L, D)
    if a.case == "self":
        fn = lambda: kb.attn_self(out, q, k, v, B, T, H, qn_w=w, kn_w=w, rope_cos=cos, rope_sin=sin, workspace=ws)
        flop = 4.0 * T * T * 128 * H * B
    elif a.case == "cross":
        V = a.valid if a.valid > 0 else L
        fn = lambda: kb.attn_cross(out[:T], q[:T], kp, vp, T, V, L - V, H, qn_w=w, workspace=ws)
        flop = 4.0 * T * V * 128 * H
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
    extra = f", {flop / us / 1e6:.1f} TFLOP/s" if flop else f", {B * T * D * (q.element_size() + 2) / us / 1e3:.0f} GB/s"
    if a.case == "cross":
        extra += f" (valid={a.valid if a.valid > 0 else L}), Q+O+K+V bytes {(2 * T + 2 * (a.valid if a.valid > 0 else L)) * D * 2 / us / 1e3:.0f} GB/s"
    print(f"case={a.case} tokens={T} batch={B} heads={H} ctx={L} dtype={a.dtype} norm={a.norm}: {us:.1f} us/call" + extra)




def _timed_us(fn, warm, reps):
    import torch
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


def bwd_case(a):
    """Attention backward (kb_attn_bwd: pre-pass if needed, forward for the statistics, D reduction, dK/dV kernel, dQ kernel) at
    --tokens queries against --tokens keys (self-attention, train.cu:344) or --ctx keys of which --valid are real (--valid > 0:
    the trainer's cross-attention call, train.cu:334). Algorithmic flops: the reference's five products, 10 * Tq * Tk * 128 * H."""
    import torch
    import kiln_b200 as kb
    T, H = a.tokens, a.heads
    D = H * 128
    cross = a.valid > 0
    Tk, npad = (a.valid, a.ctx - a.valid) if cross else (T, 0)
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[a.dtype]
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    rn = lambda r: torch.randn(r, D, device="cuda", generator=g).to(dt)
    q, k, v, do = rn(T), rn(Tk), rn(Tk), rn(T)
    dq, dk, dv = torch.empty(T, D, device="cuda"), torch.empty(Tk, D, device="cuda"), torch.empty(Tk, D, device="cuda")
    ws = torch.empty(kb.lib().kb_attn_bwd_workspace_bytes(1, T, Tk, H, kb.ops._dt(q)), dtype=torch.uint8, device="cuda")
    fn = lambda: kb.attn_bwd(dq, dk, dv, q, k, v, do, 1, T, Tk, npad, H, workspace=ws)
    us = _timed_us(fn, a.warm, a.reps)
    assert kb.check_status() == 0
    flop = 10.0 * T * Tk * 128 * H
    print(f"case=bwd tokens={T} keys={Tk} npad={npad} heads={H} dtype={a.dtype}: {us:.1f} us/call (all launches), {flop / us / 1e6:.1f} TFLOP/s")
    fwd = torch.empty(T, D, device="cuda", dtype=torch.float32)
    ws2 = torch.empty(max(16, kb.workspace_bytes(T, Tk, H, q.dtype, False, False)), dtype=torch.uint8, device="cuda")
    us_f = _timed_us(lambda: kb.attn_cross(fwd, q, k, v, T, Tk, npad, H, workspace=ws2), a.warm, a.reps)
    print(f"  forward alone on the same operands: {us_f:.1f} us/call")


def linear_cases(a):
    import torch
    import kiln_b200 as kb
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
        us = _timed_us(fn, a.warm, a.reps)
        assert kb.check_status() == 0
        print(f"case=linear M={M} N={N} K={K} epi={a.epi}: {us:.1f} us/call, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
        if a.cublas and epi == ops.EPI_F16:                 # the library GEMM on the same operands, for scale

            def mm():
                it[0] = (it[0] + 1) % nset
                torch.matmul(xs[it[0]], wts[it[0]].T, out=c)
            us = _timed_us(mm, a.warm, a.reps)
            print(f"  cuBLAS (torch.matmul) fp16: {us:.1f} us/call, {2.0 * M * N * K / us / 1e6:.1f} TFLOP/s")
        if a.lora_rank > 0:                                 # the engine's unmerged LoRA path: t = x A_cat^T, then the layer with the second product
            R = a.lora_rank
            acat, bcat = rn(R, K, 0.02), rn(N, R, 0.02)
            t = torch.empty(M, R, device="cuda", dtype=torch.float16)

            def with_lora():
                it[0] = (it[0] + 1) % nset
                ops.linear16(t, xs[it[0]], acat, ops.EPI_F16)
                ops.linear16(c, xs[it[0]], wts[it[0]], epi, lora=(t, bcat), **kw)
            us = _timed_us(with_lora, a.warm, a.reps)
            ops.linear16(t, xs[0], acat, ops.EPI_F16)
            us_down = _timed_us(lambda: ops.linear16(t, xs[0], acat, ops.EPI_F16), a.warm, a.reps)
            print(f"  with a stacked LoRA rank of {R} (down-projection launch + second product): {us:.1f} us/call; the down-projection alone {us_down:.1f} us")
        if a.ctx > 0 and a.cross_kv:                        # the cross-attention K/V producer on a [ctx, 1024] fp32 context
            ctx = torch.randn(a.ctx, 1024, device="cuda", generator=g)
            wk, wv = rn(2048, 1024, 0.03), rn(2048, 1024, 0.03)
            k16 = torch.empty(a.ctx, 2048, device="cuda", dtype=torch.float16)
            v16 = torch.empty_like(k16)
            wsx = torch.empty(a.ctx * 1024 * 2, dtype=torch.uint8, device="cuda")
            us = _timed_us(lambda: ops.cross_kv(k16, v16, ctx, wk, wv, kn_w=hw, workspace=wsx), a.warm, a.reps)
            print(f"  cross-attention K/V producer, {a.ctx} x 1024 fp32 context -> fp16 K (normalised), V [{a.ctx}, 2048]: {us:.1f} us/call (two launches)")
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
        us = _timed_us(fn, a.warm, a.reps)
        assert kb.check_status() == 0
        print(f"case=block tokens={T} heads={H} [{name}]: {us:.1f} us/block-half, {flop / us / 1e6:.1f} TFLOP/s")




def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--all-configs", action="store_true", help="one JSON line per benchmark configuration (1 GPU) instead of the benchmark line")
    ap.add_argument("--case", default=None, choices=["self", "cross", "nag", "prep", "linear", "block", "bwd"], help="run one kernel family a few times (for profilers)")
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--epi", default="f16", choices=["f32", "f16", "gelu16", "resid", "heads16"])
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--valid", type=int, default=0, help="cross: real keys of the padded context (0 = all)")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16", "f32"])
    ap.add_argument("--norm", action="store_true", help="Q/K RMSNorm (+ RoPE for self) through the staging pre-pass")
    ap.add_argument("--no-graph", action="store_true", help="time eager calls instead of a CUDA graph of the step")
    ap.add_argument("--cublas", action="store_true", help="linear: also time torch.matmul on the same operands")
    ap.add_argument("--lora-rank", type=int, default=0, help="linear: also time the layer with a stacked LoRA of this rank")
    ap.add_argument("--cross-kv", action="store_true", help="linear: also time kb_cross_kv on a [--ctx, 1024] context")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warm", type=int, default=2)
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.all_configs:
        run_all_configs(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
