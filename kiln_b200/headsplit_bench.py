"""Head-split attention at batch 1 across the GPUs of one node: timing and a self-consistency check.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 --master-port 29511 \
        -m kiln_b200.headsplit_bench [--tokens 4096] [--heads 16] [--ctx 512] [--reps 20] [--check]

Per rank: self-attention of its H/G heads with the output pushed to every rank (fused path) against local
attention + ncclAllGather (baseline), and head-split NAG (norm exchange inside the kernel, final tiles pushed).
Times are CUDA-event times on the device, max over ranks. --check compares every rank's gathered result with the
single-GPU kernels of this library run on all heads on that rank (parity against the CPU oracle lives in tests/).
`measure()` is what bench.py calls for its `headsplit` object. Prints one JSON line on rank 0.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from . import headsplit, ops


def measure(T=4096, H=16, L=512, reps=20, check=True, seed=7):
    """Runs on every rank of an initialised NCCL process group (current device set); returns the result dict."""
    G = dist.get_world_size()
    D = H * 128
    bf = torch.bfloat16
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)                                      # every rank draws the same full tensors, then slices its heads
    full = {n: torch.randn(r, D, device="cuda", generator=g).to(bf) for n, r in
            (("q", T), ("k", T), ("v", T), ("q2", T), ("kp", L), ("vp", L), ("kn", L), ("vn", L))}
    wq = (1 + 0.02 * torch.randn(128, device="cuda", generator=g)).to(bf)
    hs = headsplit.HeadSplit(T, H, bf)
    cols = slice(hs.col0, hs.col0 + hs.hl * 128)
    mine = {n: t[:, cols].contiguous() for n, t in full.items()}
    ws = torch.empty(max(16, ops.workspace_bytes(T, max(T, L), hs.hl, bf, True, False), ops.workspace_bytes(T, L, hs.hl, bf, True, False, n_ctx=2)),
                     dtype=torch.uint8, device="cuda")
    result = {"n_gpus": G, "tokens": T, "heads": H, "heads_per_gpu": hs.hl, "ctx": L}

    def nag_call():
        out = hs.nag(mine["q2"], mine["kp"], mine["vp"], L, 0, mine["kn"], mine["vn"], L, 0, 5.0, 2.5, 0.25, qn_w=wq, workspace=ws)
        hs.release(0)
        return out

    def self_call():
        out = hs.attention(1, mine["q"], mine["k"], mine["v"], T, workspace=ws)
        hs.release(1)
        return out

    if check:
        # the same work with all heads on this GPU, by the single-GPU entry points
        ws1 = torch.empty(max(ops.workspace_bytes(T, T, H, bf), ops.workspace_bytes(T, L, H, bf, True, False, n_ctx=2)), dtype=torch.uint8, device="cuda")
        ref_self = torch.empty(T, D, device="cuda", dtype=bf)
        ops.attn_self(ref_self, full["q"], full["k"], full["v"], 1, T, H, workspace=ws1)
        ref_nag = torch.empty(T, D, device="cuda", dtype=bf)
        ops.attn_nag(ref_nag, full["q2"], full["kp"], full["vp"], L, 0, full["kn"], full["vn"], L, 0, 5.0, 2.5, 0.25, T, H, qn_w=wq, workspace=ws1)
        e = []
        for _ in range(2):                                   # twice: the second call reuses buffers and the exchange area
            e.append((self_call().float() - ref_self.float()).abs().max().item())
            e.append((nag_call().float() - ref_nag.float()).abs().max().item())
        base = headsplit.nccl_all_gather_attention(mine["q"], mine["k"], mine["v"], T, T, hs.hl, G, workspace=ws)
        e.append((base.permute(1, 0, 2).reshape(T, D).float() - ref_self.float()).abs().max().item())
        assert ops.check_status() == 0
        errs = torch.tensor(e, device="cuda")
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        result["max_abs_vs_single_gpu"] = {"self_fused": max(errs[0].item(), errs[2].item()), "nag_fused": max(errs[1].item(), errs[3].item()),
                                           "self_nccl": errs[4].item()}
        # same arithmetic per head (the split of key blocks over SMs may differ: fp16 weights against another running maximum);
        # bf16 storage of O(0.1) values allows one 2^-9 step
        assert max(e) < 2e-3, result

    def timed(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    flop_self = 4.0 * T * T * 128 * H
    us = timed(self_call)
    result["self_fused_us"] = us
    result["self_fused_tflops"] = flop_self / us / 1e6
    us = timed(lambda: headsplit.nccl_all_gather_attention(mine["q"], mine["k"], mine["v"], T, T, hs.hl, G, workspace=ws))
    result["self_nccl_us"] = us
    local_out = torch.empty(T, hs.hl * 128, device="cuda", dtype=bf)
    us = timed(lambda: ops.attn_cross(local_out, mine["q"], mine["k"], mine["v"], T, T, 0, hs.hl, workspace=ws))
    result["self_local_only_us"] = us
    result["nag_fused_us"] = timed(nag_call)
    # bytes each rank pushes to remote GPUs per call (final tiles only; NAG adds 16 bytes per token and local head)
    result["remote_bytes_per_rank"] = (G - 1) * T * hs.hl * 128 * 2
    result["push_gbs_per_rank"] = result["remote_bytes_per_rank"] / max(result["self_fused_us"] - result["self_local_only_us"], 1e-3) / 1e3
    result["nvlink_peak_gbs_per_direction"] = 900
    assert ops.check_status() == 0
    hs.close()
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=512)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--check", action="store_true")
    a = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    result = measure(a.tokens, a.heads, a.ctx, a.reps, a.check)
    if dist.get_rank() == 0:
        print(json.dumps(result), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
