"""One rank of the 2+-GPU head-split parity check, started under torchrun by tests/test_headsplit.py:
head-split self-attention and head-split NAG (fused Q RMSNorm, norm exchange inside the kernel) against the CPU oracle
on sampled rows, twice in a row (buffer and exchange-area reuse), tolerance max-abs 2e-3 / mean-rel 1e-3 plus the bf16
storage step of the output."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")):
    sys.path.insert(0, p)
import oracle  # noqa: E402
from kiln_b200 import headsplit, ops  # noqa: E402
from util_gpu import assert_close_bf16_storage, sample_rows, seeded  # noqa: E402


def main():
    T, H, L = int(sys.argv[1]), 16, 512
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    D = H * 128
    q, k, v, q2 = (seeded(s, T, D, "bf16") for s in (61, 62, 63, 64))
    kp, vp, kn, vn = (seeded(s, L, D, "bf16") for s in (65, 66, 67, 68))
    wq = oracle.round16(1 + 0.02 * oracle.randn(69, 128), 1)
    bits = (wq.view(np.uint32) >> 16).astype(np.uint16)
    hs = headsplit.HeadSplit(T, H, torch.bfloat16)
    cols = slice(hs.col0, hs.col0 + hs.hl * 128)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a[:, cols])).cuda().bfloat16()
    ws = torch.empty(max(ops.workspace_bytes(T, T, hs.hl, torch.bfloat16), ops.workspace_bytes(T, L, hs.hl, torch.bfloat16, True, False, n_ctx=2)),
                     dtype=torch.uint8, device="cuda")
    rows = sample_rows(T, 24, seed=dist.get_rank())
    ref_self = oracle.attention(q[rows], k, v, H)
    qn = oracle.rmsnorm(q2, bits, H)[rows]
    Tp, Tn = 333, 45
    zp = oracle.attention(qn, kp[:Tp], vp[:Tp], H, L - Tp)
    zn = oracle.attention(qn, kn[:Tn], vn[:Tn], H, L - Tn)
    ref_nag = oracle.nag(zp, zn, 5.0, 2.5, 0.25)
    dw = torch.from_numpy(wq).cuda().bfloat16()
    for rep in range(2):
        out = hs.attention(1, d(q), d(k), d(v), T, workspace=ws).float().cpu().numpy()
        hs.release(1)
        assert ops.check_status() == 0
        assert_close_bf16_storage(out[rows], ref_self, f"head-split self-attention, call {rep}")
        out = hs.nag(d(q2), d(kp), d(vp), Tp, L - Tp, d(kn), d(vn), Tn, L - Tn, 5.0, 2.5, 0.25, qn_w=dw, workspace=ws).float().cpu().numpy()
        hs.release(0)
        assert ops.check_status() == 0
        assert_close_bf16_storage(out[rows], ref_nag, f"head-split NAG, call {rep}")
    hs.close()
    dist.destroy_process_group()
    print("HEADSPLIT PARITY OK", flush=True)


if __name__ == "__main__":
    main()
