"""Generates tests/golden/ref_gemm_fixtures.npz from the REFERENCE'S OWN fp16 GEMM kernel, run on a B200.

Needs a GPU and oracle/_ref/libkiln_ref.so (built by `python oracle/build.py --ref <kiln tree>`, which compiles the
reference's CUDA sources where they lie; nothing is copied). Run once:

    python tests/golden/make_ref_gemm_fixtures.py [out.npz]

Inputs are regenerated from seeds by the oracle's torch-compatible randn; the fixture holds the outputs of
  tc16::k_gemm16  engine/src/tcgemm16.cuh:57-175  through tc16::launch (the kernel behind linear16,
                  engine/src/kernels.cu:559-609), epilogues fp32 / fp16 / fp16 GELU / gated residual add.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

# (name, M, N, K): small so the fixture stays ~200 KB; K a multiple of 64, N of 128, M ragged
GEMM_CASES = [("ragged", 100, 128, 192), ("long_k", 40, 128, 2048), ("two_tiles", 130, 256, 64)]
EPIS = {"f32": 0, "f16": 1, "gelu16": 2, "resid": 3}


def gemm_inputs(case):
    """Activations ~ N(0,1) and weights ~ 0.03 N(0,1) (the scale of a 2048-wide linear layer), fp16-exact;
    the gate and the residual stream (EPI_RESID) ~ N(0,1) fp32."""
    name, M, N, K = case
    seed = 3000 + 10 * GEMM_CASES.index(case)
    x = oracle.round16(oracle.randn(seed, M * K), 0).reshape(M, K)
    w = oracle.round16(oracle.randn(seed + 1, N * K) * np.float32(0.03), 0).reshape(N, K)
    gate = oracle.randn(seed + 2, max(N, 16))[:N].copy()
    resid = oracle.randn(seed + 3, M * N).reshape(M, N)
    return x, w, gate, resid


def main(out_path):
    R = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so"))
    vp, i = ctypes.c_void_p, ctypes.c_int
    R.kref_linear16.argtypes = [vp, i, vp, vp, i, i, i, i, vp]
    out = {}
    for case in GEMM_CASES:
        name, M, N, K = case
        x, w, gate, resid = gemm_inputs(case)
        dx, dw = torch.from_numpy(x).cuda().half(), torch.from_numpy(w).cuda().half()
        dg = torch.from_numpy(gate).cuda()
        for ename, epi in EPIS.items():
            if epi in (0, 3):
                c = torch.from_numpy(resid).cuda().clone() if epi == 3 else torch.full((M, N), float("nan"), device="cuda")
            else:
                c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
            rc = R.kref_linear16(c.data_ptr(), N, dx.data_ptr(), dw.data_ptr(), M, N, K, epi, dg.data_ptr() if epi == 3 else None)
            torch.cuda.synchronize()
            assert rc == 0, (name, ename, rc)
            out[f"{name}/{ename}"] = c.cpu().numpy()
            assert not np.isnan(out[f"{name}/{ename}"].astype(np.float32)).any()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_gemm_fixtures.npz"))
