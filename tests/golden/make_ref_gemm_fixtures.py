"""Generates tests/golden/ref_gemm_fixtures.npz from the REFERENCE'S OWN fp16 GEMM kernel, run on a B200.

Needs a GPU and oracle/_ref/libkiln_ref.so (built by `python oracle/build.py --ref <kiln tree>`, which compiles the
reference's CUDA sources where they lie; nothing is copied). Run once:

    python tests/golden/make_ref_gemm_fixtures.py [out.npz]

Inputs are regenerated from seeds by the oracle's torch-compatible randn; the fixture holds the outputs of
  tc16::k_gemm16  engine/src/tcgemm16.cuh:57-175  through tc16::launch (the kernel behind linear16,
                  engine/src/kernels.cu:559-609), epilogues fp32 / fp16 / fp16 GELU / gated residual add,
  and, for LORA_CASES, of the same kernel with its second product (Args::A2 / W2 / K2, tcgemm16.cuh:26-28) fed
  as linear16 feeds it: k_lora_pack (kernels.cu:548-554) builds A_cat and B_cat from bf16 LoRA matrices, padded to
  the reference's 32-wide k tile, and t = fp16(x . A_cat^T) (kernels.cu:591-595; computed here by a torch fp16
  matmul, which like the reference's cublasGemmEx call accumulates in fp32). Keys "<case>/lora_t", "<case>/lora_b"
  (the packed operands) and "<case>/lora_<epilogue>".
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
# (GEMM case, LoRA ranks, scales): the stacked rank is padded to 32 by the reference
LORA_CASES = {"ragged": ([16], [2.0]), "two_tiles": ([8, 40], [1.5, -0.75]), "long_k": ([24, 24, 32], [1.0, 2.0, 0.5])}


def lora_inputs(case):
    """bf16-exact LoRA matrices ~ 0.05 N(0,1) — far larger than trained LoRAs, so that the second product is of the
    first product's size and an error in it cannot hide: [(A [r, in], B [out, r], scale), ...]."""
    name, M, N, K = case
    ranks, scales = LORA_CASES[name]
    seed = 3500 + 10 * GEMM_CASES.index(case)
    out = []
    for j, (r, s) in enumerate(zip(ranks, scales)):
        a = oracle.round16(oracle.randn(seed + 2 * j, max(r * K, 16))[:r * K] * np.float32(0.05), 1).reshape(r, K)
        b = oracle.round16(oracle.randn(seed + 2 * j + 1, max(N * r, 16))[:N * r] * np.float32(0.05), 1).reshape(N, r)
        out.append((a, b, s))
    return out


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
    R.kref_linear16_lora.argtypes = [vp, i, vp, vp, vp, vp, i, i, i, i, i, vp]
    R.kref_lora_pack.argtypes = [vp, i, i, vp, i, i, ctypes.c_float]
    for case in GEMM_CASES:
        name, M, N, K = case
        if name not in LORA_CASES:
            continue
        x, w, gate, resid = gemm_inputs(case)
        loras = lora_inputs(case)
        Rk = sum(a.shape[0] for a, _, _ in loras)
        R32 = (Rk + 31) // 32 * 32
        dx, dw = torch.from_numpy(x).cuda().half(), torch.from_numpy(w).cuda().half()
        dg = torch.from_numpy(gate).cuda()
        ac = torch.zeros(R32, K, device="cuda", dtype=torch.float16)
        bc = torch.zeros(N, R32, device="cuda", dtype=torch.float16)
        o = 0
        for a, b, s in loras:
            da, db = torch.from_numpy(a).cuda().bfloat16(), torch.from_numpy(b).cuda().bfloat16()
            assert R.kref_lora_pack(ac[o:].data_ptr(), K, 0, da.data_ptr(), a.shape[0], K, 1.0) == 0
            assert R.kref_lora_pack(bc.data_ptr(), R32, o, db.data_ptr(), N, a.shape[0], float(s)) == 0
            o += a.shape[0]
        torch.cuda.synchronize()
        t = (dx @ ac.t()).contiguous()
        out[f"{name}/lora_t"] = t.cpu().numpy()
        out[f"{name}/lora_b"] = bc.cpu().numpy()
        for ename, epi in EPIS.items():
            if epi in (0, 3):
                c = torch.from_numpy(resid).cuda().clone() if epi == 3 else torch.full((M, N), float("nan"), device="cuda")
            else:
                c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.float16)
            rc = R.kref_linear16_lora(c.data_ptr(), N, dx.data_ptr(), dw.data_ptr(), t.data_ptr(), bc.data_ptr(), R32, M, N, K, epi,
                                      dg.data_ptr() if epi == 3 else None)
            torch.cuda.synchronize()
            assert rc == 0, (name, ename, rc)
            out[f"{name}/lora_{ename}"] = c.cpu().numpy()
            assert not np.isnan(out[f"{name}/lora_{ename}"].astype(np.float32)).any()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_gemm_fixtures.npz"))
