"""Generates tests/golden/ref_fixtures.npz from the REFERENCE'S OWN KERNELS, run on a B200.

Needs a GPU and oracle/_ref/libkiln_ref.so (built by `python oracle/build.py --ref <kiln tree>`,
which compiles the reference's CUDA sources where they lie; nothing is copied). Run once:

    python tests/golden/make_ref_fixtures.py [out.npz]

Inputs are regenerated from seeds by the oracle's torch-compatible randn, so the fixture stores only
the seeds' SHA-256 (to detect a libm that rounds differently) and the reference kernels' outputs:
  ref_attn        bench/tfa_test.cu:11-33            fp32 attention incl. analytic npad
  tfa::k_flash    engine/src/tcflash.cuh:20-157      tensor-core attention, fp16 output (what attention16 returns)
  k_rmsnorm_warp  engine/src/kernels.cu:656-666
  k_rope_half     engine/src/kernels.cu:759-772      with the tables of cosmos_rope, engine/src/dit.cu:196-215
  k_nag<float>, k_nag<__half>  engine/src/dit.cu:295-324
"""
import ctypes
import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

# (name, Tq, Tk, npad, H): shapes kept small so the fixture stays a few hundred KB
ATTN_CASES = [("self_ragged", 96, 96, 0, 2), ("cross_pad", 70, 26, 486, 2), ("cross_ragged", 64, 130, 0, 2),
              ("cross_pad_multi", 40, 200, 312, 2)]
NAG_T, NAG_DIM = 6, 2048
NAG_PARAMS = [(5.0, 2.5, 0.25), (6.0, 2.5, 0.25), (3.0, 1.0, 0.5)]


def attn_inputs(case):
    """fp32 inputs with the reference harness's distribution (bench/tfa_test.cu:37-43): Q, K ~ 1.5 N(0,1), V ~ N(0,1),
    rounded through fp16 so that fp32-input and 16-bit-input kernels see identical values."""
    name, Tq, Tk, npad, H = case
    seed = 1000 + 10 * ATTN_CASES.index(case)
    q = oracle.round16(oracle.randn(seed, Tq * H * 128) * 1.5, 0).reshape(Tq, H * 128)
    k = oracle.round16(oracle.randn(seed + 1, Tk * H * 128) * 1.5, 0).reshape(Tk, H * 128)
    v = oracle.round16(oracle.randn(seed + 2, Tk * H * 128), 0).reshape(Tk, H * 128)
    return q, k, v


def norm_inputs():
    rows, H = 48, 2
    x = oracle.randn(2000, rows * H * 128).reshape(rows, H * 128)
    w = oracle.round16(1.0 + 0.02 * oracle.randn(2001, 128), 1)          # bf16-exact weights, as the engine stores them
    w_bits = (w.view(np.uint32) >> 16).astype(np.uint16)
    return x, w_bits, H


def rope_inputs():
    Hp, Wp, H = 6, 8, 2
    x = oracle.randn(2100, Hp * Wp * H * 128).reshape(Hp * Wp, H * 128)
    return x, Hp, Wp, H


def nag_inputs():
    zp = oracle.randn(2200, NAG_T * NAG_DIM).reshape(NAG_T, NAG_DIM) * 0.3
    zn = oracle.randn(2201, NAG_T * NAG_DIM).reshape(NAG_T, NAG_DIM) * 0.3
    zp[3] *= 0.01                                                          # a row where the clamp certainly triggers
    return zp.astype(np.float32), zn.astype(np.float32)


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main(out_path):
    R = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so"))
    dev = "cuda"
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    f = ctypes.c_float
    fx = {}
    for case in ATTN_CASES:
        name, Tq, Tk, npad, H = case
        q, k, v = attn_inputs(case)
        fx[f"{name}/digest"] = np.array(digest(q, k, v))
        dq, dk, dv = (torch.from_numpy(a).to(dev) for a in (q, k, v))
        ld = H * 128
        o = torch.zeros(Tq, ld, device=dev)
        assert R.kref_ref_attn(P(o), P(dq), P(dk), P(dv), Tq, Tk, H, ld, npad) == 0
        torch.cuda.synchronize()
        fx[f"{name}/ref_attn"] = o.cpu().numpy()
        o3 = torch.zeros(Tq, ld, device=dev, dtype=torch.float16)
        assert R.kref_tfa_f16(P(o3), ld, P(dq), ld, P(dk), ld, P(dv), ld, Tq, Tk, H, npad) == 0
        torch.cuda.synchronize()
        fx[f"{name}/tfa_f16"] = o3.cpu().numpy()
    x, w_bits, H = norm_inputs()
    fx["rmsnorm/digest"] = np.array(digest(x, w_bits))
    dx = torch.from_numpy(x).to(dev)
    dw = torch.from_numpy(w_bits.view(np.int16)).to(dev)
    y = torch.zeros_like(dx)
    assert R.kref_rmsnorm(P(y), P(dx), P(dw), x.shape[0] * H, 128, f(1e-6)) == 0
    torch.cuda.synchronize()
    fx["rmsnorm/out"] = y.cpu().numpy()
    x, Hp, Wp, H = rope_inputs()
    c = np.zeros((Hp * Wp, 64), np.float32)
    s = np.zeros_like(c)
    R.kref_cosmos_rope(c.ctypes.data_as(ctypes.c_void_p), s.ctypes.data_as(ctypes.c_void_p), Hp, Wp)
    fx["rope/digest"] = np.array(digest(x))
    fx["rope/cos"], fx["rope/sin"] = c, s
    dx = torch.from_numpy(x).to(dev)
    dc, ds = torch.from_numpy(c).to(dev), torch.from_numpy(s).to(dev)
    assert R.kref_rope_half(P(dx), Hp * Wp, H, 128, P(dc), P(ds)) == 0
    torch.cuda.synchronize()
    fx["rope/out"] = dx.cpu().numpy()
    zp, zn = nag_inputs()
    fx["nag/digest"] = np.array(digest(zp, zn))
    for i, (sc, tau, alpha) in enumerate(NAG_PARAMS):
        a = torch.from_numpy(zp).to(dev)
        n = torch.from_numpy(zn).to(dev)
        assert R.kref_nag_f32(P(a), P(n), NAG_T, NAG_DIM, f(sc), f(tau), f(alpha)) == 0
        torch.cuda.synchronize()
        fx[f"nag/f32_{i}"] = a.cpu().numpy()
        a16 = torch.from_numpy(zp).to(dev).half()
        n16 = torch.from_numpy(zn).to(dev).half()
        assert R.kref_nag_f16(P(a16), P(n16), NAG_T, NAG_DIM, f(sc), f(tau), f(alpha)) == 0
        torch.cuda.synchronize()
        fx[f"nag/f16_{i}"] = a16.cpu().numpy()
    np.savez_compressed(out_path, **fx)
    print("wrote", out_path, os.path.getsize(out_path), "bytes,", len(fx), "arrays")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_fixtures.npz"))
