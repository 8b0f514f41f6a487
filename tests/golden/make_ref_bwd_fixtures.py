"""Generates tests/golden/ref_bwd_fixtures.npz from the REFERENCE'S OWN attention backward, run on a B200.

Needs a GPU and oracle/_ref/libkiln_ref.so (python oracle/build.py --ref <kiln tree>). Run once:

    python tests/golden/make_ref_bwd_fixtures.py [out.npz]

The fixture holds dq, dk, dv of  attention_bwd  engine/src/train.cu:216-242  (16 heads of 128, fp32, cuBLAS SGEMM with
k_softmax_pad / k_dsoftmax) on inputs regenerated from seeds by the oracle's torch-compatible randn; to keep it small only the
columns of the first KEEP_HEADS heads are stored.
"""
import ctypes
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle  # noqa: E402

H, D = 16, 2048
KEEP_HEADS = 3
# (name, Tq, Tk, npad): a self-attention shape (train.cu:344) and a cross-attention shape with padding (train.cu:334)
BWD_CASES = [("self_ragged", 150, 150, 0), ("cross_pad", 200, 26, 486)]


def bwd_inputs(case):
    """q, k ~ 1.5 N(0,1) (the scale of normalised, rotated Q/K as in bench/tfa_test.cu:37-43), v, dout ~ N(0,1), fp32."""
    name, Tq, Tk, npad = case
    seed = 4000 + 10 * BWD_CASES.index(case)
    q = oracle.randn(seed, Tq * D).reshape(Tq, D) * np.float32(1.5)
    k = oracle.randn(seed + 1, Tk * D).reshape(Tk, D) * np.float32(1.5)
    v = oracle.randn(seed + 2, Tk * D).reshape(Tk, D)
    dout = oracle.randn(seed + 3, Tq * D).reshape(Tq, D)
    return q, k, v, dout


def load_ref():
    R = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libkiln_ref.so"))
    R.kref_engine_init.argtypes = [ctypes.c_size_t, ctypes.c_char_p, ctypes.c_int]
    R.kref_attention_bwd.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 3 + [ctypes.c_char_p, ctypes.c_int]
    err = ctypes.create_string_buffer(512)
    assert R.kref_engine_init(3 << 30, err, 512) == 0, err.value
    return R


def run_ref(R, q, k, v, dout, npad):
    """The reference's attention_bwd on device copies of the inputs; returns numpy dq, dk, dv."""
    dq_, dk_, dv_, dd = (torch.from_numpy(a).cuda() for a in (q, k, v, dout))
    gq, gk, gv = torch.full_like(dq_, float("nan")), torch.full_like(dk_, float("nan")), torch.full_like(dv_, float("nan"))
    err = ctypes.create_string_buffer(512)
    rc = R.kref_attention_bwd(gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), dq_.data_ptr(), dk_.data_ptr(), dv_.data_ptr(), dd.data_ptr(),
                              q.shape[0], k.shape[0], npad, err, 512)
    torch.cuda.synchronize()
    assert rc == 0, err.value
    return gq.cpu().numpy(), gk.cpu().numpy(), gv.cpu().numpy()


def main(out_path):
    R = load_ref()
    out = {}
    for case in BWD_CASES:
        q, k, v, dout = bwd_inputs(case)
        for name, g in zip(("dq", "dk", "dv"), run_ref(R, q, k, v, dout, case[3])):
            assert not np.isnan(g).any()
            out[f"{case[0]}/{name}"] = g[:, :KEEP_HEADS * 128].copy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "ref_bwd_fixtures.npz"))
