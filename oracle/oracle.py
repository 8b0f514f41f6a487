"""ctypes wrapper of the CPU oracle (oracle/kiln_oracle.c). TEST INFRASTRUCTURE ONLY:
imported by tests/, the smoke check and the benchmark's CPU baseline, never by the library."""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "libkiln_oracle.so")
        if not os.path.exists(path):
            import importlib.util
            spec = importlib.util.spec_from_file_location("_kiln_oracle_build", os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        L = ctypes.CDLL(path)
        vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.ko_max_threads.restype = i
        for name in ("ko_attention_f32", "ko_attention_f64"):
            getattr(L, name).argtypes = [vp, i, vp, i, vp, i, vp, i, i, i, i, i]
            getattr(L, name).restype = None
        L.ko_rmsnorm.argtypes = [vp, vp, vp, ctypes.c_size_t, i, f]
        L.ko_rope_half.argtypes = [vp, i, i, i, vp, vp]
        L.ko_cosmos_rope.argtypes = [vp, vp, i, i]
        L.ko_nag.argtypes = [vp, vp, i, i, f, f, f, i]
        L.ko_linear16.argtypes = [vp, i, vp, i, vp, i, i, i, i, i, vp]
        L.ko_attention_bwd.argtypes = [vp, i, vp, i, vp, i, vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, i]
        L.ko_attention_bwd.restype = None
        L.ko_torch_randn.argtypes = [ctypes.c_uint64, ctypes.c_size_t, vp]
        L.ko_torch_randn.restype = i
        L.ko_round16.argtypes = [vp, ctypes.c_size_t, i]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def max_threads():
    return lib().ko_max_threads()


def set_threads(n):
    """Size of the OpenMP team used by the following calls."""
    lib().ko_set_num_threads.argtypes = [ctypes.c_int]
    lib().ko_set_num_threads(int(n))


def randn(seed, n):
    """torch.manual_seed(seed); torch.randn(n) on CPU, restated (reference: engine/src/pipeline.cu:16-64)."""
    out = np.empty(n, np.float32)
    if lib().ko_torch_randn(seed, n, _p(out)) != 0:
        raise ValueError("n must be >= 16")
    return out


def round16(x, kind):
    """Round an fp32 array through fp16 (kind 0) or bf16 (kind 1), returning fp32."""
    x = _f32(x).copy()
    lib().ko_round16(_p(x), x.size, kind)
    return x


def attention(q, k, v, H, npad=0, acc64=True):
    """q [Tq, >=H*128], k/v [Tk, >=H*128] fp32 -> out [Tq, H*128] (reference: bench/tfa_test.cu:11-33)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    Tq, Tk = q.shape[0], k.shape[0]
    out = np.zeros((Tq, H * 128), np.float32)
    fn = lib().ko_attention_f64 if acc64 else lib().ko_attention_f32
    fn(_p(out), out.shape[1], _p(q), q.shape[1], _p(k), k.shape[1], _p(v), v.shape[1], Tq, Tk, H, npad)
    return out


def attention_bwd(q, k, v, dout, H, npad=0, key_rows=None):
    """Exact attention backward in double (reference: engine/src/train.cu:216-242): returns (dq [Tq, H*128], dk, dv [rows, H*128]).

    key_rows = (j0, j1) restricts dk / dv to those key rows (dq is always complete for the query rows given; to sample query rows,
    pass a subset of q and dout - but then dk / dv are meaningless)."""
    q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
    Tq, Tk = q.shape[0], k.shape[0]
    j0, j1 = (0, Tk) if key_rows is None else key_rows
    D = H * 128
    dq = np.zeros((Tq, D), np.float32)
    dk = np.zeros((j1 - j0, D), np.float32)
    dv = np.zeros((j1 - j0, D), np.float32)
    lib().ko_attention_bwd(_p(dq), D, _p(dk), D, _p(dv), D, _p(q), q.shape[1], _p(k), k.shape[1], _p(v), v.shape[1], _p(dout), dout.shape[1],
                           Tq, Tk, H, npad, j0, j1)
    return dq, dk, dv


def rmsnorm(x, w_bf16_bits, H, eps=1e-6):
    """x [rows, H*128] -> per (row, head) RMSNorm with bf16 weight bits [128] (reference: engine/src/kernels.cu:656-666)."""
    x = _f32(x)
    assert x.shape[1] == H * 128
    y = np.empty_like(x)
    w = None if w_bf16_bits is None else np.ascontiguousarray(w_bf16_bits, dtype=np.uint16)
    lib().ko_rmsnorm(_p(y), _p(x), None if w is None else _p(w), x.shape[0] * H, 128, eps)
    return y


def rope_half(x, T, H, cos_t, sin_t):
    """In-place rotate-half RoPE on a copy of x [T, H*128] (reference: engine/src/kernels.cu:759-772)."""
    x = _f32(x).copy()
    assert x.shape == (T, H * 128)
    lib().ko_rope_half(_p(x), T, H, 128, _p(_f32(cos_t)), _p(_f32(sin_t)))
    return x


def cosmos_rope(Hp, Wp):
    """cos, sin tables [Hp*Wp, 64] (reference: engine/src/dit.cu:196-215)."""
    c = np.empty((Hp * Wp, 64), np.float32)
    s = np.empty_like(c)
    lib().ko_cosmos_rope(_p(c), _p(s), Hp, Wp)
    return c, s


def nag(zp, zn, s, tau, alpha, acc64=True):
    """NAG combine of Z+ and Z- [T, dim] -> [T, dim] (reference: engine/src/dit.cu:295-324)."""
    a = _f32(zp).copy()
    n = _f32(zn)
    lib().ko_nag(_p(a), _p(n), a.shape[0], a.shape[1], s, tau, alpha, int(acc64))
    return a


def lora_operands(x, loras):
    """The operands of the LoRA second product as linear16 composes them (reference: engine/src/kernels.cu:578-596).

    x [M, in] fp16-exact; loras = [(A [r, in], B [out, r], scale), ...] with bf16-exact A and B. Returns
    (t, b_cat): b_cat = [s1 B1 | s2 B2 | ...] rounded to fp16 ([out, R], k_lora_pack at kernels.cu:548-554) and
    t = fp16(x . A_cat^T) ([M, R]; the reference's cublasGemmEx with an fp16 result and fp32 accumulation, summed in
    double here). The reference pads R to its k tile with zero columns, which add nothing to the product."""
    a_cat = np.concatenate([round16(_f32(a), 0) for a, _, _ in loras], axis=0)
    b_cat = np.concatenate([round16(np.float32(s) * _f32(b), 0) for _, b, s in loras], axis=1)
    return linear16(x, a_cat, 1), b_cat


def linear16(x, w, epi=0, gate=None, c=None, lora=None):
    """epi(x [M, K] . w [N, K]^T) with fp16-exact inputs (reference: engine/src/tcgemm16.cuh:57-175).

    epi 0 fp32, 1 fp16-rounded, 2 fp16-rounded GELU, 3 c + gate * acc (c is the fp32 residual stream, copied).
    lora = (t [M, K2], b_cat [N, K2]): the second product joins the accumulator before the epilogue
    (tcgemm16.cuh:70-76), which is one product over the concatenated k range.
    """
    x, w = _f32(x), _f32(w)
    if lora is not None:
        x = np.concatenate([x, _f32(lora[0])], axis=1)
        w = np.concatenate([w, _f32(lora[1])], axis=1)
    M, K = x.shape
    N = w.shape[0]
    out = np.zeros((M, N), np.float32) if c is None else _f32(c).copy()
    g = None if gate is None else _f32(gate)
    lib().ko_linear16(_p(out), N, _p(x), K, _p(w), K, M, N, K, epi, None if g is None else _p(g))
    return out


def linear_heads16(x, w, H, head_w_bits=None, cos_t=None, sin_t=None, eps=1e-6):
    """The engine's q / k projection chain: linear16 (fp32 out), per-head RMSNorm, rotate-half RoPE
    (reference: engine/src/dit.cu:461-468), then the fp16 rounding the attention kernel applies while staging
    (engine/src/tcflash.cuh:56-64). Returns fp32 holding fp16-exact values."""
    y = linear16(x, w, 0)
    if head_w_bits is not None:
        y = rmsnorm(y, head_w_bits, H, eps)
    if cos_t is not None:
        y = rope_half(y, y.shape[0], H, cos_t, sin_t)
    return round16(y, 0)
