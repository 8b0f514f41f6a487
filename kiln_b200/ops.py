"""ctypes binding of the C ABI (include/kiln_b200.h) plus thin torch-tensor helpers.

The helpers take torch CUDA tensors only to get device pointers, strides and the current stream;
all arithmetic happens in the library's kernels. Argument names and meaning follow the engine's
op set (reference: engine/src/gpu.h:149-156): row-major [rows, ld] activations, head h at columns
[h*128, (h+1)*128), `npad` zero keys joining the softmax.
"""
import ctypes
import os

KB_F16, KB_BF16, KB_F32 = 0, 1, 2

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("KILN_B200_LIB") or os.path.join(_PKG, "lib", "libkiln_b200.so")   # override: an alternative build of the same ABI
_lib = None


class KilnError(RuntimeError):
    """A C-ABI call returned a non-zero status (the engine's shim throws std::runtime_error here)."""

    def __init__(self, code, what):
        self.code = code
        super().__init__(f"{what}: {lib().kb_error_string(code).decode()} ({code})")


def lib():
    """Load the in-tree library; fails loudly when it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise FileNotFoundError(f"{_LIB_PATH} is missing: run `python -m kiln_b200.build` (nvcc, sm_100a)")
        L = ctypes.CDLL(_LIB_PATH)
        vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
        L.kb_error_string.restype = ctypes.c_char_p
        L.kb_error_string.argtypes = [i]
        L.kb_version.restype = i
        L.kb_init.restype = i
        L.kb_attn_workspace_bytes.restype = sz
        L.kb_attn_workspace_bytes.argtypes = [i, i, i, i, i, i, i]
        L.kb_attn_self.restype = i
        L.kb_attn_self.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, f, vp, sz, vp]
        L.kb_attn_self_static.restype = i
        L.kb_attn_self_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, f, vp]
        L.kb_attn_cross.restype = i
        L.kb_attn_cross.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, f, vp, sz, vp]
        L.kb_attn_nag.restype = i
        L.kb_attn_nag.argtypes = [vp, vp, vp, vp, vp, i, i, vp, vp, i, i, f, f, f, i, i, i, i, i, i, i, f, vp, sz, vp]
        L.kb_qk_prep.restype = i
        L.kb_qk_prep.argtypes = [vp, i, i, vp, i, i, i, i, i, vp, f, vp, vp, vp]
        L.kb_linear16.restype = i
        L.kb_linear16.argtypes = [vp, i, vp, i, vp, i, i, i, i, i, vp, vp, vp, vp, i, f, vp]
        L.kb_linear16_lora.restype = i
        L.kb_linear16_lora.argtypes = [vp, i, vp, i, vp, i, vp, i, vp, i, i, i, i, i, i, vp, vp, vp, vp, i, f, vp]
        pi = ctypes.POINTER(i)
        pvp = ctypes.POINTER(vp)
        L.kb_linear16_qkv_lora.restype = i
        L.kb_linear16_qkv_lora.argtypes = [pvp, i, vp, i, pvp, i, pvp, pi, pvp, pi, pi, i, i, i, pvp, pi, vp, vp, i, f, vp]
        L.kb_lora_pack.restype = i
        L.kb_lora_pack.argtypes = [vp, i, i, vp, i, i, f, vp]
        L.kb_attn_bwd_workspace_bytes.restype = ctypes.c_size_t
        L.kb_attn_bwd_workspace_bytes.argtypes = [i, i, i, i, i]
        L.kb_attn_bwd.restype = i
        L.kb_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, i, i, i, vp, ctypes.c_size_t, vp]
        L.kb_cross_kv.restype = i
        L.kb_cross_kv.argtypes = [vp, vp, i, vp, i, i, i, i, i, vp, vp, i, vp, f, vp, ctypes.c_size_t, vp]
        L.kb_linear16_qkv.restype = i
        L.kb_linear16_qkv.argtypes = [ctypes.POINTER(vp), i, vp, i, ctypes.POINTER(vp), i, i, i, i, ctypes.POINTER(vp), ctypes.POINTER(i), vp, vp, i, f, vp]
        L.kb_status.restype = i
        L.kb_status.argtypes = [ctypes.POINTER(ctypes.c_uint)]
        ull = ctypes.c_ulonglong
        L.kb_nag_combine.restype = i
        L.kb_nag_combine.argtypes = [vp, vp, i, i, i, i, f, f, f, i, vp]
        L.kb_peer_alloc.restype = i
        L.kb_peer_alloc.argtypes = [sz, ctypes.POINTER(vp)]
        L.kb_peer_free.restype = i
        L.kb_peer_free.argtypes = [vp]
        L.kb_ipc_export.restype = i
        L.kb_ipc_export.argtypes = [vp, ctypes.c_char_p]
        L.kb_ipc_import.restype = i
        L.kb_ipc_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.kb_ipc_close.restype = i
        L.kb_ipc_close.argtypes = [vp]
        L.kb_attn_push.restype = i
        L.kb_attn_push.argtypes = [ctypes.POINTER(vp), ctypes.POINTER(vp), i, i, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, i, f, vp, sz, vp]
        L.kb_attn_nag_push.restype = i
        L.kb_attn_nag_push.argtypes = [ctypes.POINTER(vp)] * 4 + [i, i, i, i, i, ctypes.c_uint, vp, vp, vp, vp, i, i, vp, vp, i, i, f, f, f,
                                       i, i, i, i, i, i, i, f, vp, sz, vp]
        L.kb_nag_exchange_bytes.restype = sz
        L.kb_nag_exchange_bytes.argtypes = [i, i]
        L.kb_nag_exchange_counter_offset.restype = sz
        L.kb_nag_exchange_counter_offset.argtypes = [i, i]
        L.kb_bump_counters.restype = i
        L.kb_bump_counters.argtypes = [ctypes.POINTER(vp), i, vp]
        L.kb_push_arrivals_per_call.restype = ull
        L.kb_push_arrivals_per_call.argtypes = [i, i, i, i]
        L.kb_wait_arrivals.restype = i
        L.kb_wait_arrivals.argtypes = [vp, ull, vp]
        L.kb_prof_enable.restype = i
        L.kb_prof_enable.argtypes = [i]
        L.kb_prof_read.restype = i
        L.kb_prof_read.argtypes = [i, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(i)]
        L.kb_selfcheck_workspace_bytes.restype = sz
        L.kb_attn_selfcheck.restype = i
        L.kb_attn_selfcheck.argtypes = [vp, sz, ctypes.POINTER(ctypes.c_float), vp]
        _lib = L
    return _lib


def _dt(t):
    import torch
    return {torch.float16: KB_F16, torch.bfloat16: KB_BF16, torch.float32: KB_F32}[t.dtype]


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _ld(t):
    assert t.dim() == 2 and t.stride(1) == 1, "activations are row-major [rows, ld]"
    return t.stride(0)


def _stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(code, what):
    if code != 0:
        raise KilnError(code, what)


def workspace_bytes(rows_q, rows_k, H, dtype, norm_q=False, norm_k=False, n_ctx=1):
    """Scratch bytes for one attention call; dtype is a KB_* code or a torch dtype."""
    if not isinstance(dtype, int):
        import torch
        dtype = {torch.float16: KB_F16, torch.bfloat16: KB_BF16, torch.float32: KB_F32}[dtype]
    return lib().kb_attn_workspace_bytes(rows_q, rows_k, n_ctx, H, dtype, int(bool(norm_q)), int(bool(norm_k)))


def _ws(workspace):
    if workspace is None:
        return None, 0
    return _ptr(workspace), workspace.numel() * workspace.element_size()


def attn_self(out, q, k, v, B, T, H, qn_w=None, kn_w=None, rope_cos=None, rope_sin=None, eps=1e-6, workspace=None):
    """Self-attention of B images of T tokens; q, k, v, out are [B*T, ld] tensors (out may be fp32)."""
    wp, wb = _ws(workspace)
    _check(lib().kb_attn_self(_ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(qn_w), _ptr(kn_w), _ptr(rope_cos), _ptr(rope_sin),
                              B, T, H, _ld(q), _ld(k), _ld(v), _ld(out), _dt(q), _dt(out), eps, wp, wb, _stream()), "kb_attn_self")
    return out


def attn_cross(out, q, k, v, Tq, Tk, npad, H, qn_w=None, eps=1e-6, workspace=None):
    """Cross-attention to one context: the first Tk rows of k, v are real, npad zero keys join the softmax."""
    wp, wb = _ws(workspace)
    _check(lib().kb_attn_cross(_ptr(out), _ptr(q), _ptr(qn_w), _ptr(k), _ptr(v), Tq, Tk, npad, H, _ld(q), _ld(k), _ld(v),
                               _ld(out), _dt(q), _dt(out), eps, wp, wb, _stream()), "kb_attn_cross")
    return out


def attn_nag(out, q, k_pos, v_pos, Tk_pos, npad_pos, k_neg, v_neg, Tk_neg, npad_neg, scale, tau, alpha, Tq, H,
             qn_w=None, eps=1e-6, workspace=None):
    """Cross-attention to a positive and a negative context followed by the NAG combine, in one kernel."""
    assert _ld(k_pos) == _ld(v_pos) == _ld(k_neg) == _ld(v_neg)
    wp, wb = _ws(workspace)
    _check(lib().kb_attn_nag(_ptr(out), _ptr(q), _ptr(qn_w), _ptr(k_pos), _ptr(v_pos), Tk_pos, npad_pos, _ptr(k_neg),
                             _ptr(v_neg), Tk_neg, npad_neg, scale, tau, alpha, Tq, H, _ld(q), _ld(k_pos), _ld(out), _dt(q),
                             _dt(out), eps, wp, wb, _stream()), "kb_attn_nag")
    return out


def nag_combine(a, an, scale, tau, alpha):
    """In-place NAG combine of a (Z+) with an (Z-), rows of all heads together (engine counterpart: k_nag)."""
    assert a.dtype == an.dtype and a.shape == an.shape
    _check(lib().kb_nag_combine(_ptr(a), _ptr(an), a.shape[0], a.shape[1], _ld(a), _ld(an), scale, tau, alpha, _dt(a), _stream()), "kb_nag_combine")
    return a


def attn_push(out_ptrs, ctr_ptrs, col0, q, k, v, B, Tq, Tk, npad, H_local, ld_o, out_dtype, qn_w=None, kn_w=None, rope_cos=None,
              rope_sin=None, eps=1e-6, workspace=None):
    """Attention over the local heads whose output tiles are stored into every peer buffer (device addresses in
    out_ptrs, this GPU's own included) at column col0, bumping the counters at ctr_ptrs. out_dtype: KB_F16 / KB_BF16."""
    n = len(out_ptrs)
    outs = (ctypes.c_void_p * n)(*out_ptrs)
    ctrs = (ctypes.c_void_p * n)(*ctr_ptrs)
    wp, wb = _ws(workspace)
    _check(lib().kb_attn_push(outs, ctrs, n, col0, _ptr(q), _ptr(k), _ptr(v), _ptr(qn_w), _ptr(kn_w), _ptr(rope_cos), _ptr(rope_sin),
                              B, Tq, Tk, npad, H_local, _ld(q), _ld(k), _ld(v), ld_o, _dt(q), out_dtype, eps, wp, wb, _stream()), "kb_attn_push")


def attn_nag_push(out_ptrs, ctr_ptrs, part_ptrs, flag_ptrs, self_index, col0, h0, heads_total, epoch, q, k_pos, v_pos, Tk_pos, npad_pos,
                  k_neg, v_neg, Tk_neg, npad_neg, scale, tau, alpha, Tq, H_local, ld_o, out_dtype, qn_w=None, eps=1e-6, workspace=None):
    """NAG cross-attention over the local heads with the norm exchange and the output tiles going to every peer
    (device addresses; this GPU's own at index self_index). See kb_attn_nag_push."""
    n = len(out_ptrs)
    arr = lambda ptrs: (ctypes.c_void_p * n)(*ptrs)
    wp, wb = _ws(workspace)
    _check(lib().kb_attn_nag_push(arr(out_ptrs), arr(ctr_ptrs), arr(part_ptrs), arr(flag_ptrs), n, self_index, col0, h0, heads_total, epoch,
                                  _ptr(q), _ptr(qn_w), _ptr(k_pos), _ptr(v_pos), Tk_pos, npad_pos, _ptr(k_neg), _ptr(v_neg), Tk_neg, npad_neg,
                                  scale, tau, alpha, Tq, H_local, _ld(q), _ld(k_pos), ld_o, _dt(q), out_dtype, eps, wp, wb, _stream()),
           "kb_attn_nag_push")


def bump_counters(ctr_ptrs):
    """Enqueue one system-scope add on each listed counter (device addresses), ordered after earlier work on the stream."""
    n = len(ctr_ptrs)
    _check(lib().kb_bump_counters((ctypes.c_void_p * n)(*ctr_ptrs), n, _stream()), "kb_bump_counters")


def wait_arrivals(ctr_ptr, target):
    """Enqueue the bounded wait for `target` tile arrivals on this GPU's counter (device address ctr_ptr)."""
    _check(lib().kb_wait_arrivals(ctypes.c_void_p(ctr_ptr), target, _stream()), "kb_wait_arrivals")


def qk_prep(out, x, rows, H, T, w=None, rope_cos=None, rope_sin=None, eps=1e-6):
    """out = rope(rmsnorm(x)) per (row, head) as 16-bit; a plain conversion when w and the tables are None."""
    _check(lib().kb_qk_prep(_ptr(out), _ld(out), _dt(out), _ptr(x), _ld(x), _dt(x), rows, H, T, _ptr(w), eps, _ptr(rope_cos),
                            _ptr(rope_sin), _stream()), "kb_qk_prep")
    return out


EPI_F32, EPI_F16, EPI_GELU16, EPI_RESID, EPI_HEADS16 = 0, 1, 2, 3, 4


def linear16(C, A, W, epi, gate=None, head_w=None, rope_cos=None, rope_sin=None, eps=1e-6, lora=None):
    """C = epilogue(A @ W.T): A [M, K] and W [N, K] fp16, fp32 accumulation (engine: linear16, engine/src/kernels.cu:559-609).

    EPI_F32 / EPI_RESID take an fp32 C, the others an fp16 C; EPI_HEADS16 applies the per-head RMSNorm (head_w bf16[128])
    and rotate-half RoPE (tables [T, 64]) to every 128-column head before the fp16 store.
    lora = (A2 [M, K2], W2 [N, K2]) fp16 adds the second product A2 @ W2.T to the accumulator before the epilogue
    (engine/src/kernels.cu:578-596).
    """
    M, K = A.shape
    N = W.shape[0]
    rope_T = rope_cos.shape[0] if rope_cos is not None else 0
    if lora is not None:
        A2, W2 = lora
        _check(lib().kb_linear16_lora(_ptr(C), _ld(C), _ptr(A), _ld(A), _ptr(W), _ld(W), _ptr(A2), _ld(A2), _ptr(W2), _ld(W2), A2.shape[1],
                                      M, N, K, epi, _ptr(gate), _ptr(head_w), _ptr(rope_cos), _ptr(rope_sin), rope_T, eps, _stream()),
               "kb_linear16_lora")
        return C
    _check(lib().kb_linear16(_ptr(C), _ld(C), _ptr(A), _ld(A), _ptr(W), _ld(W), M, N, K, epi, _ptr(gate), _ptr(head_w),
                             _ptr(rope_cos), _ptr(rope_sin), rope_T, eps, _stream()), "kb_linear16")
    return C


def lora_pack(dst, col0, src, scale=1.0):
    """dst[:, col0:col0 + cols] = fp16(scale * src) for a bf16 LoRA matrix src [rows, cols] (k_lora_pack, engine/src/kernels.cu:548-554)."""
    rows, cols = src.shape
    _check(lib().kb_lora_pack(_ptr(dst), _ld(dst), col0, _ptr(src), rows, cols, float(scale), _stream()), "kb_lora_pack")
    return dst


def linear16_qkv(Cs, A, Ws, head_ws=(None, None, None), rope_on=(True, True, False), rope_cos=None, rope_sin=None, eps=1e-6, loras=None):
    """Three projections of one activation in one launch: Cs[i] = heads16(A @ Ws[i].T), fp16; see kb_linear16_qkv.

    loras = three entries, each None or (A2 [M, K2], W2 [N, K2]) fp16: the second product of that projection."""
    M, K = A.shape
    N = Ws[0].shape[0]
    vp3 = ctypes.c_void_p * 3
    arr = lambda ts: vp3(*[None if t is None else t.data_ptr() for t in ts])
    on = (ctypes.c_int * 3)(*[int(bool(r) and rope_cos is not None) for r in rope_on])
    rope_T = rope_cos.shape[0] if rope_cos is not None else 0
    assert all(_ld(c) == _ld(Cs[0]) for c in Cs) and all(_ld(w) == _ld(Ws[0]) for w in Ws)
    if loras is not None:
        i3 = ctypes.c_int * 3
        a2 = [None if l is None else l[0] for l in loras]
        w2 = [None if l is None else l[1] for l in loras]
        _check(lib().kb_linear16_qkv_lora(arr(Cs), _ld(Cs[0]), _ptr(A), _ld(A), arr(Ws), _ld(Ws[0]), arr(a2),
                                          i3(*[0 if t is None else _ld(t) for t in a2]), arr(w2),
                                          i3(*[0 if t is None else _ld(t) for t in w2]), i3(*[0 if t is None else t.shape[1] for t in a2]),
                                          M, N, K, arr(head_ws), on, _ptr(rope_cos), _ptr(rope_sin), rope_T, eps, _stream()),
               "kb_linear16_qkv_lora")
        return Cs
    _check(lib().kb_linear16_qkv(arr(Cs), _ld(Cs[0]), _ptr(A), _ld(A), arr(Ws), _ld(Ws[0]), M, N, K, arr(head_ws), on, _ptr(rope_cos),
                                 _ptr(rope_sin), rope_T, eps, _stream()), "kb_linear16_qkv")
    return Cs


def attn_bwd(dq, dk, dv, q, k, v, dout, B, Tq, Tk, npad, H, workspace=None):
    """dq, dk, dv (fp32) of softmax(q k^T / sqrt(128)) v per head from q, k, v, dout (engine: attention_bwd,
    engine/src/train.cu:216-242). q, dout [B*Tq, >= H*128], k, v [B*Tk, >= H*128], one dtype."""
    import torch
    if workspace is None:
        workspace = torch.empty(lib().kb_attn_bwd_workspace_bytes(B, Tq, Tk, H, _dt(q)), dtype=torch.uint8, device=q.device)
    _check(lib().kb_attn_bwd(_ptr(dq), _ptr(dk), _ptr(dv), _ptr(q), _ptr(k), _ptr(v), _ptr(dout), B, Tq, Tk, npad, H, _ld(q), _ld(k), _ld(v),
                             _ld(dout), _ld(dq), _ld(dk), _ld(dv), _dt(q), _ptr(workspace), workspace.numel(), _stream()), "kb_attn_bwd")
    return dq, dk, dv


def cross_kv(k16, v16, ctx, Wk, Wv, kn_w=None, eps=1e-6, workspace=None):
    """fp16, already normalised cross-attention K and V of one context for one block: K = rmsnorm_per_head(ctx @ Wk.T),
    V = ctx @ Wv.T (engine: Dit::cache_context, engine/src/dit.cu:217-234). ctx [L, K] fp32 / fp16 / bf16; Wk, Wv fp16 [N, K]."""
    import torch
    L, K = ctx.shape
    N = Wk.shape[0]
    if workspace is None and ctx.dtype != torch.float16:
        workspace = torch.empty(max(L * K * 2, 16), dtype=torch.uint8, device=ctx.device)
    _check(lib().kb_cross_kv(_ptr(k16), _ptr(v16), _ld(k16), _ptr(ctx), _ld(ctx), _dt(ctx), L, N, K, _ptr(Wk), _ptr(Wv), _ld(Wk), _ptr(kn_w), eps,
                             _ptr(workspace), 0 if workspace is None else workspace.numel(), _stream()), "kb_cross_kv")
    return k16, v16


def check_status():
    """Synchronise and raise if any kernel since the last call gave up on a bounded wait."""
    bits = ctypes.c_uint(0)
    _check(lib().kb_status(ctypes.byref(bits)), "kb_status")
    return bits.value


PROF_NORM_ROPE, PROF_ATTENTION, PROF_NAG, PROF_LINEAR = 0, 1, 2, 3


def prof_enable(on=True):
    """Start (or stop) recording one event pair per kernel launch (engine counterpart: ProfScope)."""
    _check(lib().kb_prof_enable(int(on)), "kb_prof_enable")


def prof_read(category):
    """(total kernel milliseconds, launches) of one category since prof_enable; synchronises the device."""
    ms, n = ctypes.c_double(0), ctypes.c_int(0)
    _check(lib().kb_prof_read(category, ctypes.byref(ms), ctypes.byref(n)), "kb_prof_read")
    return ms.value, n.value
