"""Head-split attention at batch 1 over the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU (engine/src/kernels.cu:207: one cudaSetDevice, no peer access), so this has no
counterpart there. Rank g owns heads [g*H/G, (g+1)*H/G): its Q/K/V are the [T, (H/G)*128] column slices a
column-sharded QKV projection would leave on that GPU, and every rank ends up with the full [T, H*128]
output, which is what the following output projection reads.

Data paths:
  fused  : the attention kernel's epilogue stores each finished tile into every rank's output buffer over
           NVLink (peer-mapped pointers) and bumps arrival counters; a one-thread wait kernel gates what follows.
           NAG: the per-token norms of the combine span all heads, so the kernels exchange 16 bytes per token and
           head through every rank's exchange area, blend locally in fp32 and push only the final tiles.
  nccl   : local attention into a [T, (H/G)*128] buffer, then all_gather_into_tensor (layout [G][T][cols]) —
           the baseline the fused path is measured against.
torch.distributed is only plumbing here: rendezvous, the exchange of IPC handles, and the NCCL baseline.

Buffer reuse. Arrival counters tell a rank when ITS buffer is complete; nothing in them stops a fast rank from
pushing the next call into a buffer a slow rank is still reading. So a rank calls release(buf) when it has read a
gathered buffer (stream-ordered: after whatever consumes it); that bumps the buffer's `released` counter on every
rank, and the next push into `buf` first waits until this rank's own counter shows that ALL ranks released the
previous use. The NAG exchange area is protected the same way by a `kernel finished` counter. Counters only grow.
"""
import ctypes

import torch
import torch.distributed as dist

from . import ops


def plan(H, G, rank):
    """(local head count, first head, first output column) of `rank` when H heads are split over G ranks."""
    if H % G:
        raise ValueError(f"{H} heads do not split over {G} ranks")
    hl = H // G
    return hl, rank * hl, rank * hl * 128


def reuse_target(uses_so_far, G):
    """What a rank's own `released` counter must show before use number uses_so_far + 1 may be pushed:
    every one of the G ranks has released each earlier use."""
    return uses_so_far * G


class HeadSplit:
    """Peer output buffers, exchange area and counters for one (T, H) shape; one instance per process."""

    N_BUFFERS = 2
    # counters, one 128-byte line each: arrivals[buf], released[buf], then `NAG kernel finished`
    _CTR_LINE = 128

    def __init__(self, T, H, dtype=torch.bfloat16, group=None):
        self.group = group or dist.group.WORLD
        self.G = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.T, self.H, self.D, self.dtype = T, H, H * 128, dtype
        self.hl, self.h0, self.col0 = plan(H, self.G, self.rank)
        L = ops.lib()
        rc = L.kb_init()
        if rc:
            raise ops.KilnError(rc, "kb_init")
        self.buf_bytes = T * self.D * 2
        self.n_qt = (T + 127) // 128
        self.xchg_bytes = L.kb_nag_exchange_bytes(T, H)
        self.xchg_off = self.N_BUFFERS * self.buf_bytes
        self.flag_off = self.xchg_off + L.kb_nag_exchange_counter_offset(T, H)
        self.ctr_off = self.xchg_off + self.xchg_bytes
        total = self.ctr_off + (2 * self.N_BUFFERS + 1) * self._CTR_LINE
        base = ctypes.c_void_p()
        ops._check(L.kb_peer_alloc(total, ctypes.byref(base)), "kb_peer_alloc")       # zero-filled
        self.base = base.value
        if self.G > 1:
            handle = ctypes.create_string_buffer(64)
            ops._check(L.kb_ipc_export(base, handle), "kb_ipc_export")
            handles = [None] * self.G
            dist.all_gather_object(handles, handle.raw, group=self.group)
        self.peer_base = []
        for r in range(self.G):
            if r == self.rank:
                self.peer_base.append(self.base)
            else:
                p = ctypes.c_void_p()
                ops._check(L.kb_ipc_import(handles[r], ctypes.byref(p)), "kb_ipc_import")
                self.peer_base.append(p.value)
        self.uses = [0] * self.N_BUFFERS        # pushes into each buffer so far
        self.nag_calls = 0
        self.arrivals = L.kb_push_arrivals_per_call(1, T, self.hl, self.G)
        dist.barrier(group=self.group)

    # ---- addresses on every rank
    def out_ptrs(self, buf):
        return [b + buf * self.buf_bytes for b in self.peer_base]

    def ctr_ptrs(self, buf):
        return [b + self.ctr_off + buf * self._CTR_LINE for b in self.peer_base]

    def released_ptrs(self, buf):
        return [b + self.ctr_off + (self.N_BUFFERS + buf) * self._CTR_LINE for b in self.peer_base]

    def nag_done_ptrs(self):
        return [b + self.ctr_off + 2 * self.N_BUFFERS * self._CTR_LINE for b in self.peer_base]

    def output(self, buf):
        """This rank's gathered [T, H*128] buffer as a torch tensor (no copy)."""
        return _as_tensor(self.base + buf * self.buf_bytes, (self.T, self.D), self.dtype)

    # ---- protocol
    def _before_push(self, buf):
        """Wait (on the stream, bounded) until every rank has released the previous use of `buf`."""
        if self.uses[buf]:
            ops.wait_arrivals(self.released_ptrs(buf)[self.rank], reuse_target(self.uses[buf], self.G))
        self.uses[buf] += 1

    def release(self, buf):
        """This rank is done reading buffer `buf` (ordered after everything enqueued so far on the stream)."""
        ops.bump_counters(self.released_ptrs(buf))

    def wait(self, buf):
        """Gate the stream until every rank's tiles of the latest push into `buf` have landed here."""
        ops.wait_arrivals(self.ctr_ptrs(buf)[self.rank], self.uses[buf] * self.arrivals)

    def attention(self, buf, q, k, v, Tk, npad=0, wait=True, **kw):
        """Attention of the local heads (q [T, hl*128], k/v [Tk, hl*128]); tiles land in buffer `buf` of every rank.
        Call release(buf) once the gathered rows have been consumed."""
        out_dt = ops.KB_BF16 if self.dtype == torch.bfloat16 else ops.KB_F16
        self._before_push(buf)
        ops.attn_push(self.out_ptrs(buf), self.ctr_ptrs(buf), self.col0, q, k, v, 1, self.T, Tk, npad, self.hl, self.D, out_dt, **kw)
        if wait:
            self.wait(buf)
        return self.output(buf)

    def nag(self, q, kp, vp, Tp, npad_p, kn, vn, Tn, npad_n, scale, tau, alpha, buf=0, wait=True, **kw):
        """Head-split NAG cross-attention: one fused launch per rank; the blended rows land in buffer `buf` of every rank."""
        out_dt = ops.KB_BF16 if self.dtype == torch.bfloat16 else ops.KB_F16
        self._before_push(buf)
        if self.nag_calls:          # every rank has finished its previous NAG kernel: the exchange area may be overwritten
            ops.wait_arrivals(self.nag_done_ptrs()[self.rank], reuse_target(self.nag_calls, self.G))
        self.nag_calls += 1
        part = [b + self.xchg_off for b in self.peer_base]
        flag = [b + self.flag_off for b in self.peer_base]
        ops.attn_nag_push(self.out_ptrs(buf), self.ctr_ptrs(buf), part, flag, self.rank, self.col0, self.h0, self.H, self.nag_calls,
                          q, kp, vp, Tp, npad_p, kn, vn, Tn, npad_n, scale, tau, alpha, self.T, self.hl, self.D, out_dt, **kw)
        ops.bump_counters(self.nag_done_ptrs())
        if wait:
            self.wait(buf)
        return self.output(buf)

    def close(self):
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        L = ops.lib()
        for r, b in enumerate(self.peer_base):
            if r != self.rank:
                L.kb_ipc_close(ctypes.c_void_p(b))
        dist.barrier(group=self.group)
        L.kb_peer_free(ctypes.c_void_p(self.base))


class _Span:
    """Minimal __cuda_array_interface__ holder so torch can view library-owned device memory."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": shape, "typestr": typestr, "version": 2, "strides": None}


def _as_tensor(ptr, shape, dtype):
    t = torch.as_tensor(_Span(ptr, shape, "<i2"), device="cuda")      # 16-bit payload, reinterpreted below
    return t.view(dtype)


def nccl_all_gather_attention(q, k, v, T, Tk, hl, G, npad=0, group=None, **kw):
    """Baseline: local attention then ncclAllGather; returns [G, T, hl*128] (rank-major column blocks)."""
    local = torch.empty(T, hl * 128, device=q.device, dtype=q.dtype if q.dtype != torch.float32 else torch.float16)
    ops.attn_cross(local, q, k, v, T, Tk, npad, hl, **kw)
    gathered = torch.empty(G, T, hl * 128, device=q.device, dtype=local.dtype)
    dist.all_gather_into_tensor(gathered, local, group=group)
    return gathered
