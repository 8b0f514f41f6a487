"""Head-split attention at batch 1 over the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU (engine/src/kernels.cu:207: one cudaSetDevice, no peer access), so this has no
counterpart there. Rank g owns heads [g*H/G, (g+1)*H/G): its Q/K/V are the [T, (H/G)*128] column slices a
column-sharded QKV projection would leave on that GPU, and every rank ends up with the full [T, H*128]
output, which is what the following output projection reads.

Two data paths:
  fused  : the attention kernel's epilogue stores each finished tile into every rank's output buffer over
           NVLink (peer-mapped pointers) and bumps arrival counters; a one-thread wait kernel gates what follows.
  nccl   : local attention into a [T, (H/G)*128] buffer, then all_gather_into_tensor (layout [G][T][cols]) —
           the baseline the fused path is measured against.
torch.distributed is only plumbing here: rendezvous, the exchange of IPC handles, and the NCCL baseline.
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


class HeadSplit:
    """Peer output buffers and arrival counters for one (T, H) shape; one instance per process."""

    N_BUFFERS = 2      # Z+ / self output and Z- so that NAG can gather both before the blend

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
        esz = 2
        self.buf_bytes = T * self.D * esz
        total = self.N_BUFFERS * self.buf_bytes + 256            # buffers, then one 64-bit counter per buffer
        base = ctypes.c_void_p()
        ops._check(L.kb_peer_alloc(total, ctypes.byref(base)), "kb_peer_alloc")
        self.base = base.value
        handle = ctypes.create_string_buffer(64)
        ops._check(L.kb_ipc_export(base, handle), "kb_ipc_export")
        handles = [None] * self.G
        dist.all_gather_object(handles, handle.raw, group=self.group)
        self.peer_base = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.peer_base.append(self.base)
            else:
                p = ctypes.c_void_p()
                ops._check(L.kb_ipc_import(h, ctypes.byref(p)), "kb_ipc_import")
                self.peer_base.append(p.value)
        self.calls = [0] * self.N_BUFFERS
        self.arrivals = L.kb_push_arrivals_per_call(1, T, self.hl, self.G)
        dist.barrier(group=self.group)

    def out_ptrs(self, buf):
        return [b + buf * self.buf_bytes for b in self.peer_base]

    def ctr_ptrs(self, buf):
        return [b + self.N_BUFFERS * self.buf_bytes + 8 * buf for b in self.peer_base]

    def output(self, buf):
        """This rank's gathered [T, H*128] buffer as a torch tensor (no copy)."""
        return _as_tensor(self.base + buf * self.buf_bytes, (self.T, self.D), self.dtype)

    def attention(self, buf, q, k, v, Tk, npad=0, wait=True, **kw):
        """Attention of the local heads (q [T, hl*128], k/v [Tk, hl*128]); tiles land in buffer `buf` of every rank."""
        out_dt = ops.KB_BF16 if self.dtype == torch.bfloat16 else ops.KB_F16
        ops.attn_push(self.out_ptrs(buf), self.ctr_ptrs(buf), self.col0, q, k, v, 1, self.T, Tk, npad, self.hl, self.D, out_dt, **kw)
        self.calls[buf] += 1
        if wait:
            self.wait(buf)
        return self.output(buf)

    def wait(self, buf):
        ops.wait_arrivals(self.ctr_ptrs(buf)[self.rank], self.calls[buf] * self.arrivals)

    def nag(self, q, kp, vp, Tp, npad_p, kn, vn, Tn, npad_n, scale, tau, alpha, **kw):
        """Head-split NAG: gather Z+ and Z- from all ranks, then blend on full rows (the norm spans all heads)."""
        self.attention(0, q, kp, vp, Tp, npad_p, wait=False, **kw)
        self.attention(1, q, kn, vn, Tn, npad_n, wait=False, **kw)
        self.wait(0)
        self.wait(1)
        zp = self.output(0)
        ops.nag_combine(zp, self.output(1), scale, tau, alpha)
        return zp

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
