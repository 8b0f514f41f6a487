"""kiln_b200: B200 (sm_100a) attention path for the kiln engine's Anima DiT.

The product is the CUDA library behind the C ABI in include/kiln_b200.h; this package holds its
sources (csrc/), the C++ op-set shim the engine links (host/), and a ctypes binding used by the
tests and the benchmark. There is no CPU fallback: every launch entry point fails when the library
or an sm_100 device is missing.
"""
from .ops import (EPI_F16, EPI_F32, EPI_GELU16, EPI_HEADS16, EPI_RESID, KB_BF16, KB_F16, KB_F32, PROF_ATTENTION, PROF_LINEAR,  # noqa: F401
                  PROF_NAG, PROF_NORM_ROPE, KilnError, attn_bwd, attn_cross, attn_nag, attn_nag_push, attn_push, attn_self, bump_counters, check_status, lib, linear16, linear16_qkv,
                  nag_combine, prof_enable, prof_read, qk_prep, wait_arrivals, workspace_bytes)
