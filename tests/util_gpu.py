"""Helpers shared by the GPU parity tests: seeded inputs, the oracle on sampled rows, error metrics."""
import numpy as np
import torch

import oracle

TOL_MAX_ABS = 2e-3     # the path's stated tolerance against an fp32 reference
TOL_MEAN_REL = 1e-3

DT = {"f16": torch.float16, "bf16": torch.bfloat16}
KIND = {"f16": 0, "bf16": 1}


def seeded(seed, rows, cols, kind, amp=1.0):
    """fp32 N(0, amp^2) from the oracle's torch-compatible generator, rounded once through the 16-bit type."""
    x = oracle.randn(seed, rows * cols) * np.float32(amp)
    return oracle.round16(x, KIND[kind]).reshape(rows, cols)


def dev(x, kind=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t if kind is None else t.to(DT[kind])


def errors(out, ref):
    out = np.asarray(out, np.float64)
    ref = np.asarray(ref, np.float64)
    d = np.abs(out - ref)
    return d.max(), d.sum() / np.abs(ref).sum(), np.sqrt((d * d).sum() / (ref * ref).sum())


def assert_close(out, ref, what, max_abs=TOL_MAX_ABS, mean_rel=TOL_MEAN_REL):
    assert not np.isnan(np.asarray(out, np.float32)).any(), f"{what}: NaN in output"
    e_max, e_rel, e_l2 = errors(out, ref)
    assert e_max <= max_abs and e_rel <= mean_rel, f"{what}: max_abs {e_max:.3e} mean_rel {e_rel:.3e} rel_l2 {e_l2:.3e}"
    return e_max, e_rel, e_l2


def sample_rows(T, n, seed=0):
    """Row indices covering the first/last tiles plus a seeded sample: attention rows are independent,
    so the oracle on sampled query rows is exact for them at the full K/V size."""
    rng = np.random.RandomState(seed)
    fixed = [0, 1, 127, 128, 255, 256, T - 129, T - 128, T - 2, T - 1]
    idx = sorted(set([i for i in fixed if 0 <= i < T] + list(rng.randint(0, T, size=n))))
    return np.array(idx, np.int64)


def assert_close_bf16_storage(out, ref, what):
    """For outputs STORED as bf16: rounding to 8 significant bits alone moves a value by up to 2^-9 of its
    magnitude (half an ulp, 3.9e-3 for |x| in [1, 2)), so the stated tolerance applies on top of that
    quantisation. The same kernel with fp32 output is held to the plain tolerance elsewhere."""
    out = np.asarray(out, np.float64)
    ref = np.asarray(ref, np.float64)
    assert not np.isnan(out).any(), f"{what}: NaN in output"
    d = np.abs(out - ref)
    bound = TOL_MAX_ABS + np.abs(ref) * 2.0 ** -8
    assert np.all(d <= bound), f"{what}: worst excess {np.max(d - bound):.3e}"
    assert d.sum() / np.abs(ref).sum() <= TOL_MEAN_REL + 2.0 ** -9, f"{what}: mean_rel {d.sum() / np.abs(ref).sum():.3e}"
