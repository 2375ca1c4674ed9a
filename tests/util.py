"""Helpers shared by the parity tests."""
import numpy as np


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


def assert_same(got, want, what=""):
    """Bit-exact comparison (fp32 compared as bit patterns)."""
    got = np.ascontiguousarray(got); want = np.ascontiguousarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert got.dtype == want.dtype, (what, got.dtype, want.dtype)
    bad = np.count_nonzero(bits(got) != bits(want))
    assert bad == 0, f"{what}: {bad} of {got.size} elements differ"


def max_abs_rel(got, want):
    """max |got-want| / max|want|  (the 'max-abs-rel' measure of the fp32 tolerance)."""
    got = np.asarray(got, np.float64); want = np.asarray(want, np.float64)
    d = np.abs(got - want).max() if got.size else 0.0
    return d / max(np.abs(want).max(), 1e-30)


def to_np(t):
    return t.detach().cpu().numpy()
