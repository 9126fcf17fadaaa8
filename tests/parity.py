"""Comparison rules shared by the parity tests."""
import numpy as np

from onednn_b200 import dtypes as dt


def ulp_diff_f32(a, b):
    """Distance in units in the last place between two float32 arrays (NaNs must coincide)."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    ia = a.view(np.int32).astype(np.int64)
    ib = b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7FFFFFFF), ia)
    ib = np.where(ib < 0, -(ib & 0x7FFFFFFF), ib)
    return np.abs(ia - ib)


def assert_bit_exact(got, want, what=""):
    g = np.ascontiguousarray(got).view(np.uint8)
    w = np.ascontiguousarray(want).view(np.uint8)
    assert g.shape == w.shape, "%s: shape %s vs %s" % (what, g.shape, w.shape)
    bad = int((g != w).sum())
    assert bad == 0, "%s: %d of %d bytes differ" % (what, bad, g.size)


def assert_close(case, got, want, what=""):
    """Integer destinations bit-exact; float destinations within the case's tolerance."""
    if case.exact:
        return assert_bit_exact(got, want, what)
    g = dt.to_f32(got, case.dst_dt).astype(np.float64)
    w = dt.to_f32(want, case.dst_dt).astype(np.float64)
    assert np.array_equal(np.isnan(g), np.isnan(w)), "%s: NaN pattern differs" % what
    ok = np.abs(g - w) <= case.atol + case.rtol * np.abs(w)
    ok |= np.isnan(w)
    assert ok.all(), "%s: %d of %d elements outside rtol=%g atol=%g (max abs err %g)" % (
        what, int((~ok).sum()), ok.size, case.rtol, case.atol, float(np.nanmax(np.abs(g - w))))
