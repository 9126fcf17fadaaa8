"""Oracle vs the reference library run live (only where oracle/_ref was built).

Bit-for-bit equality against the reference's scalar implementations, and a
report of how the reference's own JIT differs from them.
"""
import numpy as np
import pytest

import cases
from onednn_b200 import dtypes as dt
from onednn_b200 import workloads as W
from oracle import binding as B

pytestmark = pytest.mark.skipif(not B.have_reference(), reason="oracle/_ref not built on this machine")


@pytest.mark.parametrize("name", list(cases.CASES))
def test_bit_exact_vs_reference_scalar_impl(name):
    c = cases.build(name)
    ref, impl, _, _ = B.run_reference(c, impl="ref")
    assert impl in ("ref_int8:any", "ref:any")
    out = B.run_oracle(c)
    assert np.array_equal(out.view(np.uint8), ref.view(np.uint8))


@pytest.mark.parametrize("name", cases.tame_names())
def test_exact_accumulation_bit_exact_vs_reference_on_exact_sums(name):
    """The whole int8 attribute catalogue on small integers and power-of-two scales, where the
    reference's f32 accumulation is exact: its output, the oracle's and the oracle's
    exact-accumulation mode agree bit for bit (with the portable tanh as well)."""
    c = cases.build(name)
    ref, impl, _, _ = B.run_reference(c, impl="ref")
    assert impl == "ref_int8:any"
    for kw in (dict(), dict(exact_acc=1)):
        out = B.run_oracle(c, **kw)
        assert np.array_equal(out.view(np.uint8), ref.view(np.uint8)), kw
    # the portable tanh the kernels share differs from libm's tanhf by at most an ulp of an f32
    # result; it must not move an integer output
    out = B.run_oracle(c, exact_acc=1, tanh_mode=1)
    if c.exact:
        assert np.array_equal(out.view(np.uint8), ref.view(np.uint8))
    else:
        g, w = dt.to_f32(out, c.dst_dt).astype(np.float64), dt.to_f32(ref, c.dst_dt).astype(np.float64)
        assert np.all(np.abs(g - w) <= 1e-6 + 1e-5 * np.abs(w))


def test_portable_tanh_changes_no_int8_output():
    """The kernels use a portable double-precision tanh instead of libm's tanhf; on the
    benchmark's requantised configuration that must not move any s8 output."""
    c = W.config1(512, 512, 512, dst_scale=1.0)
    ref, _, _, _ = B.run_reference(c, impl="ref")
    out = B.run_oracle(c, tanh_mode=1)
    assert int((out != ref).sum()) == 0


def test_reference_jit_vs_scalar_differs_by_at_most_one_lsb():
    c = W.config1(512, 512, 512)
    ref, _, _, _ = B.run_reference(c, impl="ref")
    jit, impl, _, _ = B.run_reference(c, impl="", weights_any=True)
    d = np.abs(ref.astype(np.int32) - jit.astype(np.int32))
    assert d.max() <= 1
    assert (d != 0).mean() < 1e-3


def test_sampled_oracle_equals_full():
    c = cases.build("c1_small_nonsat")
    full = B.run_oracle(c)
    part = B.run_oracle(c, m_step=7, n_step=5, m0=3, n0=1)
    assert np.array_equal(part[3::7, 1::5], full[3::7, 1::5])
    mask = np.ones_like(full, dtype=bool)
    mask[3::7, 1::5] = False
    assert np.array_equal(part[mask], c.dst_init[mask])


def test_exact_accumulation_mode_is_within_one_lsb_of_the_scalar_reference():
    """The tensor-core kernel is checked against the oracle's exact-accumulation mode; this
    bounds how far that mode is from the reference's scalar implementation (which
    accumulates the scaled products in f32) and from its JIT implementation."""
    c = W.config1(512, 512, 512, dst_scale=1.0)
    ref, _, _, _ = B.run_reference(c, impl="ref")
    jit, _, _, _ = B.run_reference(c, impl="", weights_any=True)
    exact = B.run_oracle(c, tanh_mode=1, exact_acc=1)
    for other in (ref, jit):
        d = np.abs(exact.astype(np.int32) - other.astype(np.int32))
        assert d.max() <= 1
        assert (d != 0).mean() < 2e-4


def test_exact_accumulation_equals_reference_when_sums_are_exact():
    """Integer products summed in f32 are exact while they stay below 2^24: there the two modes agree."""
    c = cases.build("int8_plain_s32")
    ref, _, _, _ = B.run_reference(c, impl="ref")
    assert np.array_equal(B.run_oracle(c, exact_acc=1), ref)
