"""The benchmark configurations at their full sizes.

The CPU oracle cannot compute these problems in full in a test's time, so each is checked
two ways: a sample of rows x columns against the oracle (every sampled element is a full-K
dot product plus the whole epilogue), and properties that hold for any size -- a shard
computed on its own equals the same rows / columns of the full result bit for bit, permuting
the rows of the inputs permutes the rows of the output, and scaling a power-of-two scale
scales a floating-point output exactly.
"""
import numpy as np
import pytest

from parity import assert_bit_exact
from onednn_b200 import api, dtypes as dt, workloads as W
from onednn_b200.workloads import Quant
from oracle import binding as B

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    eng = api.Engine()
    return eng, api.Stream(eng)


def _run(case, ctx):
    plan = api.CasePlan(case, *ctx, weights="any")
    plan.execute()
    return plan.result(), plan.impl


def _close(case, got, want, what):
    g = dt.to_f32(got, case.dst_dt).astype(np.float64)
    w = dt.to_f32(want, case.dst_dt).astype(np.float64)
    ok = np.abs(g - w) <= case.atol + case.rtol * np.abs(w)
    assert ok.all(), "%s: %d of %d sampled elements outside rtol=%g (max abs err %g)" % (
        what, int((~ok).sum()), ok.size, case.rtol, float(np.abs(g - w).max()))


def test_c1_int8_4096_full_epilogue(ctx):
    """s8 x s8 -> s8, per-N scales, bf16 bias, gelu_tanh + sum, dst scale and zero-point."""
    c = W.config1()
    got, impl = _run(c, ctx)
    assert impl == "cuda:sm100:tcgen05_i8"
    ms, ns = 5, 3   # 820 x 1366 = 1.1 M elements, each a full K = 4096 dot product plus the epilogue
    want = B.run_oracle(c, tanh_mode=1, exact_acc=1, m_step=ms, n_step=ns)
    assert_bit_exact(got[::ms, ::ns], want[::ms, ::ns], "c1 sampled against the oracle")
    # rows 1024..2047 as a problem of their own (M-split shard)
    part = W.shard(c, 1, 4, "m")
    got_part, _ = _run(part, ctx)
    assert_bit_exact(got_part, got[1024:2048], "c1 M-split shard")
    # a row permutation of src and of the prior dst permutes the rows of dst
    perm = np.random.default_rng(1).permutation(c.M)
    import copy
    cp = copy.copy(c)
    cp.src = np.ascontiguousarray(c.src[perm])
    cp.dst_init = np.ascontiguousarray(c.dst_init[perm])
    got_perm, _ = _run(cp, ctx)
    assert_bit_exact(got_perm, got[perm], "c1 row permutation")


@pytest.mark.parametrize("dst_scale", [1.0, 0.35])
def test_c1_epilogue_1024_every_element(ctx, dst_scale):
    """The C1 attribute set at 1024^3 with destination scales that leave most outputs unsaturated
    (the benchmark's own scale saturates six in ten, which hides rounding differences): every one
    of the million s8 outputs against the oracle, bit for bit."""
    c = W.config1(1024, 1024, 1024, seed=20240630, dst_scale=dst_scale)
    got, impl = _run(c, ctx)
    assert impl == "cuda:sm100:tcgen05_i8"
    want = B.run_oracle(c, tanh_mode=1, exact_acc=1)
    sat = float(np.mean((want == 127) | (want == -128)))
    assert sat < 0.5, "the case is meant to be mostly unsaturated (%.2f saturated)" % sat
    assert_bit_exact(got, want, "c1 epilogue at 1024^3, dst scale %g" % dst_scale)


@pytest.mark.parametrize("M", [1, 16, 128])
def test_c2_decode_4096x14336(ctx, M):
    """bf16 x u4 with K-grouped bf16 scales and u4 zero-points."""
    c = W.config2(M)
    got, impl = _run(c, ctx)
    assert impl == ("cuda:sm100:wc_gemv" if M <= 32 else "cuda:sm100:wc_tcgen05")
    ns = 1 if M == 1 else (7 if M == 16 else 61)
    want = B.run_oracle(c, n_step=ns)
    if "tcgen05" in impl:
        # This kernel rounds every decompressed weight to bf16 (relative error up to 2^-9 each,
        # which fpmath bf16 permits), so the error of a K = 4096 sum is about 1e-3 of the sum's
        # typical size whatever the element's own value: the absolute part of the tolerance is
        # 1e-2 of the root-mean-square output instead of a constant.
        import copy
        c = copy.copy(c)
        c.atol = max(c.atol, 1e-2 * float(np.sqrt(np.mean(dt.to_f32(want[:, ::ns], c.dst_dt).astype(np.float64) ** 2))))
    _close(c, got[:, ::ns], want[:, ::ns], "c2 M=%d against the oracle" % M)
    if M > 1:
        # every row on its own is the M = 1 problem of that row (other kernel variant, other
        # summation split): equal within the tolerance
        import copy
        one = copy.copy(c)
        one.M, one.src = 1, np.ascontiguousarray(c.src[M // 2:M // 2 + 1])
        got_one, _ = _run(one, ctx)
        _close(c, got_one, got[M // 2:M // 2 + 1], "c2 row %d alone" % (M // 2))


def test_c3_fp8_8192(ctx):
    c = W.config3()
    got, impl = _run(c, ctx)
    assert impl == "cuda:sm100:tcgen05_f8"
    ms, ns = 257, 263
    want = B.run_oracle(c, m_step=ms, n_step=ns)
    _close(c, got[::ms, ::ns], want[::ms, ::ns], "c3 sampled against the oracle")
    # doubling the (power-of-two) src scale and the bias doubles every bf16 output exactly
    import copy
    c2 = copy.copy(c)
    c2.src_scale = Quant(np.float32([0.5]), dt.F32, 0)
    c2.bias = dt.f32_to_bf16(dt.to_f32(c.bias, dt.BF16) * np.float32(2))
    got2, _ = _run(c2, ctx)
    a, b = dt.to_f32(got, dt.BF16), dt.to_f32(got2, dt.BF16)
    assert np.array_equal(a * np.float32(2), b), "c3: output is not linear in a power-of-two scale"


def test_c4_int8_16384x8192x28672(ctx):
    c = W.config4()
    got, impl = _run(c, ctx)
    assert impl == "cuda:sm100:tcgen05_i8"
    ms, ns = 1021, 1019
    want = B.run_oracle(c, exact_acc=1, m_step=ms, n_step=ns)
    _close(c, got[::ms, ::ns], want[::ms, ::ns], "c4 sampled against the oracle")
    # columns 3584..7167 as a problem of their own (N-split shard of 8): bit for bit
    part = W.shard(c, 1, 8, "n")
    got_part, _ = _run(part, ctx)
    ncol = c.N // 8
    assert_bit_exact(got_part, np.ascontiguousarray(got[:, ncol:2 * ncol]), "c4 N-split shard")
