"""Parity of the CUDA engine against the CPU oracle, through the public C API.

Every case of tests/cases.py is executed on cuda:0 with each implementation
that accepts it and compared with the oracle on the same seeded inputs:
  * the generic kernel performs the reference's operations in the reference's
    order, so it must match bit for bit -- integer and float destinations alike
    (the oracle runs with the portable tanh the kernels share; transcendental
    eltwise kinds other than tanh may differ by an ulp of the function value and
    are compared with rtol 1e-5);
  * the int8 tensor-core kernel sums the products exactly in s32 and applies the
    scales once, as the reference's optimised CPU implementation and its
    documented formula do, whereas the reference's scalar implementation converts
    every product to f32 and accumulates in f32.  It is therefore compared with
    the oracle in its exact-accumulation mode: integer destinations bit-exact,
    f32 within 1e-5.  tests/test_oracle_vs_reference.py bounds the distance
    between the two accumulation modes;
  * the fp8 and decode kernels accumulate in f32 in another order and are held to
    the case's tolerance (rtol 1e-2).
"""
import numpy as np
import pytest

import cases
from parity import assert_bit_exact, assert_close
from onednn_b200 import api, dtypes as dt, workloads as W
from oracle import binding as B

pytestmark = pytest.mark.gpu

LIBM_ALGS = {W.ELTWISE[k] for k in ("elu", "soft_relu", "logistic", "exp", "swish", "log", "pow", "gelu_erf", "mish")}


@pytest.fixture(scope="module")
def ctx():
    eng = api.Engine()
    return eng, api.Stream(eng)


def _uses_libm(case):
    return any(p.kind == W.PO_ELTWISE and p.alg in LIBM_ALGS for p in case.post_ops)


@pytest.mark.parametrize("name", list(cases.CASES))
def test_generic_kernel_bit_exact(ctx, name):
    c = cases.build(name)
    want = B.run_oracle(c, tanh_mode=1)
    got, impl = api.run_case(c, *ctx, weights="plain", impl="generic")
    assert impl == "cuda:generic"
    if _uses_libm(c):
        # exp / erf / log ... come from CUDA's double-precision library rounded to float,
        # the oracle's from glibc's float functions: equal up to an ulp of the function value
        c.exact, c.rtol, c.atol = False, max(c.rtol, 1e-5), max(c.atol, 1e-6)
        assert_close(c, got, want, name)
    else:
        assert_bit_exact(got, want, name)


@pytest.mark.parametrize("name", list(cases.CASES))
@pytest.mark.parametrize("weights", ["any", "plain"])
def test_dispatched_kernel(ctx, name, weights):
    c = cases.build(name)
    plan = api.CasePlan(c, *ctx, weights=weights)
    if plan.impl == "cuda:generic":
        pytest.skip("only the generic kernel accepts this case")
    plan.execute()
    got = plan.result()
    # the tensor-core kernel sums the products exactly in s32 and scales once
    want = B.run_oracle(c, tanh_mode=1, exact_acc=1 if "tcgen05_i8" in plan.impl else 0)
    if "wc_tcgen05" in plan.impl:
        # this kernel rounds every decompressed weight to bf16 (fpmath bf16 permits it): the error
        # of a sum is about 1e-3 of the sum's typical size whatever the element's own value, so the
        # absolute part of the tolerance is 1e-2 of the root-mean-square output
        c.atol = max(c.atol, 1e-2 * float(np.sqrt(np.mean(dt.to_f32(want, c.dst_dt).astype(np.float64) ** 2))))
    assert_close(c, got, want, "%s via %s" % (name, plan.impl))


@pytest.mark.parametrize("name", [n for n in cases.CASES])
def test_tensor_core_kernel_as_cta_pair(ctx, name, monkeypatch):
    """The two-CTA form of the int8 / fp8 kernel (tcgen05 cta_group::2), which the dispatcher
    picks by itself only for large problems, forced on every case with more than 128 rows:
    same result as the oracle, and bit for bit the single-CTA kernel's."""
    c = cases.build(name)
    if c.M <= 128:
        pytest.skip("one row tile: nothing to pair")
    monkeypatch.setenv("ONEDNN_B200_TC8_PAIR", "0")
    plan = api.CasePlan(c, *ctx, weights="any")
    if "tcgen05_i8" not in plan.impl and "tcgen05_f8" not in plan.impl:
        pytest.skip("not a case of this kernel")
    plan.execute()
    single = plan.result()
    monkeypatch.setenv("ONEDNN_B200_TC8_PAIR", "1")
    plan.reset_dst()
    plan.execute()
    paired = plan.result()
    assert np.array_equal(np.ascontiguousarray(single).view(np.uint8), np.ascontiguousarray(paired).view(np.uint8))
    want = B.run_oracle(c, tanh_mode=1, exact_acc=1 if "tcgen05_i8" in plan.impl else 0)
    assert_close(c, paired, want, "%s via the CTA-pair kernel" % name)


def test_fast_kernels_are_dispatched(ctx):
    eng, strm = ctx
    assert api.CasePlan(cases.build("c1_small"), eng, strm, upload=False).impl == "cuda:sm100:tcgen05_i8"
    assert api.CasePlan(cases.build("c3_small"), eng, strm, upload=False).impl == "cuda:sm100:tcgen05_f8"
    assert api.CasePlan(W.config2(1, 256, 512), eng, strm, upload=False).impl == "cuda:sm100:wc_gemv"


def test_repeated_execution_and_sum_in_place(ctx):
    """sum reads the destination in place: a second execution consumes the first one's output."""
    c = cases.build("c1_small_nonsat")
    plan = api.CasePlan(c, *ctx)
    plan.execute()
    first = plan.result()
    plan.execute()
    second = plan.result()
    c2 = cases.build("c1_small_nonsat")
    c2.dst_init = first
    assert_bit_exact(second, B.run_oracle(c2, tanh_mode=1, exact_acc=1))


def test_zero_dim_is_a_no_op(ctx):
    eng, strm = ctx
    src = api.Memory(api.MemoryDesc((0, 32), dt.S8, api.TAG_AB), eng)
    wei = api.Memory(api.MemoryDesc((32, 16), dt.S8, api.TAG_AB), eng)
    dst = api.Memory(api.MemoryDesc((0, 16), dt.S32, api.TAG_AB), eng)
    pd = api.matmul_primitive_desc(eng, src.md, wei.md, dst.md)
    api.Primitive(pd).execute(strm, {api.ARG_SRC: src, api.ARG_WEIGHTS: wei, api.ARG_DST: dst})
    strm.wait()


def test_missing_runtime_scale_argument_is_rejected(ctx):
    c = cases.build("c0_small")
    plan = api.CasePlan(c, *ctx, impl="generic", weights="plain")
    del plan.args[api.ARG_ATTR_SCALES | api.ARG_WEIGHTS]
    with pytest.raises(api.Error) as e:
        plan.execute()
    assert e.value.name == "invalid_arguments"


def test_user_scratchpad_mode(ctx):
    eng, strm = ctx
    c = W.config2(3, 256, 512)
    want = B.run_oracle(c)
    plan = api.CasePlan(c, eng, strm, upload=False)
    plan.attr.set_scratchpad_mode(1)
    plan2 = api.CasePlan(c, eng, strm)          # library mode as the yardstick
    plan2.execute()
    assert_close(c, plan2.result(), want)


def test_map_unmap_round_trip(ctx):
    eng, _ = ctx
    a = np.arange(6 * 10, dtype=np.float32).reshape(6, 10)
    m = api.Memory(api.MemoryDesc(a.shape, dt.F32, api.TAG_AB), eng)
    m.write(a)
    assert np.array_equal(m.read(np.float32, a.shape), a)


def test_reorder_plain_and_convert(ctx):
    eng, strm = ctx
    r = np.random.default_rng(3)
    a = r.normal(0, 50, (37, 53)).astype(np.float32)
    src = api.Memory(api.MemoryDesc(a.shape, dt.F32, api.TAG_AB), eng)
    src.write(a)
    # f32 ab -> s8 ba: saturate, round to nearest even, transpose
    dmd = api.MemoryDesc(a.shape, dt.S8, api.TAG_BA)
    dst = api.Memory(dmd, eng)
    api.Primitive(api.reorder_primitive_desc(eng, src.md, eng, dmd)).execute(strm, {api.ARG_FROM: src, api.ARG_TO: dst})
    strm.wait()
    got = dst.read(np.int8, (53, 37)).T
    want = np.clip(np.rint(a), -128, 127).astype(np.int8)
    assert np.array_equal(got, want)


def test_bounded_wait_reports_and_context_survives(ctx):
    """A wait that cannot succeed gives up after its bound, the stream reports
    dnnl_runtime_error once, and the same stream and context keep working."""
    eng, strm = ctx
    L = api.lib()
    L.dnnl_b200_stream_selftest_bounded_wait.argtypes = [api.C.c_void_p, api.C.c_uint]
    assert L.dnnl_b200_stream_selftest_bounded_wait(strm.h, 2000) == 0      # about 0.2 ms of polling
    with pytest.raises(api.Error) as e:
        strm.wait()
    assert e.value.status == 5                                               # dnnl_runtime_error
    strm.wait()                                                              # the flag was cleared
    c = cases.build("c1_small")
    got, impl = api.run_case(c, eng, strm)
    want = B.run_oracle(c, tanh_mode=1, exact_acc=1)
    assert_close(c, got, want, "after a reported wait timeout")
