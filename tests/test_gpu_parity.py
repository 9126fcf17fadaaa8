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
    # weights zero-points (per tensor, per column) stay on the tensor cores
    for name in ("int8_wei_zp_common", "int8_wei_zp_per_n_relu", "int8_wei_zp_gelu_sum"):
        c = cases.build(name)
        if c.K % 16 == 0:
            assert api.CasePlan(c, eng, strm, upload=False).impl == "cuda:sm100:tcgen05_i8", name


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
    """scratchpad_mode::user: the primitive allocates nothing, reports the size it needs and
    works out of the memory passed as DNNL_ARG_SCRATCHPAD; without that argument it refuses."""
    eng, strm = ctx
    c = W.config2(3, 256, 512)
    want = B.run_oracle(c)
    plan = api.CasePlan(c, eng, strm, scratchpad="user")
    assert plan.pd.scratchpad_desc().get_size() > 0 and api.ARG_SCRATCHPAD in plan.args
    for _ in range(2):  # the kernel leaves its partial sums zeroed: a second run must agree too
        plan.execute()
        assert_close(c, plan.result(), want)
    del plan.args[api.ARG_SCRATCHPAD]
    with pytest.raises(api.Error) as e:
        plan.execute()
    assert e.value.name == "invalid_arguments"
    lib_plan = api.CasePlan(c, eng, strm)
    assert lib_plan.pd.scratchpad_desc().get_size() == 0  # library mode: nothing for the user to provide


def _counter(which):
    v = api.C.c_uint64()
    assert api.lib().dnnl_b200_debug_counter(which, api.C.byref(v)) == 0
    return v.value


def test_scratchpad_is_cleared_again_after_a_reported_failure(ctx):
    """A kernel that gave up may leave partial sums behind; after the stream reported it (here:
    the host-side hook that stands for that report) the next execution of every primitive with a
    library scratchpad clears it first, exactly once."""
    eng, strm = ctx
    c = W.config2(2, 256, 512)
    want = B.run_oracle(c)
    plan = api.CasePlan(c, eng, strm)
    plan.execute()
    assert_close(c, plan.result(), want)
    before = _counter(2)
    plan.execute()
    strm.wait()
    assert _counter(2) == before               # clean: trusted
    assert api.lib().dnnl_b200_debug_mark_scratchpads_dirty() == 0
    plan.execute()
    assert_close(c, plan.result(), want)
    assert _counter(2) == before + 1           # cleared on the stream before the kernel
    plan.execute()
    assert_close(c, plan.result(), want)
    assert _counter(2) == before + 1


def test_allocation_failure_is_reported_as_out_of_memory(ctx):
    """Host-side injection: the library's next allocations fail; memory and primitive creation
    return dnnl_out_of_memory and later calls work again."""
    eng, strm = ctx
    L = api.lib()
    md = api.MemoryDesc((64, 64), dt.F32, api.TAG_AB)
    assert L.dnnl_b200_debug_fail_allocations(1) == 0
    with pytest.raises(api.Error) as e:
        api.Memory(md, eng)
    assert e.value.name == "out_of_memory"
    api.Memory(md, eng)  # the injection is used up
    c = W.config2(2, 256, 512)
    plan = api.CasePlan(c, eng, strm)
    assert L.dnnl_b200_debug_fail_allocations(1) == 0
    with pytest.raises(api.Error) as e:
        api.Primitive(plan.pd)  # its library scratchpad cannot be allocated
    assert e.value.name == "out_of_memory"
    api.Primitive(plan.pd)
    assert L.dnnl_b200_debug_fail_allocations(0) == 0


def test_stream_profiling_returns_one_entry_per_execution():
    """dnnl_stream_profiling + dnnl_query_profiling_data (reference: src/common/stream.cpp,
    include/oneapi/dnnl/dnnl.h experimental profiling): one device time per execute call."""
    eng = api.Engine()
    strm = api.Stream(eng, flags=1 | 4)  # in_order | profiling
    c = cases.build("c1_small")
    plan = api.CasePlan(c, eng, strm)
    n0 = api.C.c_int(0)
    L = api.lib()
    assert L.dnnl_reset_profiling(strm.h) == 0
    for _ in range(3):
        plan.execute()
    strm.wait()
    assert L.dnnl_query_profiling_data(strm.h, 1, api.C.byref(n0), None) == 0
    assert n0.value == 3
    data = (api.C.c_uint64 * 3)()
    assert L.dnnl_query_profiling_data(strm.h, 1, api.C.byref(n0), data) == 0
    assert all(0 < t < 10**9 for t in data)  # nanoseconds, well under a second each
    assert L.dnnl_reset_profiling(strm.h) == 0
    assert L.dnnl_query_profiling_data(strm.h, 1, api.C.byref(n0), None) == 0 and n0.value == 0
    plain = api.Stream(eng)
    assert L.dnnl_query_profiling_data(plain.h, 1, api.C.byref(n0), None) == 2  # not a profiling stream


def test_primitive_cache_hits_and_eviction(ctx):
    """Creating the same primitive twice is a cache hit; the cache never holds more entries than
    its capacity (reference: doc/advanced/primitive_cache.md)."""
    eng, strm = ctx
    L = api.lib()
    cap = api.C.c_int()
    assert L.dnnl_get_primitive_cache_capacity(api.C.byref(cap)) == 0
    try:
        assert L.dnnl_set_primitive_cache_capacity(2) == 0
        plans = [api.CasePlan(W.config0(16 * (i + 1), 32, 64), eng, strm, upload=False) for i in range(3)]
        assert _counter(1) <= 2
        hits = _counter(0)
        api.Primitive(plans[2].pd)      # most recent: still cached
        assert _counter(0) == hits + 1
        api.Primitive(plans[0].pd)      # evicted when the third was created
        assert _counter(0) == hits + 1
        assert _counter(1) <= 2
    finally:
        L.dnnl_set_primitive_cache_capacity(cap.value)


def test_verbose_lines_have_the_reference_shape(tmp_path):
    """ONEDNN_VERBOSE=2 prints one create and one exec line per call in the reference's CSV shape
    (doc/performance_considerations/verbose.md:22-45): marker, version, component, operation,
    engine, primitive, implementation, prop kind, memory descriptors, attributes, auxiliary,
    problem, time."""
    import os
    import subprocess
    import sys
    prog = (
        "import sys; sys.path.insert(0, %r); sys.path.insert(0, %r)\n"
        "import cases\nfrom onednn_b200 import api\n"
        "eng = api.Engine(); s = api.Stream(eng)\n"
        "p = api.CasePlan(cases.build('c1_small'), eng, s)\np.execute(); p.execute(); s.wait()\n"
    ) % (str(api._PKG.parent), str(api._PKG.parent / "tests"))
    env = dict(os.environ, ONEDNN_VERBOSE="2")
    out = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.startswith("onednn_verbose,")]
    execs = [l for l in lines if ",primitive,exec," in l and ",matmul," in l]
    creates = [l for l in lines if ",primitive,create:" in l and ",matmul," in l]
    assert len(execs) == 2 and len(creates) >= 1
    f = execs[0].split(",")
    assert len(f) == 13
    assert f[:4] == ["onednn_verbose", "v1", "primitive", "exec"] and f[4].startswith("gpu")
    assert f[5] == "matmul" and f[6] == "cuda:sm100:tcgen05_i8" and f[7] == "undef"
    assert f[8].startswith("src:s8::") and " wei:s8:" in f[8] and " dst:s8::" in f[8]
    assert "attr-scales:" in f[9] and "attr-post-ops:" in f[9]
    assert f[-2] == "96x256:256x128" and float(f[-1]) >= 0.0


@pytest.mark.parametrize("name", cases.tame_names())
@pytest.mark.parametrize("weights", ["any", "plain"])
def test_tensor_core_kernel_vs_reference_bytes(ctx, name, weights):
    """The int8 catalogue on data whose f32 sums are exact: there the bytes stored from the
    reference's own scalar implementation are what the tensor-core kernel must produce, with
    no oracle mode in between."""
    import hashlib
    from pathlib import Path
    from golden.make_golden import input_digest
    gold = np.load(Path(__file__).parent / "golden" / "reference_outputs.npz")
    c = cases.build(name)
    if str(gold[name + "/inputs_sha256"]) != input_digest(c):
        pytest.skip("numpy produced different inputs than when the fixture was made")
    plan = api.CasePlan(c, *ctx, weights=weights)
    if "tcgen05_i8" not in plan.impl:
        pytest.skip("not a case of the tensor-core kernel")
    plan.execute()
    got = np.ascontiguousarray(plan.result())
    raw = got.view(np.uint8).reshape(-1)
    want = gold[name + "/bytes"]
    if c.exact or not _uses_tanh_or_libm(c):
        assert np.array_equal(raw if raw.size <= 65536 else raw[::61], want)
        assert hashlib.sha256(raw.tobytes()).hexdigest() == str(gold[name + "/sha256"])
    else:
        # float destination behind a transcendental: the functions differ from glibc's by an ulp
        assert raw.size <= 65536
        w = dt.to_f32(want.view(dt.RAW[c.dst_dt]).reshape(c.M, c.N), c.dst_dt).astype(np.float64)
        g = dt.to_f32(got, c.dst_dt).astype(np.float64)
        assert np.all(np.abs(g - w) <= 1e-6 + 1e-5 * np.abs(w))


def _uses_tanh_or_libm(case):
    tanh_like = {W.ELTWISE[k] for k in ("tanh", "gelu_tanh")}
    return _uses_libm(case) or any(p.kind == W.PO_ELTWISE and p.alg in tanh_like for p in case.post_ops)


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
