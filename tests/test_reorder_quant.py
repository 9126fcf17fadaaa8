"""Quantising reorder: the oracle against the reference (stored outputs and, where the
reference library has been built, the library itself), and the CUDA engine against the oracle.

Every step of this operation is one f32 operation on one element, so every destination
type is compared bit for bit.
"""
from pathlib import Path

import numpy as np
import pytest

import cases
from golden.make_golden import reorder_input_digest
from onednn_b200 import dtypes as dt
from onednn_b200.workloads import Quant
from oracle import binding as B

GOLD = np.load(Path(__file__).parent / "golden" / "reorder_outputs.npz")
NAMES = list(cases.REORDER_CASES)


def _bytes(a):
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_golden(name):
    c = cases.build_reorder(name)
    if str(GOLD[name + "/inputs_sha256"]) != reorder_input_digest(c):
        pytest.skip("numpy produced different inputs than when the fixture was made")
    got, want = _bytes(B.run_oracle_reorder(c)), GOLD[name + "/bytes"]
    assert np.array_equal(got, want), "%d of %d bytes differ" % (int((got != want).sum()), want.size)


def test_every_reorder_case_has_a_fixture_and_both_reference_implementations_are_covered():
    impls = set()
    for name in NAMES:
        assert name + "/bytes" in GOLD.files
        impls.add(str(GOLD[name + "/impl"]))
    assert {"jit:uni", "simple:any"} <= impls


@pytest.mark.skipif(not B.have_reference(), reason="reference library not built here")
@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_library(name):
    c = cases.build_reorder(name)
    want, impl = B.run_reference_reorder(c)
    assert np.array_equal(_bytes(B.run_oracle_reorder(c)), _bytes(want)), impl


def test_oracle_formula_by_hand():
    """dst = sat_rne(src_scale * (src - zp) * (1 / dst_scale) + dst_zp), ties to even."""
    from onednn_b200.workloads import ReorderCase
    src = np.array([[-128, -3, 0, 5, 7, 127, 9, 11]], dtype=np.int8)
    c = ReorderCase("hand", 1, 8, src, dt.S8, dt.U8, src_scale=Quant(np.float32([0.5]), dt.F32, 0),
                    dst_scale=Quant(np.float32([2.0]), dt.F32, 0), src_zp=Quant(np.int32([1]), dt.S32, 0),
                    dst_zp=Quant(np.int32([10]), dt.S32, 0))
    # (s - 1) / 4 + 10: -22.25 -> 0 (saturated), 9, 9.75 -> 10, 11, 11.5 -> 12 (tie to even), 41.5 -> 42, 12, 12.5 -> 12
    assert B.run_oracle_reorder(c).tolist() == [[0, 9, 10, 11, 12, 42, 12, 12]]


# ---- the CUDA engine ---------------------------------------------------------------------------

@pytest.fixture(scope="module")
def ctx():
    from onednn_b200 import api
    eng = api.Engine()
    return eng, api.Stream(eng)


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_cuda_matches_oracle(name, ctx):
    from onednn_b200 import api
    c = cases.build_reorder(name)
    plan = api.ReorderPlan(c, *ctx)
    assert plan.impl == "cuda:reorder_quant"
    plan.execute()
    got, want = _bytes(plan.result()), _bytes(B.run_oracle_reorder(c))
    assert np.array_equal(got, want), "%s: %d of %d bytes differ" % (name, int((got != want).sum()), want.size)


@pytest.mark.gpu
@pytest.mark.parametrize("src_dt,dst_dt,per_row", [(dt.F32, dt.S8, False), (dt.BF16, dt.U8, True), (dt.F32, dt.U8, True)])
def test_cuda_quantize_activations_full_size(src_dt, dst_dt, per_row, ctx):
    """The activations of the 4096 x 4096 int8 benchmark problem, quantised on the device."""
    from onednn_b200 import api, workloads as W
    c = W.quantize_case(4096, 4096, src_dt, dst_dt, per_row=per_row)
    plan = api.ReorderPlan(c, *ctx)
    plan.execute()
    got, want = plan.result(), B.run_oracle_reorder(c)
    assert np.array_equal(got, want)
    # quantise -> dequantise returns every value to within half a quantisation step
    back = W.ReorderCase("dq", c.rows, c.cols, got, dst_dt, dt.F32, src_scale=c.dst_scale, src_zp=c.dst_zp)
    plan2 = api.ReorderPlan(back, *ctx)
    plan2.execute()
    x = dt.to_f32(c.src, src_dt)
    step = c.dst_scale.data.reshape(-1, 1) if per_row else c.dst_scale.data[0]
    lo, hi = (-128, 127) if dst_dt == dt.S8 else (0, 255)
    zp = 0 if c.dst_zp is None else int(c.dst_zp.data[0])
    inside = (x / step + zp > lo) & (x / step + zp < hi)
    err = np.abs(plan2.result() - x)
    assert (err[inside] <= (0.5 * step * np.ones_like(x))[inside] * 1.001 + 1e-6).all()


@pytest.mark.gpu
def test_dynamic_quantisation_pipeline(ctx):
    """f32 activations -> (reorder with per-row scales) -> s8 -> int8 matmul with the same per-row
    source scales and per-column weights scales -> bf16: both primitives on the device, each
    checked against the oracle, the s8 tensor handed from one to the other without leaving HBM."""
    from onednn_b200 import api, workloads as W
    from onednn_b200.workloads import MatmulCase, ReorderCase
    eng, strm = ctx
    M, K, N = 384, 512, 256
    rng = np.random.default_rng(77)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.2, 3.0, (M, 1))).astype(np.float32)
    row_scale = (np.abs(x).max(axis=1) / 127.0).astype(np.float32)
    q = ReorderCase("quantize", M, K, x, dt.F32, dt.S8, dst_scale=Quant(row_scale, dt.F32, 1))
    rplan = api.ReorderPlan(q, eng, strm)
    rplan.execute()
    xq = rplan.result()
    assert np.array_equal(xq, B.run_oracle_reorder(q))

    wei = rng.integers(-127, 128, (K, N), dtype=np.int8)
    c = MatmulCase("dynq", M, N, K, src=xq, src_dt=dt.S8, wei=wei, wei_dt=dt.S8, dst_dt=dt.BF16,
                   src_scale=Quant(row_scale, dt.F32, 3, (1, K)),
                   wei_scale=Quant(rng.uniform(1e-3, 3e-3, N).astype(np.float32), dt.F32, 2),
                   exact=False, rtol=1e-2, atol=1e-2)
    mplan = api.CasePlan(c, eng, strm, weights="any")
    assert mplan.impl == "cuda:sm100:tcgen05_i8"
    # the matmul reads the reorder's destination buffer itself
    mplan.args[api.ARG_SRC] = rplan.mem["dst"]
    mplan.execute()
    got = dt.to_f32(mplan.result(), dt.BF16)
    want = dt.to_f32(B.run_oracle(c, exact_acc=1), dt.BF16)
    assert np.allclose(got, want, rtol=1e-2, atol=1e-2)
    # and the whole thing approximates the f32 product it stands for
    ref = x @ (wei.astype(np.float32) * c.wei_scale.data)
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err < 0.02, err


# ---- tensors with more than two dims -------------------------------------------------------------

def _nd_md(shape, dtype):
    from onednn_b200 import api
    return api.MemoryDesc(tuple(shape), dtype, strides=tuple(int(np.prod(shape[i + 1:])) for i in range(len(shape))))


def test_more_than_two_dims_descriptor_host():
    """Dense row-major tensors of any rank quantised per tensor or per element of the last dim are taken;
    a mask over a middle dim is not."""
    import os
    os.environ["ONEDNN_B200_ALLOW_NO_DEVICE"] = "1"
    from onednn_b200 import api
    eng = api.Engine()
    for mask in (0, 1 << 2):
        a = api.PrimitiveAttr()
        a.set_scales(api.ARG_DST, mask, (), dt.F32)
        pd = api.reorder_primitive_desc(eng, _nd_md((4, 50, 96), dt.F32), eng, _nd_md((4, 50, 96), dt.S8), a)
        assert pd.impl_info_str() == "cuda:reorder_quant"
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_DST, 1 << 1, (), dt.F32)
    with pytest.raises(api.Error) as e:
        api.reorder_primitive_desc(eng, _nd_md((4, 50, 96), dt.F32), eng, _nd_md((4, 50, 96), dt.S8), a)
    assert e.value.name == "unimplemented"


@pytest.mark.gpu
@pytest.mark.parametrize("shape,per_channel", [((4, 50, 96), True), ((2, 3, 20, 64), False)])
def test_cuda_more_than_two_dims(shape, per_channel, ctx):
    """The same bytes as the 2-D reorder of the tensor folded into (prod(leading dims), last dim)."""
    from onednn_b200 import api
    from onednn_b200.workloads import ReorderCase
    eng, strm = ctx
    r = np.random.default_rng(131)
    rows, cols = int(np.prod(shape[:-1])), shape[-1]
    x = (r.standard_normal((rows, cols)) * 30).astype(np.float32)
    scale = r.uniform(0.2, 0.9, cols if per_channel else 1).astype(np.float32)
    folded = ReorderCase("nd", rows, cols, x, dt.F32, dt.U8, dst_scale=Quant(scale, dt.F32, 2 if per_channel else 0),
                         dst_zp=Quant(np.int32([100]), dt.S32, 0))
    want = B.run_oracle_reorder(folded)
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_DST, (1 << (len(shape) - 1)) if per_channel else 0, (), dt.F32)
    a.set_zero_points(api.ARG_DST, 0, (), dt.S32)
    src_md, dst_md = _nd_md(shape, dt.F32), _nd_md(shape, dt.U8)
    prim = api.Primitive(api.reorder_primitive_desc(eng, src_md, eng, dst_md, a))
    src, dst = api.Memory(src_md, eng), api.Memory(dst_md, eng)
    src.write(x)
    sc, zp = api.Memory(api.MemoryDesc((scale.size,), dt.F32, api.TAG_A), eng), api.Memory(api.MemoryDesc((1,), dt.S32, api.TAG_A), eng)
    sc.write(scale)
    zp.write(np.int32([100]))
    prim.execute(strm, {api.ARG_FROM: src, api.ARG_TO: dst, api.ARG_ATTR_SCALES | api.ARG_DST: sc,
                        api.ARG_ATTR_ZERO_POINTS | api.ARG_DST: zp})
    strm.wait()
    got = dst.read(np.uint8, (rows, cols))
    assert np.array_equal(got, want), "%d of %d bytes differ" % (int((got != want).sum()), want.size)
