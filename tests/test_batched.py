"""Batched matmul (leading batch dims, equal or broadcast): every batch index must equal the
2-D problem of its slices, which the oracle computes (src/common/matmul.cpp:374-401)."""
import os

import numpy as np
import pytest

os.environ["ONEDNN_B200_ALLOW_NO_DEVICE"] = "1"  # descriptor-only engine where there is no GPU

from onednn_b200 import api, dtypes as dt, workloads as W
from onednn_b200.workloads import MatmulCase, Quant
from oracle import binding as B


def _md(shape, dtype):
    return api.MemoryDesc(tuple(shape), dtype, strides=tuple(int(np.prod(shape[i + 1:])) for i in range(len(shape))))


def test_batched_descriptor_host():
    """Dispatch of the 2-D slice, masks moved down with the dims, queries keep the batch dims."""
    eng = api.Engine()
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_WEIGHTS, 1 << 2, (), dt.F32)          # per-N of a 3-D weights tensor
    pd = api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), _md((3, 64, 48), dt.S8), _md((3, 70, 48), dt.F32), attr=a)
    assert pd.impl_info_str() == "cuda:sm100:tcgen05_i8"
    assert pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS).dims == [48]
    assert pd.weights_desc().dims == [3, 64, 48]
    # `any` weights of a batched problem take the packed layout slice by slice: an opaque descriptor with the
    # batch dims, three times the size of a slice (each rounded up to 256 bytes)
    any_w = api.MemoryDesc((3, 64, 48), dt.S8, api.TAG_ANY)
    pd = api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), any_w, _md((3, 70, 48), dt.F32))
    wq = pd.weights_desc()
    assert wq.format_kind == 3 and wq.dims == [3, 64, 48]
    one = api.matmul_primitive_desc(eng, _md((70, 64), dt.S8), api.MemoryDesc((64, 48), dt.S8, api.TAG_ANY), _md((70, 48), dt.F32))
    slice_bytes = one.weights_desc().get_size()
    assert wq.get_size() == 3 * ((slice_bytes + 255) // 256 * 256)
    # and that descriptor is accepted back as the weights of the same problem
    pd2 = api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), wq, _md((3, 70, 48), dt.F32))
    assert pd2.impl_info_str() == pd.impl_info_str() and pd2.weights_desc() == wq
    api.reorder_primitive_desc(eng, _md((3, 64, 48), dt.S8), eng, wq)
    # broadcast weights are fine, mismatched batch dims are not
    api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), _md((1, 64, 48), dt.S8), _md((3, 70, 48), dt.F32))
    with pytest.raises(api.Error):
        api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), _md((2, 64, 48), dt.S8), _md((3, 70, 48), dt.F32))
    # weights scales over the batch dim (one set of per-N values per batch index): taken, on the fast kernel
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_WEIGHTS, 1 | 4, (), dt.F32)
    pd = api.matmul_primitive_desc(eng, _md((3, 70, 64), dt.S8), _md((3, 64, 48), dt.S8), _md((3, 70, 48), dt.F32), attr=a)
    assert pd.impl_info_str() == "cuda:sm100:tcgen05_i8"


def _run_batched(eng, strm, batch, wbatch, base: MatmulCase, binary=None, weights_any=False):
    """``base`` holds the tensors with leading batch dims; returns (result, impl).  With
    ``weights_any`` the weights go through the implementation's packed layout: queried from the
    primitive descriptor, filled by a reorder from the plain tensor."""
    nd = len(batch)
    M, N, K = base.M, base.N, base.K
    attr = api.PrimitiveAttr()
    for q, arg, is_zp in ((base.src_scale, api.ARG_SRC, False), (base.wei_scale, api.ARG_WEIGHTS, False),
                          (base.dst_scale, api.ARG_DST, False), (base.src_zp, api.ARG_SRC, True), (base.dst_zp, api.ARG_DST, True)):
        if q is not None:
            (attr.set_zero_points if is_zp else attr.set_scales)(arg, q.mask << nd, (), q.dt)
    po = api.PostOps()
    for e in base.post_ops:
        if e.kind == W.PO_ELTWISE:
            po.append_eltwise(e.alg, e.alpha, e.beta)
    src1_md = None
    if binary is not None:
        src1_md = _md(binary.shape, dt.F32)
        po.append_binary(W.BINARY["add"], src1_md)
    attr.set_post_ops(po)
    src_md, wei_md = _md(batch + (M, K), base.src_dt), _md(wbatch + (K, N), base.wei_dt)
    dst_md = _md(batch + (M, N), base.dst_dt)
    bias_md = _md((1,) * nd + (1, N), base.bias_dt) if base.bias is not None else None
    plain_wei_md = wei_md
    if weights_any:
        wei_md = api.MemoryDesc(wbatch + (K, N), base.wei_dt, api.TAG_ANY)
    pd = api.matmul_primitive_desc(eng, src_md, wei_md, dst_md, bias_md, attr)
    prim = api.Primitive(pd)
    mems = []

    def mem(md, arr):
        m = api.Memory(md, eng)
        m.write(np.ascontiguousarray(arr))
        mems.append(m)
        return m
    args = {api.ARG_SRC: mem(src_md, base.src), api.ARG_WEIGHTS: mem(plain_wei_md, base.wei),
            api.ARG_DST: mem(dst_md, np.zeros(batch + (M, N), dt.RAW[base.dst_dt]))}
    if weights_any:
        wq = pd.weights_desc()
        assert wq.format_kind == 3, "expected a packed layout for `any` weights"
        packed = api.Memory(wq, eng)
        mems.append(packed)
        api.Primitive(api.reorder_primitive_desc(eng, plain_wei_md, eng, wq)).execute(
            strm, {api.ARG_FROM: args[api.ARG_WEIGHTS], api.ARG_TO: packed})
        args[api.ARG_WEIGHTS] = packed
    if base.bias is not None:
        args[api.ARG_BIAS] = mem(bias_md, base.bias)
    for q, arg in ((base.src_scale, api.ARG_ATTR_SCALES | api.ARG_SRC), (base.wei_scale, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS),
                   (base.dst_scale, api.ARG_ATTR_SCALES | api.ARG_DST), (base.src_zp, api.ARG_ATTR_ZERO_POINTS | api.ARG_SRC),
                   (base.dst_zp, api.ARG_ATTR_ZERO_POINTS | api.ARG_DST)):
        if q is not None:
            args[arg] = mem(api.MemoryDesc((q.data.size,), q.dt, api.TAG_A), q.data)
    if binary is not None:
        args[api.arg_post_op(len(base.post_ops)) | api.ARG_SRC_1] = mem(src1_md, binary)
    prim.execute(strm, args)
    strm.wait()
    return args[api.ARG_DST].read(dt.RAW[base.dst_dt], batch + (M, N)), pd.impl_info_str()


def _slice_case(base, b, wb, binary=None):
    import copy
    c = copy.copy(base)
    c.src, c.wei = np.ascontiguousarray(base.src[b]), np.ascontiguousarray(base.wei[wb])
    c.post_ops = list(base.post_ops)
    if binary is not None:
        sl = binary[tuple(0 if binary.shape[d] == 1 else b[d] for d in range(len(b)))]
        c.post_ops.append(W.binary("add", np.ascontiguousarray(sl), dt.F32, sl.shape))
    return c


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["int8_3d", "int8_bcast_weights_binary", "fp8_4d", "int8_3d_packed", "fp8_4d_packed",
                                  "int8_bcast_weights_packed"])
def test_batched_matches_oracle_per_slice(kind):
    eng = api.Engine()
    strm = api.Stream(eng)
    r = np.random.default_rng(91)
    packed = kind.endswith("_packed")  # weights as format_tag::any: packed once, slice by slice
    kind = kind[:-len("_packed")] if packed else kind
    if kind == "int8_bcast_weights":
        kind = "int8_bcast_weights_binary"
    if kind == "fp8_4d":
        batch, wbatch, (M, N, K) = (2, 2), (2, 2), (40, 64, 96)
        base = W.config3(M, N, K, seed=92)
        base.src = dt.from_f32(r.uniform(-2, 2, batch + (M, K)).astype(np.float32), dt.F8_E4M3)
        base.wei = dt.from_f32(r.uniform(-2, 2, wbatch + (K, N)).astype(np.float32), dt.F8_E4M3)
    else:
        batch, (M, N, K) = (3,), (70, 48, 64)
        wbatch = (3,) if kind == "int8_3d" else (1,)
        base = MatmulCase(kind, M, N, K, src=r.integers(-128, 128, batch + (M, K), dtype=np.int8), src_dt=dt.S8,
                          wei=r.integers(-127, 128, wbatch + (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dt.F32,
                          src_scale=Quant(np.float32([0.02]), dt.F32, 0),
                          wei_scale=Quant(r.uniform(1e-3, 4e-3, N).astype(np.float32), dt.F32, 2),
                          bias=r.uniform(-1, 1, (1, N)).astype(np.float32), bias_dt=dt.F32,
                          post_ops=[W.eltwise("relu", 0.0)], exact=False, rtol=1e-5, atol=1e-5)
    binary = r.uniform(-1, 1, batch + (M, 1)).astype(np.float32) if kind == "int8_bcast_weights_binary" else None
    got, impl = _run_batched(eng, strm, batch, wbatch, base, binary, weights_any=packed)
    assert "tcgen05" in impl
    for b in np.ndindex(*batch):
        wb = tuple(0 if wbatch[d] == 1 else b[d] for d in range(len(b)))
        c = _slice_case(base, b, wb, binary)
        want = B.run_oracle(c, exact_acc=1 if "i8" in impl else 0)
        g, w = dt.to_f32(got[b], c.dst_dt).astype(np.float64), dt.to_f32(want, c.dst_dt).astype(np.float64)
        assert (np.abs(g - w) <= c.atol + c.rtol * np.abs(w)).all(), "%s batch %s" % (kind, b)


def _launches():
    import ctypes as C
    v = C.c_uint64()
    assert api.lib().dnnl_b200_debug_counter(3, C.byref(v)) == 0
    return v.value


@pytest.mark.gpu
def test_weights_scales_and_zero_points_per_batch_index():
    """Weights scales with mask batch + N (one set of per-column values per batch index) and a weights
    zero-point per batch index: every batch index equals the oracle's 2-D problem with its own values."""
    eng = api.Engine()
    strm = api.Stream(eng)
    r = np.random.default_rng(97)
    B_, M, N, K = 3, 40, 48, 64
    src = r.integers(-128, 128, (B_, M, K), dtype=np.int8)
    wei = r.integers(-127, 128, (B_, K, N), dtype=np.int8)
    wscale = r.uniform(1e-3, 4e-3, (B_, N)).astype(np.float32)
    wzp = r.integers(-5, 6, (B_,)).astype(np.int32)
    attr = api.PrimitiveAttr()
    attr.set_scales(api.ARG_SRC, 0, (), dt.F32)
    attr.set_scales(api.ARG_WEIGHTS, 1 | 4, (), dt.F32)
    attr.set_zero_points(api.ARG_WEIGHTS, 1, (), dt.S32)
    src_md, wei_md, dst_md = _md((B_, M, K), dt.S8), _md((B_, K, N), dt.S8), _md((B_, M, N), dt.F32)
    pd = api.matmul_primitive_desc(eng, src_md, wei_md, dst_md, None, attr)
    assert "tcgen05_i8" in pd.impl_info_str()
    prim = api.Primitive(pd)
    keep = []

    def mem(md, arr):
        m = api.Memory(md, eng)
        m.write(np.ascontiguousarray(arr))
        keep.append(m)
        return m
    args = {api.ARG_SRC: mem(src_md, src), api.ARG_WEIGHTS: mem(wei_md, wei), api.ARG_DST: mem(dst_md, np.zeros((B_, M, N), np.float32)),
            api.ARG_ATTR_SCALES | api.ARG_SRC: mem(api.MemoryDesc((1,), dt.F32, api.TAG_A), np.float32([0.02])),
            api.ARG_ATTR_SCALES | api.ARG_WEIGHTS: mem(api.MemoryDesc((B_ * N,), dt.F32, api.TAG_A), wscale),
            api.ARG_ATTR_ZERO_POINTS | api.ARG_WEIGHTS: mem(api.MemoryDesc((B_,), dt.S32, api.TAG_A), wzp)}
    prim.execute(strm, args)
    strm.wait()
    got = args[api.ARG_DST].read(np.float32, (B_, M, N))
    for b in range(B_):
        c = MatmulCase("slice", M, N, K, src=src[b], src_dt=dt.S8, wei=wei[b], wei_dt=dt.S8, dst_dt=dt.F32,
                       src_scale=Quant(np.float32([0.02]), dt.F32, 0), wei_scale=Quant(wscale[b], dt.F32, 2),
                       wei_zp=Quant(wzp[b:b + 1], dt.S32, 0), exact=False, rtol=1e-5, atol=1e-5)
        want = B.run_oracle(c, exact_acc=1)
        assert np.all(np.abs(got[b] - want) <= 1e-5 + 1e-5 * np.abs(want)), "batch %d" % b


@pytest.mark.gpu
def test_broadcast_weights_run_as_one_matmul():
    """Weights shared by every batch index, src and dst rows dense through the batch dim: the
    whole problem is one 2-D matmul of batch * M rows -- one pass of the kernels (weights pack,
    their column sums, matmul) instead of one per batch index -- and equals the per-index results
    of the oracle."""
    eng = api.Engine()
    strm = api.Stream(eng)
    r = np.random.default_rng(95)
    batch, wbatch, (M, N, K) = (2, 3), (1, 1), (40, 48, 64)
    base = MatmulCase("bcast", M, N, K, src=r.integers(-128, 128, batch + (M, K), dtype=np.int8), src_dt=dt.S8,
                      wei=r.integers(-127, 128, wbatch + (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dt.S8,
                      src_scale=Quant(np.float32([0.02]), dt.F32, 0),
                      wei_scale=Quant(r.uniform(1e-3, 4e-3, N).astype(np.float32), dt.F32, 2),
                      dst_scale=Quant(np.float32([0.05]), dt.F32, 0),
                      bias=r.uniform(-1, 1, (1, N)).astype(np.float32), bias_dt=dt.F32,
                      post_ops=[W.eltwise("relu", 0.0)], exact=True, rtol=0, atol=0)
    before = _launches()
    got, impl = _run_batched(eng, strm, batch, wbatch, base)
    used = _launches() - before
    assert "tcgen05_i8" in impl
    assert used <= 3, "%d launches for a problem that collapses into one matmul (six batch indices)" % used
    for b in np.ndindex(*batch):
        want = B.run_oracle(_slice_case(base, b, (0, 0)), exact_acc=1)
        assert np.array_equal(got[b], want), "batch %s" % (b,)


# ---- runtime dims ---------------------------------------------------------------------------

RT = -(1 << 63)  # DNNL_RUNTIME_DIM_VAL


def _rt_pd(eng):
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_SRC, 0, (), dt.F32)
    a.set_scales(api.ARG_WEIGHTS, 2, (), dt.F32)
    src = api.MemoryDesc((RT, 64), dt.S8, strides=(RT, 1))
    wei = api.MemoryDesc((64, 48), dt.S8, strides=(1, 64))      # K contiguous
    dst = api.MemoryDesc((RT, 48), dt.BF16, strides=(RT, 1))
    return api.matmul_primitive_desc(eng, src, wei, dst, attr=a)


def test_runtime_dims_descriptor_host():
    eng = api.Engine()
    pd = _rt_pd(eng)
    assert pd.impl_info_str() == "cuda:runtime_dims"
    assert not pd.next_impl()
    # a layout must be given when sizes are not
    with pytest.raises(api.Error):
        api.matmul_primitive_desc(eng, api.MemoryDesc((RT, 64), dt.S8, strides=(RT, 1)),
                                  api.MemoryDesc((64, 48), dt.S8, api.TAG_ANY), api.MemoryDesc((RT, 48), dt.BF16, strides=(RT, 1)))


@pytest.mark.gpu
def test_runtime_dims_execute_with_two_sizes():
    """One primitive created with an unknown M (DNNL_RUNTIME_DIM_VAL), executed with 40 and
    with 200 rows: each result equals the oracle's for that size."""
    eng = api.Engine()
    strm = api.Stream(eng)
    prim = api.Primitive(_rt_pd(eng))
    r = np.random.default_rng(93)
    wei = r.integers(-127, 128, (64, 48), dtype=np.int8)
    wscale = r.uniform(1e-3, 4e-3, 48).astype(np.float32)
    sscale = np.float32([0.03])
    wei_m = api.Memory(api.MemoryDesc((64, 48), dt.S8, strides=(1, 64)), eng)
    wei_m.write(np.ascontiguousarray(wei.T))
    ws_m = api.Memory(api.MemoryDesc((48,), dt.F32, api.TAG_A), eng)
    ws_m.write(wscale)
    ss_m = api.Memory(api.MemoryDesc((1,), dt.F32, api.TAG_A), eng)
    ss_m.write(sscale)
    for M in (40, 200):
        src = r.integers(-128, 128, (M, 64), dtype=np.int8)
        src_m = api.Memory(api.MemoryDesc((M, 64), dt.S8, api.TAG_AB), eng)
        src_m.write(src)
        dst_m = api.Memory(api.MemoryDesc((M, 48), dt.BF16, api.TAG_AB), eng)
        prim.execute(strm, {api.ARG_SRC: src_m, api.ARG_WEIGHTS: wei_m, api.ARG_DST: dst_m,
                            api.ARG_ATTR_SCALES | api.ARG_SRC: ss_m, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS: ws_m})
        strm.wait()
        got = dt.to_f32(dst_m.read(dt.RAW[dt.BF16], (M, 48)), dt.BF16)
        c = MatmulCase("rt", M, 48, 64, src=src, src_dt=dt.S8, wei=np.ascontiguousarray(wei.T), wei_dt=dt.S8, dst_dt=dt.BF16,
                       wei_tag="ba", src_scale=Quant(sscale, dt.F32, 0), wei_scale=Quant(wscale, dt.F32, 2))
        want = dt.to_f32(B.run_oracle(c, exact_acc=1), dt.BF16)
        assert np.allclose(got, want, rtol=1e-2, atol=1e-2), M
    # a memory whose fixed dim differs from the descriptor's is refused
    bad = api.Memory(api.MemoryDesc((40, 32), dt.S8, api.TAG_AB), eng)
    with pytest.raises(api.Error):
        prim.execute(strm, {api.ARG_SRC: bad, api.ARG_WEIGHTS: wei_m, api.ARG_DST: dst_m,
                            api.ARG_ATTR_SCALES | api.ARG_SRC: ss_m, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS: ws_m})


# ---- inner product -------------------------------------------------------------------------

def _ip_pd(eng, wtag=api.TAG_AB):
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_SRC, 0, (), dt.F32)
    a.set_scales(api.ARG_WEIGHTS, 1 << 0, (), dt.F32)          # per output channel of (OC, IC) weights
    po = api.PostOps()
    po.append_eltwise(W.ELTWISE["relu"], 0.0, 0.0)
    a.set_post_ops(po)
    return api.inner_product_primitive_desc(
        eng, api.MemoryDesc((150, 128), dt.S8, api.TAG_AB), api.MemoryDesc((96, 128), dt.S8, wtag),
        api.MemoryDesc((150, 96), dt.F32, api.TAG_AB), api.MemoryDesc((96,), dt.F32, api.TAG_A), a)


def test_inner_product_descriptor_host():
    """Forward inner product = matmul with the weights' dims exchanged: row-major (OC, IC) weights
    are already K-contiguous, so the tensor-core kernel takes them as they are."""
    eng = api.Engine()
    for wtag in (api.TAG_AB, api.TAG_ANY):
        pd = _ip_pd(eng, wtag)
        assert pd.impl_info_str() == "cuda:sm100:tcgen05_i8"
        assert pd.weights_desc() == api.MemoryDesc((96, 128), dt.S8, api.TAG_AB)
        assert pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS).dims == [96]
    with pytest.raises(api.Error):   # IC of src and weights differ
        api.inner_product_primitive_desc(eng, api.MemoryDesc((150, 64), dt.S8, api.TAG_AB),
                                         api.MemoryDesc((96, 128), dt.S8, api.TAG_AB), api.MemoryDesc((150, 96), dt.F32, api.TAG_AB))


@pytest.mark.gpu
def test_inner_product_matches_the_matmul_oracle():
    eng = api.Engine()
    strm = api.Stream(eng)
    prim = api.Primitive(_ip_pd(eng))
    r = np.random.default_rng(94)
    src = r.integers(-128, 128, (150, 128), dtype=np.int8)
    wei = r.integers(-127, 128, (96, 128), dtype=np.int8)       # (OC, IC)
    bias = r.uniform(-1, 1, 96).astype(np.float32)
    sscale, wscale = np.float32([0.02]), r.uniform(1e-3, 4e-3, 96).astype(np.float32)

    def mem(md, arr):
        m = api.Memory(md, eng)
        m.write(np.ascontiguousarray(arr))
        return m
    dst_m = api.Memory(api.MemoryDesc((150, 96), dt.F32, api.TAG_AB), eng)
    args = {api.ARG_SRC: mem(api.MemoryDesc((150, 128), dt.S8, api.TAG_AB), src),
            api.ARG_WEIGHTS: mem(api.MemoryDesc((96, 128), dt.S8, api.TAG_AB), wei),
            api.ARG_BIAS: mem(api.MemoryDesc((96,), dt.F32, api.TAG_A), bias), api.ARG_DST: dst_m,
            api.ARG_ATTR_SCALES | api.ARG_SRC: mem(api.MemoryDesc((1,), dt.F32, api.TAG_A), sscale),
            api.ARG_ATTR_SCALES | api.ARG_WEIGHTS: mem(api.MemoryDesc((96,), dt.F32, api.TAG_A), wscale)}
    prim.execute(strm, args)
    strm.wait()
    got = dst_m.read(np.float32, (150, 96))
    c = MatmulCase("ip", 150, 96, 128, src=src, src_dt=dt.S8, wei=wei, wei_dt=dt.S8, dst_dt=dt.F32, wei_tag="ba",
                   bias=bias.reshape(1, 96), bias_dt=dt.F32, src_scale=Quant(sscale, dt.F32, 0),
                   wei_scale=Quant(wscale, dt.F32, 2), post_ops=[W.eltwise("relu", 0.0)])
    want = B.run_oracle(c, exact_acc=1)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
