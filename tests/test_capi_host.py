"""Host-side logic of the C-ABI library, runnable without a GPU.

Covers: the library loads and exports every symbol the public headers declare;
memory descriptors; attributes and post-ops with the reference's status codes
(tests/gtests/test_matmul.cpp:398-470, test_iface_attr_quantization.cpp are the
model); matmul validation, implementation dispatch and queries on a
descriptor-only engine; and that nothing can be allocated or executed there.
"""
import ctypes as C
import os
import re
from pathlib import Path

import pytest

os.environ["ONEDNN_B200_ALLOW_NO_DEVICE"] = "1"

from onednn_b200 import api, dtypes as dt  # noqa: E402
from onednn_b200.workloads import ELTWISE, BINARY  # noqa: E402

ROOT = Path(__file__).resolve().parents[1]


def _have_gpu():
    return api.Engine.get_count() > 0


def test_library_exports_every_declared_symbol():
    L = api.lib()
    names = set()
    for h in ("onednn_b200.h", "onednn_b200_kernels.h"):
        text = (ROOT / "include" / h).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(dnnl_[a-z0-9_]+|b200_[a-z0-9_]+)\s*\(", text))
    names = {n for n in names if not n.endswith("_t")}
    assert len(names) > 80
    missing = [n for n in sorted(names) if not hasattr(L, n)]
    assert not missing, missing


def test_version_and_engine_kinds():
    L = api.lib()

    class V(C.Structure):
        _fields_ = [("major", C.c_int), ("minor", C.c_int), ("patch", C.c_int), ("hash", C.c_char_p),
                    ("cpu_runtime", C.c_uint), ("gpu_runtime", C.c_uint)]
    v = V.from_address(L.dnnl_version())
    assert (v.major, v.minor) == (3, 8) and v.cpu_runtime == 0
    # the CPU engine holds host memory and reorders for the callers either side of the matmul; it
    # computes nothing, so no fallback path exists
    assert api.Engine.get_count(1) == 1
    cpu = api.Engine(kind=1)
    with pytest.raises(api.Error) as e:
        api.Engine(kind=1, index=1)
    assert e.value.name == "invalid_arguments"
    md = api.MemoryDesc((8, 16), dt.S8, api.TAG_AB)
    with pytest.raises(api.Error) as e:
        api.matmul_primitive_desc(cpu, md, api.MemoryDesc((16, 8), dt.S8, api.TAG_AB), api.MemoryDesc((8, 8), dt.S32, api.TAG_AB))
    assert e.value.name == "unimplemented"


def _host_mem(cpu, a, dtype, tag=None, strides=None):
    md = api.MemoryDesc(a.shape, dtype, tag, strides=strides) if strides else api.MemoryDesc(a.shape, dtype, tag)
    m = api.Memory(md, cpu)
    p = C.c_void_p()
    assert api.lib().dnnl_memory_map_data(m.h, C.byref(p)) == 0
    return md, m, p


def test_host_engine_reorders_convert_like_the_reference():
    """f32 -> every integer / float type on the host engine: saturate, round to nearest even,
    bf16 with one rounding, 4-bit values packed two per byte (even index in the low nibble),
    transposed and strided destinations; and back to f32."""
    import numpy as np
    L = api.lib()
    cpu = api.Engine(kind=1)
    strm = api.Stream(cpu)
    a = np.array([[-200.5, -3.5, -2.5, -0.5, 0.5, 1.5], [2.5, 7.49, 7.5, 15.5, 127.5, 300.0]], dtype=np.float32)
    smd, src, sp = _host_mem(cpu, a, dt.F32, api.TAG_AB)
    C.memmove(sp, a.ctypes.data, a.nbytes)

    def run(dst_dt, tag=api.TAG_AB, strides=None):
        dmd, dst, dp = _host_mem(cpu, a, dst_dt, tag, strides)
        pd = api.reorder_primitive_desc(cpu, smd, cpu, dmd)
        assert pd.impl_info_str() == "host:reorder"
        api.Primitive(pd).execute(strm, {api.ARG_FROM: src, api.ARG_TO: dst})
        strm.wait()
        return dmd, dst, dp

    _, _, p = run(dt.S8)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int8)), a.shape)
    assert np.array_equal(got, np.clip(np.rint(a), -128, 127).astype(np.int8))
    _, _, p = run(dt.U8, api.TAG_BA)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), a.shape[::-1]).T
    assert np.array_equal(got, np.clip(np.rint(a), 0, 255).astype(np.uint8))
    _, _, p = run(dt.BF16)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), a.shape)
    assert np.array_equal(got, dt.f32_to_bf16(a))
    _, _, p = run(dt.U4)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), (a.size // 2,))
    want = np.clip(np.rint(a), 0, 15).astype(np.uint8).reshape(-1)
    assert np.array_equal(got, want[0::2] | (want[1::2] << 4))
    _, _, p = run(dt.S4)
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), (a.size // 2,))
    want = (np.clip(np.rint(a), -8, 7).astype(np.int8).reshape(-1) & 0xF).astype(np.uint8)
    assert np.array_equal(got, want[0::2] | (want[1::2] << 4))
    # s32 with a row pitch of 8 elements, then back to dense f32
    dmd, dst, p = run(dt.S32, strides=(8, 1))
    got = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_int32)), (2, 8))[:, :6]
    assert np.array_equal(got, np.rint(a).astype(np.int32))
    bmd, back, bp = _host_mem(cpu, a, dt.F32, api.TAG_AB)
    api.Primitive(api.reorder_primitive_desc(cpu, dmd, cpu, bmd)).execute(strm, {api.ARG_FROM: dst, api.ARG_TO: back})
    assert np.array_equal(np.ctypeslib.as_array(C.cast(bp, C.POINTER(C.c_float)), a.shape), np.rint(a))
    # quantising reorders stay with the CUDA engine
    attr = api.PrimitiveAttr()
    attr.set_scales(api.ARG_DST, 0)
    with pytest.raises(api.Error) as e:
        api.reorder_primitive_desc(cpu, smd, cpu, api.MemoryDesc(a.shape, dt.S8, api.TAG_AB), attr)
    assert e.value.name == "unimplemented"


def test_string_tags_and_runtime_strides():
    L = api.lib()
    md = C.c_void_p()
    dims = (C.c_int64 * 12)(2, 3, 5)
    assert L.dnnl_memory_desc_create_with_string_tag(C.byref(md), 3, dims, dt.F32, b"acb") == 0
    m = api.MemoryDesc(handle=md.value)
    assert m.strides == [15, 1, 3]
    # a blocked tag of another engine: an opaque descriptor that can be held and compared, its blocks
    # padded in the size; no primitive here computes on it
    assert L.dnnl_memory_desc_create_with_string_tag(C.byref(md), 3, dims, dt.F32, b"aBc16b") == 0
    blocked = api.MemoryDesc(handle=md.value)
    assert blocked.format_kind == 3 and blocked.get_size() >= 2 * 16 * 5 * 4
    assert L.dnnl_memory_desc_create_with_string_tag(C.byref(md), 3, dims, dt.F32, b"abb") == 2
    # a stride that depends on a runtime dim is a runtime value
    RT = -(2 ** 63)
    dims = (C.c_int64 * 12)(4, RT)
    assert L.dnnl_memory_desc_create_with_string_tag(C.byref(md), 2, dims, dt.S8, b"ab") == 0
    assert api.MemoryDesc(handle=md.value).strides == [RT, 1]
    assert L.dnnl_memory_desc_create_with_string_tag(C.byref(md), 2, dims, dt.S8, b"ba") == 0
    assert api.MemoryDesc(handle=md.value).strides == [1, 4]


@pytest.fixture(scope="module")
def eng():
    return api.Engine()


def test_memory_desc_tags_strides_sizes():
    ab = api.MemoryDesc((3, 5), dt.S8, api.TAG_AB)
    ba = api.MemoryDesc((3, 5), dt.S8, api.TAG_BA)
    assert ab.strides == [5, 1] and ba.strides == [1, 3]
    assert ab.get_size() == 15 and ab.dims == [3, 5] and ab.data_type == dt.S8 and ab.format_kind == 2
    assert ab != ba and ab == api.MemoryDesc((3, 5), dt.S8, strides=(5, 1))
    assert api.MemoryDesc((4, 6), dt.U4, api.TAG_AB).get_size() == 12      # two values per byte
    assert api.MemoryDesc((4, 6), dt.BF16, strides=(8, 1)).get_size() == (3 * 8 + 6) * 2
    assert api.MemoryDesc((0, 6), dt.F32, api.TAG_AB).get_size() == 0
    anymd = api.MemoryDesc((4, 6), dt.S8, api.TAG_ANY)
    assert anymd.format_kind == 1 and anymd.get_size() == 0
    for bad in (lambda: api.MemoryDesc((3, 5), dt.S8, api.TAG_ABC),          # tag / ndims mismatch
                lambda: api.MemoryDesc((3, -5), dt.S8, api.TAG_AB),
                lambda: api.MemoryDesc((3, 5), 99, api.TAG_AB),
                lambda: api.MemoryDesc((3, 5), dt.S8, strides=(1, 1))):      # overlapping strides
        with pytest.raises(api.Error) as e:
            bad()
        assert e.value.name == "invalid_arguments"


def test_memory_desc_submemory_reshape_permute():
    L = api.lib()
    md = api.MemoryDesc((8, 16), dt.F32, api.TAG_AB)
    sub = C.c_void_p()
    assert L.dnnl_memory_desc_create_submemory(C.byref(sub), md.h, api._dims((4, 8)), api._dims((2, 4))) == 0
    s = api.MemoryDesc(handle=sub.value)
    assert s.dims == [4, 8] and s.strides == [16, 1] and s._query(259, C.c_int64).value == 2 * 16 + 4
    assert L.dnnl_memory_desc_create_submemory(C.byref(sub), md.h, api._dims((4, 8)), api._dims((6, 4))) == 2
    r = C.c_void_p()
    assert L.dnnl_memory_desc_reshape(C.byref(r), md.h, 3, api._dims((2, 4, 16))) == 0
    assert api.MemoryDesc(handle=r.value).strides == [64, 16, 1]
    assert L.dnnl_memory_desc_reshape(C.byref(r), md.h, 2, api._dims((7, 16))) == 2
    p = C.c_void_p()
    perm = (C.c_int * 2)(1, 0)
    assert L.dnnl_memory_desc_permute_axes(C.byref(p), md.h, perm) == 0
    t = api.MemoryDesc(handle=p.value)
    assert t.dims == [16, 8] and t.strides == [1, 16]


def test_attr_setters_follow_reference_status_codes():
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_WEIGHTS, 3, (128, 1), dt.BF16)
    a.set_zero_points(api.ARG_WEIGHTS, 3, (128, 1), dt.U4)
    a.set_zero_points(api.ARG_SRC, 0)
    for fn, args in ((a.set_scales, (api.ARG_SRC, -1)),
                     (a.set_scales, (api.ARG_SRC, 0, (), dt.S8)),            # scales cannot be integers
                     (a.set_zero_points, (api.ARG_WEIGHTS, 0, (), dt.U4)),   # int4 zero-points need a mask
                     (a.set_zero_points, (api.ARG_DST, 2, (), dt.S8)),       # dst zero-points are s32
                     (a.set_zero_points, (api.ARG_SRC, 0, (), dt.F32))):
        with pytest.raises(api.Error) as e:
            fn(*args)
        assert e.value.name == "invalid_arguments"
    L = api.lib()
    mode, ati = C.c_int(), C.c_int()
    a.set_fpmath_mode(1, True)
    assert L.dnnl_primitive_attr_get_fpmath_mode_v2(a.h, C.byref(mode), C.byref(ati)) == 0
    assert (mode.value, ati.value) == (1, 1)
    b = C.c_void_p()
    assert L.dnnl_primitive_attr_clone(C.byref(b), a.h) == 0
    assert L.dnnl_primitive_attr_get_fpmath_mode_v2(b, C.byref(mode), C.byref(ati)) == 0 and ati.value == 1
    L.dnnl_primitive_attr_destroy(b)


def test_post_ops_append_and_query():
    L = api.lib()
    po = api.PostOps()
    po.append_sum(0.5, 3, dt.S8)
    po.append_eltwise(ELTWISE["gelu_tanh"])
    po.append_binary(BINARY["add"], api.MemoryDesc((1, 8), dt.F32, api.TAG_AB))
    po.append_prelu(2)
    assert len(po) == 4
    assert [L.dnnl_post_ops_get_kind(po.h, i) for i in range(4)] == [api.KIND_SUM, api.KIND_ELTWISE, api.KIND_BINARY,
                                                                     api.KIND_PRELU]
    sc, zp, d = C.c_float(), C.c_int32(), C.c_int()
    assert L.dnnl_post_ops_get_params_sum(po.h, 0, C.byref(sc), C.byref(zp), C.byref(d)) == 0
    assert (sc.value, zp.value, d.value) == (0.5, 3, dt.S8)
    assert L.dnnl_post_ops_get_params_sum(po.h, 1, C.byref(sc), C.byref(zp), C.byref(d)) == 2
    with pytest.raises(api.Error):
        po.append_eltwise(ELTWISE["clip"], 2.0, 1.0)       # beta < alpha
    with pytest.raises(api.Error):
        po.append_eltwise(0x7777)
    for _ in range(28):
        po.append_eltwise(ELTWISE["relu"])
    with pytest.raises(api.Error) as e:
        po.append_eltwise(ELTWISE["relu"])                 # the list holds at most 32 entries
    assert e.value.name == "out_of_memory"


def _pd(eng, M, K, N, sdt, wdt, ddt, wtag=api.TAG_AB, attr=None, bias=None, dst_dims=None, wei_dims=None):
    return api.matmul_primitive_desc(
        eng, api.MemoryDesc((M, K), sdt, api.TAG_AB), api.MemoryDesc(wei_dims or (K, N), wdt, wtag),
        api.MemoryDesc(dst_dims or (M, N), ddt, api.TAG_AB), bias, attr)


def test_matmul_dims_validation(eng):
    for kw in (dict(dst_dims=(5, 64)), dict(wei_dims=(48, 64)),
               dict(bias=api.MemoryDesc((1, 7), dt.F32, api.TAG_AB)),
               dict(bias=api.MemoryDesc((64,), dt.F32, api.TAG_A))):
        with pytest.raises(api.Error) as e:
            _pd(eng, 4, 32, 64, dt.S8, dt.S8, dt.S32, **kw)
        assert e.value.name == "invalid_arguments", kw
    with pytest.raises(api.Error) as e:          # int4 weights need an even N
        _pd(eng, 4, 32, 63, dt.BF16, dt.U4, dt.BF16)
    assert e.value.name == "invalid_arguments"


def test_matmul_attr_validation(eng):
    def attr(**kw):
        a = api.PrimitiveAttr()
        for k, v in kw.items():
            getattr(a, k)(*v)
        return a
    # zero-points on a float x float problem
    with pytest.raises(api.Error) as e:
        _pd(eng, 4, 32, 64, dt.F32, dt.F32, dt.F32, attr=attr(set_zero_points=(api.ARG_SRC, 0)))
    assert e.value.name == "unimplemented"
    # src scale per-M only
    with pytest.raises(api.Error) as e:
        _pd(eng, 4, 32, 64, dt.S8, dt.S8, dt.F32, attr=attr(set_scales=(api.ARG_SRC, 1)))
    assert e.value.name == "unimplemented"
    # weights groups along N without apply_to_int; K-group not a multiple of 32
    with pytest.raises(api.Error):
        _pd(eng, 4, 64, 64, dt.S8, dt.S8, dt.F32, attr=attr(set_scales=(api.ARG_WEIGHTS, 3, (32, 32))))
    with pytest.raises(api.Error):
        _pd(eng, 4, 64, 64, dt.S8, dt.S8, dt.F32, attr=attr(set_scales=(api.ARG_WEIGHTS, 3, (16, 1))))
    # sum with a data type of another size than dst
    po = api.PostOps()
    po.append_sum(1.0, 0, dt.F32)
    with pytest.raises(api.Error) as e:
        _pd(eng, 4, 32, 64, dt.S8, dt.S8, dt.S8, attr=attr(set_post_ops=(po,)))
    assert e.value.name == "unimplemented"
    # binary operand that does not broadcast onto dst
    po = api.PostOps()
    po.append_binary(BINARY["add"], api.MemoryDesc((3, 64), dt.F32, api.TAG_AB))
    with pytest.raises(api.Error) as e:
        _pd(eng, 4, 32, 64, dt.S8, dt.S8, dt.S8, attr=attr(set_post_ops=(po,)))
    assert e.value.name == "invalid_arguments"


def test_dispatch_and_next_impl(eng):
    pd = _pd(eng, 128, 1024, 1024, dt.U8, dt.S8, dt.F32, wtag=api.TAG_ANY)
    assert pd.impl_info_str() == "cuda:sm100:tcgen05_i8"
    w = pd.weights_desc()
    assert w.format_kind == 3                                  # opaque packed layout
    assert w.get_size() == api.lib().b200_packed_weights_bytes(C.c_int64(1024), C.c_int64(1024), dt.S8, 1)
    assert w.get_size() >= 1024 * 1024 + 4 * 1024              # data + s32 column sums
    assert pd.next_impl() and pd.impl_info_str() == "cuda:generic"
    assert pd.weights_desc() == api.MemoryDesc((1024, 1024), dt.S8, api.TAG_AB)
    assert not pd.next_impl()
    assert _pd(eng, 64, 64, 64, dt.F8_E4M3, dt.F8_E4M3, dt.BF16, wtag=api.TAG_ANY).impl_info_str() == \
        "cuda:sm100:tcgen05_f8"
    # K not a multiple of 16: no TMA row pitch -> generic
    assert _pd(eng, 8, 70, 64, dt.S8, dt.S8, dt.S32).impl_info_str() == "cuda:generic"
    a = api.PrimitiveAttr()
    a.set_fpmath_mode(1, True)
    a.set_scales(api.ARG_WEIGHTS, 3, (128, 1), dt.BF16)
    a.set_zero_points(api.ARG_WEIGHTS, 3, (128, 1), dt.U4)
    pd = _pd(eng, 1, 4096, 14336, dt.BF16, dt.U4, dt.BF16, wtag=api.TAG_ANY, attr=a)
    assert pd.impl_info_str() == "cuda:sm100:wc_gemv"
    assert pd.weights_desc().get_size() == 4096 * 14336 // 2
    assert pd.scratchpad_desc().get_size() == 0                # library mode: the user provides nothing
    mem = C.c_int64()
    assert api.lib().dnnl_primitive_desc_query(pd.h, 6, 0, C.byref(mem)) == 0   # memory_consumption_s64
    assert mem.value >= 14336 * 4
    a.set_scratchpad_mode(1)
    assert _pd(eng, 1, 4096, 14336, dt.BF16, dt.U4, dt.BF16, wtag=api.TAG_ANY, attr=a).scratchpad_desc().get_size() >= 14336 * 4
    # attr is copied into the pd: later changes do not reach it
    a.set_scales(api.ARG_WEIGHTS, 0)
    md = pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_WEIGHTS)
    assert md.dims == [32 * 14336] and md.data_type == dt.BF16
    md = pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_ZERO_POINTS | api.ARG_WEIGHTS)
    assert md.dims == [32 * 14336] and md.data_type == dt.U4


def test_reorder_pd(eng):
    plain = api.MemoryDesc((256, 128), dt.S8, api.TAG_AB)
    packed = _pd(eng, 16, 256, 128, dt.S8, dt.S8, dt.S32, wtag=api.TAG_ANY).weights_desc()
    assert api.reorder_primitive_desc(eng, plain, eng, packed).impl_info_str() == "cuda:pack_weights"
    assert api.reorder_primitive_desc(eng, plain, eng, api.MemoryDesc((256, 128), dt.S8, api.TAG_BA)) \
        .impl_info_str() == "cuda:reorder"
    with pytest.raises(api.Error):
        api.reorder_primitive_desc(eng, plain, eng, api.MemoryDesc((256, 64), dt.S8, api.TAG_AB))


def test_quantising_reorder_pd(eng):
    """Attribute checks of src/common/reorder.cpp:96-146 and simple_reorder.hpp:2498-2547."""
    f32 = api.MemoryDesc((8, 16), dt.F32, api.TAG_AB)
    s8 = api.MemoryDesc((8, 16), dt.S8, api.TAG_AB)
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_DST, 1, (), dt.F32)
    a.set_zero_points(api.ARG_DST, 0, (), dt.S32)
    pd = api.reorder_primitive_desc(eng, f32, eng, s8, a)
    assert pd.impl_info_str() == "cuda:reorder_quant"
    md = pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_DST)
    assert md.dims == [8] and md.data_type == dt.F32
    a = api.PrimitiveAttr()
    a.set_scales(api.ARG_SRC, 3, (4, 8), dt.BF16)
    a.set_zero_points(api.ARG_SRC, 0, (), dt.S32)
    pd = api.reorder_primitive_desc(eng, s8, eng, f32, a)
    md = pd.query_md(api.QUERY_EXEC_ARG_MD, api.ARG_ATTR_SCALES | api.ARG_SRC)
    assert md.dims == [2 * 2] and md.data_type == dt.BF16

    def rejected(src, dst, fill):
        a = api.PrimitiveAttr()
        fill(a)
        with pytest.raises(api.Error):
            api.reorder_primitive_desc(eng, src, eng, dst, a)
    rejected(f32, s8, lambda a: a.set_zero_points(api.ARG_SRC, 0, (), dt.S32))   # zero-point on a float tensor
    rejected(s8, f32, lambda a: a.set_zero_points(api.ARG_DST, 0, (), dt.S32))
    rejected(f32, s8, lambda a: a.set_scales(api.ARG_WEIGHTS, 0, (), dt.F32))    # scales go with src / dst only
    rejected(f32, s8, lambda a: a.set_scales(api.ARG_SRC, 3, (3, 4), dt.F32))    # groups must divide the dims
    rejected(f32, s8, lambda a: a.set_scales(api.ARG_DST, 3, (2, 2), dt.F32))    # no groups on the dst side
    rejected(f32, s8, lambda a: (a.set_scales(api.ARG_SRC, 1, (), dt.F32), a.set_scales(api.ARG_DST, 2, (), dt.F32)))
    po = api.PostOps()
    po.append_eltwise(0x20, 0.0, 0.0)
    rejected(f32, s8, lambda a: a.set_post_ops(po))                               # sum is the only post-op


@pytest.mark.skipif(_have_gpu(), reason="checks behaviour on a machine without a CUDA device")
def test_no_device_means_no_execution(eng):
    md = api.MemoryDesc((4, 4), dt.F32, api.TAG_AB)
    with pytest.raises(api.Error) as e:
        api.Memory(md, eng)                        # allocation needs a device
    assert e.value.name == "runtime_error"
    with pytest.raises(api.Error) as e:
        api.Stream(eng)
    assert e.value.name == "runtime_error"
    pd = _pd(eng, 4, 32, 64, dt.S8, dt.S8, dt.S32)
    with pytest.raises(api.Error) as e:
        api.Primitive(pd)
    assert e.value.name == "runtime_error"
    # a user pointer can be wrapped, but nothing reads it on the host
    m = api.Memory(md, eng, handle=0x1000)
    assert m.data_handle == 0x1000
