"""Python mirror of the C++ API over the C ABI of ``libonednn_b200.so``.

The classes follow the reference's header-only C++ wrapper
(``include/oneapi/dnnl/dnnl.hpp``: ``engine``, ``stream``, ``memory::desc``,
``memory``, ``primitive_attr``, ``post_ops``, ``matmul::primitive_desc``,
``reorder``, ``primitive::execute``) -- same names, same argument meaning, and
a non-success status raises :class:`Error` carrying the ``dnnl_status_t``, as
``dnnl::error`` does.  Everything here is a thin handle holder; all work happens
in the native library, which must be present: importing this module builds
nothing and falls back to nothing.
"""
import ctypes as C
from pathlib import Path

import numpy as np

from . import dtypes as dt

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libonednn_b200.so"

STATUS = {0: "success", 1: "out_of_memory", 2: "invalid_arguments", 3: "unimplemented",
          4: "last_impl_reached", 5: "runtime_error", 6: "not_required", 7: "invalid_graph"}

# argument indices (dnnl_types.h:2471-2700 in the reference)
ARG_SRC, ARG_SRC_1, ARG_DST, ARG_WEIGHTS, ARG_BIAS = 1, 2, 17, 33, 41
ARG_FROM, ARG_TO, ARG_SCRATCHPAD = 1, 17, 80
ARG_ATTR_SCALES, ARG_ATTR_ZERO_POINTS, ARG_ATTR_MULTIPLE_POST_OP_BASE = 4096, 8192, 32768
ARG_B200_DST_PEER0 = 3072  # extension: mirrors of dst in other GPUs' memory, up to seven
TAG_ANY, TAG_A, TAG_AB, TAG_BA, TAG_ABC = 1, 2, 3, 14, 4
GPU = 2
QUERY_IMPL_INFO_STR, QUERY_SRC_MD, QUERY_WEIGHTS_MD, QUERY_DST_MD, QUERY_SCRATCHPAD_MD, QUERY_EXEC_ARG_MD = \
    8, 129, 131, 133, 136, 255
KIND_SUM, KIND_ELTWISE, KIND_BINARY, KIND_PRELU = 4, 7, 13, 18
MEMORY_ALLOCATE = C.c_void_p(-1)


def arg_post_op(idx):
    return ARG_ATTR_MULTIPLE_POST_OP_BASE * (idx + 1)


class Error(RuntimeError):
    def __init__(self, status, what):
        super().__init__("%s: dnnl_%s" % (what, STATUS.get(status, status)))
        self.status = status
        self.name = STATUS.get(status, str(status))


class ExecArg(C.Structure):
    _fields_ = [("arg", C.c_int), ("memory", C.c_void_p)]


_lib = None


def lib():
    """The native library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError("%s is missing: run `python -m onednn_b200.build` (needs nvcc)" % LIB_PATH)
        _lib = C.CDLL(str(LIB_PATH))
        for name in ("dnnl_engine_get_count", "dnnl_memory_desc_get_size", "dnnl_data_type_size"):
            getattr(_lib, name).restype = C.c_size_t
        _lib.dnnl_primitive_desc_query_md.restype = C.c_void_p
        _lib.dnnl_version.restype = C.c_void_p
        _lib.b200_launch_count.restype = C.c_uint64
        _lib.b200_packed_weights_bytes.restype = C.c_size_t
    return _lib


def _ck(status, what):
    if status != 0:
        raise Error(status, what)


def _destroy(obj, fn):
    """Release a native handle; quiet during interpreter shutdown, when module globals are gone."""
    try:
        h = getattr(obj, "h", None)
        if h and _lib is not None:
            getattr(_lib, fn)(h)
    except Exception:
        pass
    obj.h = None


def _dims(v):
    a = (C.c_int64 * 12)()
    for i, x in enumerate(v):
        a[i] = int(x)
    return a


class Engine:
    def __init__(self, kind=GPU, index=0):
        self.h = C.c_void_p()
        _ck(lib().dnnl_engine_create(C.byref(self.h), kind, C.c_size_t(index)), "engine_create")

    @staticmethod
    def get_count(kind=GPU):
        return int(lib().dnnl_engine_get_count(kind))

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_engine_destroy")


class Stream:
    def __init__(self, engine, flags=1, cuda_stream=None):
        self.engine = engine
        self.h = C.c_void_p()
        if cuda_stream is None:
            _ck(lib().dnnl_stream_create(C.byref(self.h), engine.h, flags), "stream_create")
        else:
            _ck(lib().dnnl_cuda_interop_stream_create(C.byref(self.h), engine.h, C.c_void_p(cuda_stream)),
                "cuda_interop_stream_create")

    def wait(self):
        _ck(lib().dnnl_stream_wait(self.h), "stream_wait")

    @property
    def cuda_stream(self):
        p = C.c_void_p()
        _ck(lib().dnnl_cuda_interop_stream_get(self.h, C.byref(p)), "cuda_interop_stream_get")
        return p.value or 0

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_stream_destroy")


class MemoryDesc:
    """memory::desc; ``tag`` or ``strides`` picks the layout (``tag=TAG_ANY`` defers it)."""

    def __init__(self, dims=None, data_type=None, tag=None, strides=None, handle=None, borrowed=False):
        self.borrowed = borrowed
        if handle is not None:
            self.h = C.c_void_p(handle)
            return
        self.h = C.c_void_p()
        if strides is not None:
            _ck(lib().dnnl_memory_desc_create_with_strides(C.byref(self.h), len(dims), _dims(dims), data_type,
                                                           _dims(strides)), "memory_desc_create_with_strides")
        else:
            _ck(lib().dnnl_memory_desc_create_with_tag(C.byref(self.h), len(dims), _dims(dims), data_type,
                                                       TAG_AB if tag is None else tag), "memory_desc_create_with_tag")

    def get_size(self):
        return int(lib().dnnl_memory_desc_get_size(self.h))

    def __eq__(self, other):
        return bool(lib().dnnl_memory_desc_equal(self.h, other.h))

    def _query(self, what, ctype):
        v = ctype()
        _ck(lib().dnnl_memory_desc_query(self.h, what, C.byref(v)), "memory_desc_query")
        return v

    @property
    def ndims(self):
        return self._query(256, C.c_int32).value

    @property
    def dims(self):
        p = self._query(257, C.POINTER(C.c_int64))
        return [p[i] for i in range(self.ndims)]

    @property
    def strides(self):
        p = self._query(14, C.POINTER(C.c_int64))
        return [p[i] for i in range(self.ndims)]

    @property
    def data_type(self):
        return self._query(258, C.c_int).value

    @property
    def format_kind(self):
        return self._query(262, C.c_int).value

    def __del__(self, _destroy=_destroy):
        if not getattr(self, "borrowed", True):
            _destroy(self, "dnnl_memory_desc_destroy")


class Memory:
    """memory: ``handle`` is a device pointer (int), or None to let the library allocate."""

    def __init__(self, md, engine, handle=None):
        self.md, self.engine = md, engine
        self.h = C.c_void_p()
        hp = MEMORY_ALLOCATE if handle is None else C.c_void_p(handle)
        _ck(lib().dnnl_memory_create(C.byref(self.h), md.h, engine.h, hp), "memory_create")

    @property
    def data_handle(self):
        p = C.c_void_p()
        _ck(lib().dnnl_memory_get_data_handle(self.h, C.byref(p)), "memory_get_data_handle")
        return p.value or 0

    def write(self, array):
        """Host numpy array -> device through map / unmap (what the reference's examples do)."""
        a = np.ascontiguousarray(array)
        n = self.md.get_size()
        assert a.nbytes <= n, "array of %d bytes into a memory of %d" % (a.nbytes, n)
        p = C.c_void_p()
        _ck(lib().dnnl_memory_map_data(self.h, C.byref(p)), "memory_map_data")
        if a.nbytes:
            C.memmove(p, a.ctypes.data, a.nbytes)
        _ck(lib().dnnl_memory_unmap_data(self.h, p), "memory_unmap_data")

    def read(self, dtype, shape):
        out = np.empty(shape, dtype=dtype)
        p = C.c_void_p()
        _ck(lib().dnnl_memory_map_data(self.h, C.byref(p)), "memory_map_data")
        if out.nbytes:
            C.memmove(out.ctypes.data, p, out.nbytes)
        _ck(lib().dnnl_memory_unmap_data(self.h, p), "memory_unmap_data")
        return out

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_memory_destroy")


class PostOps:
    def __init__(self):
        self.h = C.c_void_p()
        self._keep = []
        _ck(lib().dnnl_post_ops_create(C.byref(self.h)), "post_ops_create")

    def append_sum(self, scale=1.0, zero_point=0, data_type=dt.UNDEF):
        _ck(lib().dnnl_post_ops_append_sum(self.h, C.c_float(scale), C.c_int32(zero_point), data_type), "append_sum")

    def append_eltwise(self, alg, alpha=0.0, beta=0.0):
        _ck(lib().dnnl_post_ops_append_eltwise(self.h, alg, C.c_float(alpha), C.c_float(beta)), "append_eltwise")

    def append_binary(self, alg, src1_md):
        self._keep.append(src1_md)
        _ck(lib().dnnl_post_ops_append_binary(self.h, alg, src1_md.h), "append_binary")

    def append_prelu(self, mask):
        _ck(lib().dnnl_post_ops_append_prelu(self.h, mask), "append_prelu")

    def __len__(self):
        return lib().dnnl_post_ops_len(self.h)

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_post_ops_destroy")


class PrimitiveAttr:
    def __init__(self):
        self.h = C.c_void_p()
        _ck(lib().dnnl_primitive_attr_create(C.byref(self.h)), "primitive_attr_create")

    def set_scales(self, arg, mask, groups=(), data_type=dt.F32):
        _ck(lib().dnnl_primitive_attr_set_scales(self.h, arg, mask, len(groups), _dims(groups), data_type), "set_scales")

    def set_scales_mask(self, arg, mask):
        _ck(lib().dnnl_primitive_attr_set_scales_mask(self.h, arg, mask), "set_scales_mask")

    def set_zero_points(self, arg, mask, groups=(), data_type=dt.S32):
        _ck(lib().dnnl_primitive_attr_set_zero_points(self.h, arg, mask, len(groups), _dims(groups), data_type),
            "set_zero_points")

    def set_zero_points_mask(self, arg, mask):
        _ck(lib().dnnl_primitive_attr_set_zero_points_mask(self.h, arg, mask), "set_zero_points_mask")

    def set_fpmath_mode(self, mode, apply_to_int=False):
        _ck(lib().dnnl_primitive_attr_set_fpmath_mode_v2(self.h, mode, 1 if apply_to_int else 0), "set_fpmath_mode")

    def set_scratchpad_mode(self, mode):
        _ck(lib().dnnl_primitive_attr_set_scratchpad_mode(self.h, mode), "set_scratchpad_mode")

    def set_post_ops(self, po):
        _ck(lib().dnnl_primitive_attr_set_post_ops(self.h, po.h), "set_post_ops")

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_primitive_attr_destroy")


class PrimitiveDesc:
    def __init__(self, handle, engine):
        self.h, self.engine = handle, engine

    def next_impl(self):
        return lib().dnnl_primitive_desc_next_impl(self.h) == 0

    def impl_info_str(self):
        s = C.c_char_p()
        _ck(lib().dnnl_primitive_desc_query(self.h, QUERY_IMPL_INFO_STR, 0, C.byref(s)), "query impl_info_str")
        return s.value.decode()

    def query_md(self, what, index=0):
        p = lib().dnnl_primitive_desc_query_md(self.h, what, index)
        if not p:
            raise Error(3, "query_md")
        md = MemoryDesc(handle=p, borrowed=True)
        md._owner = self   # the descriptor lives inside the primitive descriptor
        return md

    def src_desc(self):
        return self.query_md(QUERY_SRC_MD)

    def weights_desc(self):
        return self.query_md(QUERY_WEIGHTS_MD)

    def dst_desc(self):
        return self.query_md(QUERY_DST_MD)

    def scratchpad_desc(self):
        return self.query_md(QUERY_SCRATCHPAD_MD)

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_primitive_desc_destroy")


def matmul_primitive_desc(engine, src_md, weights_md, dst_md, bias_md=None, attr=None):
    h = C.c_void_p()
    _ck(lib().dnnl_matmul_primitive_desc_create(C.byref(h), engine.h, src_md.h, weights_md.h,
                                                bias_md.h if bias_md is not None else None, dst_md.h,
                                                attr.h if attr is not None else None), "matmul_primitive_desc_create")
    return PrimitiveDesc(h, engine)


def inner_product_primitive_desc(engine, src_md, weights_md, dst_md, bias_md=None, attr=None, prop_kind=96):
    """Forward inner product: src (N, IC), weights (OC, IC), bias (OC), dst (N, OC)."""
    h = C.c_void_p()
    _ck(lib().dnnl_inner_product_forward_primitive_desc_create(
        C.byref(h), engine.h, prop_kind, src_md.h, weights_md.h, bias_md.h if bias_md is not None else None, dst_md.h,
        attr.h if attr is not None else None), "inner_product_forward_primitive_desc_create")
    return PrimitiveDesc(h, engine)


def reorder_primitive_desc(src_engine, src_md, dst_engine, dst_md, attr=None):
    h = C.c_void_p()
    _ck(lib().dnnl_reorder_primitive_desc_create(C.byref(h), src_md.h, src_engine.h, dst_md.h, dst_engine.h,
                                                 attr.h if attr is not None else None), "reorder_primitive_desc_create")
    return PrimitiveDesc(h, dst_engine)


class Primitive:
    def __init__(self, pd):
        self.pd = pd
        self.h = C.c_void_p()
        _ck(lib().dnnl_primitive_create(C.byref(self.h), pd.h), "primitive_create")

    def execute(self, stream, args):
        """args: {arg index: Memory}"""
        arr = (ExecArg * len(args))()
        for i, (k, m) in enumerate(args.items()):
            arr[i].arg, arr[i].memory = k, m.h
        _ck(lib().dnnl_primitive_execute(self.h, stream.h, len(args), arr), "primitive_execute")

    def __del__(self, _destroy=_destroy):
        _destroy(self, "dnnl_primitive_destroy")


# ---- running a MatmulCase through the public API ------------------------------------------

def _quant_attr(attr, case):
    for q, arg, is_zp in ((case.src_scale, ARG_SRC, False), (case.wei_scale, ARG_WEIGHTS, False),
                          (case.dst_scale, ARG_DST, False), (case.src_zp, ARG_SRC, True),
                          (case.wei_zp, ARG_WEIGHTS, True), (case.dst_zp, ARG_DST, True)):
        if q is None:
            continue
        groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
        if is_zp:
            attr.set_zero_points(arg, q.mask, groups, q.dt)
        else:
            attr.set_scales(arg, q.mask, groups, q.dt)


class CasePlan:
    """A MatmulCase lowered onto the engine: descriptors, attribute, primitive, device
    memories.  ``weights="any"`` lets the implementation choose its packed weights layout
    and reorders the plain weights into it once (the reference's recommended usage);
    ``weights="plain"`` hands the plain weights to the primitive as they are."""

    def __init__(self, case, engine, stream, weights="any", impl=None, upload=True, dst_strides=None,
                 scratchpad="library"):
        from . import workloads as W
        self.case, self.engine, self.stream = case, engine, stream
        c = case
        src_md = MemoryDesc((c.M, c.K), c.src_dt, TAG_AB)
        plain_wei_md = MemoryDesc((c.K, c.N), c.wei_dt, TAG_AB if c.wei_tag == "ab" else TAG_BA)
        wei_md = MemoryDesc((c.K, c.N), c.wei_dt, TAG_ANY) if weights == "any" else plain_wei_md
        # dst_strides: dst is a block of a larger matrix; the caller supplies ARG_DST itself
        self.own_dst = dst_strides is None
        dst_md = MemoryDesc((c.M, c.N), c.dst_dt, TAG_AB) if self.own_dst else \
            MemoryDesc((c.M, c.N), c.dst_dt, strides=tuple(dst_strides))
        bias_md = None
        if c.bias is not None:
            bshape = c.bias.shape if c.bias.ndim == 2 else (1, c.bias.shape[0])
            bias_md = MemoryDesc(bshape, c.bias_dt, TAG_AB)
        attr = PrimitiveAttr()
        if c.apply_to_int:
            attr.set_fpmath_mode(1, True)
        _quant_attr(attr, c)
        self._po_mds = []
        if c.post_ops:
            po = PostOps()
            for e in c.post_ops:
                if e.kind == W.PO_SUM:
                    po.append_sum(e.scale, e.zero_point, e.dt)
                elif e.kind == W.PO_ELTWISE:
                    po.append_eltwise(e.alg, e.alpha, e.beta)
                elif e.kind == W.PO_BINARY:
                    md = MemoryDesc(e.shape, e.dt, TAG_AB)
                    self._po_mds.append(md)
                    po.append_binary(e.alg, md)
                else:
                    po.append_prelu((1 if e.shape[0] > 1 else 0) | (2 if e.shape[1] > 1 else 0))
            attr.set_post_ops(po)
        if scratchpad == "user":  # the caller owns the scratchpad and passes it as DNNL_ARG_SCRATCHPAD
            attr.set_scratchpad_mode(1)
        self.user_scratchpad = scratchpad == "user"
        self.attr = attr
        self.pd = matmul_primitive_desc(engine, src_md, wei_md, dst_md, bias_md, attr)
        if impl is not None:
            while impl not in self.pd.impl_info_str():
                if not self.pd.next_impl():
                    raise Error(3, "no implementation matching %r" % impl)
        self.impl = self.pd.impl_info_str()
        self.prim = Primitive(self.pd)
        self.mds = dict(src=src_md, wei=wei_md, plain_wei=plain_wei_md, dst=dst_md, bias=bias_md)
        self.args = {}
        self.mem = {}
        if upload:
            self.upload()

    def _mem(self, name, md, array):
        m = Memory(md, self.engine)
        if array is not None:
            m.write(array)
        self.mem[name] = m
        return m

    def upload(self):
        c = self.case
        self.args[ARG_SRC] = self._mem("src", self.mds["src"], c.src)
        wq = self.pd.weights_desc()
        if wq == self.mds["plain_wei"]:
            self.args[ARG_WEIGHTS] = self._mem("wei", self.mds["plain_wei"], c.wei)
        else:
            plain = self._mem("plain_wei", self.mds["plain_wei"], c.wei)
            packed = Memory(wq, self.engine)
            self.mem["wei"] = packed
            r = Primitive(reorder_primitive_desc(self.engine, self.mds["plain_wei"], self.engine, wq))
            r.execute(self.stream, {ARG_FROM: plain, ARG_TO: packed})
            self.stream.wait()
            self.args[ARG_WEIGHTS] = packed
        if c.bias is not None:
            self.args[ARG_BIAS] = self._mem("bias", self.mds["bias"], c.bias)
        if self.user_scratchpad:
            smd = self.pd.scratchpad_desc()
            if smd.get_size() > 0:
                self.args[ARG_SCRATCHPAD] = self._mem("scratchpad", smd, None)
        if self.own_dst:
            self.args[ARG_DST] = self._mem("dst", self.mds["dst"], c.dst_init)
        for name, q, arg in (("src_scale", c.src_scale, ARG_ATTR_SCALES | ARG_SRC),
                             ("wei_scale", c.wei_scale, ARG_ATTR_SCALES | ARG_WEIGHTS),
                             ("dst_scale", c.dst_scale, ARG_ATTR_SCALES | ARG_DST),
                             ("src_zp", c.src_zp, ARG_ATTR_ZERO_POINTS | ARG_SRC),
                             ("wei_zp", c.wei_zp, ARG_ATTR_ZERO_POINTS | ARG_WEIGHTS),
                             ("dst_zp", c.dst_zp, ARG_ATTR_ZERO_POINTS | ARG_DST)):
            if q is None:
                continue
            n = q.data.size * (2 if q.dt in (dt.S4, dt.U4) else 1)
            self.args[arg] = self._mem(name, MemoryDesc((n,), q.dt, TAG_A), q.data)
        from . import workloads as W
        bi = 0
        for i, e in enumerate(c.post_ops):
            if e.kind == W.PO_BINARY:
                self.args[arg_post_op(i) | ARG_SRC_1] = self._mem("po%d" % i, self._po_mds[bi], e.data)
                bi += 1
            elif e.kind == W.PO_PRELU:
                self.args[arg_post_op(i) | ARG_WEIGHTS] = self._mem(
                    "po%d" % i, MemoryDesc((e.data.size,), dt.F32, TAG_A), e.data)

    def reset_dst(self):
        if self.case.dst_init is not None:
            self.mem["dst"].write(self.case.dst_init)

    def execute(self):
        self.prim.execute(self.stream, self.args)

    def result(self):
        self.stream.wait()
        c = self.case
        return self.mem["dst"].read(dt.RAW[c.dst_dt], (c.M, c.N))


class ReorderPlan:
    """A :class:`onednn_b200.workloads.ReorderCase` lowered onto the engine through
    ``dnnl_reorder_primitive_desc_create`` with a scales / zero-points attribute."""

    def __init__(self, case, engine, stream):
        self.case, self.engine, self.stream = case, engine, stream
        c = case
        shape = (c.rows, c.cols)
        self.src_md = MemoryDesc(shape, c.src_dt, TAG_AB if c.src_tag == "ab" else TAG_BA)
        self.dst_md = MemoryDesc(shape, c.dst_dt, TAG_AB if c.dst_tag == "ab" else TAG_BA)
        attr = PrimitiveAttr()
        for q, arg, is_zp in ((c.src_scale, ARG_SRC, False), (c.dst_scale, ARG_DST, False),
                              (c.src_zp, ARG_SRC, True), (c.dst_zp, ARG_DST, True)):
            if q is None:
                continue
            groups = tuple(q.groups) if tuple(q.groups) != (1, 1) else ()
            (attr.set_zero_points if is_zp else attr.set_scales)(arg, q.mask, groups, q.dt)
        if c.beta != 0.0:
            po = PostOps()
            po.append_sum(c.beta, 0, dt.UNDEF)
            attr.set_post_ops(po)
        self.attr = attr
        self.pd = reorder_primitive_desc(engine, self.src_md, engine, self.dst_md, attr)
        self.impl = self.pd.impl_info_str()
        self.prim = Primitive(self.pd)
        self.mem = {}
        self.args = {ARG_FROM: self._mem("src", self.src_md, c.src),
                     ARG_TO: self._mem("dst", self.dst_md, c.dst_init)}
        for name, q, arg in (("src_scale", c.src_scale, ARG_ATTR_SCALES | ARG_SRC),
                             ("dst_scale", c.dst_scale, ARG_ATTR_SCALES | ARG_DST),
                             ("src_zp", c.src_zp, ARG_ATTR_ZERO_POINTS | ARG_SRC),
                             ("dst_zp", c.dst_zp, ARG_ATTR_ZERO_POINTS | ARG_DST)):
            if q is not None:
                self.args[arg] = self._mem(name, MemoryDesc((q.data.size,), q.dt, TAG_A), q.data)

    def _mem(self, name, md, array):
        m = Memory(md, self.engine)
        if array is not None:
            m.write(array)
        self.mem[name] = m
        return m

    def execute(self):
        self.prim.execute(self.stream, self.args)

    def result(self):
        """Raw destination in its physical order: (rows, cols) for tag ab, (cols, rows) for ba."""
        self.stream.wait()
        c = self.case
        shape = (c.rows, c.cols) if c.dst_tag == "ab" else (c.cols, c.rows)
        if c.dst_dt in (dt.S4, dt.U4):  # two values per byte along the contiguous dim
            shape = (shape[0], shape[1] // 2)
        return self.mem["dst"].read(dt.RAW[c.dst_dt], shape)


def run_case(case, engine=None, stream=None, weights="any", impl=None):
    """Execute ``case`` once on the engine; returns (raw dst array, implementation name)."""
    engine = engine or Engine()
    stream = stream or Stream(engine)
    plan = CasePlan(case, engine, stream, weights=weights, impl=impl)
    plan.execute()
    return plan.result(), plan.impl
