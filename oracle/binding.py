"""ctypes binding of the CPU oracle -- TEST INFRASTRUCTURE ONLY.

``run_oracle`` evaluates a :class:`onednn_b200.workloads.MatmulCase` with the C
restatement (``liboracle_matmul.so``); ``run_reference`` evaluates it with the
reference library itself (``_ref/librefrun.so``, present only where
``build_ref.py`` has been run).  Only tests, the smoke check and the
benchmark's CPU-baseline legs may import this module.
"""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
MAX_PO = 32


class Quant(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("nelems_is_one", C.c_int32),
                ("s0", C.c_int64), ("s1", C.c_int64), ("g0", C.c_int64), ("g1", C.c_int64)]


class PostOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("alg", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float),
                ("scale", C.c_float), ("zero_point", C.c_int32), ("dt", C.c_int32),
                ("ptr", C.c_void_p), ("sm", C.c_int64), ("sn", C.c_int64)]


class Problem(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("src", C.c_void_p), ("src_dt", C.c_int32), ("pad0", C.c_int32), ("src_sm", C.c_int64), ("src_sk", C.c_int64),
        ("wei", C.c_void_p), ("wei_dt", C.c_int32), ("pad1", C.c_int32), ("wei_sk", C.c_int64), ("wei_sn", C.c_int64),
        ("bias", C.c_void_p), ("bias_dt", C.c_int32), ("pad2", C.c_int32), ("bias_sm", C.c_int64), ("bias_sn", C.c_int64),
        ("dst", C.c_void_p), ("dst_dt", C.c_int32), ("pad3", C.c_int32), ("dst_sm", C.c_int64), ("dst_sn", C.c_int64),
        ("src_scale", Quant), ("wei_scale", Quant), ("dst_scale", Quant),
        ("src_zp", Quant), ("wei_zp", Quant), ("dst_zp", Quant),
        ("apply_to_int", C.c_int32), ("npo", C.c_int32), ("po", PostOp * MAX_PO),
        ("tanh_mode", C.c_int32), ("nthreads", C.c_int32),
        ("m0", C.c_int64), ("m_step", C.c_int64), ("n0", C.c_int64), ("n_step", C.c_int64),
        ("exact_acc", C.c_int32), ("pad4", C.c_int32),
    ]


class Reorder(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("cols", C.c_int64),
        ("src", C.c_void_p), ("src_dt", C.c_int32), ("pad0", C.c_int32), ("src_s0", C.c_int64), ("src_s1", C.c_int64),
        ("dst", C.c_void_p), ("dst_dt", C.c_int32), ("pad1", C.c_int32), ("dst_s0", C.c_int64), ("dst_s1", C.c_int64),
        ("src_scale", Quant), ("dst_scale", Quant), ("src_zp", Quant), ("dst_zp", Quant),
        ("beta", C.c_float), ("nthreads", C.c_int32),
    ]


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        so = HERE / "liboracle_matmul.so"
        src = HERE / "oracle_matmul.c"
        if not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
            subprocess.check_call(["make", "-C", str(HERE), "liboracle_matmul.so"], stdout=subprocess.DEVNULL)
        _lib = C.CDLL(str(so))
        _lib.orc_matmul.argtypes = [C.POINTER(Problem)]
        _lib.orc_matmul.restype = C.c_int
        _lib.orc_reorder.argtypes = [C.POINTER(Reorder)]
        _lib.orc_reorder.restype = C.c_int
        _lib.orc_load_float.argtypes = [C.c_int32, C.c_void_p, C.c_int64]
        _lib.orc_load_float.restype = C.c_float
        _lib.orc_store_float.argtypes = [C.c_int32, C.c_float, C.c_void_p, C.c_int64]
        _lib.orc_store_float.restype = None
        _lib.orc_eltwise.argtypes = [C.c_int32, C.c_float, C.c_float, C.c_float, C.c_int32]
        _lib.orc_eltwise.restype = C.c_float
        _lib.orc_tanh_portable.argtypes = [C.c_double]
        _lib.orc_tanh_portable.restype = C.c_double
    return _lib


def have_reference():
    return (HERE / "_ref" / "librefrun.so").exists()


def ref():
    global _ref
    if _ref is None:
        _ref = C.CDLL(str(HERE / "_ref" / "librefrun.so"), mode=os.RTLD_LOCAL)
        _ref.refrun_matmul.argtypes = [C.POINTER(Problem), C.c_char_p, C.c_int, C.c_int,
                                       C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_char_p, C.c_int]
        _ref.refrun_matmul.restype = C.c_int
        _ref.refrun_reorder.argtypes = [C.POINTER(Reorder), C.c_char_p, C.c_char_p, C.c_int]
        _ref.refrun_reorder.restype = C.c_int
    return _ref


def set_threads(n=0):
    """Number of OpenMP threads the oracle and the reference library use from now on
    (0 = all host cores).  Launchers such as torchrun export OMP_NUM_THREADS=1, which would
    otherwise turn a CPU baseline into a single-core one.  Returns the number in effect."""
    n = int(n) or (os.cpu_count() or 1)
    try:
        gomp = C.CDLL("libgomp.so.1", mode=os.RTLD_GLOBAL)
        gomp.omp_set_num_threads(n)
        return int(gomp.omp_get_max_threads())
    except OSError:
        return 1


def _ptr(a):
    return a.ctypes.data if a is not None else None


def _quant(q, kind, case):
    """kind: 'src' (m,k), 'wei' (k,n), 'dst' (m,n)."""
    out = Quant()
    if q is None:
        return out
    d0, d1 = {"src": (case.M, case.K), "wei": (case.K, case.N), "dst": (case.M, case.N)}[kind]
    g0, g1 = q.groups
    n1 = (d1 // g1) if (q.mask & 2) else 1
    out.ptr = _ptr(q.data)
    out.dt = q.dt
    out.s0 = n1 if (q.mask & 1) else 0
    out.s1 = 1 if (q.mask & 2) else 0
    out.g0, out.g1 = (g0 if (q.mask & 1) else 1), (g1 if (q.mask & 2) else 1)
    n0 = (d0 // g0) if (q.mask & 1) else 1
    out.nelems_is_one = 1 if n0 * n1 == 1 else 0
    return out


def make_problem(case, dst, tanh_mode=0, nthreads=0, m0=0, m_step=1, n0=0, n_step=1, exact_acc=0):
    """Fill an orc_problem_t for ``case``; ``dst`` is the raw (M, N) output array
    (pre-loaded with the prior dst contents when a sum post-op is present)."""
    p = Problem()
    p.M, p.N, p.K = case.M, case.N, case.K
    p.src, p.src_dt, p.src_sm, p.src_sk = _ptr(case.src), case.src_dt, case.K, 1
    p.wei, p.wei_dt = _ptr(case.wei), case.wei_dt
    if case.wei_tag == "ab":
        p.wei_sk, p.wei_sn = case.N, 1
    else:
        p.wei_sk, p.wei_sn = 1, case.K
    if case.bias is not None:
        p.bias, p.bias_dt = _ptr(case.bias), case.bias_dt
        bm, bn = case.bias.shape if case.bias.ndim == 2 else (1, case.bias.shape[0])
        p.bias_sm = case.N if (bm > 1 and bn > 1) else (1 if bm > 1 else 0)
        p.bias_sn = 1 if bn > 1 else 0
    p.dst, p.dst_dt, p.dst_sm, p.dst_sn = _ptr(dst), case.dst_dt, case.N, 1
    p.src_scale = _quant(case.src_scale, "src", case)
    p.wei_scale = _quant(case.wei_scale, "wei", case)
    p.dst_scale = _quant(case.dst_scale, "dst", case)
    p.src_zp = _quant(case.src_zp, "src", case)
    p.wei_zp = _quant(case.wei_zp, "wei", case)
    p.dst_zp = _quant(case.dst_zp, "dst", case)
    p.apply_to_int = 1 if case.apply_to_int else 0
    p.npo = len(case.post_ops)
    for i, e in enumerate(case.post_ops):
        o = p.po[i]
        o.kind, o.alg, o.alpha, o.beta, o.scale = e.kind, e.alg, e.alpha, e.beta, e.scale
        o.zero_point, o.dt = e.zero_point, e.dt
        if e.data is not None:
            o.ptr = _ptr(e.data)
            sm_, sn_ = e.shape
            o.sn = 1 if sn_ > 1 else 0
            o.sm = (sn_ if sn_ > 1 else 1) if sm_ > 1 else 0
    p.tanh_mode, p.nthreads = tanh_mode, nthreads
    p.m0, p.m_step, p.n0, p.n_step = m0, m_step, n0, n_step
    p.exact_acc = exact_acc
    return p


def new_dst(case):
    from onednn_b200 import dtypes as dt
    if case.dst_init is not None:
        return np.ascontiguousarray(case.dst_init).copy()
    return np.zeros((case.M, case.N), dtype=dt.RAW[case.dst_dt])


def run_oracle(case, tanh_mode=0, nthreads=0, m_step=1, n_step=1, m0=0, n0=0, exact_acc=0):
    dst = new_dst(case)
    p = make_problem(case, dst, tanh_mode, nthreads, m0, m_step, n0, n_step, exact_acc)
    rc = lib().orc_matmul(C.byref(p))
    if rc != 0:
        raise RuntimeError("orc_matmul failed: %d" % rc)
    return dst


def run_reference(case, impl="", weights_any=False, iters=0):
    """Returns (dst, impl_name, ms_min, ms_avg) from the reference library's CPU engine."""
    dst = new_dst(case)
    p = make_problem(case, dst)
    name = C.create_string_buffer(128)
    tmin, tavg = C.c_double(0), C.c_double(0)
    rc = ref().refrun_matmul(C.byref(p), impl.encode(), 1 if weights_any else 0, iters,
                             C.byref(tmin), C.byref(tavg), name, 128)
    if rc != 0:
        raise RuntimeError("refrun_matmul failed: %d" % rc)
    return dst, name.value.decode(), tmin.value, tavg.value


# ---- quantising reorder ---------------------------------------------------------------------

def _rquant(q, rows, cols):
    out = Quant()
    out.g0 = out.g1 = 1
    if q is None:
        return out
    g0, g1 = q.groups
    out.g0, out.g1 = (g0 if (q.mask & 1) else 1), (g1 if (q.mask & 2) else 1)
    n1 = (cols // out.g1) if (q.mask & 2) else 1
    n0 = (rows // out.g0) if (q.mask & 1) else 1
    out.ptr, out.dt = _ptr(q.data), q.dt
    out.s0 = n1 if (q.mask & 1) else 0
    out.s1 = 1 if (q.mask & 2) else 0
    out.nelems_is_one = 1 if n0 * n1 == 1 else 0
    return out


def make_reorder(case, dst, nthreads=0):
    """Fill an orc_reorder_t; ``dst`` is the raw destination in its physical order."""
    r = Reorder()
    r.rows, r.cols = case.rows, case.cols
    r.src, r.src_dt = _ptr(case.src), case.src_dt
    r.src_s0, r.src_s1 = (case.cols, 1) if case.src_tag == "ab" else (1, case.rows)
    r.dst, r.dst_dt = _ptr(dst), case.dst_dt
    r.dst_s0, r.dst_s1 = (case.cols, 1) if case.dst_tag == "ab" else (1, case.rows)
    r.src_scale = _rquant(case.src_scale, case.rows, case.cols)
    r.dst_scale = _rquant(case.dst_scale, case.rows, case.cols)
    r.src_zp = _rquant(case.src_zp, case.rows, case.cols)
    r.dst_zp = _rquant(case.dst_zp, case.rows, case.cols)
    r.beta, r.nthreads = case.beta, nthreads
    return r


def new_reorder_dst(case):
    from onednn_b200 import dtypes as dt
    shape = (case.rows, case.cols) if case.dst_tag == "ab" else (case.cols, case.rows)
    if case.dst_init is not None:
        return np.ascontiguousarray(case.dst_init).copy()
    if case.dst_dt in (dt.S4, dt.U4):  # two values per byte along the contiguous dim
        return np.zeros((shape[0], shape[1] // 2), dtype=np.uint8)
    return np.zeros(shape, dtype=dt.RAW[case.dst_dt])


def run_oracle_reorder(case, nthreads=0):
    dst = new_reorder_dst(case)
    r = make_reorder(case, dst, nthreads)
    rc = lib().orc_reorder(C.byref(r))
    if rc != 0:
        raise RuntimeError("orc_reorder failed: %d" % rc)
    return dst


def run_reference_reorder(case, impl=""):
    """Returns (dst, impl_name) from the reference library's CPU engine."""
    dst = new_reorder_dst(case)
    r = make_reorder(case, dst)
    name = C.create_string_buffer(128)
    rc = ref().refrun_reorder(C.byref(r), impl.encode(), name, 128)
    if rc != 0:
        raise RuntimeError("refrun_reorder failed: %d" % rc)
    return dst, name.value.decode()
