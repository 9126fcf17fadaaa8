"""ctypes view of the inner kernel launch ABI (``include/onednn_b200_kernels.h``).

For callers that hold device pointers already and want to launch a kernel
directly, without the descriptor / primitive layer: fill a
:class:`MatmulParams` and call ``lib().b200_matmul_*_launch``.
"""
import ctypes as C

from . import api

MAX_POSTOPS = 32
WEI_PLAIN, WEI_KMAJOR, WEI_WC4_TILED = 0, 1, 2
ERR_UNSUPPORTED, ERR_BAD_ARG, ERR_TOO_LARGE = -1, -2, -3


class Quant(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dt", C.c_int32), ("reserved", C.c_int32),
                ("s0", C.c_int64), ("s1", C.c_int64), ("g0", C.c_int64), ("g1", C.c_int64)]


class PostOp(C.Structure):
    _fields_ = [("kind", C.c_int32), ("alg", C.c_int32), ("alpha", C.c_float), ("beta", C.c_float),
                ("scale", C.c_float), ("zero_point", C.c_int32), ("dt", C.c_int32), ("reserved", C.c_int32),
                ("ptr", C.c_void_p), ("sm", C.c_int64), ("sn", C.c_int64)]


class MatmulParams(C.Structure):
    _fields_ = [
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64),
        ("src", C.c_void_p), ("src_dt", C.c_int32), ("reserved0", C.c_int32), ("src_sm", C.c_int64), ("src_sk", C.c_int64),
        ("wei", C.c_void_p), ("wei_dt", C.c_int32), ("wei_layout", C.c_int32), ("wei_sk", C.c_int64), ("wei_sn", C.c_int64),
        ("bias", C.c_void_p), ("bias_dt", C.c_int32), ("reserved1", C.c_int32), ("bias_sm", C.c_int64), ("bias_sn", C.c_int64),
        ("dst", C.c_void_p), ("dst_dt", C.c_int32), ("reserved2", C.c_int32), ("dst_sm", C.c_int64), ("dst_sn", C.c_int64),
        ("src_scale", Quant), ("wei_scale", Quant), ("dst_scale", Quant),
        ("src_zp", Quant), ("wei_zp", Quant), ("dst_zp", Quant),
        ("wei_colsum", C.c_void_p),
        ("apply_to_int", C.c_int32), ("npo", C.c_int32),
        ("po", PostOp * MAX_POSTOPS),
        ("status", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
        ("scratch_zeroed", C.c_int32), ("reserved3", C.c_int32),
        ("n_dst_peers", C.c_int32), ("reserved4", C.c_int32), ("dst_peer", C.c_void_p * 7),
        ("src_rowsum", C.c_void_p),
    ]


def quant(ptr, dt, s0=0, s1=0, g0=1, g1=1):
    q = Quant()
    q.ptr, q.dt, q.s0, q.s1, q.g0, q.g1 = ptr, dt, s0, s1, g0, g1
    return q


def lib():
    L = api.lib()
    L.b200_gather_columns_launch.restype = C.c_int
    L.b200_gather_columns_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_void_p]
    L.b200_matmul_scratch_bytes.restype = C.c_size_t
    L.b200_matmul_scratch_bytes.argtypes = [C.POINTER(MatmulParams), C.c_int]
    L.b200_matmul_wc_noalloc_max_bytes.restype = C.c_size_t
    for name in ("b200_matmul_generic_launch", "b200_matmul_tc8_launch", "b200_matmul_wc_launch",
                 "b200_matmul_wc_noalloc_launch"):
        getattr(L, name).argtypes = [C.POINTER(MatmulParams), C.c_void_p]
        getattr(L, name).restype = C.c_int
    L.b200_wc_pack_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32, C.c_void_p]
    L.b200_wc_pack_launch.restype = C.c_int
    L.b200_tc8_mma_peak_launch.argtypes = [C.c_int32, C.c_uint32, C.c_void_p, C.POINTER(C.c_uint64), C.c_void_p]
    L.b200_tc8_mma_peak_launch.restype = C.c_int
    return L
