"""Synthetic matmul problems: the benchmark's configurations and test cases.

A :class:`MatmulCase` is the host-side description of one ``dnnl::matmul``
problem: tensors as raw numpy arrays plus the primitive attribute (scales,
zero-points, post-ops, fpmath apply_to_int).  The same object drives the CUDA
engine (``onednn_b200.api.run_case``) and, in the tests, the CPU oracle.

No public dataset is involved: every tensor is drawn from a seeded numpy
generator with the shapes and value distributions the benchmark names.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import numpy as np

from . import dtypes as dt

# dnnl_alg_kind_t values (reference: include/oneapi/dnnl/dnnl_types.h:2043-2110)
ELTWISE = {
    "relu": 0x20, "tanh": 0x21, "elu": 0x22, "square": 0x23, "abs": 0x24, "sqrt": 0x25,
    "linear": 0x26, "soft_relu": 0x27, "hardsigmoid": 0x28, "logistic": 0x29, "exp": 0x2A,
    "gelu_tanh": 0x2B, "swish": 0x2C, "log": 0x2D, "clip": 0x2E, "clip_v2": 0x2F, "pow": 0x30,
    "gelu_erf": 0x31, "round": 0x32, "mish": 0x33, "hardswish": 0x34,
}
BINARY = {
    "add": 0x1FFF0, "mul": 0x1FFF1, "max": 0x1FFF2, "min": 0x1FFF3, "div": 0x1FFF4, "sub": 0x1FFF5,
    "ge": 0x1FFF6, "gt": 0x1FFF7, "le": 0x1FFF8, "lt": 0x1FFF9, "eq": 0x1FFFA, "ne": 0x1FFFB,
}
PO_SUM, PO_ELTWISE, PO_BINARY, PO_PRELU = 1, 2, 3, 4


@dataclass
class Quant:
    """A scales or zero-points argument: raw data, its type, the dnnl mask over the
    tensor's two dims (bit 0 = first dim, bit 1 = second dim) and the group sizes."""
    data: np.ndarray
    dt: int
    mask: int = 0
    groups: Tuple[int, int] = (1, 1)


@dataclass
class PostOp:
    kind: int
    alg: int = 0
    alpha: float = 0.0
    beta: float = 0.0
    scale: float = 1.0
    zero_point: int = 0
    dt: int = dt.UNDEF
    data: Optional[np.ndarray] = None       # binary src1 / prelu weights, raw
    shape: Tuple[int, int] = (1, 1)         # logical 2-D shape of data (1 = broadcast)


@dataclass
class MatmulCase:
    name: str
    M: int
    N: int
    K: int
    src: np.ndarray
    src_dt: int
    wei: np.ndarray                 # logical (K, N); 4-bit types packed along the contiguous dim
    wei_dt: int
    dst_dt: int
    wei_tag: str = "ab"             # "ab": N contiguous, "ba": K contiguous
    bias: Optional[np.ndarray] = None
    bias_dt: int = dt.UNDEF
    dst_init: Optional[np.ndarray] = None   # prior dst contents (sum post-op)
    src_scale: Optional[Quant] = None
    wei_scale: Optional[Quant] = None
    dst_scale: Optional[Quant] = None
    src_zp: Optional[Quant] = None
    wei_zp: Optional[Quant] = None
    dst_zp: Optional[Quant] = None
    post_ops: List[PostOp] = field(default_factory=list)
    apply_to_int: bool = False
    exact: bool = True              # integer dst: bit-exact; else use rtol/atol
    rtol: float = 0.0
    atol: float = 0.0

    @property
    def ops(self):
        """2*M*N*K, the reference's own count (tests/benchdnn/matmul/matmul.hpp:133-135)."""
        return 2 * self.M * self.N * self.K

    def algorithmic_bytes(self):
        """Minimum HBM traffic: every input read once, dst written once."""
        n = self.src.nbytes + self.wei.nbytes + dt.nbytes(self.dst_dt, self.M * self.N)
        if self.bias is not None:
            n += self.bias.nbytes
        for q in (self.src_scale, self.wei_scale, self.dst_scale, self.src_zp, self.wei_zp, self.dst_zp):
            if q is not None:
                n += q.data.nbytes
        for p in self.post_ops:
            if p.kind == PO_SUM:
                n += dt.nbytes(p.dt or self.dst_dt, self.M * self.N)
            elif p.data is not None:
                n += p.data.nbytes
        return n


@dataclass
class ReorderCase:
    """One quantising ``dnnl::reorder`` of a plain 2-D tensor: scales / zero-points on the
    source and destination side (masks over (rows, cols)), optional sum post-op."""
    name: str
    rows: int
    cols: int
    src: np.ndarray
    src_dt: int
    dst_dt: int
    src_tag: str = "ab"             # "ab": columns contiguous, "ba": rows contiguous
    dst_tag: str = "ab"
    src_scale: Optional[Quant] = None
    dst_scale: Optional[Quant] = None
    src_zp: Optional[Quant] = None
    dst_zp: Optional[Quant] = None
    beta: float = 0.0               # sum post-op scale (0 = none)
    dst_init: Optional[np.ndarray] = None
    exact: bool = True              # every destination type: the arithmetic is elementwise f32


def quantize_case(rows=4096, cols=4096, src_dt=dt.F32, dst_dt=dt.S8, seed=20240620, per_row=False, name=None):
    """Activations -> int8 in front of an int8 matmul: dst = sat_rne(src / scale + zp)."""
    rng = np.random.default_rng(seed)
    x = (rng.standard_normal((rows, cols)) * 1.5).astype(np.float32)
    src = x if src_dt == dt.F32 else dt.from_f32(x, src_dt)
    if per_row:
        sc = (np.abs(x).max(axis=1) / 127.0).astype(np.float32)
        dscale = Quant(sc, dt.F32, 1)
    else:
        dscale = Quant(np.float32([0.043]), dt.F32, 0)
    zp = None if dst_dt == dt.S8 else Quant(np.int32([128]), dt.S32, 0)
    return ReorderCase(name or "quantize_%dx%d" % (rows, cols), rows, cols, src, src_dt, dst_dt, dst_scale=dscale, dst_zp=zp)


def eltwise(name, alpha=0.0, beta=0.0):
    return PostOp(PO_ELTWISE, alg=ELTWISE[name], alpha=alpha, beta=beta, scale=1.0)


def sum_(scale=1.0, zero_point=0, dt_=dt.UNDEF):
    return PostOp(PO_SUM, scale=scale, zero_point=zero_point, dt=dt_)


def binary(name, data, dt_, shape):
    return PostOp(PO_BINARY, alg=BINARY[name], dt=dt_, data=data, shape=shape)


def prelu(weights_f32, shape):
    return PostOp(PO_PRELU, data=np.asarray(weights_f32, dtype=np.float32), dt=dt.F32, shape=shape)


def _f32(x):
    return np.asarray(x, dtype=np.float32)


def config0(M=128, N=1024, K=1024, seed=20240611):
    """u8 x s8 -> f32, source zero-point 128, per-N weight scales, f32 bias, ReLU."""
    r = np.random.default_rng(seed)
    return MatmulCase(
        "c0_int8_f32_relu", M, N, K,
        src=r.integers(0, 256, (M, K), dtype=np.uint8), src_dt=dt.U8,
        wei=r.integers(-127, 128, (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dt.F32,
        bias=_f32(r.uniform(-1, 1, (1, N))), bias_dt=dt.F32,
        src_scale=Quant(_f32([0.02]), dt.F32, 0),
        wei_scale=Quant(_f32(r.uniform(1e-3, 1e-2, N)), dt.F32, 2),
        src_zp=Quant(np.array([128], dtype=np.int32), dt.S32, 0),
        post_ops=[eltwise("relu")], exact=False, rtol=1e-5, atol=1e-6)


def config1(M=4096, N=4096, K=4096, seed=20240612, dst_scale=0.1):
    """s8 x s8 -> s8 with bf16 bias, GELU-tanh, sum(0.5) over a prior s8 dst, dst scale and zero-point."""
    r = np.random.default_rng(seed)
    return MatmulCase(
        "c1_int8_s8_gelu_sum", M, N, K,
        src=np.clip(np.rint(r.normal(0, 30, (M, K))), -128, 127).astype(np.int8), src_dt=dt.S8,
        wei=r.integers(-127, 128, (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dt.S8,
        bias=dt.f32_to_bf16(_f32(r.uniform(-0.5, 0.5, (1, N)))), bias_dt=dt.BF16,
        dst_init=r.integers(-64, 65, (M, N), dtype=np.int8),
        src_scale=Quant(_f32([0.05]), dt.F32, 0),
        wei_scale=Quant(_f32(r.uniform(5e-4, 5e-3, N)), dt.F32, 2),
        dst_scale=Quant(_f32([dst_scale]), dt.F32, 0),
        dst_zp=Quant(np.array([3], dtype=np.int32), dt.S32, 0),
        post_ops=[eltwise("gelu_tanh"), sum_(0.5)], exact=True)


def config2(M=1, N=14336, K=4096, seed=20240613, group=128):
    """bf16 x u4 weight decompression with K-grouped bf16 scales and u4 zero-points -> bf16."""
    r = np.random.default_rng(seed)
    ng = K // group
    return MatmulCase(
        "c2_wc_u4_m%d" % M, M, N, K,
        src=dt.f32_to_bf16(_f32(r.normal(0, 1, (M, K)))), src_dt=dt.BF16,
        wei=dt.pack_int4(r.integers(0, 16, (K, N))), wei_dt=dt.U4, dst_dt=dt.BF16,
        wei_scale=Quant(dt.f32_to_bf16(_f32(r.uniform(0.005, 0.02, (ng, N)))), dt.BF16, 3, (group, 1)),
        wei_zp=Quant(dt.pack_int4(r.integers(6, 10, (ng, N))), dt.U4, 3, (group, 1)),
        apply_to_int=True, exact=False, rtol=1e-2, atol=1e-2)


def config3(M=8192, N=8192, K=8192, seed=20240614):
    """e4m3 x e4m3 -> bf16 with per-tensor scales and bf16 bias."""
    r = np.random.default_rng(seed)

    def gen(shape):
        return dt.f32_to_e4m3(np.clip(_f32(r.standard_normal(shape, dtype=np.float32)) * 4, -448, 448))
    return MatmulCase(
        "c3_fp8_bf16", M, N, K,
        src=gen((M, K)), src_dt=dt.F8_E4M3, wei=gen((K, N)), wei_dt=dt.F8_E4M3, dst_dt=dt.BF16,
        bias=dt.f32_to_bf16(_f32(r.uniform(-1, 1, (1, N)))), bias_dt=dt.BF16,
        src_scale=Quant(_f32([0.25]), dt.F32, 0), wei_scale=Quant(_f32([0.125]), dt.F32, 0),
        exact=False, rtol=1e-2, atol=1e-2)


def config4(M=16384, N=28672, K=8192, seed=20240615):
    """Large s8 x s8 -> bf16 with per-N weight scales and bf16 bias (the sharded configuration)."""
    r = np.random.default_rng(seed)
    src = np.clip(np.rint(r.standard_normal((M, K), dtype=np.float32) * 30), -128, 127).astype(np.int8)
    return MatmulCase(
        "c4_int8_bf16", M, N, K,
        src=src, src_dt=dt.S8,
        wei=r.integers(-127, 128, (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dt.BF16,
        bias=dt.f32_to_bf16(_f32(r.uniform(-0.5, 0.5, (1, N)))), bias_dt=dt.BF16,
        src_scale=Quant(_f32([0.05]), dt.F32, 0),
        wei_scale=Quant(_f32(r.uniform(5e-4, 5e-3, N)), dt.F32, 2),
        exact=False, rtol=1e-2, atol=1e-2)


CONFIGS = [config0, config1, config2, config3, config4]


def shard(case: MatmulCase, rank: int, world: int, how: str) -> MatmulCase:
    """The part of ``case`` that rank ``rank`` of ``world`` computes.

    ``how == "m"``: rows [rank*M/world, (rank+1)*M/world) of src/dst, weights replicated.
    ``how == "n"``: columns of weights, per-N scales, bias and dst; src replicated.
    """
    import copy
    c = copy.copy(case)
    if world == 1:
        return c
    if how == "m":
        assert case.M % world == 0
        m = case.M // world
        sl = slice(rank * m, (rank + 1) * m)
        c.M = m
        c.src = np.ascontiguousarray(case.src[sl])
        if case.dst_init is not None:
            c.dst_init = np.ascontiguousarray(case.dst_init[sl])
        return c
    assert how == "n" and case.N % world == 0 and case.wei_dt not in (dt.S4, dt.U4)
    n = case.N // world
    sl = slice(rank * n, (rank + 1) * n)
    c.N = n
    c.wei = np.ascontiguousarray(case.wei[:, sl])
    if case.bias is not None:
        c.bias = np.ascontiguousarray(case.bias[:, sl])
    if case.dst_init is not None:
        c.dst_init = np.ascontiguousarray(case.dst_init[:, sl])
    if case.wei_scale is not None and case.wei_scale.mask & 2:
        q = case.wei_scale
        c.wei_scale = Quant(np.ascontiguousarray(q.data.reshape(-1, case.N)[:, sl]).reshape(-1), q.dt, q.mask, q.groups)
    return c
