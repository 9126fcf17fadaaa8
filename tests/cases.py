"""Catalogue of small seeded matmul problems shared by the parity tests.

Each entry is a zero-argument constructor of a MatmulCase.  The sizes are small
enough for the scalar CPU oracle to finish in well under a second; together
they cover the attribute space of the quantized matmul path: the five
benchmark configurations at reduced size, zero-points and scales in every mask
the reference admits, K-grouped quantisation, every post-op kind, ragged and
degenerate shapes, transposed weights and every destination type.
"""
import numpy as np

from onednn_b200 import dtypes as dt
from onednn_b200 import workloads as W
from onednn_b200.workloads import MatmulCase, Quant, ReorderCase


def _f32(x):
    return np.asarray(x, dtype=np.float32)


def _int8_base(M, N, K, seed, src_dt=dt.S8, dst_dt=dt.F32):
    r = np.random.default_rng(seed)
    if src_dt == dt.U8:
        src = r.integers(0, 256, (M, K), dtype=np.uint8)
    else:
        src = r.integers(-128, 128, (M, K), dtype=np.int8)
    return r, MatmulCase("int8", M, N, K, src=src, src_dt=src_dt,
                         wei=r.integers(-127, 128, (K, N), dtype=np.int8), wei_dt=dt.S8, dst_dt=dst_dt,
                         exact=dst_dt in (dt.S8, dt.U8, dt.S32), rtol=1e-5, atol=1e-5)


def int8_plain_s32():
    r, c = _int8_base(33, 50, 70, 1, dst_dt=dt.S32)
    return c


def int8_ragged_tiny():
    r, c = _int8_base(1, 2, 1, 2, dst_dt=dt.S32)
    return c


def int8_u8dst_binary_prelu():
    r, c = _int8_base(48, 40, 96, 3, src_dt=dt.U8, dst_dt=dt.U8)
    c.src_scale = Quant(_f32([0.01]), dt.F32, 0)
    c.wei_scale = Quant(_f32(r.uniform(1e-3, 1e-2, 40)), dt.F32, 2)
    c.src_zp = Quant(np.array([100], dtype=np.int32), dt.S32, 0)
    c.dst_scale = Quant(_f32([0.05]), dt.F32, 0)
    c.dst_zp = Quant(np.array([128], dtype=np.int32), dt.S32, 0)
    c.post_ops = [W.binary("add", _f32(r.uniform(-1, 1, (1, 40))), dt.F32, (1, 40)),
                  W.prelu(r.uniform(0.1, 0.5, (1, 40)), (1, 40)),
                  W.binary("mul", dt.f32_to_bf16(_f32(r.uniform(0.5, 1.5, (48, 1)))), dt.BF16, (48, 1)),
                  W.binary("max", _f32(r.uniform(-1, 1, (48, 40))), dt.F32, (48, 40))]
    return c


def int8_wei_zp_common():
    r, c = _int8_base(16, 24, 64, 4, dst_dt=dt.S8)
    c.src_scale = Quant(_f32([0.02]), dt.F32, 0)
    c.wei_scale = Quant(_f32([0.004]), dt.F32, 0)
    c.src_zp = Quant(np.array([-3], dtype=np.int32), dt.S32, 0)
    c.wei_zp = Quant(np.array([5], dtype=np.int32), dt.S32, 0)
    c.dst_scale = Quant(_f32([0.25]), dt.F32, 0)
    return c


def int8_wei_zp_per_n_relu():
    """Zero-points on both sides, the weights' one per column: several tiles, ragged edges,
    a straight-line post-op chain (the tensor-core kernel folds them in from the row sums of src)."""
    r, c = _int8_base(200, 328, 256, 24, src_dt=dt.U8, dst_dt=dt.S8)
    c.src_scale = Quant(_f32([0.02]), dt.F32, 0)
    c.wei_scale = Quant(_f32(r.uniform(2e-3, 6e-3, 328)), dt.F32, 2)
    c.src_zp = Quant(np.array([121], dtype=np.int32), dt.S32, 0)
    c.wei_zp = Quant(r.integers(-9, 10, 328).astype(np.int32), dt.S32, 2)
    c.dst_scale = Quant(_f32([0.125]), dt.F32, 0)
    c.dst_zp = Quant(np.array([-7], dtype=np.int32), dt.S32, 0)
    c.post_ops = [W.eltwise("relu", 0.25)]
    return c


def int8_wei_zp_gelu_sum():
    """Weights zero-point (no source zero-point) under gelu_tanh and sum: the interpreted chain."""
    r, c = _int8_base(70, 144, 128, 25, dst_dt=dt.S8)
    c.dst_init = r.integers(-128, 128, (70, 144), dtype=np.int8)
    c.src_scale = Quant(_f32([0.03]), dt.F32, 0)
    c.wei_scale = Quant(_f32([0.005]), dt.F32, 0)
    c.wei_zp = Quant(np.array([-11], dtype=np.int32), dt.S32, 0)
    c.dst_scale = Quant(_f32([0.05]), dt.F32, 0)
    c.post_ops = [W.eltwise("gelu_tanh"), W.sum_(0.5)]
    return c


def int8_sum_u8_as_s8():
    """sum post-op that reads the u8 dst as s8 with its own zero-point, then clip."""
    r, c = _int8_base(20, 32, 48, 5, dst_dt=dt.U8)
    c.dst_init = r.integers(0, 256, (20, 32), dtype=np.uint8)
    c.src_scale = Quant(_f32([0.003]), dt.F32, 0)
    c.post_ops = [W.sum_(0.75, 2, dt.S8), W.eltwise("clip_v2", -5.0, 200.0), W.eltwise("linear", 1.5, 0.25)]
    return c


def int8_bf16_dst_transposed_wei():
    r, c = _int8_base(24, 36, 80, 6, dst_dt=dt.BF16)
    c.wei = np.ascontiguousarray(c.wei.T)  # stored (N, K): tag "ba"
    c.wei_tag = "ba"
    c.wei_scale = Quant(_f32(r.uniform(1e-3, 1e-2, 36)), dt.F32, 2)
    c.bias = dt.f32_to_bf16(_f32(r.uniform(-1, 1, (1, 36))))
    c.bias_dt = dt.BF16
    c.exact, c.rtol, c.atol = False, 1e-2, 1e-2
    return c


def _elt_case(name, alpha=0.0, beta=0.0, seed=7):
    def make():
        r, c = _int8_base(16, 64, 32, seed)
        c.src_scale = Quant(_f32([0.01]), dt.F32, 0)
        c.wei_scale = Quant(_f32(r.uniform(1e-3, 5e-3, 64)), dt.F32, 2)
        c.post_ops = [W.eltwise(name, alpha, beta)]
        return c
    return make


def _wc_case(M, N, K, group, wei_dt, src_dt=dt.BF16, zp="grouped", seed=11, dst_dt=dt.BF16):
    def make():
        r = np.random.default_rng(seed)
        x = _f32(r.normal(0, 1, (M, K)))
        ng = K // group
        if wei_dt == dt.U4:
            wei = dt.pack_int4(r.integers(0, 16, (K, N)))
        elif wei_dt == dt.S4:
            wei = dt.pack_int4(r.integers(-8, 8, (K, N)))
        elif wei_dt == dt.S8:
            wei = r.integers(-128, 128, (K, N), dtype=np.int8)
        else:
            wei = r.integers(0, 256, (K, N), dtype=np.uint8)
        c = MatmulCase("wc", M, N, K, src=dt.from_f32(x, src_dt), src_dt=src_dt, wei=wei, wei_dt=wei_dt,
                       dst_dt=dst_dt, apply_to_int=True, exact=False, rtol=1e-2, atol=1e-2)
        sc = _f32(r.uniform(0.005, 0.02, (ng, N)))
        c.wei_scale = Quant(dt.f32_to_bf16(sc), dt.BF16, 3, (group, 1)) if ng > 1 else \
            Quant(dt.f32_to_bf16(sc.reshape(-1)), dt.BF16, 2)
        if zp == "grouped":
            if wei_dt in (dt.U4, dt.S4):
                lo, hi = (6, 10) if wei_dt == dt.U4 else (-2, 3)
                c.wei_zp = Quant(dt.pack_int4(r.integers(lo, hi, (ng, N))), wei_dt, 3, (group, 1))
            else:
                c.wei_zp = Quant(r.integers(-4, 5, (ng, N)).astype(np.int8), dt.S8, 3, (group, 1))
        elif zp == "common":
            c.wei_zp = Quant(np.array([3], dtype=np.int32), dt.S32, 0)
        return c
    return make


def fp8_f8dst():
    c = W.config3(24, 40, 64, seed=21)
    c.dst_dt = dt.F8_E4M3
    c.src_scale = Quant(_f32([0.05]), dt.F32, 0)
    c.exact, c.rtol, c.atol = False, 0.07, 0.02
    return c


def fp8_swish_f32():
    c = W.config3(17, 33, 48, seed=22)
    c.dst_dt = dt.F32
    c.post_ops = [W.eltwise("swish", 1.0)]
    c.rtol, c.atol = 1e-4, 1e-4
    return c


def int8_rows300_ragged_zp():
    """More than two row tiles, ragged in every dim, source zero-point, relu, s8 out."""
    r, c = _int8_base(300, 200, 144, 31, src_dt=dt.U8, dst_dt=dt.S8)
    c.src_scale = Quant(_f32([0.02]), dt.F32, 0)
    c.wei_scale = Quant(_f32(r.uniform(1e-3, 4e-3, 200)), dt.F32, 2)
    c.src_zp = Quant(np.array([120], dtype=np.int32), dt.S32, 0)
    c.dst_scale = Quant(_f32([0.4]), dt.F32, 0)
    c.dst_zp = Quant(np.array([-7], dtype=np.int32), dt.S32, 0)
    c.bias, c.bias_dt = _f32(r.uniform(-2, 2, (1, 200))), dt.F32
    c.post_ops = [W.eltwise("relu", 0.1)]
    return c


def int8_rows513_gelu_sum():
    """Five row tiles (an odd number: the last tile of a CTA pair is half empty), gelu + sum into s8."""
    c = W.config1(513, 272, 272, seed=32, dst_scale=0.9)
    return c


def fp8_rows260_bf16():
    c = W.config3(260, 520, 256, seed=33)
    return c


def int8_per_row_src_scales_bf16():
    """Dynamic (per-token) quantisation: one source scale per row (mask M+K, one group over K)."""
    r, c = _int8_base(200, 96, 128, 34, dst_dt=dt.BF16)
    c.src_scale = Quant(_f32(r.uniform(0.005, 0.05, 200)), dt.F32, 3, (1, 128))
    c.wei_scale = Quant(_f32(r.uniform(1e-3, 4e-3, 96)), dt.F32, 2)
    c.bias, c.bias_dt = dt.f32_to_bf16(_f32(r.uniform(-1, 1, (1, 96)))), dt.BF16
    c.exact, c.rtol, c.atol = False, 1e-2, 1e-2
    return c


def _int8_one_column(tag):
    """A single output column: both strides of the (K, 1) weights are 1 whatever the tag."""
    def make():
        r, c = _int8_base(40, 1, 64, 37, dst_dt=dt.S8)
        c.wei_tag = tag
        c.src_scale = Quant(_f32([0.01]), dt.F32, 0)
        c.wei_scale = Quant(_f32([0.004]), dt.F32, 2)
        c.bias, c.bias_dt = _f32(r.uniform(-1, 1, (1, 1))), dt.F32
        c.post_ops = [W.eltwise("relu", 0.25)]
        return c
    return make


def int8_per_row_src_scales_gelu_s8():
    c = W.config1(160, 64, 96, seed=35, dst_scale=0.7)
    r = np.random.default_rng(36)
    c.src_scale = Quant(_f32(r.uniform(0.02, 0.08, 160)), dt.F32, 3, (1, 96))
    return c


CASES = {
    # the benchmark's configurations at reduced size
    "c0_small": lambda: W.config0(64, 96, 128),
    "c0_full": lambda: W.config0(),
    "c1_small": lambda: W.config1(96, 128, 256),
    "c1_small_nonsat": lambda: W.config1(96, 128, 256, dst_scale=0.8),
    "c1_mid_nonsat": lambda: W.config1(256, 384, 512, dst_scale=1.0),
    "c2_m1": lambda: W.config2(1, 256, 512),
    "c2_m16": lambda: W.config2(16, 128, 256),
    "c3_small": lambda: W.config3(64, 96, 128),
    "c4_small": lambda: W.config4(64, 128, 256),
    # attribute space
    "int8_plain_s32": int8_plain_s32,
    "int8_ragged_tiny": int8_ragged_tiny,
    "int8_u8dst_binary_prelu": int8_u8dst_binary_prelu,
    "int8_wei_zp_common": int8_wei_zp_common,
    "int8_wei_zp_per_n_relu": int8_wei_zp_per_n_relu,
    "int8_wei_zp_gelu_sum": int8_wei_zp_gelu_sum,
    "int8_sum_u8_as_s8": int8_sum_u8_as_s8,
    "int8_bf16_dst_transposed_wei": int8_bf16_dst_transposed_wei,
    "elt_tanh": _elt_case("tanh"),
    "elt_logistic": _elt_case("logistic"),
    "elt_swish": _elt_case("swish", 1.0),
    "elt_gelu_erf": _elt_case("gelu_erf"),
    "elt_exp": _elt_case("exp"),
    "elt_elu": _elt_case("elu", 0.7),
    "elt_mish": _elt_case("mish"),
    "elt_hardswish": _elt_case("hardswish", 1.0 / 6, 0.5),
    "elt_abs_sqrt": lambda: _two_elt(),
    "wc_u4_g64_m3": _wc_case(3, 64, 256, 64, dt.U4),
    # decode kernel: whole strips per CTA (N / 16 >= SM count), units of one group
    "wc_u4_g128_m1_wide": _wc_case(1, 2560, 256, 128, dt.U4, seed=12),
    "wc_u4_g128_m9_wide": _wc_case(9, 2560, 256, 128, dt.U4, seed=13),
    "wc_s4_g256_m20_wide": _wc_case(20, 2432, 512, 256, dt.S4, seed=14),
    # decode kernel: few strips, K split across CTAs, strips shared between CTAs
    "wc_u4_g128_m1_deep": _wc_case(1, 64, 4096, 128, dt.U4, seed=15),
    "wc_u4_g64_m5_mid": _wc_case(5, 1040, 192, 64, dt.U4, seed=16),
    "wc_s4_perN_m2": _wc_case(2, 96, 384, 384, dt.S4, seed=17, zp="none"),
    # tensor-core weight decompression (more than 32 rows): ragged N, two passes over M, no zero-points
    "wc_tc_u4_g64_m33_ragged": _wc_case(33, 208, 128, 64, dt.U4, seed=18),
    "wc_tc_u4_g128_m40_wide": _wc_case(40, 2560, 256, 128, dt.U4, seed=20),
    "wc_tc_s4_perN_m300": _wc_case(300, 144, 192, 192, dt.S4, seed=19, zp="none"),
    # the same kernel with fewer tiles than SMs and a long K: the operand rings wrap many times
    "wc_tc_u4_g128_m40_longk": _wc_case(40, 1280, 1024, 128, dt.U4, seed=26),
    "wc_tc_s4_g256_m130_longk": _wc_case(130, 640, 2048, 256, dt.S4, seed=27),
    # 8-bit weight decompression on the tensor cores (any M): s8 with grouped f32-free bf16 scales and s8
    # zero-points, u8 per-column without zero-points, one row
    "wc8_s8_g64_m5": _wc_case(5, 200, 256, 64, dt.S8, seed=21),
    "wc8_u8_perN_m70": _wc_case(70, 136, 192, 192, dt.U8, seed=22, zp="none"),
    "wc8_s8_g128_m1_common_zp": _wc_case(1, 384, 256, 128, dt.S8, seed=23, zp="common"),
    "wc8_s8_g64_m5_longk": _wc_case(5, 1280, 1024, 64, dt.S8, seed=28),
    "wc_s4_g32_m2_f32dst": _wc_case(2, 32, 128, 32, dt.S4, dst_dt=dt.F32),
    "wc_s8_perN_common_zp": _wc_case(5, 48, 96, 96, dt.S8, zp="common"),
    "wc_u8_g32_nozp": _wc_case(4, 40, 64, 32, dt.U8, zp="none"),
    "int8_rows300_ragged_zp": int8_rows300_ragged_zp,
    "int8_rows513_gelu_sum": int8_rows513_gelu_sum,
    "fp8_rows260_bf16": fp8_rows260_bf16,
    "int8_per_row_src_scales_bf16": int8_per_row_src_scales_bf16,
    "int8_per_row_src_scales_gelu_s8": int8_per_row_src_scales_gelu_s8,
    "fp8_f8dst": fp8_f8dst,
    "fp8_swish_f32": fp8_swish_f32,
    "int8_one_column_ab": _int8_one_column("ab"),
    "int8_one_column_ba": _int8_one_column("ba"),
}


def _two_elt():
    c = _elt_case("abs")()
    c.post_ops.append(W.eltwise("sqrt"))
    c.post_ops.append(W.eltwise("soft_relu", 0.5))
    return c


def build(name):
    if name.startswith("tame/"):
        return build_tame(name[5:])
    c = CASES[name]()
    c.name = name
    return c


# ---- the int8 catalogue on data whose f32 sums are exact ------------------------------------
# The reference's scalar int8 implementation scales every product and accumulates in f32; its
# optimised implementation and the tensor-core kernel here accumulate exactly in s32 and scale
# once.  On inputs like those the reference's own test driver draws -- small integers
# (tests/benchdnn/matmul/cfg.cpp:63-134) and power-of-two scales
# (tests/benchdnn/utils/fill.cpp:118-142) -- every scaled product and every partial sum is an
# integer times a power of two below 2^24, so the f32 accumulation is exact, the two orders of
# operations give the same bits, and the exact-accumulation result can be pinned to the
# reference's own output over the whole attribute catalogue.

def _pow2(q):
    """The same scales argument with every value replaced by the nearest power of two."""
    v = dt.to_f32(q.data, q.dt).astype(np.float64)
    v = np.exp2(np.rint(np.log2(v))).astype(np.float32)
    return Quant(v if q.dt == dt.F32 else dt.from_f32(v, q.dt), q.dt, q.mask, q.groups)


def is_int8_case(c):
    return c.src_dt in (dt.S8, dt.U8) and c.wei_dt in (dt.S8, dt.U8) and not c.apply_to_int


def build_tame(name):
    c = build(name)
    assert is_int8_case(c), name
    r = np.random.default_rng(1000 + sum(map(ord, name)))
    if c.src_dt == dt.U8:
        c.src = r.integers(0, 9, c.src.shape, dtype=np.uint8)
    else:
        c.src = r.integers(-4, 5, c.src.shape, dtype=np.int8)
    c.wei = r.integers(-4, 5, c.wei.shape, dtype=np.int8)
    for attr in ("src_scale", "wei_scale"):
        q = getattr(c, attr)
        if q is not None:
            setattr(c, attr, _pow2(q))
    if c.src_zp is not None:
        c.src_zp = Quant(np.array([4], dtype=np.int32), dt.S32, c.src_zp.mask, c.src_zp.groups)
    if c.wei_zp is not None:
        c.wei_zp = Quant(np.ones(c.wei_zp.data.shape, dtype=np.int32), dt.S32, c.wei_zp.mask, c.wei_zp.groups)
    # the sums are now a few hundred at most: keep the requantised outputs inside the range
    if c.dst_scale is not None:
        c.dst_scale = Quant(_f32([2.0 ** -6]), dt.F32, 0)
    c.name = "tame/" + name
    return c


def tame_names():
    return ["tame/" + n for n in CASES if is_int8_case(CASES[n]())]


# ---- quantising reorders -------------------------------------------------------------------
# What surrounds the int8 matmul: activations quantised in front of it (per tensor, per row,
# per column), its s32 / s8 results dequantised or requantised behind it.

def _rsrc(r, rows, cols, src_dt, spread=40.0):
    if src_dt in (dt.S4, dt.U4):
        return dt.pack_int4(r.integers(0, 16, (rows, cols)))
    x = (r.standard_normal((rows, cols)) * spread).astype(np.float32)
    if src_dt == dt.S8:
        return np.clip(np.rint(x), -128, 127).astype(np.int8)
    if src_dt == dt.U8:
        return np.clip(np.rint(x + 128), 0, 255).astype(np.uint8)
    if src_dt == dt.S32:
        return np.rint(x * 1000).astype(np.int32)
    return x if src_dt == dt.F32 else dt.from_f32(x, src_dt)


def _rq(r, rows, cols, mask, lo, hi, qdt=dt.F32, groups=(1, 1)):
    n0 = rows // groups[0] if mask & 1 else 1
    n1 = cols // groups[1] if mask & 2 else 1
    v = _f32(r.uniform(lo, hi, n0 * n1))
    return Quant(v if qdt == dt.F32 else dt.from_f32(v, qdt), qdt, mask, groups)


def _zp(v):
    return Quant(np.array([v], dtype=np.int32), dt.S32, 0)


def _reorder(seed, rows, cols, src_dt, dst_dt, **kw):
    r = np.random.default_rng(seed)
    c = ReorderCase("reorder", rows, cols, _rsrc(r, rows, cols, src_dt, kw.pop("spread", 40.0)), src_dt, dst_dt)
    for k, v in kw.items():
        setattr(c, k, v(r) if callable(v) else v)
    if c.src_tag == "ba":
        c.src = np.ascontiguousarray(c.src.T)
    return c


def _sum_init(r, rows=40, cols=64):
    return r.integers(-60, 60, (rows, cols)).astype(np.int8)


REORDER_CASES = {
    "q_f32_s8_tensor": lambda: _reorder(101, 64, 128, dt.F32, dt.S8, dst_scale=lambda r: _rq(r, 64, 128, 0, 0.3, 0.4)),
    "q_f32_u8_zp": lambda: _reorder(102, 64, 128, dt.F32, dt.U8, dst_scale=lambda r: _rq(r, 64, 128, 0, 0.3, 0.4),
                                     dst_zp=_zp(128)),
    "q_bf16_s8_per_row": lambda: _reorder(103, 48, 256, dt.BF16, dt.S8, dst_scale=lambda r: _rq(r, 48, 256, 1, 0.2, 0.9)),
    "q_f32_s8_per_col": lambda: _reorder(104, 32, 96, dt.F32, dt.S8, dst_scale=lambda r: _rq(r, 32, 96, 2, 0.2, 0.9)),
    "q_f32_s8_saturating": lambda: _reorder(105, 16, 64, dt.F32, dt.S8, spread=1e9,
                                            dst_scale=lambda r: _rq(r, 16, 64, 0, 0.5, 0.6)),
    "q_f32_s8_sum": lambda: _reorder(106, 40, 64, dt.F32, dt.S8, dst_scale=lambda r: _rq(r, 40, 64, 0, 0.5, 0.6),
                                      beta=0.5, dst_init=_sum_init),
    "q_f32_s8_transposed_src": lambda: _reorder(107, 64, 48, dt.F32, dt.S8, src_tag="ba",
                                                dst_scale=lambda r: _rq(r, 64, 48, 0, 0.5, 0.6)),
    "q_f32_u8_ragged": lambda: _reorder(108, 7, 13, dt.F32, dt.U8, dst_scale=lambda r: _rq(r, 7, 13, 2, 0.3, 0.9),
                                         dst_zp=_zp(100)),
    "q_f32_bf16_scaled": lambda: _reorder(109, 32, 64, dt.F32, dt.BF16, src_scale=lambda r: _rq(r, 32, 64, 0, 0.1, 0.2)),
    "dq_s32_f32_per_col": lambda: _reorder(110, 64, 128, dt.S32, dt.F32, src_scale=lambda r: _rq(r, 64, 128, 2, 1e-4, 1e-3)),
    "dq_s8_bf16_zp": lambda: _reorder(111, 64, 128, dt.S8, dt.BF16, src_scale=lambda r: _rq(r, 64, 128, 0, 0.01, 0.1),
                                       src_zp=_zp(3)),
    "dq_u8_f32_grouped_bf16_scales": lambda: _reorder(
        112, 64, 128, dt.U8, dt.F32, src_scale=lambda r: _rq(r, 64, 128, 3, 0.01, 0.1, dt.BF16, (8, 32)), src_zp=_zp(128)),
    "dq_u8_f32_grouped_narrow": lambda: _reorder(
        113, 32, 66, dt.U8, dt.F32, src_scale=lambda r: _rq(r, 32, 66, 3, 0.01, 0.1, dt.F32, (4, 2)), src_zp=_zp(7)),
    "rq_s8_u8_both_scales": lambda: _reorder(114, 64, 128, dt.S8, dt.U8, src_scale=lambda r: _rq(r, 64, 128, 0, 0.02, 0.03),
                                             dst_scale=lambda r: _rq(r, 64, 128, 0, 0.04, 0.05), src_zp=_zp(-2),
                                             dst_zp=_zp(120)),
    "rq_s32_s8_per_col_both": lambda: _reorder(115, 32, 64, dt.S32, dt.S8,
                                               src_scale=lambda r: _rq(r, 32, 64, 2, 1e-4, 1e-3),
                                               dst_scale=lambda r: _rq(r, 32, 64, 2, 0.2, 0.5), dst_zp=_zp(-5)),
    "rq_s8_s32_transposed_dst": lambda: _reorder(116, 24, 40, dt.S8, dt.S32, dst_tag="ba",
                                                 src_scale=lambda r: _rq(r, 24, 40, 0, 3.0, 4.0)),
    # 4-bit tensors: compressed weights back to a float type (scales / zero-points per column or
    # per K group, as the decompression matmul takes them), and the plain conversions
    "dq_u4_f32_per_col_zp": lambda: _reorder(117, 64, 96, dt.U4, dt.F32, src_scale=lambda r: _rq(r, 64, 96, 2, 0.01, 0.1),
                                             src_zp=_zp(7)),
    "dq_s4_bf16_grouped": lambda: _reorder(118, 128, 48, dt.S4, dt.BF16,
                                           src_scale=lambda r: _rq(r, 128, 48, 3, 0.01, 0.1, dt.F32, (32, 1))),
    "dq_u4_f16_grouped_zp": lambda: _reorder(
        119, 64, 32, dt.U4, dt.F16, src_scale=lambda r: _rq(r, 64, 32, 3, 0.01, 0.1, dt.F32, (16, 2)),
        src_zp=lambda r: Quant(r.integers(0, 16, (64 // 16) * (32 // 2)).astype(np.int32), dt.S32, 3, (16, 2))),
    "dq_s4_f32_plain": lambda: _reorder(120, 9, 14, dt.S4, dt.F32),
    "q_f32_s4_plain": lambda: _reorder(121, 33, 20, dt.F32, dt.S4, spread=5.0),
    "q_f32_u4_plain": lambda: _reorder(122, 16, 64, dt.F32, dt.U4, spread=9.0),
}


def build_reorder(name):
    c = REORDER_CASES[name]()
    c.name = name
    return c
