"""Data-type codes and host-side (numpy) encodings used by the matmul path.

The integer codes are the values of ``dnnl_data_type_t`` in the reference's
``include/oneapi/dnnl/dnnl_common_types.h:78-110``.  Sub-byte and 16-bit
float types have no numpy dtype, so tensors of those types are carried as raw
``uint8`` / ``uint16`` arrays; the helpers here convert to and from float32.
"""
import numpy as np

UNDEF, F16, BF16, F32, S32, S8, U8 = 0, 1, 2, 3, 4, 5, 6
F8_E5M2, F8_E4M3, S4, U4 = 9, 10, 11, 12

NAMES = {F16: "f16", BF16: "bf16", F32: "f32", S32: "s32", S8: "s8", U8: "u8",
         F8_E5M2: "f8_e5m2", F8_E4M3: "f8_e4m3", S4: "s4", U4: "u4", UNDEF: "undef"}
CODES = {v: k for k, v in NAMES.items()}

# storage dtype of the raw numpy array that carries a tensor of the given type
RAW = {F16: np.uint16, BF16: np.uint16, F32: np.float32, S32: np.int32, S8: np.int8,
       U8: np.uint8, F8_E5M2: np.uint8, F8_E4M3: np.uint8, S4: np.uint8, U4: np.uint8}

BITS = {F16: 16, BF16: 16, F32: 32, S32: 32, S8: 8, U8: 8, F8_E5M2: 8, F8_E4M3: 8, S4: 4, U4: 4}


def nbytes(dt, nelems):
    return (nelems * BITS[dt] + 7) // 8


def f32_to_bf16(x):
    """float32 -> raw bf16 (round to nearest even; NaN kept quiet)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if np.any(nan):
        r = np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), r)
    return r


def bf16_to_f32(r):
    return (np.ascontiguousarray(r, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _e4m3_table():
    t = np.zeros(256, dtype=np.float32)
    for raw in range(256):
        s, e, m = raw >> 7, (raw >> 3) & 0xF, raw & 7
        if e == 0xF and m == 7:
            v = np.nan
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (8 + m) * 2.0 ** (e - 10)
        t[raw] = -v if s else v
    return t


E4M3_TABLE = _e4m3_table()


def e4m3_to_f32(r):
    return E4M3_TABLE[np.ascontiguousarray(r, dtype=np.uint8)]


def f32_to_e4m3(x):
    """float32 -> raw e4m3 for values already clipped to +-448 (nearest, ties to even)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    pos = E4M3_TABLE[:0x7F].astype(np.float64)  # 0 .. 448, ascending
    a = np.abs(x).astype(np.float64)
    hi = np.clip(np.searchsorted(pos, a, side="left"), 1, len(pos) - 1)
    lo = hi - 1
    dlo, dhi = a - pos[lo], pos[hi] - a
    pick_hi = (dhi < dlo) | ((dhi == dlo) & (hi % 2 == 0))
    code = np.where(pick_hi, hi, lo).astype(np.uint8)
    return np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)


def pack_int4(v):
    """int values (last axis even) -> packed nibbles, even index in the low nibble."""
    v = np.asarray(v).astype(np.int16) & 0xF
    return (v[..., 0::2] | (v[..., 1::2] << 4)).astype(np.uint8)


def unpack_int4(raw, signed):
    raw = np.asarray(raw, dtype=np.uint8)
    lo, hi = (raw & 0xF).astype(np.int16), (raw >> 4).astype(np.int16)
    out = np.stack([lo, hi], axis=-1).reshape(raw.shape[:-1] + (raw.shape[-1] * 2,))
    if signed:
        out = np.where(out >= 8, out - 16, out)
    return out


def to_f32(raw, dt):
    if dt == F32:
        return np.asarray(raw, dtype=np.float32)
    if dt == BF16:
        return bf16_to_f32(raw)
    if dt == F16:
        return np.asarray(raw, dtype=np.uint16).view(np.float16).astype(np.float32)
    if dt == F8_E4M3:
        return e4m3_to_f32(raw)
    if dt in (S32, S8, U8):
        return np.asarray(raw).astype(np.float32)
    if dt in (S4, U4):
        return unpack_int4(raw, dt == S4).astype(np.float32)
    raise ValueError("unsupported dt %r" % dt)


def from_f32(x, dt):
    x = np.asarray(x, dtype=np.float32)
    if dt == F32:
        return x.copy()
    if dt == BF16:
        return f32_to_bf16(x)
    if dt == F16:
        return x.astype(np.float16).view(np.uint16)
    if dt == F8_E4M3:
        return f32_to_e4m3(x)
    if dt == S32:
        return np.rint(x).astype(np.int32)
    if dt == S8:
        return np.clip(np.rint(x), -128, 127).astype(np.int8)
    if dt == U8:
        return np.clip(np.rint(x), 0, 255).astype(np.uint8)
    if dt in (S4, U4):
        return pack_int4(np.rint(x).astype(np.int16))
    raise ValueError("unsupported dt %r" % dt)
