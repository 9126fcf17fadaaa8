"""Data-type encodings: the oracle's scalar conversions against independent numpy code."""
import ctypes as C

import numpy as np

from onednn_b200 import dtypes as dt
from oracle import binding as B


def _store(dtc, vals, raw_dtype):
    out = np.zeros(len(vals), dtype=raw_dtype)
    for i, v in enumerate(vals):
        B.lib().orc_store_float(dtc, C.c_float(float(v)), out.ctypes.data, i)
    return out


def test_e4m3_decode_all_codes():
    raw = np.arange(256, dtype=np.uint8)
    got = np.array([B.lib().orc_load_float(dt.F8_E4M3, raw.ctypes.data, i) for i in range(256)], dtype=np.float32)
    want = dt.e4m3_to_f32(raw)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    assert want[0x7E] == 448.0 and want[0x08] == 2.0 ** -6 and want[0x01] == 2.0 ** -9


def test_e4m3_encode_round_trip_and_ties():
    raw = np.array([c for c in range(256) if (c & 0x7F) != 0x7F], dtype=np.uint8)
    vals = dt.e4m3_to_f32(raw)
    assert np.array_equal(_store(dt.F8_E4M3, vals, np.uint8) & 0x7F | (raw & 0x80), raw | (raw & 0x80))
    # 464 is the tie between 448 and 480 (not representable): rounds to 448; above it overflows to NaN
    assert _store(dt.F8_E4M3, [464.0, 465.0, -1000.0], np.uint8).tolist() == [0x7E, 0x7F, 0xFF]
    # ties go to the even mantissa
    assert _store(dt.F8_E4M3, [1.0625, 1.1875], np.uint8).tolist() == [0x38, 0x3A]
    r = np.random.default_rng(0)
    x = np.clip(r.normal(0, 40, 4000), -448, 448).astype(np.float32)
    # inputs that already are f16 values see a single rounding, as in the numpy helper
    x = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(_store(dt.F8_E4M3, x, np.uint8), dt.f32_to_e4m3(x))


def test_bf16_rne():
    r = np.random.default_rng(1)
    x = r.normal(0, 100, 5000).astype(np.float32)
    assert np.array_equal(_store(dt.BF16, x, np.uint16), dt.f32_to_bf16(x))
    assert _store(dt.BF16, [1.00390625], np.uint16)[0] == 0x3F80  # tie -> even


def test_int_saturation_and_rne():
    assert _store(dt.S8, [126.5, 127.5, -128.5, 0.5, 1.5, 2.5, -0.5, 300, -300], np.int8).tolist() == \
        [126, 127, -128, 0, 2, 2, 0, 127, -128]
    assert _store(dt.U8, [-3, 254.5, 255.5, 0.5], np.uint8).tolist() == [0, 254, 255, 0]
    assert _store(dt.S32, [3e9, -3e9, 2.5], np.int32).tolist() == [2147483520, -2147483648, 2]


def test_int4_nibble_order():
    raw = np.array([0x21, 0xF8], dtype=np.uint8)
    got_u = [int(B.lib().orc_load_float(dt.U4, raw.ctypes.data, i)) for i in range(4)]
    got_s = [int(B.lib().orc_load_float(dt.S4, raw.ctypes.data, i)) for i in range(4)]
    assert got_u == [1, 2, 8, 15] and got_s == [1, 2, -8, -1]
    assert dt.unpack_int4(raw, False).tolist() == got_u and dt.unpack_int4(raw, True).tolist() == got_s
    assert np.array_equal(dt.pack_int4(np.array(got_s)), raw)


def test_portable_tanh_accuracy():
    xs = np.concatenate([np.linspace(-12, 12, 4001), np.logspace(-8, 1, 500)])
    got = np.array([B.lib().orc_tanh_portable(float(x)) for x in xs])
    assert np.max(np.abs(got - np.tanh(xs)) / np.maximum(np.abs(np.tanh(xs)), 1e-300)) < 4e-15
