#!/usr/bin/env python3
"""Regenerates tests/golden/reference_outputs.npz from the reference library.

Run in a container that has the reference tree and a built
``oracle/_ref/librefrun.so`` (``python oracle/build_ref.py``).  For every case
of ``tests/cases.py`` the reference's scalar implementation (``ref_int8:any``
for int8 sources, ``ref:any`` otherwise) is executed on its CPU engine through
its public C API, and the raw destination bytes are stored: in full when they
are at most 64 KiB, otherwise as a SHA-256 digest plus every 61st byte.
The int8 cases are stored a second time under ``tame/<name>``: the same attributes on small
integers and power-of-two scales, where the reference's f32 accumulation is exact.
A digest of the regenerated inputs is stored too, so that a change in numpy's
random streams is detected instead of reported as a parity failure.

tests/golden/reorder_outputs.npz is made the same way from the quantising
reorders of ``cases.REORDER_CASES``, each run through the implementation the
reference dispatches for it (its JIT reorder or the generic ``simple:any``).
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import cases  # noqa: E402
from oracle import binding as B  # noqa: E402


def input_digest(c):
    h = hashlib.sha256()
    for a in (c.src, c.wei, c.bias, c.dst_init):
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    for q in (c.src_scale, c.wei_scale, c.dst_scale, c.src_zp, c.wei_zp, c.dst_zp):
        if q is not None:
            h.update(np.ascontiguousarray(q.data).tobytes())
    for p in c.post_ops:
        if p.data is not None:
            h.update(np.ascontiguousarray(p.data).tobytes())
    return h.hexdigest()


def reorder_input_digest(c):
    h = hashlib.sha256()
    for a in (c.src, c.dst_init):
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    for q in (c.src_scale, c.dst_scale, c.src_zp, c.dst_zp):
        if q is not None:
            h.update(np.ascontiguousarray(q.data).tobytes())
    return h.hexdigest()


def make_reorders():
    out = {}
    for name in cases.REORDER_CASES:
        c = cases.build_reorder(name)
        dst, impl = B.run_reference_reorder(c)
        raw = np.ascontiguousarray(dst).view(np.uint8).reshape(-1)
        out[name + "/impl"] = np.array(impl)
        out[name + "/inputs_sha256"] = np.array(reorder_input_digest(c))
        out[name + "/bytes"] = raw
        print("%-32s %-14s %8d bytes" % (name, impl, raw.size))
    np.savez_compressed(Path(__file__).with_name("reorder_outputs.npz"), **out)


def main():
    make_reorders()
    out = {}
    for name in list(cases.CASES) + cases.tame_names():
        c = cases.build(name)
        dst, impl, _, _ = B.run_reference(c, impl="ref")
        raw = np.ascontiguousarray(dst).view(np.uint8).reshape(-1)
        out[name + "/impl"] = np.array(impl)
        out[name + "/inputs_sha256"] = np.array(input_digest(c))
        out[name + "/sha256"] = np.array(hashlib.sha256(raw.tobytes()).hexdigest())
        out[name + "/bytes"] = raw if raw.size <= 65536 else raw[::61].copy()
        print("%-32s %-14s %8d bytes" % (name, impl, raw.size))
    np.savez_compressed(Path(__file__).with_name("reference_outputs.npz"), **out)


if __name__ == "__main__":
    main()
