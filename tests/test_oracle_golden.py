"""The CPU oracle must reproduce the reference library's stored outputs.

tests/golden/reference_outputs.npz holds, for every case of tests/cases.py,
the destination bytes the reference's own scalar matmul produced (see
tests/golden/make_golden.py).  These tests run anywhere: they need neither the
reference tree nor a GPU.
"""
import hashlib
from pathlib import Path

import numpy as np
import pytest

import cases
from golden.make_golden import input_digest
from oracle import binding as B

GOLD = np.load(Path(__file__).parent / "golden" / "reference_outputs.npz")


@pytest.mark.parametrize("name", list(cases.CASES))
def test_oracle_matches_reference_golden(name):
    c = cases.build(name)
    if str(GOLD[name + "/inputs_sha256"]) != input_digest(c):
        pytest.skip("numpy produced different inputs than when the fixture was made")
    out = np.ascontiguousarray(B.run_oracle(c)).view(np.uint8).reshape(-1)
    want = GOLD[name + "/bytes"]
    got = out if out.size <= 65536 else out[::61]
    assert np.array_equal(got, want), "%d of %d stored bytes differ" % (int((got != want).sum()), want.size)
    assert hashlib.sha256(out.tobytes()).hexdigest() == str(GOLD[name + "/sha256"])


@pytest.mark.parametrize("name", cases.tame_names())
def test_exact_accumulation_mode_matches_reference_golden_on_exact_sums(name):
    """Where every f32 partial sum is exact, the reference's scalar implementation, the oracle
    that restates it and the oracle's exact-accumulation mode (the one the tensor-core kernel is
    held to) must all give the same bytes."""
    c = cases.build(name)
    if str(GOLD[name + "/inputs_sha256"]) != input_digest(c):
        pytest.skip("numpy produced different inputs than when the fixture was made")
    want = GOLD[name + "/bytes"]
    for exact_acc in (0, 1):
        out = np.ascontiguousarray(B.run_oracle(c, exact_acc=exact_acc)).view(np.uint8).reshape(-1)
        got = out if out.size <= 65536 else out[::61]
        assert np.array_equal(got, want), "exact_acc=%d: %d of %d stored bytes differ" % (
            exact_acc, int((got != want).sum()), want.size)
        assert hashlib.sha256(out.tobytes()).hexdigest() == str(GOLD[name + "/sha256"])


def test_every_case_has_a_fixture():
    for name in list(cases.CASES) + cases.tame_names():
        assert name + "/sha256" in GOLD.files
