"""The reference's own test driver on this engine.

oracle/build_benchdnn.py compiles the reference's benchdnn (matmul driver) against
libonednn_b200.so where the reference tree is present; the binary and the driver's input files
travel with the tree.  Here it runs the reference's own matmul batch files in correctness mode
on the CUDA engine (``--engine=gpu``): the driver fills its tensors through this library's host
engine and reorders, executes the primitive, computes its own scalar reference and compares
with its own per-data-type thresholds.  Recorded per batch: passed / skipped / unimplemented
(a valid problem no implementation here takes; the driver treats it as "not a failure" only
for known gaps, so the counts are kept visible) / failed.  The bar is zero failed cases.
"""
import os
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
BD = ROOT / "oracle" / "_ref" / "benchdnn"

# batch file -> cases that must at least pass (a floor, so that a run that silently skips everything is noticed)
BATCHES = [("test_matmul_int8", 1000), ("test_matmul_fp8", 1000), ("harness_matmul_decompression", 100),
           ("test_matmul_ci", 50), ("harness_matmul_runtime_int8", 500), ("harness_matmul_strides", 200)]


BUDGET_S = int(os.environ.get("B200_BENCHDNN_BUDGET_S", "75"))  # per batch file; the full files take minutes each


def run_batch(name, budget_s=BUDGET_S):
    """Runs one batch file; returns (finished, counts) where counts come from the driver's summary
    line, or -- when the time budget ran out first (some harnesses end in shapes whose scalar CPU
    reference takes minutes per case) -- from the per-case lines printed so far."""
    cmd = [str(BD / "benchdnn"), "--matmul", "--engine=gpu", "--mode=C", "--batch=inputs/matmul/" + name]
    try:
        p = subprocess.run(cmd, cwd=str(BD), capture_output=True, text=True, timeout=budget_s)
        out = p.stdout + p.stderr
    except subprocess.TimeoutExpired as ex:
        out = (ex.stdout or b"").decode(errors="replace") + (ex.stderr or b"").decode(errors="replace")
    m = re.search(r"tests:(\d+) passed:(\d+) skipped:(\d+) mistrusted:(\d+) unimplemented:(\d+) "
                  r"invalid_arguments:(\d+) failed:(\d+)", out)
    if m:
        tests, passed, skipped, mistrusted, unimpl, invalid, failed = (int(x) for x in m.groups())
        return True, dict(tests=tests, passed=passed, skipped=skipped, mistrusted=mistrusted, unimplemented=unimpl,
                          invalid_arguments=invalid, failed=failed - unimpl - invalid), out
    c = {k: len(re.findall(r"^\d+:%s" % tag, out, re.M)) for k, tag in
         (("passed", "PASSED"), ("skipped", "SKIPPED"), ("mistrusted", "MISTRUSTED"), ("unimplemented", "UNIMPLEMENTED"),
          ("invalid_arguments", "INVALID_ARGUMENTS"), ("failed", "FAILED"))}
    c["tests"] = sum(c.values())
    return False, c, out


@pytest.mark.gpu
@pytest.mark.parametrize("name,min_passed", BATCHES)
def test_reference_matmul_batch_on_the_cuda_engine(name, min_passed):
    if not (BD / "benchdnn").exists():
        pytest.skip("benchdnn was not built (needs the reference tree: python oracle/build_benchdnn.py)")
    finished, c, out = run_batch(name)
    print("%s: %s%s" % (name, " ".join("%s %d" % kv for kv in c.items()), "" if finished else " (time budget reached)"))
    # a driver that stops on an error of its own prints neither a summary nor further cases
    assert finished or "Error: Function" not in out.splitlines()[-1], "the driver stopped:\n" + out[-2000:]
    bad = [l for l in out.splitlines() if re.match(r"^\d+:FAILED", l)][:20]
    assert c["failed"] == 0, "\n".join(bad)
    assert c["invalid_arguments"] == 0
    assert c["passed"] >= min_passed
