"""Programs written against the reference library's own headers (dnnl.hpp, dnnl.h) and linked
with libonednn_b200.so instead of libdnnl.so.

oracle/build_ref.py compiles them where the reference's headers are present and leaves, beside
each binary, a stamp of the sources it was built from (the program and this library's public
headers).  Where the reference tree is present the binaries are rebuilt before the tests run;
elsewhere the prebuilt ones travel with the tree and a stamp that no longer matches the sources
fails the test instead of running a stale program."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
BIN = ROOT / "oracle" / "_ref"
SRC = ROOT / "tests" / "consumer"
sys.path.insert(0, str(ROOT))

PROGRAMS = [("dnnl_hpp_int8_matmul.cpp", "cuda:sm100:tcgen05_i8"),
            ("dnnl_h_quantize_reorder.c", "cuda:reorder_quant"),
            ("dnnl_hpp_weights_decompression.cpp", "cuda:sm100:wc_gemv cuda:sm100:wc_tcgen05")]


def _stamp(prog):
    from oracle.build_ref import consumer_stamp
    return consumer_stamp(prog)


@pytest.fixture(scope="session")
def consumers():
    ref = Path(os.environ.get("ONEDNN_REF", "/root/reference"))
    if (ref / "include/oneapi/dnnl/dnnl.hpp").exists() and (ROOT / "onednn_b200" / "libonednn_b200.so").exists():
        stale = [p for p, _ in PROGRAMS
                 if not (BIN / ("consumer_" + Path(p).stem + ".sha256")).exists()
                 or (BIN / ("consumer_" + Path(p).stem + ".sha256")).read_text().strip() != _stamp(SRC / p)]
        if stale:
            subprocess.check_call([sys.executable, str(ROOT / "oracle" / "build_ref.py"), "--consumers-only"],
                                  stdout=subprocess.DEVNULL)
    return BIN


@pytest.mark.parametrize("prog,impl", PROGRAMS)
def test_consumer_binary_matches_its_sources(consumers, prog, impl):
    exe = consumers / ("consumer_" + Path(prog).stem)
    if not exe.exists():
        pytest.skip("%s was not built (needs the reference's headers)" % exe.name)
    stamp = consumers / (exe.name + ".sha256")
    assert stamp.exists(), "no source stamp beside %s: rebuild with oracle/build_ref.py --consumers-only" % exe.name
    assert stamp.read_text().strip() == _stamp(SRC / prog), \
        "%s is older than %s or include/*.h: rebuild with oracle/build_ref.py --consumers-only" % (exe.name, prog)


@pytest.mark.gpu
@pytest.mark.parametrize("prog,impl", PROGRAMS)
def test_reference_api_program_runs_on_the_cuda_engine(consumers, prog, impl):
    exe = consumers / ("consumer_" + Path(prog).stem)
    if not exe.exists():
        pytest.skip("%s was not built (needs the reference's headers)" % exe.name)
    stamp = consumers / (exe.name + ".sha256")
    assert stamp.exists() and stamp.read_text().strip() == _stamp(SRC / prog), "stale binary: " + exe.name
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.startswith("OK " + impl), p.stdout
