"""Programs written against the reference library's own C++ header (dnnl.hpp) and linked with
libonednn_b200.so instead of libdnnl.so (built by oracle/build_ref.py where the reference's
headers are present; the binaries travel with the tree)."""
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).resolve().parents[1] / "oracle" / "_ref"


@pytest.mark.gpu
@pytest.mark.parametrize("name,impl", [("consumer_dnnl_hpp_int8_matmul", "cuda:sm100:tcgen05_i8"),
                                       ("consumer_dnnl_h_quantize_reorder", "cuda:reorder_quant"),
                                       ("consumer_dnnl_hpp_weights_decompression", "cuda:sm100:wc_gemv cuda:sm100:wc_tcgen05")])
def test_reference_api_program_runs_on_the_cuda_engine(name, impl):
    exe = BIN / name
    if not exe.exists():
        pytest.skip("%s was not built (needs the reference's headers)" % name)
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
    assert p.stdout.startswith("OK " + impl), p.stdout
