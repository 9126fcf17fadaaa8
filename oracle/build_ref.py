#!/usr/bin/env python3
"""Compile the reference library's CPU matmul path straight from its sources.

TEST INFRASTRUCTURE ONLY.  Nothing here is part of the shipped product: the
result (``oracle/_ref/libdnnl_ref.so`` and ``oracle/_ref/librefrun.so``) is
used to pin the CPU restatement in ``oracle/oracle_matmul.c`` and as the timed
CPU baseline of ``bench.py --impl reference``.  It also compiles the programs of
``tests/consumer/`` against the reference's own ``dnnl.hpp`` and links them with the CUDA
engine's library (``oracle/_ref/consumer_*``).

The reference's own build system is not run.  This script plays the part of a
short Makefile: it lists the translation units of the reference's common
runtime and CPU engine (the same globs the reference's source lists use:
``src/common/*.cpp``, ``src/cpu/*.cpp``, ``src/cpu/{gemm,matmul,reorder,rnn,
jit_utils}/**``, ``src/cpu/x64/**``), writes the configuration headers the
sources include (``dnnl_config.h``, ``dnnl_version.h``, ``dnnl_version_hash.h``) into ``oracle/_ref/``
by filling in the reference's own templates, and calls ``g++`` on every file
where it lies in the reference tree.  No reference source is copied into this
repository; every output lands in ``oracle/_ref/`` which is git-ignored.

Usage:  python oracle/build_ref.py [--ref /path/to/oneDNN] [-j N]
"""
import argparse
import concurrent.futures as cf
import os
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"

ENABLED = {
    # only matmul and reorder implementation lists are populated
    "BUILD_TRAINING": 1, "BUILD_INFERENCE": 0,
    "BUILD_PRIMITIVE_ALL": 0, "BUILD_MATMUL": 1, "BUILD_REORDER": 1,
    "BUILD_PRIMITIVE_CPU_ISA_ALL": 1, "BUILD_PRIMITIVE_GPU_ISA_ALL": 0,
    "BUILD_GEMM_KERNELS_ALL": 1,
}
RUNTIME = {
    "DNNL_CPU_THREADING_RUNTIME": "DNNL_RUNTIME_OMP",
    "DNNL_CPU_RUNTIME": "DNNL_RUNTIME_OMP",
    "DNNL_GPU_RUNTIME": "DNNL_RUNTIME_NONE",
    "DNNL_GPU_VENDOR": "DNNL_VENDOR_NONE",
}


def gen_headers(ref: Path) -> Path:
    inc = OUT / "include" / "oneapi" / "dnnl"
    inc.mkdir(parents=True, exist_ok=True)
    text = (ref / "include/oneapi/dnnl/dnnl_config.h.in").read_text()
    out = []
    for line in text.splitlines():
        m = re.match(r"\s*#cmakedefine01\s+(\w+)", line)
        if m:
            out.append("#define %s %d" % (m.group(1), ENABLED.get(m.group(1), 0)))
            continue
        m = re.match(r"\s*#cmakedefine\s+(\w+)(.*)", line)
        if m:
            name = m.group(1)
            if name in RUNTIME:
                out.append("#define %s %s" % (name, RUNTIME[name]))
            else:
                out.append("/* #undef %s */" % name)
            continue
        out.append(line)
    (inc / "dnnl_config.h").write_text("\n".join(out) + "\n")

    top = (ref / "CMakeLists.txt").read_text()
    ver = re.search(r'PROJECT_VERSION\s+"(\d+)\.(\d+)\.(\d+)"', top)
    major, minor, patch = ver.groups() if ver else ("0", "0", "0")
    text = (ref / "include/oneapi/dnnl/dnnl_version.h.in").read_text()
    text = (text.replace("@DNNL_VERSION_MAJOR@", major)
                .replace("@DNNL_VERSION_MINOR@", minor)
                .replace("@DNNL_VERSION_PATCH@", patch)
                .replace("@DNNL_VERSION_HASH@", "unknown"))
    text = re.sub(r"@\w+@", "0", text)
    (inc / "dnnl_version.h").write_text(text)
    text = (ref / "include/oneapi/dnnl/dnnl_version_hash.h.in").read_text()
    text = text.replace("@DNNL_VERSION_HASH@", "N/A")
    (inc / "dnnl_version_hash.h").write_text(re.sub(r"@\w+@", "0", text))
    return OUT / "include"


def sources(ref: Path):
    src = ref / "src"
    files = sorted((src / "common").glob("*.cpp"))
    files = [f for f in files
             if f.name not in ("stream_threadpool.cpp", "logging.cpp")]
    files += sorted((src / "cpu").glob("*.cpp"))
    for sub in ("gemm", "matmul", "reorder", "rnn"):
        files += sorted((src / "cpu" / sub).rglob("*.cpp"))
    files += sorted((src / "cpu" / "jit_utils").glob("*.cpp"))
    files += sorted((src / "cpu" / "x64").rglob("*.cpp"))
    return files


def consumer_stamp(prog: Path) -> str:
    """Hash of everything a consumer program is compiled from on this side: its own source and
    the CUDA engine's public headers (it is compiled against the reference's headers, which do
    not change)."""
    import hashlib
    h = hashlib.sha256(prog.read_bytes())
    for hdr in sorted((HERE.parent / "include").glob("*.h")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def build_consumers(ref: Path, inc: Path, cxx: str = "/usr/bin/g++") -> int:
    """User programs written against the reference's own C and C++ headers, linked against the
    CUDA engine instead of the reference library (the drop-in claim, checked by
    tests/test_consumer.py).  Beside each binary goes ``<name>.sha256``, the stamp of the sources
    it was built from, so that a stale binary is noticed where it cannot be rebuilt."""
    eng_lib = HERE.parent / "onednn_b200" / "libonednn_b200.so"
    consumer = HERE.parent / "tests" / "consumer"
    for prog in sorted(list(consumer.glob("*.cpp")) + list(consumer.glob("*.c"))):
        if not eng_lib.exists():
            print("skipped %s: %s not built yet" % (prog.name, eng_lib.name))
            continue
        out = OUT / ("consumer_" + prog.stem)
        comp = [cxx, "-std=c++11"] if prog.suffix == ".cpp" else ["/usr/bin/gcc", "-std=c99"]
        cmd = comp + ["-O1", str(prog), "-I", str(ref / "include"), "-I", str(inc), "-L", str(eng_lib.parent),
                      "-lonednn_b200", "-lm", "-Wl,-rpath,$ORIGIN/../../onednn_b200", "-o", str(out)]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(p.stderr[-6000:])
            return 1
        (OUT / (out.name + ".sha256")).write_text(consumer_stamp(prog) + "\n")
        print("built", out)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("ONEDNN_REF", "/root/reference"))
    ap.add_argument("-j", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--cxx", default="/usr/bin/g++")
    ap.add_argument("--consumers-only", action="store_true", help="only (re)build the programs of tests/consumer")
    args = ap.parse_args()
    ref = Path(args.ref)
    if not (ref / "src/common/matmul.cpp").exists():
        print("reference tree not found at %s: nothing built" % ref)
        return 2
    inc = gen_headers(ref)
    if args.consumers_only:
        return build_consumers(ref, inc, args.cxx)
    obj = OUT / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    flags = [
        "-std=c++11", "-O2", "-fPIC", "-fopenmp", "-msse4.1", "-w",
        "-fvisibility=internal", "-fvisibility-inlines-hidden",
        "-DDNNL_DLL", "-DDNNL_DLL_EXPORTS", "-DDNNL_ENABLE_JIT_PROFILING=0",
        "-DDNNL_ENABLE_MAX_CPU_ISA", "-DDNNL_ENABLE_CPU_ISA_HINTS",
        "-D__STDC_LIMIT_MACROS", "-D__STDC_CONSTANT_MACROS", "-DNDEBUG",
        "-I", str(inc), "-I", str(ref / "include"), "-I", str(ref / "src"),
        "-I", str(ref / "third_party"),
    ]
    jobs = []
    for f in sources(ref):
        rel = f.relative_to(ref / "src")
        o = obj / (str(rel).replace("/", "__")[:-4] + ".o")
        opt = ["-O1"] if f.name.endswith("_kern_autogen.cpp") else []
        if o.exists() and o.stat().st_mtime >= f.stat().st_mtime:
            jobs.append((None, o))
        else:
            jobs.append(([args.cxx] + flags + opt + ["-c", str(f), "-o", str(o)], o))

    def run(job):
        cmd, o = job
        if cmd is None:
            return o, 0, ""
        p = subprocess.run(cmd, capture_output=True, text=True)
        return o, p.returncode, p.stderr[-2000:]

    failed = 0
    with cf.ThreadPoolExecutor(args.j) as ex:
        for i, (o, rc, err) in enumerate(ex.map(run, jobs)):
            if rc != 0:
                failed += 1
                print("FAILED %s\n%s" % (o.name, err), flush=True)
            elif i % 50 == 0:
                print("[%d/%d] %s" % (i, len(jobs), o.name), flush=True)
    if failed:
        print("%d translation units failed" % failed)
        return 1
    lib = OUT / "libdnnl_ref.so"
    cmd = [args.cxx, "-shared", "-fopenmp", "-o", str(lib)] + \
        [str(o) for _, o in jobs] + ["-Wl,-Bsymbolic", "-Wl,--no-undefined", "-s", "-ldl", "-lpthread"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        print(p.stderr[-6000:])
        return 1
    print("built", lib)
    runner = HERE / "ref_runner.cpp"
    if runner.exists():
        rlib = OUT / "librefrun.so"
        cmd = [args.cxx, "-std=c++14", "-O2", "-fPIC", "-shared", "-fopenmp",
               "-fvisibility=hidden", "-I", str(HERE), "-I", str(inc), "-I", str(ref / "include"),
               str(runner), "-o", str(rlib), "-L", str(OUT), "-ldnnl_ref",
               "-Wl,-rpath,$ORIGIN", "-Wl,-Bsymbolic"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(p.stderr[-6000:])
            return 1
        print("built", rlib)
    return build_consumers(ref, inc, args.cxx)


if __name__ == "__main__":
    sys.exit(main())
