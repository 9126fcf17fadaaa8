"""Builds libonednn_b200.so in-tree: the sm_100a kernels plus the host C API.

``python -m onednn_b200.build`` (or ``build()``) compiles every ``.cu`` and
``.cpp`` under ``onednn_b200/csrc`` with nvcc for ``sm_100a`` only and links
them, with the CUDA runtime linked statically, into
``onednn_b200/libonednn_b200.so``.  nvcc cross-compiles without a GPU.
"""
import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libonednn_b200.so"
OBJ = PKG / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall",
          "-I", str(ROOT / "include"), "-I", str(CSRC / "kernels"), "-I", str(CSRC / "api")]


def _sources():
    return sorted(CSRC.rglob("*.cu")) + sorted(CSRC.rglob("*.cpp"))


def _headers_mtime():
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


def build(verbose=False, force=False):
    OBJ.mkdir(exist_ok=True)
    hm = _headers_mtime()
    jobs = []
    objs = []
    for src in _sources():
        o = OBJ / (src.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(o)
        if not force and o.exists() and o.stat().st_mtime >= max(src.stat().st_mtime, hm):
            continue
        cmd = [NVCC] + ARCH + COMMON + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(src), "-o", str(o)]
        if src.suffix == ".cpp":
            cmd.insert(1, "-x")
            cmd.insert(2, "cu")
        jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        p = subprocess.run(cmd, capture_output=True, text=True)
        return src, p.returncode, p.stdout + p.stderr

    failed = False
    with cf.ThreadPoolExecutor(max(1, min(8, os.cpu_count() or 1))) as ex:
        for src, rc, out in ex.map(run, jobs):
            if rc != 0 or verbose:
                print("== %s (rc=%d)\n%s" % (src.name, rc, out))
            failed |= rc != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if jobs or not LIB.exists():
        cmd = [NVCC] + ARCH + ["-shared", "-cudart", "static", "-o", str(LIB)] + [str(o) for o in objs] + \
            ["-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            print(p.stdout + p.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", LIB)
