"""In-tree build of libgtopk_b200.so (sm_100a only).

Every kernel file is plain CUDA with an ``extern "C"`` launcher, so nothing
here needs the PyTorch headers and a full rebuild takes seconds.  The library
is written next to this file; a digest of the sources is stored beside it so
that an up-to-date library is never rebuilt (the GPU box receives the built
file together with the sources).

Run ``python -m gtopkssgd_b200.ops.build`` to build, ``--force`` to rebuild,
``--verbose`` to print the ptxas resource usage of every kernel.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_NAME = "libgtopk_b200.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
DIGEST_PATH = LIB_PATH + ".digest"
OBJ_DIR = os.path.join(HERE, "build")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def sources() -> list[str]:
    names = sorted(f for f in os.listdir(CSRC) if f.endswith((".cu", ".cpp")))
    return [os.path.join(CSRC, n) for n in names]


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cpp", ".cuh", ".h")):
            h.update(f.encode())
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(fh.read())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB_PATH) and os.path.exists(DIGEST_PATH)):
        return False
    with open(DIGEST_PATH) as fh:
        return fh.read().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source for sm_100a and link the shared library."""
    if not force and is_current():
        return LIB_PATH
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sources()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]
        if src.endswith(".cu") and verbose:
            cmd += ["-Xptxas", "-v"]
        if src.endswith(".cpp"):
            cmd = [nvcc, "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", CSRC, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, res.stdout, res.stderr))
        if verbose and (res.stdout or res.stderr):
            sys.stderr.write(res.stdout + res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, "-shared", *ARCH_FLAGS, "-o", tmp, *objs, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (res.stdout, res.stderr))
    os.replace(tmp, LIB_PATH)
    with open(DIGEST_PATH, "w") as fh:
        fh.write(_digest())
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
