"""Builds the CUDA library in-tree: csrc/*.cu -> libqkmoe.so (sm_100a only).

    python qwen-kernel_b200/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  Objects go to csrc/build/ (ignored by git);
the shared library sits beside this file so it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libqkmoe.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler",
              "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function", "-Xptxas", "-v"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for f in sorted(os.listdir(root)):
            p = os.path.join(root, f)
            if os.path.isfile(p) and f.endswith((".cu", ".cuh", ".h", ".inc")):
                h.update(f.encode())
                h.update(open(p, "rb").read())
    h.update(" ".join(ARCH + NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if sources changed since the last build; returns the library path."""
    bdir = os.path.join(CSRC, "build")
    os.makedirs(bdir, exist_ok=True)
    stamp = os.path.join(bdir, "stamp")
    dig = _digest()
    if not force and os.path.exists(OUT) and os.path.exists(stamp) and open(stamp).read() == dig:
        return OUT
    cc = nvcc()

    def one(src):
        obj = os.path.join(bdir, src[:-3] + ".o")
        cmd = [cc, *ARCH, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for src, obj, r in ex.map(one, _sources()):
            log = (r.stdout + r.stderr).strip()
            open(os.path.join(bdir, src[:-3] + ".log"), "w").write(log)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}:\n{log}")
            if verbose and log:
                print(f"== {src}\n{log}")
            objs.append(obj)
    r = subprocess.run([cc, *ARCH, "-shared", "-o", OUT, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    open(stamp, "w").write(dig)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
