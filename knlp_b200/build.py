"""Build libknlp_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m knlp_b200.build [--force] [--verbose]

No GPU is needed to build.  Objects go to knlp_b200/csrc/build/, the library to
knlp_b200/libknlp_b200.so.  A file is recompiled when it or a header it includes is newer
than its object (headers are found by following the #include "..." lines).
"""

from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libknlp_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
          "-I", INCLUDE]
# per-file extras: the quantizer must never contract a*b+c or use fast division
EXTRA = {"quant_append.cu": ["-fmad=false", "-prec-div=true"]}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


_INC = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _deps_mtime(path: str, seen=None) -> float:
    """Newest modification time of a source file and the local headers it includes."""
    seen = set() if seen is None else seen
    path = os.path.normpath(path)
    if path in seen or not os.path.exists(path):
        return 0.0
    seen.add(path)
    t = os.path.getmtime(path)
    with open(path) as f:
        text = f.read()
    for inc in _INC.findall(text):
        for base in (os.path.dirname(path), INCLUDE):
            cand = os.path.join(base, inc)
            if os.path.exists(cand):
                t = max(t, _deps_mtime(cand, seen))
                break
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for src in _sources():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < _deps_mtime(s):
            cmd = [nvcc, *ARCH, *COMMON, *EXTRA.get(src, []), "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    need_link = force or bool(jobs) or not os.path.exists(LIB) or any(
        os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs)
    if need_link:
        cmd = [nvcc, *ARCH, "-shared", "-o", LIB, *objs, "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
