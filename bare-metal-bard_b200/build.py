"""Build libbmb.so (the CUDA kernels and the C ABI) for sm_100a with nvcc, and the
bmb_train_gpt driver that links against it.

Run as a script (``python bare-metal-bard_b200/build.py``) or call
``build_library()``.  Objects go to ``build/`` at the repository root and the
shared library is written next to this file, where the ctypes loader in
``__init__.py`` looks for it.  Only files whose sources (or common headers)
are newer than their object are recompiled.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJDIR = os.path.join(ROOT, "build", "bmb")
LIB = os.path.join(HERE, "libbmb.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
] + os.environ.get("BMB_NVCC_FLAGS", "").split()      # e.g. -DBMB_FLASH_TRACE for the developer phase timers


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    m = 0.0
    for d in (CSRC, os.path.join(ROOT, "include")):
        for f in os.listdir(d):
            if f.endswith((".h", ".cuh")):
                m = max(m, os.path.getmtime(os.path.join(d, f)))
    return m


def _compile(src, hdr_m, verbose):
    obj = os.path.join(OBJDIR, src[:-3] + ".o")
    srcp = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(srcp), hdr_m):
        return obj, ""
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", srcp, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj, r.stderr


def build_library(verbose=False, force=False):
    os.makedirs(OBJDIR, exist_ok=True)
    hdr_m = float("inf") if force else _headers_mtime()
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        res = list(ex.map(lambda s: _compile(s, hdr_m, verbose), srcs))
    objs = [o for o, _ in res]
    if verbose:
        for _, log in res:
            if log:
                sys.stderr.write(log)
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < newest:
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs + [
            "-lcuda", "-ldl", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    build_cli()
    return LIB


def build_cli():
    """bmb_train_gpt, the training driver over the C ABI (host C++ only), next to the library."""
    src = os.path.join(HERE, "cli", "bmb_train_gpt.cpp")
    exe = os.path.join(HERE, "bmb_train_gpt")
    newest = max(os.path.getmtime(src), os.path.getmtime(LIB), os.path.getmtime(os.path.join(ROOT, "include", "bmb.h")))
    if os.path.exists(exe) and os.path.getmtime(exe) > newest:
        return exe
    cmd = ["nvcc", "-O2", "-std=c++17", "-I", os.path.join(ROOT, "include"), src, "-o", exe, "-L", HERE, "-lbmb",
           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building bmb_train_gpt failed:\n%s\n%s" % (r.stdout, r.stderr))
    return exe


if __name__ == "__main__":
    print(build_library(verbose="-v" in sys.argv, force="-f" in sys.argv))
