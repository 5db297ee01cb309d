"""Compile the CUDA sources under csrc/ into ucmx/_lib/libucmx.so for sm_100a, and the CPython front of the
retrieval object (csrc/pybackend.c, plain C) into ucmx/_lib/_ucmx_fast.<abi>.so.

Usage: python build.py [--force] [--verbose]
The library links the CUDA runtime statically and depends on nothing else, so the built file can
be carried to another machine with the same driver.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "ucmx", "_lib")
OUT = os.path.join(OUT_DIR, "libucmx.so")
STAMP = os.path.join(OUT_DIR, "libucmx.stamp")
PY_SRC = os.path.join(CSRC, "pybackend.c")
PY_OUT = os.path.join(OUT_DIR, "_ucmx_fast" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    files = _sources() + [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(".cuh")]
    files.append(os.path.join(INCLUDE, "ucmx.h"))
    files.append(PY_SRC)
    for f in files:
        with open(f, "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def up_to_date() -> bool:
    if not (os.path.exists(OUT) and os.path.exists(STAMP) and os.path.exists(PY_OUT)):
        return False
    with open(STAMP) as fh:
        return fh.read().strip() == _digest()


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and up_to_date():
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in _sources():
        obj = os.path.join(OUT_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, "-c", src, "-o", obj, "-I", INCLUDE] + NVCC_FLAGS
        if verbose:
            cmd += ["-Xptxas", "-v"]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{out}\n")
        elif verbose or "warning" in out:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("CUDA build failed")
    link = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                   "-cudart", "static", "-Xcompiler", "-fPIC"]
    subprocess.run(link, check=True)
    for o in objs:
        os.remove(o)
    build_python_front()
    with open(STAMP, "w") as fh:
        fh.write(_digest())
    return OUT


def build_python_front() -> str:
    """gcc: the CPython module that fronts ucmx_retrieval_* (no CUDA, no link against libucmx.so)."""
    import numpy
    cc = os.environ.get("CC") or shutil.which("gcc") or shutil.which("cc")
    if not cc:
        raise RuntimeError("no C compiler found (set CC)")
    cmd = [cc, "-O2", "-fPIC", "-shared", "-Wall", "-o", PY_OUT, PY_SRC,
           "-I", sysconfig.get_paths()["include"], "-I", numpy.get_include()]
    subprocess.run(cmd, check=True)
    return PY_OUT


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
