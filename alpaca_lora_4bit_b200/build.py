"""Builds ``libq4b200.so`` (all CUDA kernels + the C ABI) in-tree with nvcc for sm_100a.

    python -m alpaca_lora_4bit_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is rebuilt when any source under ``csrc/`` or
``include/`` is newer than the ``.so``.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libq4b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    deps.append(os.path.abspath(__file__))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; libq4b200.so cannot be built")
    objdir = os.path.join(PKG, "build")
    os.makedirs(objdir, exist_ok=True)
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0 or verbose:
            sys.stderr.write(f"--- {os.path.basename(src)} ---\n{out}\n")
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = LIB + ".tmp"
    subprocess.check_call([nvcc, "-shared", "-o", tmp, *objs, "-Xcompiler", "-fPIC"])
    os.replace(tmp, LIB)
    return LIB


CALL_SRC = os.path.join(CSRC, "host", "q4call.c")
CALL_LIB = os.path.join(PKG, "_q4call.so")


def build_call(force: bool = False) -> str:
    """Builds ``_q4call.so`` (the CPython module that makes the per-token foreign call) with the C compiler."""
    if not force and os.path.exists(CALL_LIB) and os.path.getmtime(CALL_LIB) >= os.path.getmtime(CALL_SRC):
        return CALL_LIB
    import sysconfig
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        raise RuntimeError("no C compiler; _q4call.so cannot be built")
    tmp = CALL_LIB + ".tmp"
    subprocess.check_call([cc, "-O2", "-shared", "-fPIC", "-I", sysconfig.get_paths()["include"], CALL_SRC, "-o", tmp])
    os.replace(tmp, CALL_LIB)
    return CALL_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_call(force="--force" in sys.argv))
