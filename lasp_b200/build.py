"""Build liblasp_b200.so in-tree with nvcc for sm_100a.

    python -m lasp_b200.build          # incremental
    python -m lasp_b200.build --force

The library links the CUDA runtime statically; the driver entry point of the TMA
tensor-map encoder is looked up at run time.  It has no torch dependency.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "liblasp_b200.so")
SOURCES = ["api.cu", "simt_kernels.cu", "fault_word.cu", "walk_kernels.cu", "relay_kernels.cu", "static_scratch.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _stale(out: str, deps) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu under csrc/ and link liblasp_b200.so; returns its path."""
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(ROOT, "include", "lasp_b200.h"))
    objs = []
    common = ARCH + ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-I", os.path.join(ROOT, "include"),
                     "-I", CSRC]
    if verbose:
        common += ["-Xptxas", "-v"]
    if os.environ.get("LASP_TRACE") == "1":
        common += ["-DLASP_TRACE"]
    procs = []
    for src in SOURCES:
        path = os.path.join(CSRC, src)
        if not os.path.exists(path):
            continue
        obj = os.path.join(CSRC, src[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [path] + headers):
            procs.append((src, subprocess.Popen([nvcc, "-c", path, "-o", obj] + common,
                                                stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if out.strip():
            print(f"[{src}]\n{out}", file=sys.stderr)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if force or procs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ARCH + ["-cudart", "static"]
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
