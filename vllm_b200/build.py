"""Build libb200q.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m vllm_b200.build [--force] [--verbose]

The library has no dependency on torch or Python; it is loaded with ctypes by
``vllm_b200._lib``.  Translation units are compiled in parallel.
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
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libb200q.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _units():
    """(source, object name, extra defines)"""
    units = [("capi.cu", "capi.o", []), ("repack.cu", "repack.o", [])]
    for bf16 in (0, 1):
        for bits in (4, 8):
            units.append(("gemm_stream_inst.cu", f"gemm_stream_{'bf16' if bf16 else 'f16'}_w{bits}.o",
                          [f"-DINST_BF16={bf16}", f"-DINST_BITS={bits}"]))
    for extra in ("gemm_tc.cu", "noalloc.cu", "allreduce.cu", "elementwise.cu"):
        if os.path.exists(os.path.join(CSRC, extra)):
            units.append((extra, extra.replace(".cu", ".o"), []))
    return units


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)) + ["../../include/b200q.h"]:
        path = os.path.join(CSRC, name)
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("B200Q_EXTRA_NVCC_FLAGS", "").encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    stamp = os.path.join(OBJ, "stamp")
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return LIB
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    nvcc = _nvcc()
    flags = NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    flags = flags + os.environ.get("B200Q_EXTRA_NVCC_FLAGS", "").split()

    def compile_one(unit):
        src, obj, defs = unit
        cmd = [nvcc, *flags, *defs, "-c", os.path.join(CSRC, src), "-o", os.path.join(OBJ, obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return unit, r

    units = _units()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        for unit, r in ex.map(compile_one, units):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"--- {unit[1]}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {unit[0]} {unit[2]}")
    objs = [os.path.join(OBJ, u[1]) for u in units]
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}{r.stderr}")
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
