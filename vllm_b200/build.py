"""Build the two in-tree libraries.

    python -m vllm_b200.build [--force] [--verbose]

lib/libb200q.so     the C-ABI CUDA library: nvcc, sm_100a, no dependency on torch or Python
                    (loaded with ctypes by ``vllm_b200._lib``); translation units are compiled
                    in parallel
lib/b200q_torch.so  the torch operator registration (csrc/torch_bindings.cpp): host compiler
                    only, against the torch of the running interpreter, linked to libb200q.so
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
TORCH_LIB = os.path.join(HERE, "lib", "b200q_torch.so")

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
        units.append((extra, extra.replace(".cu", ".o"), []))
    return units


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def _digest() -> str:
    h = hashlib.sha256()
    for name in sorted(n for n in os.listdir(CSRC) if n != "torch_bindings.cpp") + ["../../include/b200q.h"]:
        path = os.path.join(CSRC, name)
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("B200Q_EXTRA_NVCC_FLAGS", "").encode())
    return h.hexdigest()


def build_torch_extension(force: bool = False, verbose: bool = False) -> str:
    """g++ on csrc/torch_bindings.cpp -> lib/b200q_torch.so (needs lib/libb200q.so)."""
    import torch
    from torch.utils import cpp_extension as ce
    src = os.path.join(CSRC, "torch_bindings.cpp")
    h = hashlib.sha256()
    for path in (src, os.path.join(HERE, "..", "include", "b200q.h")):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(torch.__version__.encode())
    digest = h.hexdigest()
    stamp = os.path.join(OBJ, "stamp_torch")
    if not force and os.path.exists(TORCH_LIB) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return TORCH_LIB
    os.makedirs(OBJ, exist_ok=True)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", src, "-o", TORCH_LIB]
    cmd += [f"-I{p}" for p in ce.include_paths()] + [f"-I{os.path.join(cuda_home, 'include')}"]
    cmd += [f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", "-ltorch_cuda",
            f"-L{os.path.dirname(LIB)}", "-lb200q", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(f"--- b200q_torch.so\n{r.stdout}{r.stderr}\n")
    if r.returncode != 0:
        raise RuntimeError("g++ failed for torch_bindings.cpp")
    with open(stamp, "w") as f:
        f.write(digest)
    return TORCH_LIB


def build(force: bool = False, verbose: bool = False) -> str:
    _build_cuda_library(force, verbose)
    build_torch_extension(force, verbose)
    return LIB


def _build_cuda_library(force: bool = False, verbose: bool = False) -> str:
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
