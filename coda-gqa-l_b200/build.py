"""Build libcoda_b200.so (sm_100a) from csrc/ with nvcc, and the torch custom-op layer
libcoda_b200_torch.so (torch_ext/torch_binding.cpp, host C++ only) on top of it; no GPU is needed to compile.

    python coda-gqa-l_b200/build.py [--force] [--verbose]

Both libraries are written next to the Python package (coda_gqa_l_b200/).
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
OUT = os.path.join(HERE, "coda_gqa_l_b200", "libcoda_b200.so")
OBJ = os.path.join(HERE, "build")
TORCH_EXT_SRC = os.path.join(HERE, "torch_ext", "torch_binding.cpp")
TORCH_EXT_OUT = os.path.join(HERE, "coda_gqa_l_b200", "libcoda_b200_torch.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I", INCLUDE, "-I", CSRC,
]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for root in (CSRC, INCLUDE):
        for f in sorted(os.listdir(root)):
            p = os.path.join(root, f)
            if os.path.isfile(p):
                h.update(f.encode())
                h.update(open(p, "rb").read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    """g++ torch_ext/torch_binding.cpp -> libcoda_b200_torch.so, linked against libcoda_b200.so (found through
    $ORIGIN) and the installed torch.  Registers torch.ops.coda_b200.* when loaded with torch.ops.load_library."""
    import torch
    from torch.utils import cpp_extension
    h = hashlib.sha256()
    for p in (TORCH_EXT_SRC, os.path.join(INCLUDE, "coda_b200.h")):
        h.update(open(p, "rb").read())
    h.update(torch.__version__.encode())
    dig = h.hexdigest()
    stamp = os.path.join(OBJ, "torch_ext_digest.txt")
    if not force and os.path.exists(TORCH_EXT_OUT) and os.path.exists(stamp) and open(stamp).read() == dig:
        return TORCH_EXT_OUT
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-I", INCLUDE,
           *[a for d in cpp_extension.include_paths() for a in ("-isystem", d)], "-isystem", os.path.join(cuda_home, "include"),
           TORCH_EXT_SRC, "-o", TORCH_EXT_OUT, "-L", os.path.dirname(OUT), "-l:libcoda_b200.so", "-L", tlib,
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(f"== torch_binding.cpp\n{r.stdout}{r.stderr}\n")
    if r.returncode != 0:
        raise RuntimeError("building the torch custom-op layer failed")
    open(stamp, "w").write(dig)
    return TORCH_EXT_OUT


def build(force: bool = False, verbose: bool = False) -> str:
    path = build_kernels(force=force, verbose=verbose)
    build_torch_ext(force=force, verbose=verbose)
    return path


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    stamp = os.path.join(OBJ, "digest.txt")
    dig = _digest()
    if not force and os.path.exists(OUT) and os.path.exists(stamp) and open(stamp).read() == dig:
        return OUT
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(OBJ, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    objs = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        for src, obj, r in ex.map(compile_one, _sources()):
            if verbose or r.returncode != 0:
                sys.stderr.write(f"== {src}\n{r.stdout}{r.stderr}\n")
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src}")
            objs.append(obj)
    r = subprocess.run([nvcc, "-shared", "-o", OUT, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-lcuda"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    open(stamp, "w").write(dig)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
