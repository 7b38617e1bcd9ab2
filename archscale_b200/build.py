"""Build the in-tree sm_100a extension ``archscale_b200/_C.so``.

Kernels (``ops/csrc/*.cu``) are compiled straight with ``nvcc -gencode arch=compute_100a,code=sm_100a``
— they include no torch headers, so each takes seconds — and linked with the one torch-aware
translation unit ``bindings.cpp``.  Nothing is cached outside the repository: object files live in
``archscale_b200/_build/`` and are rebuilt when their source (or a header) is newer.

    python -m archscale_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import glob
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "ops", "csrc")
BUILD = os.path.join(PKG, "_build")
OUT = os.path.join(PKG, "_C.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(src: str, dst: str, headers) -> bool:
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(f) > t for f in [src, *headers])


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout, r.stderr)
    return r


def build(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(BUILD, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + \
        glob.glob(os.path.join(CSRC, "*.inc"))
    cu_files = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    jobs = []
    objs = []
    for src in cu_files:
        obj = os.path.join(BUILD, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            jobs.append([NVCC, *ARCH, "-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
                         "-Xptxas", "-v" if verbose else "-O3", "-I", CSRC, "-c", src, "-o", obj])
    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{sysconfig.get_paths()['include']}", f"-I{CSRC}"]
    bobj = os.path.join(BUILD, "bindings.cpp.o")
    bsrc = os.path.join(CSRC, "bindings.cpp")
    if force or _newer(bsrc, bobj, headers):
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        jobs.append(["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
                     "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-c", bsrc, "-o", bobj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    if jobs or force or not os.path.exists(OUT):
        libdirs = ce.library_paths(device_type="cuda")
        link = ["g++", "-shared", "-o", OUT, bobj, *objs]
        for d in libdirs:
            link += [f"-L{d}", f"-Wl,-rpath,{d}"]
        link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"]
        _run(link, verbose)
    return OUT


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))


if __name__ == "__main__":
    main()
